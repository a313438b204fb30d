"""The tensors that describe one step to the parts: which tokens, of which
sequences, at which positions, and where their keys and values live.

The reference passes ``(token, position)`` for one sequence
(inference/InferenceEngine.java:180-182) and keeps ``[position, seqLen]`` on the
device so that a captured graph can be replayed (java21
inference/CudaForwardPass.java:138-141, :1283-1292). Here a step carries the new
tokens of a whole batch, packed sequence after sequence; all of its integers go
to the device in one copy.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch


@dataclass(frozen=True)
class SequenceStep:
    """One sequence's share of a step."""
    slot: int
    start: int            # offset of its first new token among the step's tokens
    num_new: int
    first_position: int   # position of its first new token = its length before the step


class Workspace:
    """Named scratch buffers that persist across steps and only ever grow."""

    def __init__(self, device):
        self.device = device
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self.version = 0      # bumped whenever a buffer moved (captured graphs are stale then)

    def get(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        count = 1
        for s in shape:
            count *= int(s)
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < count:
            buf = torch.empty(max(count, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.version += 1
        return buf[:count].view(*shape)


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class StepContext:
    """Device-side description of a step plus the host-side list of its sequences.

    Device tensors (all int32): ``tokens[T]``, ``positions[T]``, ``seq_ids[T]``
    (index of the token's sequence in this step), ``slots[B]``, ``q_start[B+1]``,
    ``kv_len[B]`` (length after the step), ``page_tables[g][B, P_g]`` per cache group,
    ``rows[W]`` (tokens whose logits are wanted).
    """

    def __init__(self, workspace: Workspace, sequences: List[SequenceStep], tokens: Sequence[int],
                 page_tables: List[List[List[int]]], wanted_rows: Sequence[int], *,
                 min_table_width: int = 1, meta_name: str = "step_meta"):
        self.workspace = workspace
        self.sequences = sequences
        self.num_tokens = T = len(tokens)
        self.num_sequences = B = len(sequences)
        self.max_new = max((s.num_new for s in sequences), default=0)
        self.all_single = all(s.num_new == 1 for s in sequences)
        self.max_kv_len = max((s.first_position + s.num_new for s in sequences), default=0)
        self.num_wanted = W = len(wanted_rows)

        widths = [max([min_table_width] + [len(t) for t in group]) for group in page_tables]
        sizes = [T, T, T, B, B + 1, B] + [B * w for w in widths] + [W]
        offsets, total = [], 0
        for n in sizes:
            offsets.append(total)
            total += _round_up(max(n, 1), 4)          # keep every array 16-byte aligned
        host = torch.zeros(total, dtype=torch.int32)
        view = host.numpy()
        o = offsets
        view[o[0]:o[0] + T] = tokens
        for i, s in enumerate(sequences):
            view[o[1] + s.start:o[1] + s.start + s.num_new] = range(s.first_position, s.first_position + s.num_new)
            view[o[2] + s.start:o[2] + s.start + s.num_new] = i
            view[o[3] + i] = s.slot
            view[o[4] + i] = s.start
            view[o[5] + i] = s.first_position + s.num_new
        view[o[4] + B] = T
        for g, group in enumerate(page_tables):
            base, w = o[6 + g], widths[g]
            for i, table in enumerate(group):
                view[base + i * w:base + i * w + len(table)] = table
        view[o[-1]:o[-1] + W] = wanted_rows

        meta = workspace.get(meta_name, (total,), torch.int32)
        self.h2d_bytes = total * 4
        meta.copy_(host.pin_memory() if torch.cuda.is_available() else host, non_blocking=False)
        self.meta = meta
        self.tokens = meta[o[0]:o[0] + T]
        self.positions = meta[o[1]:o[1] + T]
        self.seq_ids = meta[o[2]:o[2] + T]
        self.slots = meta[o[3]:o[3] + B]
        self.q_start = meta[o[4]:o[4] + B + 1]
        self.kv_len = meta[o[5]:o[5] + B]
        self.page_tables = [meta[o[6 + g]:o[6 + g] + B * w].view(B, w) for g, w in enumerate(widths)]
        self.rows = meta[o[-1]:o[-1] + W]

    def buffer(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        return self.workspace.get(name, shape, dtype)

    # A norm can zero, on the side, the buffer that the product after it sums into. The
    # block says so here, and the product picks the note up (once).
    _cleared = False

    def note_cleared(self) -> None:
        self._cleared = True

    def take_cleared(self) -> bool:
        was, self._cleared = self._cleared, False
        return was
