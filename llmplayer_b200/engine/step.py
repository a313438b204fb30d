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


class _NoEvent:
    """Stands in for a CUDA event where copies are synchronous (no GPU)."""

    def record(self) -> None:
        pass

    def synchronize(self) -> None:
        pass


class Workspace:
    """Named scratch buffers that persist across steps and only ever grow."""

    def __init__(self, device):
        self.device = device
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._pinned: Dict[str, tuple] = {}
        self._kept_zero = set()
        self.version = 0      # bumped whenever a buffer moved (captured graphs are stale then)

    def pinned(self, name: str, count: int):
        """A page-locked int32 host buffer of at least ``count`` entries and the event that marks
        the end of the last copy out of it; both persist, and the buffer is waited for before reuse."""
        entry = self._pinned.get(name)
        if entry is None or entry[0].numel() < count:
            host = torch.zeros(max(count, 256), dtype=torch.int32)
            event = None
            if torch.cuda.is_available() and torch.device(self.device).type == "cuda":
                host = host.pin_memory()
                event = torch.cuda.Event()
            entry = (host, event if event is not None else _NoEvent())
            self._pinned[name] = entry
        else:
            entry[1].synchronize()
        return entry

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

    def get_zeroed(self, name: str, count: int) -> torch.Tensor:
        """A float32 buffer of ``count`` values that is zero when first handed out and that its users
        promise to leave zero again after each use (partial sums that meet in atomics)."""
        key = (name, torch.float32)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < count:
            buf = torch.zeros(max(count, 1), dtype=torch.float32, device=self.device)
            self._buffers[key] = buf
            self._kept_zero.add(key)
            self.version += 1
        return buf[:count]

    def get_counters(self, name: str, count: int) -> torch.Tensor:
        """An int32 buffer of ``count`` counters that is zero when first handed out and that its users leave
        zero again after each use (CTAs that count themselves; the last one sets the counter back)."""
        key = (name, torch.int32)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < count:
            buf = torch.zeros(max(count, 1024), dtype=torch.int32, device=self.device)
            self._buffers[key] = buf
            self._kept_zero.add(key)
            self.version += 1
        return buf[:count]

    def restore_zeroes(self) -> None:
        """After a step that broke off half-way: the buffers and counters that are zero between uses are
        made zero again."""
        for key in self._kept_zero:
            self._buffers[key].zero_()


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class StepContext:
    """Device-side description of a step plus the host-side list of its sequences.

    Device tensors (all int32, views of one buffer that is filled by one copy): ``tokens[T]``,
    ``positions[T]``, ``kv_len[B]`` (length after the step), ``seq_ids[T]`` (index of the token's
    sequence in this step), ``slots[B]``, ``q_start[B+1]``, ``page_tables[g][B, P_g]`` per cache
    group, ``rows[W]`` (tokens whose logits are wanted).

    A context of one token per sequence can be moved on to the next step of the same sequences
    (:meth:`advance`): only the tokens, positions and lengths are copied again.
    """

    def __init__(self, workspace: Workspace, sequences: List[SequenceStep], tokens: Sequence[int],
                 page_tables: List[List[List[int]]], wanted_rows: Sequence[int], *,
                 min_table_width: int = 1, meta_name: str = "step_meta"):
        self.workspace = workspace
        self._sequences: Optional[List[SequenceStep]] = sequences
        self.slot_list = [s.slot for s in sequences]
        self.first_positions = [s.first_position for s in sequences]
        self.new_counts = [s.num_new for s in sequences]
        self.num_tokens = T = len(tokens)
        self.num_sequences = B = len(sequences)
        self.max_new = max((s.num_new for s in sequences), default=0)
        self.all_single = all(s.num_new == 1 for s in sequences)
        self.max_kv_len = max((s.first_position + s.num_new for s in sequences), default=0)
        self.num_wanted = W = len(wanted_rows)
        self.wanted_rows = list(wanted_rows)
        # one token for each sequence and every sequence's logits wanted: the shape a decode step continues in
        self.continues_all = self.all_single and self.wanted_rows == list(range(B))

        widths = [max([min_table_width] + [len(t) for t in group]) for group in page_tables]
        self._widths = widths
        self._table_lengths = [[len(t) for t in group] for group in page_tables]
        # the arrays that change from one decode step to the next come first and lie together
        sizes = [T, T, B, T, B, B + 1] + [B * w for w in widths] + [W]
        offsets, total = [], 0
        for n in sizes:
            offsets.append(total)
            total += _round_up(max(n, 1), 4)          # keep every array 16-byte aligned
        self._offsets = o = offsets
        self._moving = offsets[3]                      # tokens, positions, kv_len: the first `_moving` ints
        host, self._copied = workspace.pinned(meta_name, total)
        self._host = host
        view = self._view = host.numpy()
        view[:total] = 0
        view[o[0]:o[0] + T] = tokens
        for i, s in enumerate(sequences):
            view[o[1] + s.start:o[1] + s.start + s.num_new] = range(s.first_position, s.first_position + s.num_new)
            view[o[2] + i] = s.first_position + s.num_new
            view[o[3] + s.start:o[3] + s.start + s.num_new] = i
            view[o[4] + i] = s.slot
            view[o[5] + i] = s.start
        view[o[5] + B] = T
        for g, group in enumerate(page_tables):
            base, w = o[6 + g], widths[g]
            for i, table in enumerate(group):
                view[base + i * w:base + i * w + len(table)] = table
        view[o[-1]:o[-1] + W] = wanted_rows

        meta = workspace.get(meta_name, (total,), torch.int32)
        self._total = total
        self.meta = meta
        self._upload_views: Dict[int, tuple] = {}
        self._pinned = host.is_pinned()
        self.graph_key = None                          # set by the engine: what a captured graph of this step depends on
        self.fused_key = None
        self.host_pointer = host.data_ptr()
        self.moving_offsets = (o[0], o[1], o[2])
        self.moving_bytes = self._moving * 4
        self._upload(total)
        self.tokens = meta[o[0]:o[0] + T]
        self.positions = meta[o[1]:o[1] + T]
        self.kv_len = meta[o[2]:o[2] + B]
        self.seq_ids = meta[o[3]:o[3] + T]
        self.slots = meta[o[4]:o[4] + B]
        self.q_start = meta[o[5]:o[5] + B + 1]
        self.page_tables = [meta[o[6 + g]:o[6 + g] + B * w].view(B, w) for g, w in enumerate(widths)]
        self.rows = meta[o[-1]:o[-1] + W]

    @property
    def sequences(self) -> List[SequenceStep]:
        """The step's sequences (rebuilt on demand after :meth:`advance`, which only moves the positions on)."""
        if self._sequences is None:
            self._sequences = [SequenceStep(slot, i, 1, pos)
                               for i, (slot, pos) in enumerate(zip(self.slot_list, self.first_positions))]
        return self._sequences

    def _upload(self, count: int, record: bool = True) -> None:
        """Copy the first ``count`` integers of the pinned host image to the device, asynchronously;
        the event lets the next writer of the host image wait until the copy has read it
        (``record=False`` while a graph is being captured: the graph's user waits for the whole step)."""
        self.h2d_bytes = count * 4
        views = self._upload_views.get(count)
        if views is None:
            views = self._upload_views[count] = (self.meta[:count], self._host[:count])
        if self._pinned:
            views[0].copy_(views[1], non_blocking=True)
            if record:
                self._copied.record()
        else:
            views[0].copy_(views[1])

    def upload_all(self) -> None:
        self._upload(self._total)

    def upload_moving(self, record: bool = True) -> None:
        """Copy tokens, positions and lengths (what changes from one decode step to the next) to the device."""
        self._upload(self._moving, record)

    def moved_on(self, steps: int) -> None:
        """The host image was moved on by ``steps`` further decode steps outside this object (the native
        host loop): bring the host-side counters along."""
        if steps:
            self.first_positions = [p + steps for p in self.first_positions]
            self._sequences = None
            self.max_kv_len += steps

    def advance(self, tokens: Sequence[int], page_tables: List[List[List[int]]], upload: bool = True):
        """Move a context of one token per sequence on by one step: new tokens, positions and
        lengths one further, page tables as they are now. None if the tables outgrew the
        context's shape (the caller then builds a new context); else whether the page tables changed.
        ``upload=False``: only the host image is written; the caller copies it to the device."""
        o, B = self._offsets, self.num_sequences
        grown = False
        for g, group in enumerate(page_tables):
            for i, table in enumerate(group):
                if len(table) > self._widths[g]:
                    return None
                if len(table) != self._table_lengths[g][i]:
                    grown = True
        self._copied.synchronize()                     # the previous copy has read the host image
        view = self._view
        view[o[0]:o[0] + B] = tokens
        view[o[1]:o[1] + B] += 1
        view[o[2]:o[2] + B] += 1
        if grown:
            for g, group in enumerate(page_tables):
                base, w = o[6 + g], self._widths[g]
                for i, table in enumerate(group):
                    view[base + i * w:base + i * w + len(table)] = table
                    self._table_lengths[g][i] = len(table)
        self.first_positions = [p + 1 for p in self.first_positions]
        self._sequences = None
        self.max_kv_len += 1
        self._cleared = False
        if upload:
            self._upload(self._total if grown else self._moving)
        return grown

    def buffer(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        return self.workspace.get(name, shape, dtype)

    def angles(self, rotation) -> torch.Tensor:
        """(cos, sin) of every token's position times each of the rotation's frequencies, float32
        [T, rotary_dim / 2, 2]; formed once per step and table of frequencies."""
        from ..kernels import ops
        cache = self.__dict__.setdefault("_angles", {})
        key = (rotation.inv_freq.data_ptr(), rotation.rotary_dim)
        table = cache.get(key)
        if table is None:
            table = self.workspace.get(f"angles{len(cache)}", (self.num_tokens, rotation.rotary_dim // 2, 2), torch.float32)
            ops.rope_angles(self.positions, rotation, table)
            cache[key] = table
        return table

    def counters(self, name: str, count: int) -> torch.Tensor:
        return self.workspace.get_counters(name, count)

    # A norm can zero, on the side, the buffer that the product after it sums into. The
    # block says so here, and the product picks the note up (once).
    _cleared = False

    def note_cleared(self) -> None:
        self._cleared = True

    def take_cleared(self) -> bool:
        was, self._cleared = self._cleared, False
        return was
