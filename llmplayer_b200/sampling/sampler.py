"""Per-request sampler state on the host and the batched call of the sampling kernel.

The reference keeps, per request, a random generator, the recently sampled tokens
(at most max(64, dry range)) and the mirostat threshold mu
(sampler/CompositeSampler.java:14-31). The same state lives here in
:class:`SequenceSampler`; what depends on the logits runs on the device, one
block per sequence (csrc/sampling.cu).
"""
from __future__ import annotations

import math
from collections import Counter
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from ..kernels import ops
from .java_random import JavaRandom
from .params import SamplerConfig

PARAMS_DTYPE = np.dtype([
    ("inv_temperature", "<f4"), ("top_k", "<i4"), ("top_p", "<f4"), ("min_p", "<f4"),
    ("mirostat_threshold", "<f4"), ("uniform", "<f4"), ("edit_begin", "<i4"), ("edit_count", "<i4"),
    ("logits_row", "<i4"),
])


class SequenceSampler:
    def __init__(self, config: SamplerConfig):
        self.config = config
        self.rng = JavaRandom(config.seed)
        self.recent: List[int] = []
        self.max_recent = max(64, config.dry_range)
        self.mu = 2.0 * config.mirostat_tau
        self._powers = [1.0]         # powers of the repetition penalty, by number of occurrences
        # the first maximum of the logits as they are: nothing of this state enters the choice
        self.plain_greedy = config.is_greedy and config.repetition_penalty == 1.0 and config.dry_multiplier <= 0

    # ------------------------------------------------------------------ before a draw
    def edit_lists(self) -> Tuple[List[int], List[float], List[float]]:
        """The tokens whose logit changes, in ascending order, with the amount to subtract from each (DRY)
        and the factor of its repetition penalty: the penalty once per occurrence among the recent
        tokens (sampler/CompositeSampler.java:45-55), so the factor is the penalty multiplied up that often."""
        c = self.config
        counts = Counter(self.recent) if c.repetition_penalty != 1.0 else {}
        if c.dry_multiplier > 0:
            subtract: Dict[int, float] = {}
            for tok, pen in self._dry_penalties():
                subtract[tok] = subtract.get(tok, 0.0) + pen
            tokens = sorted(set(subtract) | set(counts))
            return (tokens, [subtract.get(tok, 0.0) for tok in tokens],
                    [self._penalty_power(counts.get(tok, 0)) for tok in tokens])
        if not counts:
            return [], [], []
        tokens = sorted(counts)
        self._penalty_power(max(counts.values()))
        powers = self._powers
        return tokens, [0.0] * len(tokens), [powers[counts[tok]] for tok in tokens]

    def logit_edits(self) -> List[Tuple[int, float, float]]:
        """(token, amount to subtract, penalty factor) for every token whose logit changes."""
        return list(zip(*self.edit_lists()))

    def _penalty_power(self, times: int) -> float:
        """1 * penalty * penalty ... (``times`` factors), multiplied up in that order."""
        powers = self._powers
        while len(powers) <= times:
            powers.append(powers[-1] * self.config.repetition_penalty)
        return powers[times]

    def _dry_penalties(self):
        """sampler/CompositeSampler.java:150-192: for each earlier occurrence of the last token,
        the length of the repeated suffix ending there; the token that followed it is penalised
        by multiplier * base^(length - allowed) once the length reaches the allowed one."""
        c, rec = self.config, self.recent
        n = len(rec)
        if n < 2:
            return
        start = n - min(n, c.dry_range)
        last = rec[-1]
        for p in range(start, n - 1):
            if rec[p] != last:
                continue
            length, pi, ni = 1, p - 1, n - 2
            while pi >= start and ni > p and rec[pi] == rec[ni]:
                length, pi, ni = length + 1, pi - 1, ni - 1
            if length >= c.dry_allowed_length:
                yield rec[p + 1], c.dry_multiplier * math.pow(c.dry_base, length - c.dry_allowed_length)

    def draw(self) -> float:
        """One uniform number per sampled token; none for a greedy choice."""
        return 0.0 if self.config.is_greedy else self.rng.next_float()

    def mirostat_threshold(self) -> float:
        return math.pow(2.0, -self.mu) if (self.config.mirostat == 2 and not self.config.is_greedy) else -1.0

    # ------------------------------------------------------------------ after a draw
    def accept(self, token: int, observed_probability: float) -> None:
        c = self.config
        if c.mirostat == 2 and not c.is_greedy and observed_probability > 0:
            surprise = -math.log2(observed_probability)
            self.mu -= c.mirostat_eta * (surprise - c.mirostat_tau)
        self.recent.append(int(token))
        if len(self.recent) > self.max_recent:
            self.recent.pop(0)


class BatchSampler:
    """Draws one token for each of several sequences from their rows of logits."""

    def __init__(self, vocab_size: int, device):
        self.vocab_size = vocab_size
        self.device = device
        self._work = None
        self._out = None
        self._host = None            # page-locked landing place of the results
        self._staging = None         # page-locked staging of the parameters and logit edits
        self._done = None
        self._constant = {}          # greedy batches without logit edits: parameters stay on the device
        self._dummy = None
        self._select = None          # scratch of the two-stage top-k
        self._slice_capacity = None
        self.last_h2d_bytes = 0
        self.last_d2h_bytes = 0

    def _stage(self, packed: np.ndarray) -> torch.Tensor:
        """``packed`` in page-locked memory that is kept from call to call (the previous call's copy out of it
        has finished: every call ends by waiting for its results)."""
        n = packed.size
        if self._staging is None or self._staging.numel() < n:
            self._staging = torch.empty(max(2 * n, 4096), dtype=torch.int32).pin_memory()
        self._staging[:n].numpy()[:] = packed
        return self._staging[:n]

    def _read_back(self, count: int, while_waiting) -> torch.Tensor:
        """The first ``count`` result words on the host. The copy is asynchronous into page-locked memory;
        ``while_waiting`` (a callable or None) runs on the host until the device has got there."""
        if self._host is None or self._host.numel() < count:
            self._host = torch.empty(max(count, 64), dtype=torch.int32).pin_memory()
            self._done = torch.cuda.Event()
        host = self._host[:count]
        host.copy_(self._out[:count], non_blocking=True)
        self._done.record()
        if while_waiting is not None:
            while_waiting()
        self._done.synchronize()
        return host

    def sample(self, logits: torch.Tensor, rows: Sequence[int], samplers: Sequence[SequenceSampler],
               while_waiting=None) -> List[int]:
        B = len(samplers)
        dev = self.device
        if self._work is None or self._work.shape[0] < B:
            self._work = torch.empty((B, self.vocab_size), dtype=torch.float32, device=dev)
            self._out = torch.empty(2 * B, dtype=torch.int32, device=dev)
            self._dummy = (torch.zeros(1, dtype=torch.int32, device=dev), torch.ones(1, dtype=torch.float32, device=dev))
            self._select = torch.empty(B * ops.sample_select_words(), dtype=torch.int32, device=dev)
            self._slice_capacity = ops.sample_slice_capacity(self.vocab_size)
        out_tok = self._out[:B]
        out_prob = self._out[B:2 * B].view(torch.float32)
        all_edits = [s.edit_lists() for s in samplers]
        plain_greedy = all(s.config.is_greedy for s in samplers) and not any(e[0] for e in all_edits)
        key = tuple(rows)
        if plain_greedy and list(rows) == list(range(B)) and logits.shape[0] == B:
            # first-maximum argmax of every row, spread over many blocks
            with ops.section("sample"):
                ops.argmax(logits, self._work.view(-1), out_tok)
            self.last_h2d_bytes = 0
            self.last_d2h_bytes = 4 * B
            chosen = self._read_back(B, while_waiting).tolist()
            for s, tok in zip(samplers, chosen):
                s.accept(tok, 1.0)
            return chosen
        if plain_greedy and key in self._constant:
            params_dev, edit_tok, edit_sub, edit_fac = self._constant[key], self._dummy[0], self._dummy[1], self._dummy[1]
            self.last_h2d_bytes = 0
        else:
            params = np.zeros(B, dtype=PARAMS_DTYPE)
            tokens, subs, facs = [], [], []
            for i, (row, s, (edit_tokens, edit_subs, edit_facs)) in enumerate(zip(rows, samplers, all_edits)):
                c = s.config
                params[i] = (0.0 if c.is_greedy else 1.0 / np.float32(c.temperature), c.top_k, c.top_p, c.min_p,
                             s.mirostat_threshold(), s.draw(), len(tokens), len(edit_tokens), row)
                tokens.extend(edit_tokens)
                subs.extend(edit_subs)
                facs.extend(edit_facs)
            # one upload: parameter records, then the edits' tokens, amounts and factors (4-byte units)
            n = max(1, len(tokens))
            packed = np.zeros(B * PARAMS_DTYPE.itemsize // 4 + 3 * n, dtype=np.int32)
            head = B * PARAMS_DTYPE.itemsize // 4
            packed[:head] = params.view(np.int32)
            packed[head:head + len(tokens)] = np.asarray(tokens, dtype=np.int32)
            packed[head + n:head + n + len(tokens)] = np.asarray(subs, dtype=np.float32).view(np.int32)
            fac_arr = np.ones(n, dtype=np.float32)
            fac_arr[:len(tokens)] = np.asarray(facs, dtype=np.float32)
            packed[head + 2 * n:head + 3 * n] = fac_arr.view(np.int32)
            blob = self._stage(packed).to(dev, non_blocking=True)
            self.last_h2d_bytes = packed.nbytes
            params_dev = blob[:head].view(torch.uint8)
            edit_tok = blob[head:head + n]
            edit_sub = blob[head + n:head + 2 * n].view(torch.float32)
            edit_fac = blob[head + 2 * n:head + 3 * n].view(torch.float32)
            if plain_greedy:
                if len(self._constant) > 256:
                    self._constant.clear()
                self._constant[key] = params_dev
        # a small top-k: several blocks per row find the candidates before one block draws among them
        sliced = any(not s.config.is_greedy and 0 < s.config.top_k <= self._slice_capacity for s in samplers)
        with ops.section("sample"):
            ops.sample(logits, self._work[:B], params_dev, edit_tok, edit_sub, edit_fac, out_tok, out_prob,
                       select=self._select if sliced else None)
        host = self._read_back(2 * B, while_waiting)         # one copy back: tokens, then probabilities
        self.last_d2h_bytes = 8 * B
        chosen = host[:B].tolist()
        probs = host[B:].view(torch.float32).tolist()
        for s, tok, pr in zip(samplers, chosen, probs):
            s.accept(tok, pr)
        return chosen
