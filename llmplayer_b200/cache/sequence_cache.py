"""The cache of a model: per-sequence slots, paged keys and values in groups of
layers with equal needs, and a per-sequence state area of fixed size.

What a run of a layer needs is said by its mixer (a :class:`KVRequest`, a
:class:`StateRequest` or nothing). Runs with the same key/value geometry and
window share one :class:`KVGroup` — one storage tensor and one page map —
so layers that keep all keys and layers that keep a window of them have storage
of their own. State requests get one row per slot each, zeroed when the slot is
taken (a recurrent state must not start from a former sequence's values; key and
value pages need no clearing because lengths mask them).

Reference: inference/KVCache.java:87-136 (one array per layer and request),
inference/InferenceState.java:24-58 (per-request buffers); the fixed-size states of
its recurrent architectures live in per-request objects too
(inference/Qwen35State.java:39-42).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..errors import CacheError, CacheFull
from .pages import PAGE_SIZE, FreeList, PageMap


@dataclass(frozen=True)
class KVRequest:
    """Keys and values of every position (or of a window of positions) of a sequence."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """A block of fixed shape per sequence, zero at the sequence's start."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class KVGroup:
    """Storage of the runs that share one :class:`KVRequest`.

    ``storage[i]`` is the tensor of the i-th run of the group:
    [num_pages, 2 (keys, values), kv heads, PAGE_SIZE, head_dim].
    """

    def __init__(self, request: KVRequest, runs: Sequence[int], num_pages: int, dtype: torch.dtype, device):
        self.request = request
        self.runs = list(runs)
        self.pages = PageMap(num_pages, window=request.window)
        # zeros once, so that stale rows are always finite; never cleared again
        self.storage = torch.zeros(
            (len(self.runs), num_pages, 2, request.num_kv_heads, PAGE_SIZE, request.head_dim),
            dtype=dtype, device=device)

    def bytes_per_token(self) -> int:
        r = self.request
        return len(self.runs) * 2 * r.num_kv_heads * r.head_dim * self.storage.element_size()

    def view_of(self, run: int) -> torch.Tensor:
        return self.storage[self.runs.index(run)]


class KVView:
    """What an attention run sees of the cache: its storage and its group's index."""

    def __init__(self, group_index: int, pages: torch.Tensor):
        self.group_index = group_index
        self.pages = pages


class StateView:
    """What a run with fixed-size state sees: one row per slot."""

    def __init__(self, rows: torch.Tensor):
        self.rows = rows


class SequenceCache:
    def __init__(self, requests: Sequence[object], *, max_tokens: int, max_slots: Optional[int], kv_dtype: torch.dtype,
                 device):
        """``requests[i]``: what run i of the schedule keeps (KVRequest, StateRequest or None)."""
        if max_tokens <= 0:
            raise CacheError(f"max_tokens must be positive, got {max_tokens}")
        self.device = device
        self.num_pages = -(-max_tokens // PAGE_SIZE)
        self.max_slots = max_slots if max_slots is not None else self.num_pages
        if self.max_slots <= 0:
            raise CacheError(f"max_slots must be positive, got {self.max_slots}")
        self.slots = FreeList(self.max_slots, "slot")
        self._length: Dict[int, int] = {}
        self.groups: List[KVGroup] = []
        self._views: List[object] = [None] * len(requests)
        by_request: Dict[KVRequest, List[int]] = {}
        for run, req in enumerate(requests):
            if isinstance(req, KVRequest):
                by_request.setdefault(req, []).append(run)
        for req, runs in by_request.items():
            group = KVGroup(req, runs, self.num_pages, kv_dtype, device)
            for run in runs:
                self._views[run] = KVView(len(self.groups), group.view_of(run))
            self.groups.append(group)
        self._state_rows: List[torch.Tensor] = []
        for run, req in enumerate(requests):
            if isinstance(req, StateRequest):
                rows = torch.zeros((self.max_slots,) + tuple(req.shape), dtype=req.dtype, device=device)
                self._state_rows.append(rows)
                self._views[run] = StateView(rows)
            elif req is not None and not isinstance(req, KVRequest):
                raise CacheError(f"run {run}: unknown cache request {req!r}")

    # ------------------------------------------------------------------ slots
    def acquire(self) -> int:
        slot = self.slots.take()
        self._length[slot] = 0
        for group in self.groups:
            group.pages.open(slot)
        for rows in self._state_rows:
            rows[slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not held (freed twice?)")
        for group in self.groups:
            group.pages.close(slot)
        del self._length[slot]
        self.slots.give_back(slot)

    def length(self, slot: int) -> int:
        try:
            return self._length[slot]
        except KeyError:
            raise CacheError(f"slot {slot} is not held") from None

    def view(self, run: int):
        return self._views[run]

    # ------------------------------------------------------------------ a step
    def reserve(self, slots: Sequence[int], new_tokens: Sequence[int]) -> None:
        """Give every slot the pages its new tokens need; nothing changes if they do not all fit."""
        seen = set()
        for slot in slots:
            if slot in seen:
                raise CacheError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            self.length(slot)
        for group in self.groups:
            need = sum(group.pages.pages_needed(s, self._length[s] + n) for s, n in zip(slots, new_tokens))
            if need > group.pages.pool.num_free:
                raise CacheFull(
                    f"the cache is full: this step needs {need} more page(s) of {PAGE_SIZE} positions, "
                    f"{group.pages.pool.num_free} of {group.pages.pool.count} are free")
        for group in self.groups:
            for s, n in zip(slots, new_tokens):
                group.pages.extend(s, self._length[s] + n)

    def reserve_up_to(self, slots: Sequence[int], lengths: Sequence[int]) -> None:
        """Pages for every slot up to the given total length, ahead of the steps that fill them."""
        self.reserve(slots, [max(0, n - self.length(s)) for s, n in zip(slots, lengths)])

    def commit(self, slots: Sequence[int], new_tokens: Sequence[int]) -> None:
        """The step ran: lengths grow, pages behind a window go back."""
        for s, n in zip(slots, new_tokens):
            self._length[s] += n
            for group in self.groups:
                group.pages.trim(s, self._length[s])

    def page_tables(self, slots: Sequence[int]) -> List[List[List[int]]]:
        """Per group, per slot of the step: page id of each block of positions."""
        return [[group.pages.table(s) for s in slots] for group in self.groups]

    # ------------------------------------------------------------------ reporting
    def memory_bytes(self) -> int:
        total = sum(g.storage.numel() * g.storage.element_size() for g in self.groups)
        total += sum(r.numel() * r.element_size() for r in self._state_rows)
        return total

    def free_pages(self) -> List[int]:
        return [g.pages.pool.num_free for g in self.groups]
