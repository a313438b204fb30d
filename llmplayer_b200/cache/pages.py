"""Host-side bookkeeping of the cache: slots for sequences and pages for keys and values.

The reference gives every request a state object of its own with
``maxSeqLen`` rows per layer (inference/KVCache.java:108-136,
inference/InferenceState.java:24-58). Here a sequence holds a *slot* (its row in
the per-sequence state area and its identity in the page maps) and, in each
group of layers, as many *pages* of ``PAGE_SIZE`` positions as its length needs.
Slots and pages go back to their free lists when the sequence ends and are
handed out again; nothing is cleared, so no kernel may read what its sequence
did not write.
"""
from __future__ import annotations

from typing import Dict, List, Optional

from ..errors import CacheError, CacheFull

PAGE_SIZE = 64


class FreeList:
    """Identifiers 0..n-1, each either free or held; hands out the lowest free one."""

    def __init__(self, count: int, what: str):
        if count < 0:
            raise CacheError(f"cannot make {count} {what}s")
        self.count = count
        self.what = what
        self._held = [False] * count
        self._free = list(range(count - 1, -1, -1))   # pop() yields the lowest id first

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} left (all {self.count} are held)")
        ident = self._free.pop()
        self._held[ident] = True
        return ident

    def give_back(self, ident: int) -> None:
        if not 0 <= ident < self.count:
            raise CacheError(f"{self.what} {ident} does not exist (there are {self.count})")
        if not self._held[ident]:
            raise CacheError(f"{self.what} {ident} is not held (freed twice?)")
        self._held[ident] = False
        self._free.append(ident)
        self._free.sort(reverse=True)

    def is_held(self, ident: int) -> bool:
        return 0 <= ident < self.count and self._held[ident]

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.count - len(self._free)


class PageMap:
    """Pages of one group of layers: which page holds which block of positions of which slot.

    ``window`` (in positions) lets the map give back pages that no later query
    can reach; ``None`` keeps every page until the slot is released.
    """

    def __init__(self, num_pages: int, window: Optional[int] = None, page_size: int = PAGE_SIZE):
        self.page_size = page_size
        self.window = window
        self.pool = FreeList(num_pages, "page")
        self._pages: Dict[int, List[int]] = {}     # slot -> page id per block of positions (-1: given back)

    def open(self, slot: int) -> None:
        if slot in self._pages:
            raise CacheError(f"slot {slot} already has pages in this group")
        self._pages[slot] = []

    def pages_needed(self, slot: int, length: int) -> int:
        have = len(self._pages[slot])
        need = -(-length // self.page_size)
        return max(0, need - have)

    def extend(self, slot: int, length: int) -> None:
        """Make sure positions [0, length) of ``slot`` have pages (all or nothing)."""
        pages = self._pages[slot]
        need = self.pages_needed(slot, length)
        if need > self.pool.num_free:
            raise CacheFull(
                f"the cache is full: slot {slot} needs {need} more page(s) of {self.page_size} positions "
                f"for length {length}, {self.pool.num_free} of {self.pool.count} are free")
        for _ in range(need):
            pages.append(self.pool.take())

    def trim(self, slot: int, length: int) -> None:
        """After a step that left ``slot`` at ``length``: give back the pages whose
        positions all lie before the window of the next query (position ``length``)."""
        if self.window is None:
            return
        first_needed = length - self.window + 1
        pages = self._pages[slot]
        for block in range(min(len(pages), max(0, first_needed) // self.page_size)):
            if pages[block] >= 0:
                self.pool.give_back(pages[block])
                pages[block] = -1

    def close(self, slot: int) -> None:
        for page in self._pages.pop(slot):
            if page >= 0:
                self.pool.give_back(page)

    def table(self, slot: int) -> List[int]:
        return self._pages[slot]

    def holds(self, slot: int) -> bool:
        return slot in self._pages
