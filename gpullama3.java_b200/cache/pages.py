"""Host-side bookkeeping of cache pages and sequence slots: pure Python, no device memory.

A page holds the keys and values of ``PAGE_TOKENS`` consecutive positions of one sequence (for
every cache entry of its group).  Pages and slots are handed out from free lists and must come
back exactly once; both allocators refuse a double free or a foreign id, which is what the
cache tests lean on (no page or slot lost, held twice or freed twice)."""
from __future__ import annotations

PAGE_TOKENS = 64


class CacheFull(RuntimeError):
    """The cache has no free page or slot left for what was asked."""


class CacheError(RuntimeError):
    """A slot or page was used in a way its state forbids (double free, unknown id, ...)."""


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages < 0:
            raise ValueError("n_pages must be >= 0")
        self.n_pages = n_pages
        self._free = list(range(n_pages - 1, -1, -1))  # pop() hands out low ids first
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n_pages - len(self._free)

    def alloc(self, n: int) -> list[int]:
        if n > len(self._free):
            raise CacheFull(f"need {n} cache page(s) of {PAGE_TOKENS} tokens, {len(self._free)} of {self.n_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def free(self, pages) -> None:
        pages = list(pages)
        for p in pages:
            if not (0 <= p < self.n_pages):
                raise CacheError(f"page {p} does not belong to this pool of {self.n_pages}")
            if not self._held[p]:
                raise CacheError(f"page {p} freed twice")
            self._held[p] = False
        self._free.extend(reversed(pages))


class SlotTable:
    def __init__(self, max_slots: int):
        if max_slots < 1:
            raise ValueError("max_slots must be >= 1")
        self.max_slots = max_slots
        self._free = list(range(max_slots - 1, -1, -1))
        self._live = [False] * max_slots

    @property
    def n_free(self) -> int:
        return len(self._free)

    def is_live(self, slot: int) -> bool:
        return 0 <= slot < self.max_slots and self._live[slot]

    def acquire(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.max_slots} sequence slots are in use")
        s = self._free.pop()
        self._live[s] = True
        return s

    def release(self, slot: int) -> None:
        if not (0 <= slot < self.max_slots):
            raise CacheError(f"slot {slot} does not exist")
        if not self._live[slot]:
            raise CacheError(f"slot {slot} released twice (or never acquired)")
        self._live[slot] = False
        self._free.append(slot)

    def live_slots(self) -> list[int]:
        return [s for s in range(self.max_slots) if self._live[s]]
