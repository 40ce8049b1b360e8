"""The cache: a slot for each live sequence, keys and values for each cache entry, each
sequence's own length, and fixed-size per-sequence state beside them.

The reference keeps one contiguous ``[layers, context, kv_dim]`` pair of arrays for its single
sequence (inference/state/LlamaState.java:44-46,61-64 of the reference project).  Here:

* a *cache entry* is what one run of a mixer keeps (the schedule names it by an integer);
* what an entry keeps is described by its *need* (a small frozen record); entries with the same
  need form a *group* with storage of its own.  Which class holds the storage of a need is looked
  up in a registry (``register_cache_group``), so a mixer that keeps something else brings its
  need type and its group class with it;
* a *paged group* grows with the sequence: it owns a pool of pages of ``PAGE_TOKENS`` positions and
  one page table per sequence (shared by the group's entries).  ``KVGroup`` is the paged group of
  attention: keys ``[entry][page][kv_head][64][head_dim]``, values transposed
  ``[entry][page][kv_head][head_dim][64]``; with a ``window`` it only keeps the pages a query can
  still reach;
* a *slot group* has a fixed size per sequence: ``StateGroup`` owns ``[entry][slot][...shape]``,
  zeroed when a slot is acquired;
* a *slot* is acquired when a sequence starts and released when it ends; its pages go back to
  the pools and are handed to later sequences without clearing (positions at or beyond a
  sequence's length are never read).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .pages import PAGE_TOKENS, CacheError, CacheFull, PagePool, SlotTable, pages_for


@dataclass(frozen=True)
class KVCacheNeed:
    """Growing keys and values: one [kv_heads, head_dim] row per position; ``window`` = how many
    of the latest positions a query reads (None: all of them)."""
    n_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """Per-sequence state of fixed size, carried from step to step."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class CacheSizes:
    """What a group is sized by."""
    n_pages: int        # pages of PAGE_TOKENS positions the cache was promised
    max_slots: int
    dtype: torch.dtype  # the run's precision
    device: torch.device
    window_slack: int   # the most tokens one sequence adds in one step


class CacheGroup:
    """Storage of the cache entries that share one need.  ``paged`` groups grow with their sequences and
    have a page table in every step's context; the others have a fixed size per slot."""
    paged = False

    def __init__(self, need, entries: list[int], sizes: CacheSizes):
        self.need, self.entries = need, list(entries)
        self.entry_pos = {e: i for i, e in enumerate(self.entries)}
        self.index = -1   # position among the cache's paged (or slot) groups, set by the cache

    def acquire(self, slot: int) -> None:
        """A new sequence takes ``slot``."""

    def release(self, slot: int) -> None:
        """The sequence in ``slot`` is over."""

    def view(self, entry: int):
        """What the mixer of ``entry`` is handed in ``forward``."""
        raise NotImplementedError

    def bytes_per_token(self) -> int:
        """Bytes one cached position takes over the group's entries (0 for fixed-size state)."""
        return 0

    def check(self) -> None:
        """Raise CacheError if the group's bookkeeping is inconsistent."""


class PagedGroup(CacheGroup):
    """Bookkeeping of a group that grows page by page; subclasses own the device storage and the view."""
    paged = True

    def __init__(self, need, entries, sizes: CacheSizes, window: int | None = None):
        super().__init__(need, entries, sizes)
        self.window = window
        n_pages = sizes.n_pages
        if window is not None:   # a windowed group never holds more than this, whatever the promised total
            per_seq = pages_for(window + max(sizes.window_slack, 1)) + 1
            n_pages = min(n_pages, sizes.max_slots * per_seq)
        self.pool = PagePool(n_pages)
        # per live slot: logical page index -> physical page, -1 where a windowed group let go
        self.rows: dict[int, list[int]] = {}

    def acquire(self, slot):
        self.rows[slot] = []

    def release(self, slot):
        self.pool.free([p for p in self.rows.pop(slot) if p >= 0])

    def pages_needed(self, slot: int, new_length: int) -> int:
        return max(0, pages_for(new_length) - len(self.rows[slot]))

    def reserve(self, slot: int, new_length: int) -> None:
        extra = self.pages_needed(slot, new_length)
        if extra > 0:
            self.rows[slot].extend(self.pool.alloc(extra))

    def commit(self, slot: int, new_length: int) -> None:
        """The sequence now holds ``new_length`` tokens: let go of pages no later query can reach."""
        if self.window is None:
            return
        first_needed = max(0, new_length - self.window + 1)  # the next query sits at position `new_length`
        dead = first_needed // PAGE_TOKENS
        row = self.rows[slot]
        drop = [p for p in row[:dead] if p >= 0]
        if drop:
            self.pool.free(drop)
            for i in range(dead):
                row[i] = -1

    def check(self):
        held = [p for row in self.rows.values() for p in row if p >= 0]
        if len(held) != len(set(held)):
            raise CacheError(f"paged group {self.index}: a page is held twice")
        if len(held) != self.pool.n_held:
            raise CacheError(f"paged group {self.index}: {self.pool.n_held} pages are out but slots hold {len(held)}")


@dataclass
class KVView:
    """What a mixer sees of its growing cache entry: the entry's page pools and the id of the
    group whose page table (in the step context) addresses them."""
    group: int
    k: torch.Tensor  # [n_pages, kv_heads, PAGE_TOKENS, head_dim]
    v: torch.Tensor  # [n_pages, kv_heads, head_dim, PAGE_TOKENS]
    window: int | None


class KVGroup(PagedGroup):
    def __init__(self, need: KVCacheNeed, entries, sizes: CacheSizes):
        super().__init__(need, entries, sizes, window=need.window)
        n = self.pool.n_pages
        # keys: a row per position; values: transposed, a row per dimension (positions contiguous)
        self.k = torch.zeros((len(self.entries), n, need.n_kv_heads, PAGE_TOKENS, need.head_dim), dtype=sizes.dtype,
                             device=sizes.device)
        self.v = torch.zeros((len(self.entries), n, need.n_kv_heads, need.head_dim, PAGE_TOKENS), dtype=sizes.dtype,
                             device=sizes.device)

    def view(self, entry):
        i = self.entry_pos[entry]
        return KVView(group=self.index, k=self.k[i], v=self.v[i], window=self.need.window)

    def bytes_per_token(self):
        return 2 * len(self.entries) * self.need.n_kv_heads * self.need.head_dim * self.k.element_size()


@dataclass
class StateView:
    """What a mixer sees of its fixed-size state: ``data[slot]`` is the state of that sequence."""
    data: torch.Tensor  # [max_slots, *shape]


class StateGroup(CacheGroup):
    def __init__(self, need: StateNeed, entries, sizes: CacheSizes):
        super().__init__(need, entries, sizes)
        self.data = torch.zeros((len(self.entries), sizes.max_slots, *need.shape), dtype=need.dtype, device=sizes.device)

    def acquire(self, slot):
        self.data[:, slot].zero_()

    def view(self, entry):
        return StateView(data=self.data[self.entry_pos[entry]])


_GROUP_CLASSES: dict[type, type] = {}


def register_cache_group(need_type: type, group_class: type, *, replace: bool = False) -> None:
    """Entries whose need is a ``need_type`` are stored by ``group_class(need, entries, sizes)``, a
    ``PagedGroup`` (grows with the sequence) or a plain ``CacheGroup`` (fixed size per slot).  Needs must be
    hashable and comparable: entries with equal needs share one group."""
    if need_type in _GROUP_CLASSES and not replace:
        raise CacheError(f"cache need {need_type.__name__} already has a group class")
    _GROUP_CLASSES[need_type] = group_class


def unregister_cache_group(need_type: type) -> None:
    _GROUP_CLASSES.pop(need_type, None)


def _group_class(need) -> type:
    for t in type(need).__mro__:
        if t in _GROUP_CLASSES:
            return _GROUP_CLASSES[t]
    raise TypeError(f"no cache group is registered for the need {need!r}; "
                    f"registered: {', '.join(sorted(t.__name__ for t in _GROUP_CLASSES))}")


register_cache_group(KVCacheNeed, KVGroup)
register_cache_group(StateNeed, StateGroup)


class SequenceCache:
    def __init__(self, needs: dict[int, object], *, max_tokens: int, max_slots: int | None = None,
                 dtype: torch.dtype = torch.bfloat16, device="cuda", window_slack: int = 0):
        """``needs``: cache entry id -> what its mixer keeps.  ``max_tokens``: the most tokens all
        live sequences hold together, each sequence counted in whole pages.  ``window_slack``: the
        most tokens one sequence adds in one step (a windowed group keeps window + slack)."""
        if max_tokens < PAGE_TOKENS:
            raise ValueError(f"max_tokens must be at least one page ({PAGE_TOKENS} tokens)")
        self.max_tokens = max_tokens
        self.n_pages = max_tokens // PAGE_TOKENS
        self.max_slots = max_slots if max_slots is not None else min(self.n_pages, 1024)
        self.dtype = dtype
        self.device = torch.device(device)
        self.slots = SlotTable(self.max_slots)
        self.window_slack = window_slack
        sizes = CacheSizes(self.n_pages, self.max_slots, dtype, self.device, window_slack)

        by_need: dict = {}
        for entry in sorted(needs):
            by_need.setdefault(needs[entry], []).append(entry)
        self.paged_groups: list[PagedGroup] = []
        self.slot_groups: list[CacheGroup] = []
        self._entry_group: dict[int, CacheGroup] = {}
        for need, entries in by_need.items():
            g = _group_class(need)(need, entries, sizes)
            family = self.paged_groups if g.paged else self.slot_groups
            g.index = len(family)
            family.append(g)
            for e in entries:
                self._entry_group[e] = g
        self._length: dict[int, int] = {}
        # counts acquisitions and releases: while it stands still, a slot number means the same sequence
        self.ownership_changes = 0

    @property
    def groups(self) -> list[CacheGroup]:
        return [*self.paged_groups, *self.slot_groups]

    # ---- slots
    def acquire(self) -> int:
        slot = self.slots.acquire()
        self.ownership_changes += 1
        self._length[slot] = 0
        for g in self.groups:
            g.acquire(slot)
        return slot

    def release(self, slot: int) -> None:
        if not self.slots.is_live(slot):
            raise CacheError(f"slot {slot} is not live")
        del self._length[slot]
        self.ownership_changes += 1
        for g in self.groups:
            g.release(slot)
        self.slots.release(slot)

    def length(self, slot: int) -> int:
        return self._length[slot]

    def live_slots(self) -> list[int]:
        return sorted(self._length)

    # ---- pages
    def pages_needed(self, requests: list[tuple[int, int]]) -> list[int]:
        """Per paged group, how many new pages ``[(slot, n_new_tokens)]`` would take."""
        return [sum(g.pages_needed(slot, self._length[slot] + n_new) for slot, n_new in requests)
                for g in self.paged_groups]

    def reserve(self, requests: list[tuple[int, int]]) -> None:
        """Make room for ``n_new`` more tokens in each slot, or raise CacheFull and change nothing."""
        for slot, _ in requests:
            if slot not in self._length:
                raise CacheError(f"slot {slot} is not live")
        for g, n in zip(self.paged_groups, self.pages_needed(requests)):
            if n > g.pool.n_free:
                raise CacheFull(f"cache group {g.index} needs {n} more page(s) of {PAGE_TOKENS} tokens, "
                                f"{g.pool.n_free} of {g.pool.n_pages} are free")
        for slot, n_new in requests:
            for g in self.paged_groups:
                g.reserve(slot, self._length[slot] + n_new)

    def commit(self, slot: int, n_new: int) -> None:
        """The step wrote ``n_new`` tokens: advance the length, let windowed groups drop pages that
        no later query can reach."""
        self._length[slot] += n_new
        for g in self.paged_groups:
            g.commit(slot, self._length[slot])

    def page_rows(self, group: int, slots: list[int]) -> list[list[int]]:
        rows = self.paged_groups[group].rows
        return [rows[s] for s in slots]

    def pages_for_planning(self) -> int:
        """The fewest pages any paged group can give all sequences together (a very large number if the model
        keeps nothing that grows)."""
        return min((g.pool.n_pages for g in self.paged_groups), default=1 << 30)

    # ---- what mixers see
    def view(self, entry: int):
        return self._entry_group[entry].view(entry)

    def bytes_per_token(self) -> int:
        """Bytes one cached position takes over all growing entries."""
        return sum(g.bytes_per_token() for g in self.paged_groups)

    def check_invariants(self) -> None:
        """Every page is free or held by exactly one live slot; used by tests."""
        for g in self.groups:
            g.check()
            if g.paged and set(g.rows) != set(self._length):
                raise CacheError(f"paged group {g.index}: page rows exist for slots {sorted(g.rows)}, "
                                 f"live are {sorted(self._length)}")
