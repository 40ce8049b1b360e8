"""The cache: a slot for each live sequence, keys and values for each cache entry, each
sequence's own length, and fixed-size per-sequence state beside them.

The reference keeps one contiguous ``[layers, context, kv_dim]`` pair of arrays for its single
sequence (inference/state/LlamaState.java:44-46,61-64 of the reference project).  Here:

* a *cache entry* is what one run of a mixer keeps (the schedule names it by an integer);
* entries with the same need form a *group* with storage of its own: a group of growing
  key/value entries owns a pool of pages (keys ``[entry][page][kv_head][64][head_dim]``, values
  transposed ``[entry][page][kv_head][head_dim][64]``) and one page
  table per sequence (shared by the group's entries); a group whose need has a ``window`` only
  keeps the pages that a query can still reach; a group of fixed-size state owns
  ``[entry][slot][...shape]``, zeroed when a slot is acquired;
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


class KVGroup:
    def __init__(self, index: int, need: KVCacheNeed, entries: list[int], n_pages: int, dtype, device):
        self.index = index
        self.need = need
        self.entries = entries
        self.pool = PagePool(n_pages)
        # keys: a row per position; values: transposed, a row per dimension (positions contiguous)
        self.k = torch.zeros((len(entries), n_pages, need.n_kv_heads, PAGE_TOKENS, need.head_dim), dtype=dtype, device=device)
        self.v = torch.zeros((len(entries), n_pages, need.n_kv_heads, need.head_dim, PAGE_TOKENS), dtype=dtype, device=device)
        self.entry_pos = {e: i for i, e in enumerate(entries)}


class StateGroup:
    def __init__(self, index: int, need: StateNeed, entries: list[int], max_slots: int, device):
        self.index = index
        self.need = need
        self.entries = entries
        self.data = torch.zeros((len(entries), max_slots, *need.shape), dtype=need.dtype, device=device)
        self.entry_pos = {e: i for i, e in enumerate(entries)}


@dataclass
class KVView:
    """What a mixer sees of its growing cache entry: the entry's page pools and the id of the
    group whose page table (in the step context) addresses them."""
    group: int
    k: torch.Tensor  # [n_pages, kv_heads, PAGE_TOKENS, head_dim]
    v: torch.Tensor  # [n_pages, kv_heads, head_dim, PAGE_TOKENS]
    window: int | None


@dataclass
class StateView:
    """What a mixer sees of its fixed-size state: ``data[slot]`` is the state of that sequence."""
    data: torch.Tensor  # [max_slots, *shape]


class _Slot:
    __slots__ = ("length", "pages")

    def __init__(self, n_groups: int):
        self.length = 0
        # per KV group: logical page index -> physical page, -1 where a windowed group let go
        self.pages: list[list[int]] = [[] for _ in range(n_groups)]


class SequenceCache:
    def __init__(self, needs: dict[int, KVCacheNeed | StateNeed], *, max_tokens: int, max_slots: int | None = None,
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

        by_need: dict = {}
        for entry in sorted(needs):
            by_need.setdefault(needs[entry], []).append(entry)
        self.kv_groups: list[KVGroup] = []
        self.state_groups: list[StateGroup] = []
        self._entry_group: dict[int, tuple[str, int]] = {}
        for need, entries in by_need.items():
            if isinstance(need, KVCacheNeed):
                n_pages = self.n_pages
                if need.window is not None:
                    per_seq = pages_for(need.window + max(window_slack, 1)) + 1
                    n_pages = min(n_pages, self.max_slots * per_seq)
                g = KVGroup(len(self.kv_groups), need, entries, n_pages, dtype, self.device)
                self.kv_groups.append(g)
                for e in entries:
                    self._entry_group[e] = ("kv", g.index)
            elif isinstance(need, StateNeed):
                g = StateGroup(len(self.state_groups), need, entries, self.max_slots, self.device)
                self.state_groups.append(g)
                for e in entries:
                    self._entry_group[e] = ("state", g.index)
            else:
                raise TypeError(f"cache entry needs must be KVCacheNeed or StateNeed, got {need!r}")
        self._slot: dict[int, _Slot] = {}
        # counts acquisitions and releases: while it stands still, a slot number means the same sequence
        self.ownership_changes = 0

    # ---- slots
    def acquire(self) -> int:
        slot = self.slots.acquire()
        self.ownership_changes += 1
        self._slot[slot] = _Slot(len(self.kv_groups))
        for g in self.state_groups:
            g.data[:, slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        if not self.slots.is_live(slot):
            raise CacheError(f"slot {slot} is not live")
        s = self._slot.pop(slot)
        self.ownership_changes += 1
        for g, pages in zip(self.kv_groups, s.pages):
            g.pool.free([p for p in pages if p >= 0])
        self.slots.release(slot)

    def length(self, slot: int) -> int:
        return self._slot[slot].length

    def live_slots(self) -> list[int]:
        return sorted(self._slot)

    # ---- pages
    def pages_needed(self, requests: list[tuple[int, int]]) -> list[int]:
        """Per KV group, how many new pages ``[(slot, n_new_tokens)]`` would take."""
        need = [0] * len(self.kv_groups)
        for slot, n_new in requests:
            s = self._slot[slot]
            for gi in range(len(self.kv_groups)):
                need[gi] += max(0, pages_for(s.length + n_new) - len(s.pages[gi]))
        return need

    def reserve(self, requests: list[tuple[int, int]]) -> None:
        """Make room for ``n_new`` more tokens in each slot, or raise CacheFull and change nothing."""
        for slot, _ in requests:
            if slot not in self._slot:
                raise CacheError(f"slot {slot} is not live")
        need = self.pages_needed(requests)
        for g, n in zip(self.kv_groups, need):
            if n > g.pool.n_free:
                raise CacheFull(f"cache group {g.index} needs {n} more page(s) of {PAGE_TOKENS} tokens, "
                                f"{g.pool.n_free} of {g.pool.n_pages} are free")
        for slot, n_new in requests:
            s = self._slot[slot]
            for gi, g in enumerate(self.kv_groups):
                extra = pages_for(s.length + n_new) - len(s.pages[gi])
                if extra > 0:
                    s.pages[gi].extend(g.pool.alloc(extra))

    def commit(self, slot: int, n_new: int) -> None:
        """The step wrote ``n_new`` tokens: advance the length, let windowed groups drop pages that
        no later query can reach."""
        s = self._slot[slot]
        s.length += n_new
        for gi, g in enumerate(self.kv_groups):
            w = g.need.window
            if w is None:
                continue
            first_needed = max(0, s.length - w + 1)  # the next query sits at position `length`
            dead = first_needed // PAGE_TOKENS
            drop = [p for p in s.pages[gi][:dead] if p >= 0]
            if drop:
                g.pool.free(drop)
                for i in range(dead):
                    s.pages[gi][i] = -1

    def page_rows(self, group: int, slots: list[int]) -> list[list[int]]:
        return [self._slot[s].pages[group] for s in slots]

    # ---- what mixers see
    def view(self, entry: int) -> KVView | StateView:
        kind, gi = self._entry_group[entry]
        if kind == "kv":
            g = self.kv_groups[gi]
            i = g.entry_pos[entry]
            return KVView(group=gi, k=g.k[i], v=g.v[i], window=g.need.window)
        g = self.state_groups[gi]
        return StateView(data=g.data[g.entry_pos[entry]])

    def bytes_per_token(self) -> int:
        """Key and value bytes one cached position takes over all growing entries."""
        el = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(g.entries) * g.need.n_kv_heads * g.need.head_dim * el for g in self.kv_groups)

    def check_invariants(self) -> None:
        """Every page is free or held by exactly one live slot; used by tests."""
        for gi, g in enumerate(self.kv_groups):
            held = [p for s in self._slot.values() for p in s.pages[gi] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"group {gi}: a page is held twice")
            if len(held) != g.pool.n_held:
                raise CacheError(f"group {gi}: {g.pool.n_held} pages are out but slots hold {len(held)}")
