"""The paged key/value cache: a slot per sequence, pages of PAGE tokens, one group of
storage per kind of need.

Every schedule entry whose mixer keeps something per token gets a cache of its own.
Entries with the same `CacheNeed` (kind, per-token tensors, window) form a group; a group
owns its storage (per declared tensor [entries, pages, *outer, PAGE, inner]; for attention
the one tensor "kv" [entries, pages, 2 (K,V), kv_heads, PAGE, head_dim]), its page pool
and, for each slot, one page table shared by the group's entries (they all hold the same
positions).  A "full" group keeps every position of a sequence; a "window" group gives a
page back as soon as all of its positions lie before the window of the next query, so its
pool can be smaller.  Slots and pages return to their pools when a sequence ends and are
handed out again; nothing is cleared, since a position is readable only after it has
been written (each sequence's length bounds every read).

The reference's cache is one sequence's [layers][ctx][kv_heads*head_dim] float32 arrays
with the context fixed at 512 (core/model.hpp:29-54, core/model.cpp:64).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..csrc.ops import PAGE
from .slots import CacheFull, PagePool, SlotAllocator


@dataclass
class CacheView:
    """What a mixer sees of its entry: the entry's tensors (name -> [pages, *outer, PAGE,
    inner], as its CacheNeed declared them) and its group's page tables for the sequences of
    the current step ([B, max_pages] int32 on the device)."""
    tensors: dict | None
    tables: torch.Tensor | None
    group: int

    @property
    def kv(self):
        """Attention's tensor [pages, 2, kv_heads, PAGE, head_dim]."""
        return None if self.tensors is None else self.tensors["kv"]


def page_shape(per_token_shape) -> tuple:
    """A page of a tensor with this per-token shape: the tokens run along the last but one axis."""
    shape = tuple(int(d) for d in per_token_shape)
    if not shape or min(shape) < 1:
        raise ValueError(f"a cached tensor needs a per-token shape of positive sizes, got {per_token_shape}")
    return shape[:-1] + (PAGE, shape[-1])


class CacheGroup:
    def __init__(self, index: int, need, entries: list[int], n_pages: int, n_slots: int, max_pages_per_seq: int):
        self.index = index
        self.need = need
        self.entries = entries
        self.pool = PagePool(n_pages)
        self.tables = np.full((n_slots, max_pages_per_seq), -1, dtype=np.int32)
        # per slot: pages [lo, hi) are mapped (lo > 0 only in window groups)
        self.lo = np.zeros(n_slots, dtype=np.int64)
        self.hi = np.zeros(n_slots, dtype=np.int64)
        self.storage: dict | None = None        # tensor name -> [entries, pages, *outer, PAGE, inner]

    def allocate(self, dtype, device) -> None:
        self.storage = {name: torch.zeros((len(self.entries), self.pool.n) + page_shape(shape), dtype=dtype,
                                          device=device)
                        for name, shape in self.need.tensors}

    def bytes_per_page(self, itemsize: int) -> int:
        return len(self.entries) * PAGE * self.need.elements_per_token() * itemsize


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


class KVCache:
    def __init__(self, needs, max_tokens: int, max_seq_len: int, dtype=torch.bfloat16, device=None,
                 n_slots: int | None = None, allocate: bool = True, window_pool_tokens: int | None = None):
        """needs: per schedule entry a CacheNeed or None.  max_tokens: the most tokens the
        live sequences hold together, each sequence's count rounded up to a multiple of
        PAGE.  max_seq_len: the longest a single sequence may grow."""
        if max_tokens < PAGE:
            raise ValueError(f"the cache needs room for at least one page of {PAGE} tokens")
        self.max_tokens = (max_tokens // PAGE) * PAGE
        self.max_seq_len = min(max_seq_len, self.max_tokens)
        n_pages = self.max_tokens // PAGE
        self.n_slots = n_slots or n_pages
        self.max_pages_per_seq = pages_for(self.max_seq_len)
        self.slots = SlotAllocator(self.n_slots)
        self.lengths = np.zeros(self.n_slots, dtype=np.int64)
        self.version = 0                       # grows whenever any page table changes
        self.groups: list[CacheGroup] = []
        self.entry_group: dict[int, tuple[int, int]] = {}      # entry -> (group, index in group)
        by_need: dict = {}
        for e, need in enumerate(needs):
            if need is None:
                continue
            if need.kind not in ("full", "window"):
                raise ValueError(f"entry {e}: unknown cache kind {need.kind!r}")
            if need.kind == "window" and need.window < 1:
                raise ValueError(f"entry {e}: a window cache needs window >= 1")
            names = [name for name, _ in need.tensors]
            if not names or len(set(names)) != len(names):
                raise ValueError(f"entry {e}: a cache need declares at least one tensor, each name once")
            for _, shape in need.tensors:
                page_shape(shape)
            by_need.setdefault(need, []).append(e)
        for gi, (need, entries) in enumerate(by_need.items()):
            pages = n_pages
            if need.kind == "window" and window_pool_tokens is not None:
                pages = min(n_pages, max(1, window_pool_tokens // PAGE))
            g = CacheGroup(gi, need, entries, pages, self.n_slots, self.max_pages_per_seq)
            self.groups.append(g)
            for j, e in enumerate(entries):
                self.entry_group[e] = (gi, j)
        if allocate:
            for g in self.groups:
                g.allocate(dtype, device)

    # ------------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        s = self.slots.alloc()
        self.lengths[s] = 0
        return s

    def free_slot(self, slot: int) -> None:
        """Gives the slot and every page it holds back."""
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is not held (freed twice, or never allocated)")
        for g in self.groups:
            row = g.tables[slot]
            for i in np.nonzero(row >= 0)[0]:
                g.pool.release(int(row[i]))
            row[:] = -1
            g.lo[slot] = g.hi[slot] = 0
        self.version += 1
        self.lengths[slot] = 0
        self.slots.free(slot)

    def length(self, slot: int) -> int:
        return int(self.lengths[slot])

    # ------------------------------------------------------------------ pages
    def reserve(self, slot: int, new_len: int) -> bool:
        """Makes positions [length, new_len) of `slot` writable in every group (and, in
        window groups, releases pages no query of this step can reach).  Returns True if
        any page table changed.  Raises CacheFull before changing anything it cannot
        finish for this slot."""
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is not held")
        cur = int(self.lengths[slot])
        if new_len > self.max_seq_len:
            raise CacheFull(f"sequence would reach {new_len} tokens; the cache allows {self.max_seq_len}")
        need_hi = pages_for(new_len)
        for g in self.groups:                       # the common case: every page is there already
            if need_hi > g.hi[slot] or (g.need.kind == "window"
                                        and max(0, cur - g.need.window + 1) // PAGE > g.lo[slot]):
                break
        else:
            return False
        changed = False
        first_needed_page = {}
        for g in self.groups:
            lo_page = 0
            if g.need.kind == "window":
                lo_page = max(0, cur - g.need.window + 1) // PAGE     # oldest key the first new query reads
            first_needed_page[g.index] = lo_page
            row = g.tables[slot]
            releasable = int(((row[:lo_page] >= 0).sum()))
            want = [p for p in range(lo_page, pages_for(new_len)) if row[p] < 0]
            if len(want) > g.pool.n_free + releasable:
                raise CacheFull(f"cache group {g.index} ({g.need.kind}) has {g.pool.n_free} free pages, "
                                f"{len(want)} more are needed; size the cache for more tokens")
        for g in self.groups:
            row = g.tables[slot]
            lo_page = first_needed_page[g.index]
            for p in np.nonzero(row[:lo_page] >= 0)[0]:
                g.pool.release(int(row[p]))
                row[p] = -1
                changed = True
            for p in range(lo_page, pages_for(new_len)):
                if row[p] < 0:
                    row[p] = g.pool.alloc()
                    changed = True
            g.lo[slot] = lo_page
            g.hi[slot] = max(int(g.hi[slot]), pages_for(new_len))
        if changed:
            self.version += 1
        return changed

    def commit(self, slot: int, new_len: int) -> None:
        self.lengths[slot] = new_len

    def tables_for(self, group: int, slots) -> np.ndarray:
        """[len(slots), max_pages] page table rows; a slot < 0 (padding) gives -1 rows."""
        g = self.groups[group]
        out = np.full((len(slots), self.max_pages_per_seq), -1, dtype=np.int32)
        for i, s in enumerate(slots):
            if s >= 0:
                out[i] = g.tables[s]
        return out

    def storage_of(self, entry: int):
        """The entry's tensors: name -> [pages, *outer, PAGE, inner] (None before allocation)."""
        gi, j = self.entry_group[entry]
        st = self.groups[gi].storage
        return None if st is None else {name: t[j] for name, t in st.items()}

    def group_of(self, entry: int) -> int:
        return self.entry_group[entry][0]

    def total_bytes(self, itemsize: int) -> int:
        return sum(g.bytes_per_page(itemsize) * g.pool.n for g in self.groups)

    def check(self) -> None:
        """No slot or page lost or held twice; free slots hold no pages."""
        self.slots.check()
        for g in self.groups:
            g.pool.check()
            held = g.tables[g.tables >= 0]
            assert len(held) == len(set(held.tolist())), "a page is mapped twice"
            assert set(held.tolist()) == g.pool._used, "page tables and pool disagree"
            for s in range(self.n_slots):
                if not self.slots.is_held(s):
                    assert (g.tables[s] < 0).all(), f"free slot {s} still maps pages"
