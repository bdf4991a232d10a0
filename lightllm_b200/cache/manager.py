"""The cache manager: pages of keys and values with a block table per request and per group,
and slots for per-request state of fixed size.

The reference keeps one ``BlockAllocator`` per layer with a FIFO free list and reference counts
(src/kv_cache/block_allocator.cpp:16-79,138-147), one identical ``BlockTable`` per layer per
request (:236-248, src/engine/engine_server.cpp:1426-1438), and prints ``FATAL`` and carries on
when the pool is empty (:1427-1432).  Here:

* one pool of page ids per *group* of cache planes with equal needs; all planes of a group
  share a request's block table, each has its own storage;
* the free list is a stack, so a page that was just given back is the next one handed out and
  a stale read shows at once;
* pages are taken by :meth:`CacheManager.reserve` before a step runs (all or nothing, so a step
  never fails midway), and given back by :meth:`close` when a request ends or by
  :meth:`advance` when a window has passed them;
* every request also holds one state slot; planes of fixed-size state are indexed by it.

All bookkeeping is on the host and has no dependency on a GPU; the storage tensors are only
allocated when a device is given.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Hashable, List, Optional, Sequence

import numpy as np

import torch

from .spec import CacheLayout, KVSpec


class CacheError(RuntimeError):
    """A fault in the use of the cache manager (double free, unknown request, ...)."""


class OutOfPages(CacheError):
    """Not enough free pages (or slots) for what was asked; nothing was taken."""


class PagePool:
    """Page ids ``0..num_pages-1`` of one group, with an owner for every page in use."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # stack; page 0 on top
        self._owner: List[Optional[Hashable]] = [None] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, owner: Hashable) -> int:
        if owner is None:
            raise CacheError("a page needs an owner")
        if not self._free:
            raise OutOfPages("no free page")
        page = self._free.pop()
        if self._owner[page] is not None:
            raise CacheError(f"page {page} on the free list is owned by {self._owner[page]!r}")
        self._owner[page] = owner
        return page

    def take_many(self, owner: Hashable, n: int) -> List[int]:
        """``n`` pages at once, in the order ``take`` would give them."""
        if owner is None:
            raise CacheError("a page needs an owner")
        if n > len(self._free):
            raise OutOfPages(f"{n} pages asked for, {len(self._free)} free")
        if n <= 0:
            return []
        pages = self._free[-n:][::-1]
        del self._free[-n:]
        for page in pages:
            if self._owner[page] is not None:
                raise CacheError(f"page {page} on the free list is owned by {self._owner[page]!r}")
            self._owner[page] = owner
        return pages

    def give(self, page: int, owner: Hashable) -> None:
        if not 0 <= page < self.num_pages:
            raise CacheError(f"page {page} is outside the pool of {self.num_pages}")
        if self._owner[page] is None:
            raise CacheError(f"page {page} is freed twice")
        if self._owner[page] != owner:
            raise CacheError(f"page {page} belongs to {self._owner[page]!r}, not to {owner!r}")
        self._owner[page] = None
        self._free.append(page)

    def owner_of(self, page: int) -> Optional[Hashable]:
        return self._owner[page]

    def check(self) -> None:
        """No page lost, none held twice, none both free and owned."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError("a page is on the free list twice")
        for p in range(self.num_pages):
            if (p in free) == (self._owner[p] is not None):
                raise CacheError(f"page {p} is {'free and owned' if p in free else 'neither free nor owned'}")


@dataclass
class SeqCache:
    """What one live request holds: a state slot, its length, and a block table per group
    (physical page of each logical page; -1 once a window has passed it)."""

    seq_id: Hashable
    slot: int
    length: int = 0
    tables: List[List[int]] = field(default_factory=list)
    first_live: List[int] = field(default_factory=list)    # first logical page not yet released
    version: int = 0                                       # bumped whenever a table changes
    _np: Dict[int, Any] = field(default_factory=dict)      # group -> (version, int32 array of the table)


class CacheManager:
    def __init__(self, layout: CacheLayout, page_size: int, num_pages, max_seqs: int, max_seq_len: int,
                 dtype: torch.dtype = torch.float32, device: Optional[torch.device] = None):
        if page_size <= 0 or max_seqs <= 0 or max_seq_len <= 0:
            raise CacheError("page_size, max_seqs and max_seq_len must be positive")
        self.layout = layout
        self.page_size = page_size
        self.max_seqs = max_seqs
        self.max_seq_len = max_seq_len
        self.max_pages_per_seq = (max_seq_len + page_size - 1) // page_size
        ngroups = len(layout.groups)
        if isinstance(num_pages, int):
            num_pages = [num_pages] * ngroups
        if len(num_pages) != ngroups:
            raise CacheError(f"num_pages has {len(num_pages)} entries for {ngroups} groups")
        self.pools = [PagePool(n) for n in num_pages]
        self._free_slots: List[int] = list(range(max_seqs - 1, -1, -1))
        self.seqs: Dict[Hashable, SeqCache] = {}
        self.dtype = dtype
        self.device = device
        # Storage: per group [planes, 2 (k, v), pages, page_size, kv_heads, head_dim]; per state plane [max_seqs, *shape].
        self.kv: List[Optional[torch.Tensor]] = [None] * ngroups
        self.state: List[Optional[torch.Tensor]] = [None] * len(layout.state_planes)
        if device is not None:
            for g, (spec, planes) in enumerate(zip(layout.groups, layout.planes_per_group)):
                self.kv[g] = torch.zeros((planes, 2, num_pages[g], page_size, spec.kv_heads, spec.head_dim),
                                         dtype=dtype, device=device)
            for i, s in enumerate(layout.state_planes):
                self.state[i] = torch.zeros((max_seqs, *s.shape), dtype=getattr(torch, s.dtype), device=device)

    # ---- requests -------------------------------------------------------------------------
    def open(self, seq_id: Hashable) -> SeqCache:
        """Admit a request: it gets a state slot and empty block tables."""
        if seq_id in self.seqs:
            raise CacheError(f"request {seq_id!r} is already open")
        if not self._free_slots:
            raise OutOfPages(f"all {self.max_seqs} request slots are in use")
        slot = self._free_slots.pop()
        n = len(self.pools)
        seq = SeqCache(seq_id, slot, 0, [[] for _ in range(n)], [0] * n)
        self.seqs[seq_id] = seq
        return seq

    def get(self, seq_id: Hashable) -> SeqCache:
        try:
            return self.seqs[seq_id]
        except KeyError:
            raise CacheError(f"request {seq_id!r} is not open") from None

    def pages_needed(self, seq_id: Hashable, n_tokens: int) -> List[int]:
        """New pages per group that holding ``n_tokens`` more tokens takes."""
        seq = self.get(seq_id)
        total = (seq.length + n_tokens + self.page_size - 1) // self.page_size
        return [max(0, total - len(t)) for t in seq.tables]

    def can_reserve(self, seq_id: Hashable, n_tokens: int) -> bool:
        seq = self.get(seq_id)
        if seq.length + n_tokens > self.max_seq_len:
            return False
        return all(need <= pool.free_count for need, pool in zip(self.pages_needed(seq_id, n_tokens), self.pools))

    def reserve(self, seq_id: Hashable, n_tokens: int) -> None:
        """Take the pages that ``n_tokens`` more tokens need, in every group, or none at all."""
        seq = self.get(seq_id)
        if seq.length + n_tokens > self.max_seq_len:
            raise OutOfPages(f"request {seq_id!r} would hold {seq.length + n_tokens} tokens; "
                             f"the limit is {self.max_seq_len}")
        needs = self.pages_needed(seq_id, n_tokens)
        for g, (need, pool) in enumerate(zip(needs, self.pools)):
            if need > pool.free_count:
                raise OutOfPages(f"group {g}: {need} pages needed, {pool.free_count} free")
        for g, (need, pool) in enumerate(zip(needs, self.pools)):
            if need:
                seq.tables[g].extend(pool.take_many(seq_id, need))
                seq.version += 1

    def can_reserve_all(self, asks) -> bool:
        """Whether every ``(request, n_tokens)`` of ``asks`` can get its pages at the same time."""
        total = [0] * len(self.pools)
        for seq_id, n in asks:
            if self.get(seq_id).length + n > self.max_seq_len:
                return False
            for g, need in enumerate(self.pages_needed(seq_id, n)):
                total[g] += need
        return all(t <= pool.free_count for t, pool in zip(total, self.pools))

    def reserve_all(self, asks) -> None:
        """:meth:`reserve` for several requests at once: all of them get their pages, or none does."""
        asks = list(asks)
        if not self.can_reserve_all(asks):
            for seq_id, n in asks:
                if self.get(seq_id).length + n > self.max_seq_len:
                    raise OutOfPages(f"request {seq_id!r} would hold {self.get(seq_id).length + n} tokens; "
                                     f"the limit is {self.max_seq_len}")
            raise OutOfPages("not enough free pages for this step: free per group "
                             f"{[p.free_count for p in self.pools]}")
        for seq_id, n in asks:
            self.reserve(seq_id, n)

    def advance(self, seq_id: Hashable, n_tokens: int) -> None:
        """The request now holds ``n_tokens`` more tokens (their keys and values are written).
        Pages that every later query's window has passed are given back."""
        seq = self.get(seq_id)
        new_len = seq.length + n_tokens
        for g, table in enumerate(seq.tables):
            if new_len > len(table) * self.page_size:
                raise CacheError(f"request {seq_id!r} advanced to {new_len} tokens without pages for them")
        seq.length = new_len
        for g, spec in enumerate(self.layout.groups):
            if spec.window is None:
                continue
            first_needed_pos = new_len - spec.window + 1       # the next query sees keys from here
            dead = max(0, first_needed_pos) // self.page_size   # logical pages wholly before it
            table = seq.tables[g]
            for lp in range(seq.first_live[g], min(dead, len(table))):
                self.pools[g].give(table[lp], seq_id)
                table[lp] = -1
                seq.version += 1
            seq.first_live[g] = max(seq.first_live[g], min(dead, len(table)))

    def close(self, seq_id: Hashable) -> None:
        """Give back everything the request holds."""
        seq = self.get(seq_id)
        for g, table in enumerate(seq.tables):
            for page in table:
                if page >= 0:
                    self.pools[g].give(page, seq_id)
        self._free_slots.append(seq.slot)
        del self.seqs[seq_id]

    # ---- views for the step function ----------------------------------------------------------
    def slot_mapping(self, seq_id: Hashable, group: int, start: int, n: int) -> List[int]:
        """Cache row (page * page_size + offset) of positions ``start .. start+n-1``."""
        table = self.get(seq_id).tables[group]
        ps = self.page_size
        out = []
        for pos in range(start, start + n):
            page = table[pos // ps]
            if page < 0:
                raise CacheError(f"position {pos} of request {seq_id!r} lies in a page that was given back")
            out.append(page * ps + pos % ps)
        return out

    def block_table(self, seq_id: Hashable, group: int) -> List[int]:
        return self.get(seq_id).tables[group]

    def block_table_array(self, seq_id: Hashable, group: int) -> "np.ndarray":
        """The block table as an int32 array, rebuilt only when the table has changed."""
        seq = self.get(seq_id)
        hit = seq._np.get(group)
        if hit is None or hit[0] != seq.version:
            hit = (seq.version, np.asarray(seq.tables[group], dtype=np.int32))
            seq._np[group] = hit
        return hit[1]

    def plane_kv(self, group: int, plane: int):
        """(k, v) storage of one plane, each ``[pages * page_size, kv_heads, head_dim]``."""
        t = self.kv[group]
        if t is None:
            raise CacheError("the cache has no device storage")
        k, v = t[plane, 0], t[plane, 1]
        return k.view(-1, k.shape[-2], k.shape[-1]), v.view(-1, v.shape[-2], v.shape[-1])

    # ---- accounting --------------------------------------------------------------------------
    def free_pages(self, group: int = 0) -> int:
        return self.pools[group].free_count

    def used_pages(self, group: int = 0) -> int:
        return self.pools[group].used_count

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def check(self) -> None:
        """Invariants: pools consistent; every owned page is in exactly one table; slots unique."""
        for g, pool in enumerate(self.pools):
            pool.check()
            seen = {}
            for seq in self.seqs.values():
                for page in seq.tables[g]:
                    if page < 0:
                        continue
                    if page in seen:
                        raise CacheError(f"group {g}: page {page} is held by {seen[page]!r} and {seq.seq_id!r}")
                    seen[page] = seq.seq_id
                    if pool.owner_of(page) != seq.seq_id:
                        raise CacheError(f"group {g}: page {page} in the table of {seq.seq_id!r} "
                                         f"is owned by {pool.owner_of(page)!r}")
            if len(seen) != pool.used_count:
                raise CacheError(f"group {g}: {pool.used_count} pages in use but {len(seen)} in tables (a page is lost)")
        slots = [s.slot for s in self.seqs.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a state slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_seqs:
            raise CacheError("a state slot is lost")
