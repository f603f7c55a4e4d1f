"""The cache manager: keys and values in pages, a block table per request, and
slots for per-request state of fixed size.

The reference keeps one contiguous key/value extent per sequence slot
(runtime/backends/cuda/native/kv_cache_gpu.cu:32-35) and a host-side page
accountant that no kernel ever sees (runtime/kv_cache/paged_kv_cache.h:14-20);
sequence slots are leased with a generation stamp so that a stale free is refused
(runtime/scheduler/sequence_slot_manager.h:17-347).  Here the pages are the device
storage itself.

Caches (one per schedule entry that writes) with the same needs - same heads, head
size and window - form a group.  A group has its own pool
[caches_in_group, pages, 2 (K, V), kv_heads, page_size, head_dim], its own page
allocator and its own block table [max_seqs, max_blocks] on the device, indexed by
the request's slot: one page id serves every cache of the group.  A request's
pages are given back when it ends, and, in a group with a window, as soon as
the window has moved past them.  Entries of the device block table change only
through the updates a step drains with `drain_table_updates`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from ..config.plan import ScheduleEntry
from ..parts.base import KVCacheSpec, StateSpec
from .pages import OutOfPages, PageAccountingError, PageAllocator


class OutOfSlots(RuntimeError):
    """Every request slot is taken."""


@dataclass
class CacheView:
    """What a mixer sees of the cache during one step."""
    kv: Optional[torch.Tensor]              # [pages, 2, kv_heads, page_size, head_dim] or None
    block_table: Optional[torch.Tensor]     # int32 [max_seqs, max_blocks], rows indexed by request slot
    page_size: int
    state: Optional[torch.Tensor]           # [max_seqs, *state shape] or None
    writes: bool                            # False: read what another entry stored, store nothing
    group: int = -1


@dataclass
class _Request:
    rid: Hashable
    slot: int
    generation: int
    length: int = 0                                              # tokens whose keys/values are stored
    blocks: List[Dict[int, int]] = field(default_factory=list)   # per group: logical block -> page
    # per group: blocks [lo, hi) are held (blocks are taken upward without gaps inside what is still
    # needed, and given back from below), so counting what a step needs is O(1)
    lo: List[int] = field(default_factory=list)
    hi: List[int] = field(default_factory=list)


class _Group:
    def __init__(self, spec: KVCacheSpec, cache_ids: List[int], num_pages: int, page_size: int,
                 max_seqs: int, max_blocks: int, dtype, device):
        self.spec = spec
        self.cache_ids = cache_ids
        self.alloc = PageAllocator(num_pages)
        self.pool = torch.zeros((len(cache_ids), num_pages, 2, spec.num_kv_heads, page_size, spec.head_dim),
                                dtype=dtype, device=device)
        self.table = torch.zeros((max_seqs, max_blocks), dtype=torch.int32, device=device)
        self.updates: List[Tuple[int, int]] = []                 # (flat index into table, page)


class CacheManager:
    def __init__(self, cache_specs: Sequence[Tuple[Optional[KVCacheSpec], Optional[StateSpec]]],
                 page_size: int, num_pages: int, max_seqs: int, max_seq_len: int,
                 dtype=torch.bfloat16, device="cpu"):
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        if max_seqs <= 0:
            raise ValueError(f"max_seqs must be positive, got {max_seqs}")
        self.page_size = int(page_size)
        self.num_pages = int(num_pages)
        self.max_seqs = int(max_seqs)
        self.max_seq_len = int(max_seq_len)
        self.max_blocks = -(-self.max_seq_len // self.page_size)
        self.device = torch.device(device)
        self.dtype = dtype

        # ---- groups of caches with the same needs
        self.groups: List[_Group] = []
        self._cache_group: List[Optional[Tuple[int, int]]] = []          # cache -> (group, index in group)
        by_spec: Dict[KVCacheSpec, int] = {}
        members: Dict[int, List[int]] = {}
        for c, (kv, _state) in enumerate(cache_specs):
            if kv is None:
                self._cache_group.append(None)
                continue
            if kv not in by_spec:
                by_spec[kv] = len(by_spec)
                members[by_spec[kv]] = []
            g = by_spec[kv]
            self._cache_group.append((g, len(members[g])))
            members[g].append(c)
        for kv, g in sorted(by_spec.items(), key=lambda it: it[1]):
            self.groups.append(_Group(kv, members[g], self.num_pages, self.page_size, self.max_seqs,
                                      self.max_blocks, dtype, self.device))

        # ---- slots of fixed-size state, one per live request (even when no cache has state)
        self.state: List[Optional[torch.Tensor]] = []
        for _kv, st in cache_specs:
            self.state.append(None if st is None else
                              torch.zeros((self.max_seqs,) + tuple(st.shape), dtype=st.dtype, device=self.device))
        self._free_slots: List[int] = list(range(self.max_seqs - 1, -1, -1))
        self._generation: List[int] = [0] * self.max_seqs
        self._requests: Dict[Hashable, _Request] = {}

    # ------------------------------------------------------------------ requests
    def __contains__(self, rid) -> bool:
        return rid in self._requests

    def live_requests(self):
        return list(self._requests)

    def length(self, rid) -> int:
        return self._requests[rid].length

    def slot(self, rid) -> int:
        return self._requests[rid].slot

    def generation(self, rid) -> int:
        return self._requests[rid].generation

    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def add_request(self, rid) -> int:
        """Give `rid` a slot (its state zeroed) and empty block lists."""
        if rid in self._requests:
            raise KeyError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise OutOfSlots(f"all {self.max_seqs} request slots are taken")
        slot = self._free_slots.pop()
        self._generation[slot] += 1
        for st in self.state:
            if st is not None:
                st[slot].zero_()
        n = len(self.groups)
        self._requests[rid] = _Request(rid, slot, self._generation[slot], 0, [dict() for _ in self.groups],
                                       [0] * n, [0] * n)
        return slot

    def free(self, rid, generation: Optional[int] = None) -> None:
        """Give back everything `rid` holds.  A generation that is not the live one
        (a stale handle to a slot that has since been given to someone else) is refused."""
        req = self._requests.get(rid)
        if req is None:
            raise KeyError(f"request {rid!r} is not live (freed twice?)")
        if generation is not None and generation != req.generation:
            raise PageAccountingError(f"stale free of request {rid!r}: generation {generation}, "
                                      f"live generation {req.generation}")
        for g, held in zip(self.groups, req.blocks):
            g.alloc.release(list(held.values()), owner=rid)
            held.clear()
        self._free_slots.append(req.slot)
        del self._requests[rid]

    # --------------------------------------------------------------------- pages
    def _first_needed_block(self, group: _Group, next_position: int) -> int:
        """Lowest block a query at `next_position` (and any later one) still reads."""
        w = group.spec.window
        if w is None:
            return 0
        return max(0, next_position - w + 1) // self.page_size

    def pages_needed(self, rid, new_len: int) -> List[int]:
        """Per group, how many pages a step that extends `rid` to `new_len` tokens must take."""
        req = self._requests[rid]
        last = -(-new_len // self.page_size)
        need = []
        for gi, g in enumerate(self.groups):
            first = self._first_needed_block(g, req.length)
            need.append(max(0, last - max(first, req.hi[gi])))
        return need

    def pages_needed_fresh(self, new_len: int) -> List[int]:
        """The same for a request that is not live yet."""
        return [-(-new_len // self.page_size) for _ in self.groups]

    def free_pages(self) -> List[int]:
        return [g.alloc.num_free for g in self.groups]

    def can_reserve(self, rid, new_len: int) -> bool:
        if new_len > self.max_seq_len:
            return False
        return all(n <= g.alloc.num_free for n, g in zip(self.pages_needed(rid, new_len), self.groups))

    def reserve(self, rid, new_len: int) -> None:
        """Take the pages that positions [length, new_len) of `rid` need, in every
        group or in none."""
        req = self._requests[rid]
        if new_len < req.length:
            raise ValueError(f"request {rid!r} holds {req.length} tokens, cannot shrink to {new_len}")
        if new_len > self.max_seq_len:
            raise OutOfPages(f"request {rid!r}: {new_len} tokens exceed the longest sequence the cache "
                             f"was made for ({self.max_seq_len})")
        need = self.pages_needed(rid, new_len)
        for n, g in zip(need, self.groups):
            if n > g.alloc.num_free:
                raise OutOfPages(f"request {rid!r} needs {need} pages per group to reach {new_len} tokens, "
                                 f"free: {self.free_pages()}")
        last = -(-new_len // self.page_size)
        for gi, (g, held) in enumerate(zip(self.groups, req.blocks)):
            first = self._first_needed_block(g, req.length)
            start = max(first, req.hi[gi])
            if start >= last:
                continue
            pages = g.alloc.allocate(last - start, owner=rid)
            for b, p in zip(range(start, last), pages):
                held[b] = p
                g.updates.append((req.slot * self.max_blocks + b, p))
            if not held or req.hi[gi] <= req.lo[gi]:
                req.lo[gi] = start
            req.hi[gi] = last

    def release_uncommitted(self, rid) -> None:
        """Give back the blocks that `reserve` took beyond what the committed length needs (a step
        that reserved and then failed before `commit`)."""
        req = self._requests[rid]
        keep = -(-req.length // self.page_size)
        for gi, (g, held) in enumerate(zip(self.groups, req.blocks)):
            dead = [b for b in held if b >= keep]
            if dead:
                g.alloc.release([held[b] for b in dead], owner=rid)
                for b in dead:
                    del held[b]
                gone = {req.slot * self.max_blocks + b for b in dead}
                g.updates = [(i, p) for i, p in g.updates if i not in gone]     # the table never learns of them
            req.hi[gi] = max(req.lo[gi], min(req.hi[gi], keep))

    def commit(self, rid, new_len: int) -> None:
        """The step has stored positions up to new_len - 1; pages that a window has
        moved past are given back."""
        req = self._requests[rid]
        req.length = new_len
        for gi, (g, held) in enumerate(zip(self.groups, req.blocks)):
            if g.spec.window is None:
                continue
            first = min(self._first_needed_block(g, new_len), req.hi[gi])
            if req.lo[gi] < first:
                dead = [b for b in range(req.lo[gi], first) if b in held]
                if dead:
                    g.alloc.release([held[b] for b in dead], owner=rid)
                    for b in dead:
                        del held[b]
                req.lo[gi] = first

    def drain_table_updates(self) -> List[List[Tuple[int, int]]]:
        """Per group, the (flat index, page) pairs that the device block table has
        not seen yet; the caller writes them before the next kernel reads the table."""
        out = []
        for g in self.groups:
            out.append(g.updates)
            g.updates = []
        return out

    # --------------------------------------------------------------------- views
    def view(self, entry: ScheduleEntry) -> CacheView:
        where = self._cache_group[entry.cache]
        state = self.state[entry.cache]
        if where is None:
            return CacheView(None, None, self.page_size, state, entry.writes_cache)
        gi, idx = where
        g = self.groups[gi]
        return CacheView(g.pool[idx], g.table, self.page_size, state, entry.writes_cache, gi)

    def pages_of(self, rid, group: int = 0) -> Dict[int, int]:
        return dict(self._requests[rid].blocks[group])

    # -------------------------------------------------------------------- checks
    def check(self) -> None:
        """No page lost, held twice or freed twice; no slot lost or held twice."""
        for gi, g in enumerate(self.groups):
            g.alloc.check()
            seen = {}
            for rid, req in self._requests.items():
                for b, p in req.blocks[gi].items():
                    if p in seen:
                        raise PageAccountingError(f"group {gi}: page {p} is held by {seen[p]!r} and {rid!r}")
                    if g.alloc.owner_of(p) != rid:
                        raise PageAccountingError(f"group {gi}: page {p} of {rid!r} has owner "
                                                  f"{g.alloc.owner_of(p)!r}")
                    seen[p] = rid
            if len(seen) != g.alloc.num_used:
                raise PageAccountingError(f"group {gi}: {g.alloc.num_used} pages are taken but requests hold "
                                          f"{len(seen)} (a page is lost)")
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise PageAccountingError("a request slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_seqs:
            raise PageAccountingError("a request slot is lost")

    def stats(self) -> dict:
        return {"groups": [{"window": g.spec.window, "caches": len(g.cache_ids), "pages": g.alloc.num_pages,
                            "free": g.alloc.num_free, "allocations": g.alloc.allocations}
                           for g in self.groups],
                "live_requests": len(self._requests), "free_slots": len(self._free_slots)}
