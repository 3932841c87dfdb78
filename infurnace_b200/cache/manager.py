"""The cache manager: pages of keys and values with a block table for each request, in
groups, and slots for per-request state of fixed size.

The reference keeps one contiguous region per slot (``kv[layer, 2, slot, position,
kv_head, head_dim]``, src/infurnace/executor/tinygrad/buffers.py:36-45) and reserves it at
admission (src/infurnace/scheduler/scheduler.py:56-62); its paged design exists as text
only (docs/architecture.md:219-257: logical pages, block tables, a page-granular store).
This file is that design.

Groups.  The layer calls of a model are grouped by what they need
(``cache_need().group_key``): all calls that keep every key share one group; calls
with a window of w keys form another; calls with fixed-size state a third.  A key/value
group has a page pool and, for each request, a block table of its own, because its
pages come and go by its own rule: a full-attention group holds a request's pages
until the request ends, a window group gives a page back as soon as every key in it
lies below the window of the request's next query.  Each cache entry (one per layer
call that stores) of a group has a tensor ``[pages, 2, kv_heads, page_size, head_dim]``
(keys and values of one shape), or, for a need whose streams differ in shape (values narrower
than keys, a latent beside a small rotated key), one tensor ``[pages, heads, page_size, width]``
per stream; the entries of one group share page ids, so one block table serves them all.

State slots.  A request gets a slot id when it is added and returns it when it ends.
The id is the row of the request in every fixed-size state tensor ``[slots, *shape]``
(zeroed when the slot is granted).  A model without such state, like Qwen3, has slots
that own no memory.

Accounting.  ``allocate(rid, n)`` takes the pages that n further tokens need, in every
group or in none.  ``commit(rid, n)`` records that n tokens were stored and releases
pages that a window has passed.  ``free_request`` gives everything back, once.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from ..config.specs import KVCacheNeed, ModelPlan, PagedCacheNeed, StateNeed
from ..errors import CacheError, OutOfPages
from .block_pool import BlockPool

RELEASED = -1      # block-table entry of a logical page that was given back


@dataclass
class KVGroup:
    need: KVCacheNeed
    cache_ids: List[int]
    pool: BlockPool
    page_size: int
    tables: Dict[str, List[int]] = field(default_factory=dict)
    tensors: Dict[int, object] = field(default_factory=dict)      # cache id -> device tensor (None: streams of unequal shape)
    streams: Dict[int, Dict[str, object]] = field(default_factory=dict)      # cache id -> stream name -> device tensor

    @property
    def uniform(self) -> bool:
        """All streams have one shape, so an entry is a single tensor with a stream axis."""
        st = self.need.streams
        return all((x.heads, x.width) == (st[0].heads, st[0].width) for x in st)

    def first_needed_page(self, next_position: int) -> int:
        """Index of the first logical page that the query at ``next_position`` can read."""
        if self.need.window is None:
            return 0
        return max(0, next_position - self.need.window + 1) // self.page_size


@dataclass
class StateGroup:
    need: StateNeed
    cache_ids: List[int]
    tensors: Dict[int, object] = field(default_factory=dict)      # cache id -> [slots, *shape]


class CacheLayout:
    """Which cache entries a plan has and how they group."""

    def __init__(self, plan: ModelPlan):
        self.kv: Dict[tuple, Tuple[KVCacheNeed, List[int]]] = {}
        self.state: Dict[tuple, Tuple[StateNeed, List[int]]] = {}
        self.group_of: Dict[int, tuple] = {}
        for call in plan.resolved_schedule():
            need = plan.layers[call.layer].cache_need()
            if need is None:
                continue
            key = need.group_key
            if call.cache in self.group_of:
                if self.group_of[call.cache] != key:
                    raise CacheError(f"cache entry {call.cache} is read by a layer with a different need "
                                     f"({key}) than the layer that stores it ({self.group_of[call.cache]})")
                continue
            self.group_of[call.cache] = key
            table = self.kv if isinstance(need, (KVCacheNeed, PagedCacheNeed)) else self.state
            table.setdefault(key, (need, []))[1].append(call.cache)


class CacheManager:
    def __init__(self, plan: ModelPlan, page_size: int, num_pages, max_requests: int,
                 dtype=None, device=None, allocate_tensors: bool = True):
        """``num_pages``: pages of every key/value group (an int), or a dict from group key
        to its count.  ``allocate_tensors`` False gives a manager that only does the
        accounting (tests without a device)."""
        if page_size < 1:
            raise CacheError("page_size must be positive")
        if max_requests < 1:
            raise CacheError("max_requests must be positive")
        self.page_size = page_size
        self.max_requests = max_requests
        self.layout = CacheLayout(plan)
        self.kv_groups: List[KVGroup] = []
        self.state_groups: List[StateGroup] = []
        self._group_index: Dict[int, Tuple[str, int]] = {}           # cache id -> ("kv"|"state", index)
        for key, (need, ids) in self.layout.kv.items():
            n = num_pages[key] if isinstance(num_pages, dict) else int(num_pages)
            g = KVGroup(need, ids, BlockPool(n), page_size)
            for cid in ids:
                self._group_index[cid] = ("kv", len(self.kv_groups))
            self.kv_groups.append(g)
        for key, (need, ids) in self.layout.state.items():
            g = StateGroup(need, ids)
            for cid in ids:
                self._group_index[cid] = ("state", len(self.state_groups))
            self.state_groups.append(g)
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self._slot_of: Dict[str, int] = {}
        self._computed: Dict[str, int] = {}
        self._epoch: Dict[str, int] = {}          # rid -> serial number of its current life (ids may be reused)
        self._lives = 0
        if allocate_tensors:
            import torch
            for g in self.kv_groups:
                st = g.need.streams
                for cid in g.cache_ids:
                    if g.uniform:
                        t = torch.zeros((g.pool.num_pages, len(st), st[0].heads, page_size, st[0].width),
                                        dtype=dtype, device=device)
                        g.tensors[cid] = t
                        g.streams[cid] = {x.name: t[:, i] for i, x in enumerate(st)}
                    else:
                        g.tensors[cid] = None
                        g.streams[cid] = {x.name: torch.zeros((g.pool.num_pages, x.heads, page_size, x.width),
                                                              dtype=dtype, device=device) for x in st}
            for g in self.state_groups:
                for cid in g.cache_ids:
                    g.tensors[cid] = torch.zeros((max_requests, *g.need.shape), dtype=torch.float32, device=device)

    # ------------------------------------------------------------------ lookups
    def kv_group_of(self, cache_id: int) -> int:
        kind, idx = self._group_index[cache_id]
        if kind != "kv":
            raise CacheError(f"cache entry {cache_id} holds fixed-size state, not keys and values")
        return idx

    def state_group_of(self, cache_id: int) -> int:
        kind, idx = self._group_index[cache_id]
        if kind != "state":
            raise CacheError(f"cache entry {cache_id} holds keys and values, not fixed-size state")
        return idx

    def has_request(self, rid: str) -> bool:
        return rid in self._slot_of

    def num_computed(self, rid: str) -> int:
        return self._computed[rid]

    def slot_of(self, rid: str) -> int:
        return self._slot_of[rid]

    def epoch_of(self, rid: str) -> int:
        """A number that differs between two lives of the same request id."""
        return self._epoch[rid]

    def block_table(self, rid: str, group: int) -> List[int]:
        return self.kv_groups[group].tables[rid]

    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.kv_groups]

    def bytes_per_token(self) -> int:
        total = 0
        for g in self.kv_groups:
            for streams in g.streams.values():
                for x in g.need.streams:
                    total += x.heads * x.width * streams[x.name].element_size()
        return total

    # ------------------------------------------------------------------ life of a request
    def add_request(self, rid: str) -> int:
        """Grant a state slot.  Raises :class:`CacheError` if the id is live or no slot is free."""
        if rid in self._slot_of:
            raise CacheError(f"request {rid!r} is already live in the cache")
        if not self._free_slots:
            raise CacheError("no state slot is free")
        slot = self._free_slots.pop()
        self._slot_of[rid] = slot
        self._computed[rid] = 0
        self._lives += 1
        self._epoch[rid] = self._lives
        for g in self.kv_groups:
            g.tables[rid] = []
        for g in self.state_groups:
            for t in g.tensors.values():
                t[slot].zero_()
        return slot

    def pages_needed(self, rid: str, num_new_tokens: int) -> List[int]:
        """Pages each key/value group lacks for ``num_new_tokens`` more tokens of ``rid``."""
        end = self._computed[rid] + num_new_tokens
        want = -(-end // self.page_size)
        return [max(0, want - len(g.tables[rid])) for g in self.kv_groups]

    def can_allocate(self, rid: str, num_new_tokens: int, reserved: Optional[List[int]] = None) -> bool:
        """``reserved``: pages of each group already promised to others in the same plan."""
        need = self.pages_needed(rid, num_new_tokens)
        for i, g in enumerate(self.kv_groups):
            if need[i] > g.pool.num_free - (reserved[i] if reserved else 0):
                return False
        return True

    def allocate(self, rid: str, num_new_tokens: int) -> None:
        """Take the pages for ``num_new_tokens`` more tokens: in every group, or in none."""
        if num_new_tokens < 1:
            raise CacheError("a request advances by at least one token")
        need = self.pages_needed(rid, num_new_tokens)
        taken: List[Tuple[KVGroup, List[int]]] = []
        try:
            for g, n in zip(self.kv_groups, need):
                taken.append((g, g.pool.allocate(n)))
        except OutOfPages:
            for g, pages in taken:
                g.pool.free(pages)
            raise
        for g, pages in taken:
            g.tables[rid].extend(pages)

    def release_allocation(self, rid: str) -> None:
        """Undo ``allocate`` calls that no ``commit`` followed: give back the pages above
        what the committed tokens need."""
        keep = -(-self._computed[rid] // self.page_size)
        for g in self.kv_groups:
            table = g.tables[rid]
            extra = [p for p in table[keep:] if p != RELEASED]
            del table[keep:]
            g.pool.free(extra)

    def slots_for(self, rid: str, group: int, num_new_tokens: int) -> List[int]:
        """Where the next tokens are stored: page * page_size + offset for each."""
        g = self.kv_groups[group]
        table, start, ps = g.tables[rid], self._computed[rid], self.page_size
        out = []
        for pos in range(start, start + num_new_tokens):
            page = table[pos // ps]
            if page == RELEASED:
                raise CacheError(f"request {rid!r} would store position {pos} in a page it gave back")
            out.append(page * ps + pos % ps)
        return out

    def slots_array(self, rid: str, group: int, num_new_tokens: int):
        """``slots_for`` as an int32 numpy array, without a Python loop over the tokens."""
        import numpy as np
        g = self.kv_groups[group]
        table, start, ps = g.tables[rid], self._computed[rid], self.page_size
        pos = np.arange(start, start + num_new_tokens, dtype=np.int64)
        first, last = start // ps, (start + num_new_tokens - 1) // ps
        pages = np.asarray(table[first:last + 1], dtype=np.int64)
        if (pages == RELEASED).any():
            raise CacheError(f"request {rid!r} would store in a page it gave back")
        return (pages[pos // ps - first] * ps + pos % ps).astype(np.int32)

    def commit(self, rid: str, num_new_tokens: int) -> None:
        """``num_new_tokens`` were stored.  Pages that every later query's window has passed
        go back to their pool; their block-table entries become ``RELEASED``."""
        self._computed[rid] += num_new_tokens
        nxt = self._computed[rid]
        for g in self.kv_groups:
            if len(g.tables[rid]) < -(-nxt // self.page_size):
                raise CacheError(f"request {rid!r} committed tokens for which it holds no pages")
        for g in self.kv_groups:
            if g.need.window is None:
                continue
            table = g.tables[rid]
            first = min(g.first_needed_page(nxt), len(table))
            gone = [p for p in table[:first] if p != RELEASED]
            if gone:
                for i in range(first):
                    table[i] = RELEASED
                g.pool.free(gone)

    def free_request(self, rid: str) -> None:
        """Give back every page and the state slot of ``rid``.  A second call is an error."""
        if rid not in self._slot_of:
            raise CacheError(f"request {rid!r} is not live in the cache (freed twice?)")
        for g in self.kv_groups:
            g.pool.free([p for p in g.tables.pop(rid) if p != RELEASED])
        self._free_slots.append(self._slot_of.pop(rid))
        del self._computed[rid]
        del self._epoch[rid]

    # ------------------------------------------------------------------ invariants
    def check(self) -> None:
        """No page lost, held twice or freed twice; slots likewise."""
        for g in self.kv_groups:
            g.pool.check()
            owned = [p for t in g.tables.values() for p in t if p != RELEASED]
            if len(set(owned)) != len(owned):
                raise CacheError("a page is in two block tables")
            for p in owned:
                if not g.pool.is_held(p):
                    raise CacheError(f"page {p} is in a block table but free in the pool")
            if len(owned) != g.pool.num_held:
                raise CacheError(f"{g.pool.num_held - len(owned)} pages are held by no request")
        slots = list(self._slot_of.values())
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a state slot is granted twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("a state slot is lost")
