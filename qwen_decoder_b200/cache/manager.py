"""The cache manager: what each run of a layer caches, grouped by need, in pages.

A mixer declares its need: ``PagedKV`` (keys and values per token, all of them or a
window) or ``FixedState`` (a per-request tensor of fixed size), or nothing.  Runs
with equal paged needs form a *group*: one page id serves every layer of the group
(as one page serves all layers in the reference, kv_cache.h:16-29), and every group
has pages and block tables of its own, so that a windowed group can give pages back
while a full group keeps them.  Pages are taken lazily, as the reference's
``ensure_blocks`` does (scheduler.cpp:67-80), and given back when a request ends
(scheduler.cpp:43-52) or when a window has passed them.

Device layout of a group: ``[layer in group, page, K|V, kv head, offset in page,
head_dim]``, so that one (layer, page, K or V, kv head) tile is contiguous.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .pages import BlockTable, CacheAccountingError, OutOfPages, PagePool, StateSlots
from .prefix import PrefixIndex


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of ``num_kv_heads`` x ``head_dim`` per token; ``window`` = None keeps
    all of them, an integer keeps the last ``window`` positions readable."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """A per-request tensor of fixed ``shape`` (zero when a request starts)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class CacheGroup:
    need: PagedKV
    entries: List[int] = field(default_factory=list)   # schedule entries that own a layer here


@dataclass
class CacheLayout:
    """Where each schedule entry's cache lives.

    ``paged[e] = (group, layer_in_group)`` and ``fixed[e] = index into state tensors`` for
    entries that own a cache; entries that read another entry's cache map to the same place.
    """
    groups: List[CacheGroup]
    paged: Dict[int, Tuple[int, int]]
    fixed: Dict[int, int]
    fixed_needs: List[FixedState]
    owners: Dict[int, int]      # schedule entry -> entry whose cache it uses

    @classmethod
    def from_needs(cls, needs: Sequence[Optional[object]], cache_of: Sequence[Optional[int]]) -> "CacheLayout":
        """``needs[e]``: the need of schedule entry e's mixer; ``cache_of[e]``: None or an earlier entry."""
        groups: List[CacheGroup] = []
        paged: Dict[int, Tuple[int, int]] = {}
        fixed: Dict[int, int] = {}
        fixed_needs: List[FixedState] = []
        owners: Dict[int, int] = {}
        by_need: Dict[PagedKV, int] = {}
        for e, (need, src) in enumerate(zip(needs, cache_of)):
            if src is not None:
                if not (0 <= src < e) or cache_of[src] is not None:
                    raise ValueError(f"schedule entry {e}: cache_of must name an earlier entry that owns its cache")
                if needs[src] != need:
                    raise ValueError(f"schedule entry {e} reads the cache of entry {src}, whose need differs")
                owners[e] = src
                if src in paged:
                    paged[e] = paged[src]
                if src in fixed:
                    fixed[e] = fixed[src]
                continue
            owners[e] = e
            if need is None:
                continue
            if isinstance(need, PagedKV):
                g = by_need.get(need)
                if g is None:
                    g = len(groups)
                    by_need[need] = g
                    groups.append(CacheGroup(need))
                paged[e] = (g, len(groups[g].entries))
                groups[g].entries.append(e)
            elif isinstance(need, FixedState):
                fixed[e] = len(fixed_needs)
                fixed_needs.append(need)
            else:
                raise TypeError(f"schedule entry {e}: unknown cache need {need!r}")
        return cls(groups, paged, fixed, fixed_needs, owners)


class RequestCache:
    """What one live request holds: a block table per group and a state slot."""

    def __init__(self, request_id, num_groups: int, state_slot: int):
        self.request_id = request_id
        self.num_tokens = 0                      # tokens whose cache entries are written
        self.tables = [BlockTable() for _ in range(num_groups)]
        self.state_slot = state_slot
        self.closed = False
        # prefix cache: the tokens cached so far and the index entry of each full page (-1: none)
        self.token_log: List[int] = []
        self.prefix_ids: List[int] = []


class CacheManager:
    """Pools, tables and state slots of all live requests; device tensors if ``device`` is given."""

    def __init__(self, layout: CacheLayout, num_pages: int, page_size: int, max_requests: int,
                 dtype: torch.dtype = torch.bfloat16, device=None, prefix_cache: bool = False):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.layout = layout
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.pools = [PagePool(num_pages) for _ in layout.groups]
        self.slots = StateSlots(max_requests)
        self.live: Dict[object, RequestCache] = {}
        # Sharing pages of a common prefix needs every group to keep all keys and no per-request state:
        # a windowed group gives pages back early and a fixed-size state cannot be shared.
        self.prefix: Optional[PrefixIndex] = None
        if prefix_cache and layout.groups and not layout.fixed_needs and \
                all(g.need.window is None for g in layout.groups):
            self.prefix = PrefixIndex(self.pools, page_size)
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else None
        self.kv: List[Optional[torch.Tensor]] = [None] * len(layout.groups)
        self.states: List[Optional[torch.Tensor]] = [None] * len(layout.fixed_needs)
        if self.device is not None:
            # one page more than the pool hands out: the rows that pad a batch write their keys and values there
            for g, grp in enumerate(layout.groups):
                n = grp.need
                self.kv[g] = torch.zeros(
                    (len(grp.entries), num_pages + 1, 2, n.num_kv_heads, page_size, n.head_dim),
                    dtype=dtype, device=self.device)
            # one slot more than requests: the padding rows of a padded decode batch update that one
            for i, need in enumerate(layout.fixed_needs):
                self.states[i] = torch.zeros((max_requests + 1,) + tuple(need.shape), dtype=need.dtype,
                                             device=self.device)

    @property
    def scratch_page(self) -> int:
        """The page (of every group) that belongs to no request: rows that pad a batch write to it."""
        return self.num_pages

    @property
    def scratch_slot(self) -> int:
        """The state slot that belongs to no request: rows that pad a batch read and write it."""
        return self.max_requests

    # ---- sizes ---------------------------------------------------------
    @staticmethod
    def bytes_per_page(layout: CacheLayout, page_size: int, dtype: torch.dtype) -> int:
        """Device bytes one page id costs over all groups and layers."""
        es = torch.empty((), dtype=dtype).element_size()
        return sum(len(g.entries) * 2 * g.need.num_kv_heads * g.need.head_dim * page_size * es
                   for g in layout.groups)

    def _pages_for(self, g: int, first_token: int, total_tokens: int) -> range:
        """Logical pages of group g that tokens [first_token, total_tokens) touch."""
        ps = self.page_size
        return range(first_token // ps, (total_tokens + ps - 1) // ps)

    def _first_needed_page(self, g: int, next_pos: int) -> int:
        """Lowest logical page a query at position >= next_pos may still read."""
        w = self.layout.groups[g].need.window
        if w is None:
            return 0
        return max(0, next_pos - w + 1) // self.page_size

    def pages_missing(self, rc: RequestCache, total_tokens: int) -> List[int]:
        """Pages per group that ``ensure(rc, total_tokens)`` would have to take."""
        out = []
        for g, table in enumerate(self.tables_of(rc)):
            need_upto = (total_tokens + self.page_size - 1) // self.page_size
            out.append(max(0, need_upto - len(table)))
        return out

    def tables_of(self, rc: RequestCache) -> List[BlockTable]:
        return rc.tables

    def free_pages(self) -> List[int]:
        return [p.num_free for p in self.pools]

    # ---- life of a request ----------------------------------------------
    def open(self, request_id, tokens: Optional[Sequence[int]] = None) -> RequestCache:
        """Start a request.  With the prefix cache on and the request's ``tokens`` given, full pages
        that an earlier request cached for the same beginning are shared: ``num_tokens`` then starts
        above zero and the caller feeds only the rest."""
        if request_id in self.live:
            raise CacheAccountingError(f"request {request_id!r} is already live")
        slot = self.slots.allocate()
        rc = RequestCache(request_id, len(self.pools), slot)
        self.live[request_id] = rc
        for st in self.states:
            if st is not None:
                st[slot].zero_()
        if self.prefix is not None and tokens is not None:
            for eid in self.prefix.match(tokens):
                pages = self.prefix.acquire(eid)
                for g, p in enumerate(pages):
                    rc.tables[g].pages.append(p)
                rc.prefix_ids.append(eid)
            n = len(rc.prefix_ids) * self.page_size
            rc.num_tokens = n
            rc.token_log = [int(t) for t in tokens[:n]]
        return rc

    def ensure(self, rc: RequestCache, total_tokens: int) -> None:
        """Make pages exist for token positions < total_tokens in every group; takes all or nothing."""
        missing = self.pages_missing(rc, total_tokens)
        for g, m in enumerate(missing):
            if m > self.pools[g].num_free:
                raise OutOfPages(
                    f"request {rc.request_id!r} needs {m} more pages in cache group {g}, "
                    f"{self.pools[g].num_free} free")
        for g, m in enumerate(missing):
            for _ in range(m):
                rc.tables[g].pages.append(self.pools[g].allocate())

    def commit(self, rc: RequestCache, n_tokens: int, tokens: Optional[Sequence[int]] = None) -> None:
        """The step wrote ``n_tokens`` more tokens (``tokens``: which ones, for the prefix cache; a caller
        that does not know them yet gives None and calls ``log_tokens`` later); give back pages a
        window has passed."""
        rc.num_tokens += n_tokens
        if tokens is not None:
            self.log_tokens(rc, tokens)
        for g, table in enumerate(rc.tables):
            if rc.num_tokens > len(table) * self.page_size:
                raise CacheAccountingError(
                    f"request {rc.request_id!r} holds {rc.num_tokens} tokens but only {len(table)} pages")
            first = min(self._first_needed_page(g, rc.num_tokens), len(table))
            for p in range(table.first_live, first):
                if table.pages[p] != BlockTable.RELEASED:
                    self.pools[g].release(table.pages[p])
                    table.pages[p] = BlockTable.RELEASED
            table.first_live = max(table.first_live, first)

    def log_tokens(self, rc: RequestCache, tokens: Sequence[int]) -> None:
        """Tell the prefix cache which tokens the request's next cached positions hold; every page that is
        full of known tokens is recorded."""
        if self.prefix is None or rc.closed or len(rc.token_log) + len(tokens) > rc.num_tokens:
            return
        rc.token_log.extend(int(t) for t in tokens)
        ps = self.page_size
        while (len(rc.prefix_ids) + 1) * ps <= len(rc.token_log):
            i = len(rc.prefix_ids)
            parent = rc.prefix_ids[-1] if rc.prefix_ids else PrefixIndex.ROOT
            if parent < 0:
                rc.prefix_ids.append(-1)          # the chain broke earlier: nothing below is recorded
                continue
            rc.prefix_ids.append(self.prefix.record(parent, rc.token_log[i * ps:(i + 1) * ps],
                                                    [t.pages[i] for t in rc.tables]))

    def close(self, rc: RequestCache) -> None:
        """Give back everything the request holds (last page first, as kv_cache.h:231-236)."""
        if rc.closed:
            raise CacheAccountingError(f"request {rc.request_id!r} closed twice")
        for g, table in enumerate(rc.tables):
            for p in reversed(table.pages):
                if p != BlockTable.RELEASED:
                    self.pools[g].release(p)
            table.pages.clear()
        self.slots.release(rc.state_slot)
        rc.closed = True
        del self.live[rc.request_id]

    def check(self) -> None:
        """Invariants: every page is free or held by exactly the tables that name it."""
        for g, pool in enumerate(self.pools):
            pool.check()
            held: Dict[int, int] = {}
            for rc in self.live.values():
                for p in rc.tables[g].live_pages():
                    held[p] = held.get(p, 0) + 1
            for p in range(pool.num_pages):
                if pool.ref_count(p) != held.get(p, 0):
                    raise CacheAccountingError(
                        f"group {g} page {p}: reference count {pool.ref_count(p)} but named by {held.get(p, 0)} tables")

    # ---- views for the step ------------------------------------------------
    def layer_kv(self, entry: int) -> torch.Tensor:
        g, l = self.layout.paged[entry]
        return self.kv[g][l]

    def layer_state(self, entry: int) -> torch.Tensor:
        return self.states[self.layout.fixed[entry]]
