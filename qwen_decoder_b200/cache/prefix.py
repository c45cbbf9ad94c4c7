"""Prefix cache: requests whose prompts begin alike share the full cache pages of the common part.

The reference keys each full page by an FNV-1a hash of all tokens up to its end and trusts the
hash (prefix_cache.cpp:14-24, 37-43); it looks prompts up at admission, shares live pages or takes
freed ones back from the free list (prefix_cache.cpp:26-62), records pages when a prompt is done
(prefix_cache.cpp:64-88) and forgets a page when the pool hands it out again
(prefix_cache.cpp:9-11, kv_cache.cpp:67-74).  Here the index is a trie keyed by (parent entry,
the page's tokens), so a hit is exact; pages are recorded as soon as they are full (generated
tokens too), and a match always leaves at least one token to compute (prefix_cache.cpp:29-32).
The index holds no references: a recorded page that nobody holds sits on the free list and is
lost when it is handed out again.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

from .pages import PagePool


@dataclass
class PrefixEntry:
    key: Tuple[int, Tuple[int, ...]]      # (parent entry id, tokens of the page)
    pages: Tuple[int, ...]                # the page of each cache group


class PrefixIndex:
    ROOT = 0

    def __init__(self, pools: Sequence[PagePool], page_size: int):
        self.pools = list(pools)
        self.page_size = page_size
        self._next_id = 1
        self.children: Dict[Tuple[int, Tuple[int, ...]], int] = {}
        self.entries: Dict[int, PrefixEntry] = {}
        self._by_page: List[Dict[int, int]] = [dict() for _ in pools]     # group -> page -> entry id
        self.hits = 0
        for g, pool in enumerate(self.pools):
            pool.on_allocate = (lambda page, g=g: self._forget(g, page))

    def _forget(self, group: int, page: int) -> None:
        eid = self._by_page[group].pop(page, None)
        if eid is None:
            return
        e = self.entries.pop(eid)
        self.children.pop(e.key, None)
        for g, p in enumerate(e.pages):          # the entry is void in every group
            if g != group:
                self._by_page[g].pop(p, None)

    def match(self, tokens: Sequence[int]) -> List[int]:
        """Entry ids of the longest recorded chain of full pages that ``tokens`` begins with, leaving
        at least one token uncovered."""
        ps = self.page_size
        out: List[int] = []
        parent = self.ROOT
        for i in range(max(0, (len(tokens) - 1) // ps)):
            eid = self.children.get((parent, tuple(tokens[i * ps:(i + 1) * ps])))
            if eid is None:
                break
            out.append(eid)
            parent = eid
        return out

    def acquire(self, eid: int) -> Tuple[int, ...]:
        """Hold the pages of an entry for one more request (taking them off the free list if nobody
        held them); returns the page of each group."""
        e = self.entries[eid]
        for g, p in enumerate(e.pages):
            if self.pools[g].ref_count(p) == 0:
                self.pools[g].take(p)
            else:
                self.pools[g].retain(p)
        self.hits += 1
        return e.pages

    def record(self, parent: int, page_tokens: Sequence[int], pages: Sequence[int]) -> int:
        """Record a full page; returns the id of its entry (an older entry with the same content wins)."""
        key = (parent, tuple(page_tokens))
        eid = self.children.get(key)
        if eid is not None:
            return eid
        if any(p in self._by_page[g] for g, p in enumerate(pages)):
            return -1                      # the page already stands for other content (cannot happen for owned pages)
        eid = self._next_id
        self._next_id += 1
        self.children[key] = eid
        self.entries[eid] = PrefixEntry(key, tuple(pages))
        for g, p in enumerate(pages):
            self._by_page[g][p] = eid
        return eid
