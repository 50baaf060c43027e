"""Page bookkeeping per cache group: full attention, sliding window, chunked-local attention.

Role of the reference's single-type managers and their coordinator
(easydel/inference/esurge/core/single_type_cache_manager.py:404 ``SlidingWindowManager``, :528
``ChunkedLocalAttentionManager``, :170 ``FullAttentionManager``; core/kv_cache_coordinator.py): every group of layers
with the same retention rule owns a :class:`PagePool` and one page list per request. A request's lists all have one
entry per 128-token page of its context, so a token position indexes every group's list the same way; a page that a
window-bounded group no longer needs is given back to that group's pool and its entry becomes the null page (the
attention kernels skip key tiles in front of the window, so the entry is never dereferenced).

Prefix caching: a cached prefix of ``n`` pages can be reused if every unbounded group still holds all ``n`` pages and
every bounded group still holds the pages its window reaches back to from position ``n * 128``.
"""

from __future__ import annotations

import typing as tp

from ...caching.specs import KVCacheGroup, KVCacheSpec, cdiv
from .page_pool import NULL_PAGE, PagePool


class GroupManager:
    """One group's pool plus the retention rule of its layers."""

    def __init__(self, spec: KVCacheSpec, num_pages: int, enable_caching: bool = True, layers: tp.Sequence[int] = ()):
        self.spec = spec
        self.layers = list(layers)
        self.pool = PagePool(num_pages, enable_caching=enable_caching)
        self.bounded = spec.kind in ("sliding", "chunked")

    # -- allocation
    def pages_needed(self, pages: list[int], upto_tokens: int) -> int:
        return max(0, cdiv(upto_tokens, self.spec.page_size) - len(pages))

    def release(self, pages: list[int]) -> None:
        self.pool.release([p for p in pages if p != NULL_PAGE])
        pages.clear()

    def remove_skipped(self, pages: list[int], num_computed_tokens: int) -> int:
        """Gives back the pages that lie entirely in front of the first key any later query can read."""
        if not self.bounded:
            return 0
        upto = min(self.spec.first_useful_token(num_computed_tokens) // self.spec.page_size, len(pages))
        freed = []
        for i in range(upto - 1, -1, -1):
            if pages[i] == NULL_PAGE:     # everything further left went in an earlier call
                break
            freed.append(pages[i])
            pages[i] = NULL_PAGE
        if freed:
            self.pool.release(freed)      # reversed inside: the oldest page becomes evictable first
        return len(freed)

    # -- prefix cache
    def window_start_page(self, num_pages_hit: int) -> int:
        """First page a hit of ``num_pages_hit`` pages must still hold."""
        if not self.bounded:
            return 0
        return self.spec.first_useful_token(num_pages_hit * self.spec.page_size) // self.spec.page_size

    def holds(self, hashes: tp.Sequence[bytes], n: int) -> bool:
        cached = self.pool.cached
        return all(hashes[i] in cached for i in range(self.window_start_page(n), n))

    def take_cached(self, hashes: tp.Sequence[bytes], n: int) -> list[int]:
        lo = self.window_start_page(n)
        got = [self.pool.cached[hashes[i]] for i in range(lo, n)]
        self.pool.touch(got)
        self.pool.stats.queries += n
        self.pool.stats.hits += n
        return [NULL_PAGE] * lo + got


class KVCacheCoordinator:
    """All groups of one engine. ``req.pages`` is the list of group 0, ``req.group_pages[g - 1]`` that of group g."""

    def __init__(self, groups: tp.Sequence[KVCacheGroup], enable_caching: bool = True):
        if not groups:
            raise ValueError("a cache needs at least one group")
        self.managers = [GroupManager(g.spec, g.num_pages, enable_caching, g.layers) for g in groups]
        self.page_size = groups[0].spec.page_size
        self.enable_caching = enable_caching

    @classmethod
    def single(cls, pool: PagePool, page_size: int = 128) -> "KVCacheCoordinator":
        """One full-attention group over an existing pool."""
        from ...caching.specs import FullAttentionSpec

        self = cls.__new__(cls)
        m = GroupManager.__new__(GroupManager)
        m.spec, m.layers, m.pool, m.bounded = FullAttentionSpec(page_size=page_size), [], pool, False
        self.managers, self.page_size, self.enable_caching = [m], page_size, pool.enable_caching
        return self

    @property
    def pool(self) -> PagePool:
        return self.managers[0].pool

    @property
    def num_groups(self) -> int:
        return len(self.managers)

    def lists(self, req) -> list[list[int]]:
        extra = req.group_pages
        while len(extra) < len(self.managers) - 1:
            extra.append([])
        return [req.pages, *extra]

    # -- allocation
    def try_allocate(self, req, upto_tokens: int) -> bool:
        lists = self.lists(req)
        need = [m.pages_needed(pl, upto_tokens) for m, pl in zip(self.managers, lists)]
        if any(n > m.pool.num_free for n, m in zip(need, self.managers)):
            return False
        for n, m, pl in zip(need, self.managers, lists):
            if n:
                pl.extend(m.pool.allocate(n))
        return True

    def release(self, req) -> None:
        for m, pl in zip(self.managers, self.lists(req)):
            m.release(pl)

    def remove_skipped(self, req) -> int:
        n = 0
        for m, pl in zip(self.managers, self.lists(req)):
            n += m.remove_skipped(pl, req.num_computed_tokens)
        return n

    # -- prefix cache
    def admit_with_prefix(self, req, usable_hashes: tp.Sequence[bytes]) -> int:
        """Takes the longest reusable prefix for ``req`` (its page lists must be empty); returns its page count."""
        if not self.enable_caching or not usable_hashes:
            return 0
        unbounded = [m for m in self.managers if not m.bounded]
        n = len(usable_hashes)
        for m in unbounded:
            n = min(n, len(m.pool.lookup(usable_hashes[:n])))
        bounded = [m for m in self.managers if m.bounded]
        if bounded:
            if not unbounded:
                for m in bounded:
                    m.pool.stats.queries += 1
            while n > 0 and not all(m.holds(usable_hashes, n) for m in bounded):
                n -= 1
        if n == 0:
            return 0
        for m, pl in zip(self.managers, self.lists(req)):
            if m.bounded:
                pl[:] = m.take_cached(usable_hashes, n)
            else:
                hit = [m.pool.cached[h] for h in usable_hashes[:n]]
                m.pool.touch(hit)
                pl[:] = hit
        return n

    def register(self, req, index: int, page_hash: bytes) -> None:
        for m, pl in zip(self.managers, self.lists(req)):
            if index < len(pl) and pl[index] != NULL_PAGE:
                m.pool.register(pl[index], page_hash)

    # -- reporting
    def usage(self) -> float:
        return max(m.pool.usage for m in self.managers)

    def pages_held(self, req) -> list[int]:
        return [sum(1 for p in pl if p != NULL_PAGE) for pl in self.lists(req)]
