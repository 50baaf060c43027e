"""KV page pool with reference counts and hash-chained prefix caching.

Behaviour of the reference's ``PagePool`` / ``CacheManager`` (easydel/inference/esurge/core/
page_pool.py, manager.py, utils.py ``hash_page_tokens``): a free queue of page ids, reference
counts for pages shared between requests, a map from the chained hash of a *full* page's tokens
to the page that holds them, LRU-ish eviction of unreferenced cached pages, and a null page (id 0)
that is never handed out. Everything here is host-side Python over small integers; the device
only ever sees page tables.
"""

from __future__ import annotations

import collections
import hashlib
import os
import typing as tp
from dataclasses import dataclass, field

NULL_PAGE = 0


def _seed() -> bytes:
    return os.environ.get("PYTHONHASHSEED", "0").encode()


def hash_page_tokens(parent_hash: bytes | None, tokens: tp.Sequence[int], extra_keys: tp.Any = None) -> bytes:
    """Hash of one full page given the hash of the pages before it (prefix identity, not content only)."""
    h = hashlib.blake2b(digest_size=16, key=_seed()[:64] or b"0")
    h.update(parent_hash or b"\x00")
    h.update(b",".join(str(int(t)).encode() for t in tokens))
    if extra_keys is not None:
        h.update(repr(extra_keys).encode())
    return h.digest()


def hash_request_pages(tokens: tp.Sequence[int], page_size: int, extra_keys: tp.Any = None) -> list[bytes]:
    """Chained hashes of every *full* page of a token list (native 128-bit mixer when the library is built,
    keyed BLAKE2b otherwise; one process always uses the same one)."""
    if _NATIVE is not None:
        extra = 0 if extra_keys is None else int.from_bytes(
            hashlib.blake2b(repr(extra_keys).encode(), digest_size=8).digest(), "little")
        return _NATIVE.hash_pages(tokens, page_size, _SEED_INT, extra)
    out, parent = [], None
    for i in range(0, len(tokens) - len(tokens) % page_size, page_size):
        parent = hash_page_tokens(parent, tokens[i:i + page_size], extra_keys)
        out.append(parent)
    return out


def _pick_native():
    try:
        from ...data import _native

        return _native if _native.available() else None
    except Exception:
        return None


_NATIVE = _pick_native()
_SEED_INT = int.from_bytes(hashlib.blake2b(_seed(), digest_size=8).digest(), "little")


@dataclass
class PoolStats:
    queries: int = 0
    hits: int = 0
    evictions: int = 0

    @property
    def hit_rate(self) -> float:
        return self.hits / self.queries if self.queries else 0.0


class PagePool:
    def __init__(self, num_pages: int, enable_caching: bool = True):
        if num_pages < 2:
            raise ValueError("a page pool needs at least 2 pages (one is the null page)")
        self.num_pages = num_pages
        self.enable_caching = enable_caching
        self.ref = [0] * num_pages
        self.page_hash: list[bytes | None] = [None] * num_pages
        # free pages in eviction order: pages freed earliest are reused first; cached pages stay findable
        self.free: collections.OrderedDict[int, None] = collections.OrderedDict((i, None) for i in range(1, num_pages))
        self.cached: dict[bytes, int] = {}
        self.stats = PoolStats()

    # ------------------------------------------------------------------ queries
    @property
    def num_free(self) -> int:
        return len(self.free)

    @property
    def usage(self) -> float:
        return 1.0 - self.num_free / max(1, self.num_pages - 1)

    def lookup(self, page_hashes: tp.Sequence[bytes]) -> list[int]:
        """Longest prefix of ``page_hashes`` present in the cache -> their page ids (no reference taken)."""
        out = []
        if not self.enable_caching:
            return out
        for h in page_hashes:
            self.stats.queries += 1
            pid = self.cached.get(h)
            if pid is None:
                break
            self.stats.hits += 1
            out.append(pid)
        return out

    # ------------------------------------------------------------------ allocation
    def touch(self, pages: tp.Sequence[int]) -> None:
        """Takes a reference on cached pages (removing them from the free/evictable queue)."""
        for pid in pages:
            if self.ref[pid] == 0:
                self.free.pop(pid, None)
            self.ref[pid] += 1

    def allocate(self, n: int) -> list[int]:
        if n > len(self.free):
            raise MemoryError(f"page pool exhausted: need {n}, have {len(self.free)}")
        out = []
        for _ in range(n):
            pid, _ = self.free.popitem(last=False)
            h = self.page_hash[pid]
            if h is not None:  # evict whatever prefix this page was caching
                if self.cached.get(h) == pid:
                    del self.cached[h]
                self.page_hash[pid] = None
                self.stats.evictions += 1
            self.ref[pid] = 1
            out.append(pid)
        return out

    def release(self, pages: tp.Sequence[int]) -> None:
        """Drops one reference per page; unreferenced pages become evictable (tail pages first in, so that a
        request's prefix outlives its suffix)."""
        for pid in reversed(list(pages)):
            if pid == NULL_PAGE:
                continue
            self.ref[pid] -= 1
            if self.ref[pid] < 0:
                raise RuntimeError(f"page {pid} released more often than referenced")
            if self.ref[pid] == 0:
                self.free[pid] = None

    def register(self, pid: int, page_hash: bytes) -> int:
        """Publishes a full page under its chained hash. If another page already holds that prefix the
        existing page id is returned (the caller keeps using its own copy)."""
        if not self.enable_caching:
            return pid
        other = self.cached.get(page_hash)
        if other is not None and other != pid:
            return other
        self.cached[page_hash] = pid
        self.page_hash[pid] = page_hash
        return pid

    def reset_cache(self) -> None:
        self.cached.clear()
        self.page_hash = [None] * self.num_pages
