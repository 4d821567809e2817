"""A pool of fixed-size cache pages with reference counts and shared-prefix lookup.

Semantics follow the reference's block allocator (utils/kv_cache.py:91-189): pages leave a FIFO
free list with one reference, ``retain`` adds a reference, ``release`` drops one, and a page whose
count reaches zero goes back to the free list, unless it holds a complete, hashed block of a
prompt: then it is parked in an idle list (least recently used first) from which a later request
with the same prefix can take it again, and from which it is evicted only when the free list is
empty.  Idle pages count as available.
"""
from __future__ import annotations

from collections import OrderedDict, deque
from typing import Dict, List, Optional


class KVCacheExhaustedError(BufferError):
    """No free and no idle page is left (utils/kv_cache.py:516-517)."""


class KVCacheStateError(RuntimeError):
    """The cache was asked for something its bookkeeping forbids: a double free, a page that is
    not allocated, a table that does not belong to the request (utils/kv_cache.py:519-520)."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"num_pages must be positive: {num_pages}")
        self.num_pages = num_pages
        self.free: deque = deque(range(num_pages))
        self.references: Dict[int, int] = {}
        self.digest_of: Dict[int, str] = {}      # page -> digest of the prompt block it holds
        self.page_of: Dict[str, int] = {}        # digest -> page
        self.idle: "OrderedDict[int, None]" = OrderedDict()  # unreferenced hashed pages, oldest first
        self.allocations = 0
        self.evictions = 0

    # ------------------------------------------------------------------ counts
    @property
    def num_free(self) -> int:
        return len(self.free)

    @property
    def num_idle(self) -> int:
        return len(self.idle)

    @property
    def num_available(self) -> int:
        return len(self.free) + len(self.idle)

    @property
    def num_allocated(self) -> int:
        return len(self.references)

    # ------------------------------------------------------------------ allocation
    def allocate(self) -> int:
        if self.free:
            page = self.free.popleft()
        elif self.idle:
            page, _ = self.idle.popitem(last=False)
            self._forget_digest(page)
            self.evictions += 1
        else:
            raise KVCacheExhaustedError("no free page is left in the cache")
        self.references[page] = 1
        self.allocations += 1
        return page

    def retain(self, page: int) -> None:
        self._check_id(page)
        if page in self.idle:
            del self.idle[page]
            self.references[page] = 1
            return
        if page not in self.references:
            raise KVCacheStateError(f"page {page} is not allocated and cannot be retained")
        self.references[page] += 1

    def release(self, page: int) -> None:
        self._check_id(page)
        if page not in self.references:
            raise KVCacheStateError(f"page {page} is not allocated (freed twice?)")
        self.references[page] -= 1
        if self.references[page] > 0:
            return
        del self.references[page]
        if page in self.digest_of:
            self.idle[page] = None
        else:
            self.free.append(page)

    # ------------------------------------------------------------------ shared prefixes
    def register_digest(self, page: int, digest: str) -> None:
        """Marks an allocated page as holding the complete prompt block named by ``digest``.
        The first page registered under a digest keeps it (utils/engine.py:399-400)."""
        if page not in self.references:
            raise KVCacheStateError(f"page {page} is not allocated and cannot be hashed")
        if digest in self.page_of and self.page_of[digest] != page:
            return
        old = self.digest_of.get(page)
        if old is not None and old != digest:
            self.page_of.pop(old, None)
        self.digest_of[page] = digest
        self.page_of[digest] = page

    def lookup(self, digest: str) -> Optional[int]:
        return self.page_of.get(digest)

    def share(self, digest: str, table: List[int]) -> Optional[int]:
        """Appends the page holding ``digest`` to ``table`` with a new reference, or returns None.
        A page may appear once in a table (utils/kv_cache.py:124-135)."""
        page = self.page_of.get(digest)
        if page is None:
            return None
        if self.digest_of.get(page) != digest:
            raise KVCacheStateError(f"hash table and page {page} disagree about digest {digest[:12]}")
        if page in table:
            raise ValueError(f"page {page} is already in the block table")
        self.retain(page)
        table.append(page)
        return page

    # ------------------------------------------------------------------ helpers
    def _forget_digest(self, page: int) -> None:
        digest = self.digest_of.pop(page, None)
        if digest is not None and self.page_of.get(digest) == page:
            del self.page_of[digest]

    def _check_id(self, page: int) -> None:
        if not isinstance(page, int) or not 0 <= page < self.num_pages:
            raise ValueError(f"page id {page!r} is outside 0..{self.num_pages - 1}")

    def check_invariants(self) -> None:
        """Every page is in exactly one of: free list, idle list, referenced."""
        free, idle, held = set(self.free), set(self.idle), set(self.references)
        if len(free) != len(self.free):
            raise AssertionError("a page is in the free list twice")
        if free & idle or free & held or idle & held:
            raise AssertionError("a page is in two places at once")
        if len(free) + len(idle) + len(held) != self.num_pages:
            raise AssertionError(f"pages lost: {len(free)} free + {len(idle)} idle + {len(held)} held != {self.num_pages}")
        if any(count <= 0 for count in self.references.values()):
            raise AssertionError("a held page has no reference")
        for page in idle:
            if page not in self.digest_of:
                raise AssertionError(f"idle page {page} has no digest")
        for digest, page in self.page_of.items():
            if self.digest_of.get(page) != digest:
                raise AssertionError("digest tables disagree")
