"""Page pool of one cache group: free list, reference counts, and the index of
published (reusable) prompt-prefix pages. The pool itself is C++
(vosti_b200/csrc/host/engine_core.cpp); this class is its Python face.

Behaviour follows the reference's cache scheduler: vacant ids start in order
0..N-1, allocation pops the front and a released page is put back at the front
(src/exec/cache_scheduler/availability_queue.rs:746-780, 377, 246;
reclamation.rs:119, 1185), which is what makes a page come back into use soon.
A published page whose last holder left stays resident at reference count 0 in a
queue of evictable pages and is evicted, oldest first, only when an allocation
would otherwise fail (reclamation.rs:13-334; eviction_policy.rs:34-65). A page is
found again by the hash chain of its tokens, but a match is accepted only after
depth, parent page and all tokens have been compared (prefix_cache.rs:3155-3469),
so nothing depends on the hash being collision-free.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Sequence, Tuple

from .. import host
from ..host import OutOfPages, PageAccountingError

__all__ = ["OutOfPages", "PageAccountingError", "PagePool", "chain_hash"]


def chain_hash(previous: int, tokens: Sequence[int]) -> int:
    """Hash of a page given the hash of the page before it (FNV-1a steps over the
    token ids; the reference chains pages the same way, cache_scheduler/mod.rs:939-958)."""
    tokens = list(tokens)
    return int(host.library().vh_chain_hash(ctypes.c_uint64(previous), host.ints(tokens), len(tokens)))


class PagePool:
    def __init__(self, num_pages: int = 0, *, borrowed=None):
        """A pool of its own, or (borrowed) the pool of a cache manager's group."""
        self._lib = host.library()
        if borrowed is not None:
            self._ptr, self._owned = borrowed, False
        else:
            if num_pages <= 0:
                raise ValueError("a page pool needs at least one page")
            self._ptr, self._owned = self._lib.vh_pool_create(num_pages), True
        self._h = host.handle(self._ptr)
        self.num_pages = self._lib.vh_pool_num_pages(self._h)

    def __del__(self):
        if getattr(self, "_owned", False) and self._ptr:
            self._lib.vh_pool_destroy(self._h)
            self._ptr = None

    # ------------------------------------------------------------ counts
    def available(self) -> int:
        """Pages an allocation can get: vacant ones plus evictable published ones."""
        return self._lib.vh_pool_available(self._h)

    def held(self) -> int:
        return self.num_pages - self.available()

    @property
    def evictions(self) -> int:
        return int(self._lib.vh_pool_evictions(self._h))

    def _list(self, which: int) -> List[int]:
        buf = (ctypes.c_int32 * self.num_pages)()
        n = self._lib.vh_pool_list(self._h, which, buf, self.num_pages)
        return list(buf[:n])

    @property
    def free(self) -> List[int]:
        return self._list(0)

    @property
    def evictable(self) -> List[int]:
        """Published pages nobody holds, oldest first."""
        return self._list(1)

    @property
    def published(self) -> List[int]:
        return self._list(2)

    @property
    def refcount(self) -> List[int]:
        return [self._lib.vh_pool_refcount(self._h, page) for page in range(self.num_pages)]

    # ------------------------------------------------------------ allocate / release
    def allocate(self, count: int) -> List[int]:
        """`count` fresh pages, all or nothing; evicts published pages only if needed."""
        buf = (ctypes.c_int32 * max(count, 1))()
        host.check(self._lib.vh_pool_allocate(self._h, count, buf))
        return list(buf[:count])

    def acquire(self, page: int) -> None:
        """One more holder of a resident page (prefix reuse)."""
        host.check(self._lib.vh_pool_acquire(self._h, page))

    def release(self, page: int) -> None:
        """One holder less; the last one returns the page to the pool."""
        host.check(self._lib.vh_pool_release(self._h, page))

    # ------------------------------------------------------------ published prefixes
    def publish(self, page: int, tokens: Sequence[int], previous_hash: int, depth: int,
                parent: int) -> Tuple[int, int]:
        """Make a full, held page findable. Returns (hash of this page, the page a
        following page names as its parent): the first page published under a hash
        keeps the entry, a later twin with equal content chains through it."""
        tokens = list(tokens)
        next_parent = ctypes.c_int32(-1)
        h = self._lib.vh_pool_publish(self._h, page, host.ints(tokens), len(tokens), ctypes.c_uint64(previous_hash),
                                      depth, parent, ctypes.byref(next_parent))
        return int(h), int(next_parent.value)

    def match(self, tokens: Sequence[int], page_size: int) -> List[int]:
        """Longest chain of published pages equal to the start of `tokens`, never
        reaching the page that holds the last token."""
        tokens = list(tokens)
        buf = (ctypes.c_int32 * max(self.num_pages, 1))()
        n = self._lib.vh_pool_match(self._h, host.ints(tokens), len(tokens), page_size, buf, self.num_pages)
        return list(buf[:n])

    def _set_published_tokens(self, page: int, tokens: Sequence[int]) -> None:
        """Test hook: remember a published page with other tokens, as a hash collision would."""
        tokens = list(tokens)
        host.check(self._lib.vh_pool_set_published_tokens(self._h, page, host.ints(tokens), len(tokens)))

    # ------------------------------------------------------------ checks
    def check(self, holders: Dict[int, int]) -> None:
        """Every page is vacant, evictable or held, exactly once; `holders` maps a page
        to how many requests list it."""
        pages = list(holders)
        host.check(self._lib.vh_pool_check(self._h, host.ints(pages), host.ints([holders[p] for p in pages]),
                                           len(pages)))
