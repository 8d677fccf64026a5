"""Page pool of one cache group: free list, reference counts, and the index of
published (reusable) prompt-prefix pages.

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

from collections import OrderedDict, deque
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

_MASK = (1 << 64) - 1
_ROOT = 0xCBF29CE484222325


class OutOfPages(RuntimeError):
    """An allocation asked for more pages than are free or evictable."""


class PageAccountingError(AssertionError):
    """A page was released twice, acquired while vacant, or lost."""


def chain_hash(previous: int, tokens: Sequence[int]) -> int:
    """Hash of a page given the hash of the page before it (FNV-1a steps over the
    token ids; the reference chains pages the same way, cache_scheduler/mod.rs:939-958)."""
    h = (previous ^ _ROOT) & _MASK
    for token in tokens:
        h ^= int(token) & _MASK
        h = (h * 0x100000001B3) & _MASK
    return h or 1


@dataclass
class PublishedPage:
    tokens: Tuple[int, ...]
    hash_value: int
    depth: int            # number of pages from the start of the prompt, this one included
    parent: int           # page id of the page before it, -1 at the start


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self.free: deque[int] = deque(range(num_pages))
        self.refcount: List[int] = [0] * num_pages
        self.published: Dict[int, PublishedPage] = {}
        self.hash_to_page: Dict[int, int] = {}
        self.evictable: "OrderedDict[int, None]" = OrderedDict()
        self.evictions = 0

    # ------------------------------------------------------------ counts
    def available(self) -> int:
        """Pages an allocation can get: vacant ones plus evictable published ones."""
        return len(self.free) + len(self.evictable)

    def held(self) -> int:
        return self.num_pages - self.available()

    # ------------------------------------------------------------ allocate / release
    def _evict_one(self) -> None:
        page, _ = self.evictable.popitem(last=False)
        info = self.published.pop(page)
        if self.hash_to_page.get(info.hash_value) == page:
            del self.hash_to_page[info.hash_value]
        self.free.appendleft(page)
        self.evictions += 1

    def allocate(self, count: int) -> List[int]:
        """`count` fresh pages, all or nothing; evicts published pages only if needed."""
        if count < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if count > self.available():
            raise OutOfPages(f"{count} pages wanted, {self.available()} available")
        while len(self.free) < count:
            self._evict_one()
        pages = [self.free.popleft() for _ in range(count)]
        for page in pages:
            if self.refcount[page] != 0:
                raise PageAccountingError(f"vacant page {page} has holders")
            self.refcount[page] = 1
        return pages

    def acquire(self, page: int) -> None:
        """One more holder of a resident page (prefix reuse)."""
        if self.refcount[page] == 0:
            if page not in self.evictable:
                raise PageAccountingError(f"page {page} is vacant and cannot be acquired")
            del self.evictable[page]
        self.refcount[page] += 1

    def release(self, page: int) -> None:
        """One holder less; the last one returns the page to the pool."""
        if not 0 <= page < self.num_pages or self.refcount[page] <= 0:
            raise PageAccountingError(f"page {page} released but not held")
        self.refcount[page] -= 1
        if self.refcount[page] == 0:
            if page in self.published:
                self.evictable[page] = None
            else:
                self.free.appendleft(page)

    # ------------------------------------------------------------ published prefixes
    def publish(self, page: int, tokens: Sequence[int], previous_hash: int, depth: int,
                parent: int) -> Tuple[int, int]:
        """Make a full, held page findable. Returns (hash of this page, the page a
        following page names as its parent): the first page published under a hash
        keeps the entry, a later twin with equal content chains through it."""
        h = chain_hash(previous_hash, tokens)
        tokens = tuple(int(t) for t in tokens)
        if page in self.published:
            return h, page
        owner = self.hash_to_page.get(h)
        if owner is not None:
            twin = self.published[owner]
            if twin.tokens == tokens and twin.depth == depth and twin.parent == parent:
                return h, owner
            return h, page          # a true collision: this page stays private
        self.published[page] = PublishedPage(tokens, h, depth, parent)
        self.hash_to_page[h] = page
        return h, page

    def match(self, tokens: Sequence[int], page_size: int) -> List[int]:
        """Longest chain of published pages equal to the start of `tokens`, never
        reaching the page that holds the last token (at least one token stays to be
        computed)."""
        pages: List[int] = []
        previous_hash, parent = 0, -1
        limit = (len(tokens) - 1) // page_size
        for j in range(limit):
            chunk = tuple(int(t) for t in tokens[j * page_size:(j + 1) * page_size])
            h = chain_hash(previous_hash, chunk)
            page = self.hash_to_page.get(h)
            if page is None:
                break
            info = self.published[page]
            if info.depth != j + 1 or info.parent != parent or info.tokens != chunk:
                break
            pages.append(page)
            previous_hash, parent = h, page
        return pages

    # ------------------------------------------------------------ checks
    def check(self, holders: Dict[int, int]) -> None:
        """Every page is vacant, evictable or held, exactly once; `holders` maps a page
        to how many requests list it."""
        seen = set()
        for page in self.free:
            if page in seen or self.refcount[page] != 0 or page in self.published:
                raise PageAccountingError(f"page {page} is in the free list wrongly")
            seen.add(page)
        for page in self.evictable:
            if page in seen or self.refcount[page] != 0 or page not in self.published:
                raise PageAccountingError(f"page {page} is in the evictable queue wrongly")
            seen.add(page)
        for page in range(self.num_pages):
            count = holders.get(page, 0)
            if self.refcount[page] != count:
                raise PageAccountingError(f"page {page}: reference count {self.refcount[page]}, "
                                          f"{count} holders")
            if count > 0:
                if page in seen:
                    raise PageAccountingError(f"page {page} is held and also vacant")
                seen.add(page)
        if len(seen) != self.num_pages:
            missing = sorted(set(range(self.num_pages)) - seen)
            raise PageAccountingError(f"pages lost: {missing}")
        for h, page in self.hash_to_page.items():
            if page not in self.published or self.published[page].hash_value != h:
                raise PageAccountingError(f"hash index names page {page} wrongly")
