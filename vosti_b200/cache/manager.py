"""The cache manager: keys and values in pages with a block table per request, one
page pool per group of layers with the same needs, and slots for per-request state
of fixed size.

Layers whose mixers keep everything share one group (one id space, one block table,
as the reference's layers do: python/vosti_kernels/physical.py:124-147, 329-339);
layers that only ever read a window of the past form a group of their own, whose pages
are given back as soon as the window has passed them. A slot is ``page * page_size +
offset`` (kernels/triton_kernels/store_kv_cache.py:21-25); a layer's storage is
``[num_pages, heads, page_size, width]``, so the tokens one head holds in a page are
contiguous (the reference keeps ``[pages, page_size, heads, width]``).

Pages come back when a request finishes, when a window has passed them, and (for
published prefix pages nobody holds) when an allocation needs them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import PagedCacheSpec, StateSpec
from .pages import OutOfPages, PageAccountingError, PagePool

RELEASED = -1  # block-table entry of a page a window has passed


class OutOfSlots(RuntimeError):
    pass


@dataclass
class LayerCache:
    """What one layer's mixer gets: its group, its page storage and its state."""

    group: int = -1
    tensors: Tuple[torch.Tensor, ...] = ()
    state: Optional[torch.Tensor] = None
    page_size: int = 0

    @property
    def k(self):
        return self.tensors[0] if self.tensors else None

    @property
    def v(self):
        return self.tensors[1] if len(self.tensors) > 1 else None


@dataclass
class CacheGroup:
    window: int
    layers: List[int]
    pool: PagePool


@dataclass
class Residency:
    """What a live request holds."""

    request_id: object
    slot: int
    length: int = 0                       # tokens whose cache entries exist
    pages: List[List[int]] = field(default_factory=list)   # per group, by page index
    cached_prefix_pages: int = 0
    published_pages: int = 0
    last_hash: int = 0
    last_parent: int = -1


class CacheManager:
    def __init__(self, cache_specs: Sequence[Optional[PagedCacheSpec]],
                 state_specs: Sequence[Optional[StateSpec]], *, num_pages: int, page_size: int,
                 max_requests: int, device: Optional[torch.device] = None,
                 dtype: torch.dtype = torch.bfloat16, prefix_reuse: bool = True):
        if page_size <= 0 or num_pages <= 0 or max_requests <= 0:
            raise ValueError("page_size, num_pages and max_requests must be positive")
        self.page_size, self.num_pages, self.max_requests = page_size, num_pages, max_requests
        self.groups: List[CacheGroup] = []
        self.layer_caches: List[LayerCache] = []
        by_window: Dict[int, int] = {}
        for layer, spec in enumerate(cache_specs):
            cache = LayerCache(page_size=page_size)
            if spec is not None:
                if spec.window not in by_window:
                    by_window[spec.window] = len(self.groups)
                    self.groups.append(CacheGroup(spec.window, [], PagePool(num_pages)))
                cache.group = by_window[spec.window]
                self.groups[cache.group].layers.append(layer)
                if device is not None:
                    cache.tensors = tuple(
                        torch.empty((num_pages, spec.heads, page_size, spec.width), dtype=dtype, device=device)
                        for _ in range(spec.entries))
            self.layer_caches.append(cache)
        for layer, spec in enumerate(state_specs):
            if spec is not None and device is not None:
                self.layer_caches[layer].state = torch.zeros((max_requests, *spec.shape), dtype=spec.dtype,
                                                             device=device)
        self.has_state = any(s is not None for s in state_specs)
        # A published page stands for the keys of every layer; with a windowed group or
        # per-request state a prefix would need more than pages to be reused.
        self.prefix_reuse = (prefix_reuse and len(self.groups) == 1 and self.groups[0].window == 0
                             and not self.has_state)
        self.free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self.live: Dict[object, Residency] = {}
        self.reused_prefix_pages = 0
        self.requests_with_reuse = 0

    # ------------------------------------------------------------ sizes
    def bytes_per_token(self) -> int:
        total = 0
        for cache in self.layer_caches:
            for t in cache.tensors:
                total += t.shape[1] * t.shape[3] * t.element_size()      # heads * width
        return total

    def pages_for(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size

    def available_pages(self) -> int:
        return min((g.pool.available() for g in self.groups), default=self.num_pages)

    # ------------------------------------------------------------ requests
    def begin(self, request_id, prompt_for_reuse: Optional[Sequence[int]] = None) -> Residency:
        """Admit a request: a state slot, and (if reuse is on and a prompt is given) the
        published pages that already hold the start of the prompt."""
        if request_id in self.live:
            raise ValueError(f"request {request_id!r} is already live")
        if not self.free_slots:
            raise OutOfSlots(f"all {self.max_requests} request slots are taken")
        slot = self.free_slots.pop()
        res = Residency(request_id, slot, pages=[[] for _ in self.groups])
        for cache in self.layer_caches:
            if cache.state is not None:
                cache.state[slot].zero_()
        if self.prefix_reuse and prompt_for_reuse is not None:
            pool = self.groups[0].pool
            matched = pool.match(prompt_for_reuse, self.page_size)
            for page in matched:
                pool.acquire(page)
            if matched:
                res.pages[0] = list(matched)
                res.length = len(matched) * self.page_size
                res.cached_prefix_pages = res.published_pages = len(matched)
                info = pool.published[matched[-1]]
                res.last_hash, res.last_parent = info.hash_value, matched[-1]
                self.reused_prefix_pages += len(matched)
                self.requests_with_reuse += 1
        self.live[request_id] = res
        return res

    def pages_needed(self, request_id, new_tokens: int) -> int:
        """Fresh pages (in the most demanding group) that `extend` would take."""
        res = self.live[request_id]
        need = self.pages_for(res.length + new_tokens)
        return max((need - len(res.pages[g]) for g in range(len(self.groups))), default=0)

    def can_extend(self, request_id, new_tokens: int) -> bool:
        res = self.live[request_id]
        need = self.pages_for(res.length + new_tokens)
        return all(need - len(res.pages[g]) <= group.pool.available()
                   for g, group in enumerate(self.groups))

    def extend(self, request_id, new_tokens: int) -> List[List[int]]:
        """Reserve cache entries for the request's next `new_tokens` tokens. Returns, per
        group, the slot of each new token. All groups or none."""
        res = self.live[request_id]
        if new_tokens <= 0:
            raise ValueError("extend needs at least one token")
        if not self.can_extend(request_id, new_tokens):
            raise OutOfPages(f"request {request_id!r}: not enough pages for {new_tokens} more tokens")
        need = self.pages_for(res.length + new_tokens)
        slots: List[List[int]] = []
        P = self.page_size
        for g, group in enumerate(self.groups):
            extra = need - len(res.pages[g])
            if extra > 0:
                res.pages[g].extend(group.pool.allocate(extra))
            row = res.pages[g]
            slots.append([row[pos // P] * P + pos % P for pos in range(res.length, res.length + new_tokens)])
        res.length += new_tokens
        return slots

    def trim(self, request_id) -> int:
        """Give back the pages a window has passed: every query from now on sits at a
        position >= length and reads keys > position - window only."""
        res = self.live[request_id]
        freed = 0
        for g, group in enumerate(self.groups):
            if group.window <= 0:
                continue
            first_needed = res.length - group.window + 1
            if first_needed <= 0:
                continue
            for index in range(min(first_needed // self.page_size, len(res.pages[g]))):
                page = res.pages[g][index]
                if page != RELEASED:
                    group.pool.release(page)
                    res.pages[g][index] = RELEASED
                    freed += 1
        return freed

    def publish(self, request_id, tokens: Sequence[int]) -> int:
        """Make the request's full pages findable by later prompts; `tokens` are the
        tokens whose cache entries exist (at least `length` of them)."""
        if not self.prefix_reuse:
            return 0
        res = self.live[request_id]
        pool, P = self.groups[0].pool, self.page_size
        full = res.length // P
        done = 0
        while res.published_pages < full:
            i = res.published_pages
            page = res.pages[0][i]
            res.last_hash, res.last_parent = pool.publish(
                page, tokens[i * P:(i + 1) * P], res.last_hash, i + 1, res.last_parent)
            res.published_pages += 1
            done += 1
        return done

    def finish(self, request_id) -> None:
        """The request ends: all its pages and its slot are given back."""
        res = self.live.pop(request_id)
        for g, group in enumerate(self.groups):
            for page in reversed(res.pages[g]):   # leaves before their parents
                if page != RELEASED:
                    group.pool.release(page)
        self.free_slots.append(res.slot)

    # ------------------------------------------------------------ views for the step
    def block_row(self, request_id, group: int) -> List[int]:
        return self.live[request_id].pages[group]

    def length(self, request_id) -> int:
        return self.live[request_id].length

    def slot(self, request_id) -> int:
        return self.live[request_id].slot

    # ------------------------------------------------------------ checks
    def check(self) -> None:
        """No page lost, held twice without being shared on purpose, or vacant while held."""
        slots = [r.slot for r in self.live.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self.free_slots):
            raise PageAccountingError("a state slot is held twice or is also free")
        if len(slots) + len(self.free_slots) != self.max_requests:
            raise PageAccountingError("a state slot was lost")
        for g, group in enumerate(self.groups):
            holders: Dict[int, int] = {}
            for res in self.live.values():
                own = [p for p in res.pages[g] if p != RELEASED]
                if len(set(own)) != len(own):
                    raise PageAccountingError(f"request {res.request_id!r} lists a page twice")
                for page in own:
                    holders[page] = holders.get(page, 0) + 1
            if not self.prefix_reuse and any(c > 1 for c in holders.values()):
                raise PageAccountingError("a page is held by two requests without prefix reuse")
            group.pool.check(holders)
