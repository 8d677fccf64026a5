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
published prefix pages nobody holds) when an allocation needs them. The accounting is
C++ (vosti_b200/csrc/host/engine_core.cpp); device storage is allocated here.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import ctypes

import torch

from .. import host
from ..host import OutOfSlots
from ..parts.base import PagedCacheSpec, StateSpec
from .pages import OutOfPages, PageAccountingError, PagePool

RELEASED = -1  # block-table entry of a page a window has passed


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
    """What a live request holds (a snapshot read from the C++ core)."""

    request_id: object
    slot: int
    length: int = 0                       # tokens whose cache entries exist
    pages: List[List[int]] = field(default_factory=list)   # per group, by page index
    cached_prefix_pages: int = 0
    published_pages: int = 0


class _LiveView:
    """`manager.live`: the live requests, by request id."""

    def __init__(self, manager: "CacheManager"):
        self._m = manager

    def __contains__(self, request_id) -> bool:
        h = self._m._handles.get(request_id)
        return h is not None and bool(self._m._lib.vh_is_live(self._m._h, ctypes.c_int64(h)))

    def __getitem__(self, request_id) -> Residency:
        m = self._m
        if request_id not in self:
            raise KeyError(request_id)
        rid = ctypes.c_int64(m._handles[request_id])
        return Residency(request_id, m._lib.vh_slot(m._h, rid), m._lib.vh_length(m._h, rid),
                         [m.block_row(request_id, g) for g in range(len(m.groups))],
                         m._lib.vh_residency_field(m._h, rid, 0), m._lib.vh_residency_field(m._h, rid, 1))

    def _ids(self):
        m = self._m
        count = int(m._lib.vh_counter(m._h, 5))
        buf = (ctypes.c_int64 * max(count, 1))()
        m._lib.vh_live_ids(m._h, buf, count)
        return [m._names[h] for h in buf[:count]]

    def __len__(self) -> int:
        return int(self._m._lib.vh_counter(self._m._h, 5))

    def __iter__(self):
        return iter(self._ids())

    def values(self):
        return [self[rid] for rid in self._ids()]


class CacheManager:
    def __init__(self, cache_specs: Sequence[Optional[PagedCacheSpec]],
                 state_specs: Sequence[Optional[StateSpec]], *, num_pages: int, page_size: int,
                 max_requests: int, device: Optional[torch.device] = None,
                 dtype: torch.dtype = torch.bfloat16, prefix_reuse: bool = True):
        if page_size <= 0 or num_pages <= 0 or max_requests <= 0:
            raise ValueError("page_size, num_pages and max_requests must be positive")
        self.page_size, self.num_pages, self.max_requests = page_size, num_pages, max_requests
        self.layer_caches: List[LayerCache] = []
        windows: List[int] = []
        layers_of: List[List[int]] = []
        by_window: Dict[int, int] = {}
        for layer, spec in enumerate(cache_specs):
            cache = LayerCache(page_size=page_size)
            if spec is not None:
                if spec.window not in by_window:
                    by_window[spec.window] = len(windows)
                    windows.append(spec.window)
                    layers_of.append([])
                cache.group = by_window[spec.window]
                layers_of[cache.group].append(layer)
                if device is not None:
                    # zeros, not empty: the decode kernel reads whole boxes of 16 keys and masks
                    # afterwards, so slots nobody wrote yet must hold finite values
                    cache.tensors = tuple(
                        torch.zeros((num_pages, spec.heads, page_size, spec.width), dtype=dtype, device=device)
                        for _ in range(spec.entries))
            self.layer_caches.append(cache)
        for layer, spec in enumerate(state_specs):
            if spec is not None and device is not None:
                self.layer_caches[layer].state = torch.zeros((max_requests, *spec.shape), dtype=spec.dtype,
                                                             device=device)
        # Beside the mixers' state, every request slot holds four 64-bit words for the engine: the
        # sampler's state (temperature as float bits, seed, index of the next token) and the
        # position of the last sampled token's input, written at admission and advanced on the
        # device (src/exec/request_state.rs:213-226 keeps the same per request on the host).
        self.request_state = (torch.zeros((max_requests, 4), dtype=torch.int64, device=device)
                              if device is not None else None)
        self.has_state = any(s is not None for s in state_specs)
        # The accounting itself is C++. A published page stands for the keys of every layer;
        # with a windowed group or per-request state a prefix would need more than pages to
        # be reused, so the core switches reuse off then.
        self._lib = host.library()
        self._ptr = self._lib.vh_create(len(windows), host.ints(windows), num_pages, page_size, max_requests,
                                        int(prefix_reuse), int(self.has_state), max_requests, 4096, 0, 0, 0)
        if not self._ptr:
            raise ValueError("the host core refused the cache geometry")
        self._h = host.handle(self._ptr)
        self.prefix_reuse = bool(self._lib.vh_prefix_reuse(self._h))
        self.has_windows = any(w > 0 for w in windows)
        self.groups: List[CacheGroup] = [
            CacheGroup(window, layers, PagePool(borrowed=self._lib.vh_group_pool(self._h, g)))
            for g, (window, layers) in enumerate(zip(windows, layers_of))]
        self._handles: Dict[object, int] = {}
        self._names: Dict[int, object] = {}
        self._next_handle = 1
        self._fresh = (ctypes.c_int32 * max_requests)()
        self.live = _LiveView(self)

    def __del__(self):
        if getattr(self, "_ptr", None):
            self._lib.vh_destroy(self._h)
            self._ptr = None

    def handle_of(self, request_id) -> int:
        """The integer the C++ core knows the request by."""
        h = self._handles.get(request_id)
        if h is None:
            h = self._next_handle
            self._next_handle += 1
            self._handles[request_id] = h
            self._names[h] = request_id
        return h

    def forget(self, request_id) -> None:
        """Drop the name of a request that is no longer live, so that what the host keeps does
        not grow with the number of requests served."""
        if request_id in self.live:
            raise ValueError(f"request {request_id!r} is still live")
        h = self._handles.pop(request_id, None)
        if h is not None:
            self._names.pop(h, None)

    def clear_fresh_state(self) -> int:
        """Zero the state slots that were handed out since the last call, on the current
        stream. Requests are admitted (and re-admitted after a preemption) inside the C++ core,
        by `begin` here or by the scheduler's plan; whichever did it, the slot still holds its
        last tenant's state until this runs, so the step function calls it before every step."""
        if not self.has_state:
            return 0
        count = self._lib.vh_take_fresh_slots(self._h, self._fresh, self.max_requests)
        for slot in self._fresh[:count]:
            for cache in self.layer_caches:
                if cache.state is not None:
                    cache.state[slot].zero_()
        return count

    def _rid(self, request_id) -> ctypes.c_int64:
        h = self._handles.get(request_id)
        if h is None:
            raise KeyError(f"request {request_id!r} is not live")
        return ctypes.c_int64(h)

    # ------------------------------------------------------------ sizes
    @property
    def reused_prefix_pages(self) -> int:
        return int(self._lib.vh_counter(self._h, 0))

    @property
    def requests_with_reuse(self) -> int:
        return int(self._lib.vh_counter(self._h, 1))

    @property
    def free_slots(self) -> List[int]:
        buf = (ctypes.c_int32 * self.max_requests)()
        n = self._lib.vh_free_slots(self._h, buf, self.max_requests)
        return list(buf[:n])

    def bytes_per_token(self) -> int:
        total = 0
        for cache in self.layer_caches:
            for t in cache.tensors:
                total += t.shape[1] * t.shape[3] * t.element_size()      # heads * width
        return total

    def pages_for(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size

    def available_pages(self) -> int:
        return self._lib.vh_available_pages(self._h)

    # ------------------------------------------------------------ requests
    def begin(self, request_id, prompt_for_reuse: Optional[Sequence[int]] = None) -> Residency:
        """Admit a request: a state slot, and (if reuse is on and a prompt is given) the
        published pages that already hold the start of the prompt."""
        if request_id in self.live:
            raise ValueError(f"request {request_id!r} is already live")
        rid = ctypes.c_int64(self.handle_of(request_id))
        if prompt_for_reuse is not None and self.prefix_reuse:
            prompt = list(prompt_for_reuse)
            slot = host.check(self._lib.vh_begin(self._h, rid, host.ints(prompt), len(prompt)))
        else:
            host.check(self._lib.vh_begin(self._h, rid, None, 0))
        self.clear_fresh_state()
        return self.live[request_id]

    def pages_needed(self, request_id, new_tokens: int) -> int:
        """Fresh pages (in the most demanding group) that `extend` would take."""
        return host.check(self._lib.vh_pages_needed(self._h, self._rid(request_id), new_tokens))

    def can_extend(self, request_id, new_tokens: int) -> bool:
        return bool(host.check(self._lib.vh_can_extend(self._h, self._rid(request_id), new_tokens)))

    def extend(self, request_id, new_tokens: int) -> List[List[int]]:
        """Reserve cache entries for the request's next `new_tokens` tokens. Returns, per
        group, the slot of each new token. All groups or none."""
        groups = len(self.groups)
        buf = (ctypes.c_int32 * max(groups * max(new_tokens, 0), 1))()
        host.check(self._lib.vh_extend(self._h, self._rid(request_id), new_tokens, buf))
        return [list(buf[g * new_tokens:(g + 1) * new_tokens]) for g in range(groups)]

    def trim(self, request_id) -> int:
        """Give back the pages a window has passed: every query from now on sits at a
        position >= length and reads keys > position - window only."""
        return host.check(self._lib.vh_trim(self._h, self._rid(request_id)))

    def publish(self, request_id, tokens: Sequence[int]) -> int:
        """Make the request's full pages findable by later prompts; `tokens` are the
        tokens whose cache entries exist (at least `length` of them)."""
        if not self.prefix_reuse:
            return 0
        tokens = list(tokens)
        return host.check(self._lib.vh_publish(self._h, self._rid(request_id), host.ints(tokens), len(tokens)))

    def finish(self, request_id) -> None:
        """The request ends: all its pages and its slot are given back."""
        host.check(self._lib.vh_finish(self._h, self._rid(request_id)))

    # ------------------------------------------------------------ views for the step
    def block_row(self, request_id, group: int) -> List[int]:
        capacity = self.num_pages + 1024
        buf = (ctypes.c_int32 * capacity)()
        n = host.check(self._lib.vh_block_row(self._h, self._rid(request_id), group, buf, capacity))
        if n > capacity:
            buf = (ctypes.c_int32 * n)()
            host.check(self._lib.vh_block_row(self._h, self._rid(request_id), group, buf, n))
        return list(buf[:n])

    def length(self, request_id) -> int:
        return host.check(self._lib.vh_length(self._h, self._rid(request_id)))

    def slot(self, request_id) -> int:
        return host.check(self._lib.vh_slot(self._h, self._rid(request_id)))

    # ------------------------------------------------------------ checks
    def check(self) -> None:
        """No page lost, held twice without being shared on purpose, or vacant while held."""
        host.check(self._lib.vh_check(self._h))
