"""The flat batch one step runs: what the parts see of it (`StepContext`) and how it
is laid out for a single host-to-device copy.

The reference describes a step to its model by the same flat index tensors
(input_ids, positions, slot_mapping, block_table, cu_seqlens_q/k:
src/exec/cache_scheduler/mod.rs:824-930, python/vosti_kernels/kernels.py:519-626) and
builds each with its own copy; here all of them are sections of one pinned int32
buffer that is copied once.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import ctypes

import numpy as np
import torch

from .. import host, ops
from ..parts.base import step_layout_providers


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them whose
    logits are wanted."""

    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class GroupView:
    """One cache group as the step sees it."""

    block_table: torch.Tensor     # int32 [requests, max_pages]
    slot_mapping: torch.Tensor    # int32 [tokens]
    page_size: int
    max_pages: int


@dataclass
class StepContext:
    num_tokens: int
    num_requests: int
    tokens: torch.Tensor          # int32 [T]
    positions: torch.Tensor       # int32 [T], absolute position of each token
    request_of: torch.Tensor      # int32 [T], row of the request each token belongs to
    cu_q: torch.Tensor            # int32 [B+1], cumulative token counts
    kv_len: torch.Tensor          # int32 [B], keys of each request after this step
    state_slots: torch.Tensor     # int32 [B], per-request state slot
    want_rows: torch.Tensor       # int32 [W], flat token indices whose logits are wanted
    groups: List[GroupView]
    status: torch.Tensor          # int32 [1], device fault bits
    dtype: torch.dtype
    device: torch.device
    # host copies, for parts that loop over requests on the host
    host_q_lens: List[int] = field(default_factory=list)
    host_kv_lens: List[int] = field(default_factory=list)
    host_state_slots: List[int] = field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0
    all_decode: bool = False
    extras: dict = field(default_factory=dict)   # further per-step device arrays by name
    # extras["feedback"] (int32 [T], -1 or an index) names tokens to take from this device array
    # instead of `tokens`: what the step before sampled and the host has not read yet
    feedback_values: Optional[torch.Tensor] = None
    # what the registered step-layout providers made of the step's shape, by provider name: host
    # values here, their int32 arrays on the device in `extras` under "<name>.<array>"
    layout: dict = field(default_factory=dict)

    def group(self, index: int) -> GroupView:
        return self.groups[index]


class StagingBuffer:
    """Pinned host memory and its device twin, grown on demand."""

    def __init__(self, device: torch.device, capacity: int = 1 << 18):
        self.device = device
        self.copied = None          # event after the last host-to-device copy
        self.last_upload_bytes = 0
        self._alloc(capacity)

    def _alloc(self, capacity: int) -> None:
        self.capacity = capacity
        self.host = torch.empty(capacity, dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()
        self.dev = torch.empty(capacity, dtype=torch.int32, device=self.device)

    def reserve(self, count: int) -> None:
        """Make room for `count` ints; waits until the previous copy has left the host
        buffer before it may be overwritten."""
        if self.copied is not None:
            self.copied.synchronize()
        if count > self.capacity:
            torch.cuda.current_stream(self.device).synchronize()
            self._alloc(max(count, 2 * self.capacity))

    def upload(self, count: int) -> None:
        self.dev[:count].copy_(self.host[:count], non_blocking=True)
        self.last_upload_bytes = 4 * count
        if self.copied is None:
            self.copied = torch.cuda.Event()
        self.copied.record()


def _round_up(value: int, multiple: int) -> int:
    return (value + multiple - 1) // multiple * multiple


def build_context(staging: StagingBuffer, cache, entries: Sequence[StepEntry], status: torch.Tensor,
                  dtype: torch.dtype, extras: Optional[dict] = None, min_pages: int = 0, kv_bucket: int = 0,
                  position_limit: int = 0) -> StepContext:
    """Reserve cache entries for the step's tokens (all requests or none), lay the batch out
    in the pinned staging buffer and copy it. The reservation and the index arrays
    (positions, slots, block tables, ...) are written by the C++ host core straight into the
    staging buffer; tokens and wanted rows come from the entries."""
    B = len(entries)
    if B == 0:
        raise ValueError("a step needs at least one entry")
    q_lens = [len(e.tokens) for e in entries]
    known = cache._handles
    try:
        handles = [known[e.request_id] for e in entries]
    except KeyError as missing:
        raise KeyError(f"request {missing.args[0]!r} is not live") from None
    G = len(cache.groups)
    ids = (ctypes.c_int64 * B)(*handles)
    counts = (ctypes.c_int32 * B)(*q_lens)
    starts = (ctypes.c_int32 * B)()
    widest = (ctypes.c_int32 * max(G, 1))()
    lib = host.library()
    host.check(lib.vh_step_extend(cache._h, ids, counts, B, position_limit, starts, widest))
    T = sum(q_lens)
    W = sum(len(e.want) for e in entries)
    max_pages = [max(min_pages, _round_up(max(widest[g], 1), 4)) for g in range(G)]
    # sections are padded to 4 ints so that every section starts 16-byte aligned
    sizes = [T, T, T, B + 1, B, B, W] + [x for g in range(G) for x in (T, B * max_pages[g])]
    offsets, total = [], 0
    for s in sizes:
        offsets.append(total)
        total += _round_up(max(s, 1), 4)
    extras = dict(extras or {})
    single = T == B                    # a decode-only step: one token per request
    layout = {}
    for name, provider in step_layout_providers().items():
        arrays, layout[name] = provider(q_lens)
        for key, array in arrays.items():
            extras[f"{name}.{key}"] = np.asarray(array, dtype=np.int32)
    extra_at = {}
    for name, array in extras.items():
        words = np.ascontiguousarray(array).view(np.int32)
        extra_at[name] = (total, words, array.dtype)
        total += _round_up(max(words.size, 1), 4)
    staging.reserve(total)
    buf = staging.host_np
    o_tok, o_pos, o_req, o_cu, o_kv, o_slot, o_want = offsets[:7]
    if single and W == B and all(len(e.want) == 1 and e.want[0] == 0 for e in entries):
        buf[o_tok:o_tok + B] = [e.tokens[0] for e in entries]
        buf[o_want:o_want + B] = np.arange(B, dtype=np.int32)
    else:
        cursor, wcursor = 0, 0
        for i, e in enumerate(entries):
            n = q_lens[i]
            buf[o_tok + cursor:o_tok + cursor + n] = e.tokens
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.request_id!r}: wanted place {w} outside its {n} tokens")
                buf[o_want + wcursor] = cursor + w
                wcursor += 1
            cursor += n
    base = staging.host.data_ptr()
    at = lambda offset: ctypes.cast(base + 4 * offset, host.i32p)
    slot_ptrs = (host.i32p * max(G, 1))(*[at(offsets[7 + 2 * g]) for g in range(G)])
    table_ptrs = (host.i32p * max(G, 1))(*[at(offsets[8 + 2 * g]) for g in range(G)])
    widths = (ctypes.c_int32 * max(G, 1))(*max_pages)
    host.check(lib.vh_step_fill(cache._h, ids, counts, starts, B, at(o_pos), at(o_req), at(o_cu), at(o_kv),
                                at(o_slot), slot_ptrs, table_ptrs, widths))
    for name, (where, words, _) in extra_at.items():
        buf[where:where + words.size] = words
    staging.upload(total)
    dev = staging.dev
    torch_types = {np.dtype(np.float32): torch.float32, np.dtype(np.int64): torch.int64,
                   np.dtype(np.int32): torch.int32}
    extra_views = {name: dev[where:where + words.size].view(torch_types[np.dtype(kind)])
                   for name, (where, words, kind) in extra_at.items()}
    groups = [GroupView(block_table=dev[offsets[8 + 2 * g]:offsets[8 + 2 * g] + B * max_pages[g]].view(B, max_pages[g]),
                        slot_mapping=dev[offsets[7 + 2 * g]:offsets[7 + 2 * g] + T], page_size=cache.page_size,
                        max_pages=max_pages[g]) for g in range(G)]
    kv_lens = (np.frombuffer(starts, dtype=np.int32, count=B) + np.asarray(q_lens, dtype=np.int32)).tolist()
    state_slots = buf[o_slot:o_slot + B].tolist()
    return StepContext(
        num_tokens=T, num_requests=B, tokens=dev[o_tok:o_tok + T], positions=dev[o_pos:o_pos + T],
        request_of=dev[o_req:o_req + T], cu_q=dev[o_cu:o_cu + B + 1], kv_len=dev[o_kv:o_kv + B],
        state_slots=dev[o_slot:o_slot + B], want_rows=dev[o_want:o_want + W], groups=groups, status=status,
        dtype=dtype, device=staging.device, host_q_lens=q_lens, host_kv_lens=kv_lens,
        host_state_slots=state_slots, max_q_len=max(q_lens, default=0),
        max_kv_len=max(kv_bucket, max(kv_lens, default=0)), all_decode=all(n == 1 for n in q_lens), extras=extra_views,
        layout=layout)
