"""Continuous-batching scheduler: admits requests, cuts prompts into portions under a
token budget, decodes, finishes and frees.

Shape and policy follow the reference's cache scheduler (plan / commit split with
requests added only between steps, src/exec/engine.rs:2620-2622;
src/exec/cache_scheduler/planning.rs):

* decode rows first: the longest prefix of the running requests, in admission order and
  at most `max_num_seqs`, whose new pages fit (planning.rs:247-338); a request that does
  not fit sits the step out;
* then admissions from the head of the waiting queue only (head-of-line blocking,
  planning.rs:1002-1091), each matched against published prefix pages;
* a prompt that does not fit the remaining token budget is cut: the whole remainder if it
  fits, else the largest multiple of the page size (planning.rs:11-49); only the portion
  that reaches the end of the known tokens samples;
* decode rows are not limited by the token budget but use it up (planning.rs:965-970).

Differences, decided here: a request keeps the pages of its earlier portions while it
waits for the next one (the reference gives them back and finds them again through the
prefix cache, request_lifecycle.rs:187-316); pages are reserved per portion, not for the
whole prompt; and when pages run out so that no row at all can be scheduled, the youngest
running request is preempted: its pages are given back and it returns to the head of the
waiting queue to be recomputed (the reference schedules nothing and does not guarantee
progress, cache_scheduler/mod.rs:8-12). A request that could not fit even into an empty
cache is finished with reason "capacity".
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from .. import host
from ..cache import CacheManager
from .request import MAX_EOS_TOKEN_IDS, AdmissionStatus, Request


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 4096
    prefill_chunk_size: int = 0      # 0: limited by the token budget only
    vocab_size: int = 0              # 0: prompt tokens are not range-checked here
    max_context: int = 0             # 0: no limit
    keep_finished: int = 1024        # records of finished requests kept for `finished[...]`; older ones go

    def validate(self, page_size: int = 0) -> None:
        if self.max_num_seqs <= 0 or self.max_num_batched_tokens <= 0:
            raise ValueError("max_num_seqs and max_num_batched_tokens must be positive")
        if self.prefill_chunk_size < 0:
            raise ValueError("prefill_chunk_size must be >= 0")
        if self.keep_finished < 0:
            raise ValueError("keep_finished must be >= 0")
        # A prompt longer than a step's cap is cut into whole pages; a cap below one page would
        # leave nothing to schedule for it.
        cap = min(self.max_num_batched_tokens, self.prefill_chunk_size or self.max_num_batched_tokens)
        if page_size and cap < page_size:
            raise ValueError(f"a step may take at most {cap} tokens of a prompt (the smaller of "
                             f"max_num_batched_tokens={self.max_num_batched_tokens} and prefill_chunk_size="
                             f"{self.prefill_chunk_size or 'unset'}), which is less than one page of {page_size} "
                             f"tokens: prompts are cut into whole pages, so raise it to at least {page_size}")


@dataclass
class PlanRow:
    request: Request
    start: int                 # position of the row's first token
    count: int                 # tokens the row computes
    sample: bool               # the row reaches the end of the known tokens
    slot: int = -1             # the request's slot of per-request state in this step


@dataclass
class StepPlan:
    rows: List[PlanRow] = field(default_factory=list)
    preempted: List[object] = field(default_factory=list)
    dropped: List[object] = field(default_factory=list)

    def num_tokens(self) -> int:
        return sum(r.count for r in self.rows)


_ADMISSION = [AdmissionStatus.ACCEPTED, AdmissionStatus.DUPLICATE_ID, AdmissionStatus.EMPTY_PROMPT,
              AdmissionStatus.BAD_EOS, AdmissionStatus.ZERO_BUDGET, AdmissionStatus.TOO_LONG,
              AdmissionStatus.BAD_TOKEN, AdmissionStatus.BAD_SAMPLING]
_FINISH = {1: "length", 2: "eos", 3: "capacity", 4: "aborted"}


class Scheduler:
    """Python face of the C++ scheduler (vosti_b200/csrc/host/engine_core.cpp), which shares
    its state with the cache manager's core. `Request` objects are kept here and updated from
    what the core decides."""

    def __init__(self, cache: CacheManager, config: SchedulerConfig):
        config.validate(cache.page_size)
        self.cache, self.config = cache, config
        self._lib, self._h = host.library(), cache._h
        self._lib.vh_configure_scheduler(self._h, config.max_num_seqs, config.max_num_batched_tokens,
                                         config.prefill_chunk_size, config.vocab_size, config.max_context)
        self._requests: Dict[object, Request] = {}
        self.accepted_ids = set()            # ids are never reused (src/exec/cache_scheduler/types.rs:162-165)
        self.finished: Dict[object, Request] = {}
        capacity = max(config.max_num_seqs, cache.max_requests, 1) + 8
        self._capacity = capacity
        self._ids = (ctypes.c_int64 * capacity)()
        self._rows = (ctypes.c_int32 * (4 * capacity))()
        self._side = (ctypes.c_int64 * 4096)()
        self._side2 = (ctypes.c_int64 * 4096)()

    # ------------------------------------------------------------ counters and queues
    @property
    def admitted_requests(self) -> int:
        return int(self._lib.vh_counter(self._h, 2))

    @property
    def preemptions(self) -> int:
        return int(self._lib.vh_counter(self._h, 3))

    def _queue(self, which: int) -> List[Request]:
        buf = (ctypes.c_int64 * 65536)()
        n = min(self._lib.vh_queue(self._h, which, buf, 65536), 65536)
        return [self._requests[self.cache._names[h]] for h in buf[:n]]

    @property
    def waiting(self) -> List[Request]:
        return self._queue(0)

    @property
    def running(self) -> List[Request]:
        return self._queue(1)

    # ------------------------------------------------------------ admission
    def add_request(self, request: Request) -> AdmissionStatus:
        if request.request_id in self.accepted_ids:
            return AdmissionStatus.DUPLICATE_ID
        prompt = [int(t) for t in request.prompt_tokens]
        if any(not -2 ** 31 <= t < 2 ** 31 for t in prompt):
            return AdmissionStatus.BAD_TOKEN
        eos = [int(t) for t in request.eos_token_ids]
        rid = self.cache.handle_of(request.request_id)
        temperature = request.temperature if request.temperature == request.temperature else -1.0
        code = self._lib.vh_add_request(self._h, ctypes.c_int64(rid), host.ints(prompt), len(prompt),
                                        int(request.max_tokens) if request.max_tokens < 2 ** 31 else 2 ** 31 - 1,
                                        host.ints(eos[:4]), len(eos), int(request.ignore_eos),
                                        ctypes.c_float(temperature))
        status = _ADMISSION[code]
        if status is AdmissionStatus.ACCEPTED:
            self.accepted_ids.add(request.request_id)
            self._requests[request.request_id] = request
        return status

    def abort(self, request_id) -> bool:
        """End a request now: it leaves its queue and gives back what it holds."""
        request = self._requests.get(request_id)
        if request is None or request.finished:
            return False
        if not self._lib.vh_abort(self._h, ctypes.c_int64(self.cache.handle_of(request_id))):
            return False
        self._retire(request, "aborted")
        return True

    def _retire(self, request: Request, reason: Optional[str] = None) -> None:
        """A request has ended and its last token has been handed out: keep its record among the
        `keep_finished` newest ones and drop everything else the host holds for it (the core's
        copy of its tokens, its handle), so that a long-lived engine does not grow."""
        if reason is not None:
            request.finished, request.finish_reason = True, reason
        rid = request.request_id
        if self._requests.pop(rid, None) is None:
            return
        self.finished[rid] = request
        while len(self.finished) > self.config.keep_finished:
            del self.finished[next(iter(self.finished))]
        h = self.cache._handles.get(rid)
        if h is not None:
            self._lib.vh_forget(self._h, ctypes.c_int64(h))
            self.cache.forget(rid)

    def release(self, request_id) -> bool:
        """Drop the record of a finished request."""
        return self.finished.pop(request_id, None) is not None

    def has_unfinished(self) -> bool:
        return bool(self._lib.vh_unfinished(self._h))

    # ------------------------------------------------------------ planning
    def plan(self) -> StepPlan:
        """Decide the next step's batch. Never returns an empty plan while a request is
        live: it preempts (or, for a request no cache could hold, drops) until a row fits."""
        n_pre, n_drop = ctypes.c_int32(0), ctypes.c_int32(0)
        n = host.check(self._lib.vh_plan(self._h, self._ids, self._rows, self._capacity, self._side,
                                         ctypes.byref(n_pre), self._side2, ctypes.byref(n_drop), 4096))
        names = self.cache._names
        plan = StepPlan()
        for h in self._side[:n_pre.value]:
            request = self._requests[names[h]]
            request.computed = 0
            request.preemptions += 1
            plan.preempted.append(request.request_id)
        for h in self._side2[:n_drop.value]:
            request = self._requests[names[h]]
            plan.dropped.append(request.request_id)
            self._retire(request, "capacity")
        rows = self._rows
        for i in range(n):
            request = self._requests[names[self._ids[i]]]
            request.computed = rows[4 * i]
            plan.rows.append(PlanRow(request, rows[4 * i], rows[4 * i + 1], bool(rows[4 * i + 2]), rows[4 * i + 3]))
        return plan

    # ------------------------------------------------------------ commit
    def commit(self, plan: StepPlan, sampled: Sequence[Optional[int]]) -> Dict[object, int]:
        """Apply a step's results: `sampled[i]` is the token of row i (ignored for rows that
        do not sample). Returns request id -> emitted token."""
        count = len(plan.rows)
        tokens = []
        for row, token in zip(plan.rows, sampled):
            if row.sample and token is None:
                raise ValueError(f"row of request {row.request.request_id!r} samples but got no token")
            tokens.append(int(token) if row.sample else -1)
        finished = (ctypes.c_int32 * max(count, 1))()
        host.check(self._lib.vh_commit(self._h, host.ints(tokens), count, finished))
        emitted: Dict[object, int] = {}
        for i, row in enumerate(plan.rows):
            request = row.request
            request.computed += row.count
            if not row.sample:
                continue
            request.generated.append(tokens[i])
            emitted[request.request_id] = tokens[i]
            if finished[i]:
                self._retire(request, _FINISH[finished[i]])
        return emitted

    # ------------------------------------------------------------ the commit in two halves
    PENDING = -1          # a sampled token the host has not read yet

    def commit_ahead(self, plan: StepPlan) -> List[int]:
        """Apply what a step's commit does without its tokens (counts, publication, the end by
        length); sampling rows get the token PENDING. Returns a state per row: -1 for a row
        whose request had ended before (it is ignored from here on)."""
        count = len(plan.rows)
        state = (ctypes.c_int32 * max(count, 1))()
        host.check(self._lib.vh_commit_ahead(self._h, state))
        for i, row in enumerate(plan.rows):
            if state[i] < 0:
                continue
            request = row.request
            request.computed += row.count
            if row.sample:
                request.generated.append(self.PENDING)
                if state[i]:       # ended by length; its record is retired when its token is resolved
                    request.finished, request.finish_reason = True, _FINISH[state[i]]
        return list(state[:count])

    def resolve(self, plan: StepPlan, sampled: Sequence[Optional[int]]) -> Dict[object, int]:
        """Write the tokens of a step that commit_ahead took in and apply the end by EOS.
        Returns request id -> emitted token."""
        count = len(plan.rows)
        tokens = [int(t) if (row.sample and t is not None) else 0 for row, t in zip(plan.rows, sampled)]
        finished = (ctypes.c_int32 * max(count, 1))()
        host.check(self._lib.vh_resolve(self._h, host.ints(tokens), count, finished))
        emitted: Dict[object, int] = {}
        for i, row in enumerate(plan.rows):
            if not row.sample or finished[i] < 0:
                continue
            request = row.request
            index = row.start + row.count - len(request.prompt_tokens)
            request.generated[index] = tokens[i]
            emitted[request.request_id] = tokens[i]
            if finished[i]:
                self._retire(request, None if request.finished else _FINISH[finished[i]])
        return emitted
