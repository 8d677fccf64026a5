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

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from ..cache import CacheManager
from .request import MAX_EOS_TOKEN_IDS, AdmissionStatus, Request


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 4096
    prefill_chunk_size: int = 0      # 0: limited by the token budget only
    vocab_size: int = 0              # 0: prompt tokens are not range-checked here
    max_context: int = 0             # 0: no limit

    def validate(self) -> None:
        if self.max_num_seqs <= 0 or self.max_num_batched_tokens <= 0:
            raise ValueError("max_num_seqs and max_num_batched_tokens must be positive")
        if self.prefill_chunk_size < 0:
            raise ValueError("prefill_chunk_size must be >= 0")


@dataclass
class PlanRow:
    request: Request
    start: int                 # position of the row's first token
    count: int                 # tokens the row computes
    sample: bool               # the row reaches the end of the known tokens


@dataclass
class StepPlan:
    rows: List[PlanRow] = field(default_factory=list)
    preempted: List[object] = field(default_factory=list)
    dropped: List[object] = field(default_factory=list)

    def num_tokens(self) -> int:
        return sum(r.count for r in self.rows)


class Scheduler:
    def __init__(self, cache: CacheManager, config: SchedulerConfig):
        config.validate()
        self.cache, self.config = cache, config
        self.waiting: List[Request] = []
        self.running: List[Request] = []
        self.accepted_ids = set()            # ids are never reused (src/exec/cache_scheduler/types.rs:162-165)
        self.finished: Dict[object, Request] = {}
        self.admitted_requests = 0
        self.preemptions = 0

    # ------------------------------------------------------------ admission
    def add_request(self, request: Request) -> AdmissionStatus:
        cfg = self.config
        if request.request_id in self.accepted_ids:
            return AdmissionStatus.DUPLICATE_ID
        if len(request.prompt_tokens) == 0:
            return AdmissionStatus.EMPTY_PROMPT
        if not request.ignore_eos and not 1 <= len(request.eos_token_ids) <= MAX_EOS_TOKEN_IDS:
            return AdmissionStatus.BAD_EOS
        if len(request.eos_token_ids) > MAX_EOS_TOKEN_IDS:
            return AdmissionStatus.BAD_EOS
        if request.max_tokens <= 0:
            return AdmissionStatus.ZERO_BUDGET
        if not (request.temperature >= 0.0 and request.temperature < float("inf")):
            return AdmissionStatus.BAD_SAMPLING
        if cfg.max_context and len(request.prompt_tokens) + request.max_tokens > cfg.max_context:
            return AdmissionStatus.TOO_LONG
        if cfg.vocab_size and any(not 0 <= int(t) < cfg.vocab_size for t in request.prompt_tokens):
            return AdmissionStatus.BAD_TOKEN
        self.accepted_ids.add(request.request_id)
        self.waiting.append(request)
        return AdmissionStatus.ACCEPTED

    def abort(self, request_id) -> bool:
        """End a request now: it leaves its queue and gives back what it holds."""
        for queue in (self.waiting, self.running):
            for request in queue:
                if request.request_id == request_id:
                    queue.remove(request)
                    if request_id in self.cache.live:
                        self.cache.finish(request_id)
                    request.finished, request.finish_reason = True, "aborted"
                    self.finished[request_id] = request
                    return True
        return False

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------ planning
    def _chunk(self, remaining: int, budget: int) -> int:
        """Tokens of the next portion: everything if it fits, else whole pages."""
        cap = budget
        if self.config.prefill_chunk_size:
            cap = min(cap, self.config.prefill_chunk_size)
        if remaining <= cap:
            return remaining
        return cap // self.cache.page_size * self.cache.page_size

    def _plan_once(self) -> StepPlan:
        cache, cfg = self.cache, self.config
        plan = StepPlan()
        budget = cfg.max_num_batched_tokens
        reserved = 0

        # 1. decode rows: a prefix of the running requests
        for request in self.running:
            if not request.is_decoding():
                continue
            if len(plan.rows) >= cfg.max_num_seqs:
                break
            need = cache.pages_needed(request.request_id, 1)
            if reserved + need > cache.available_pages():
                break
            plan.rows.append(PlanRow(request, request.computed, 1, True))
            reserved += need
            budget -= 1

        # 2. running requests in the middle of their prompt
        for request in self.running:
            if request.is_decoding() or len(plan.rows) >= cfg.max_num_seqs:
                continue
            count = self._chunk(request.remaining(), max(budget, 0))
            if count <= 0:
                continue
            need = cache.pages_needed(request.request_id, count)
            if reserved + need > cache.available_pages():
                continue
            plan.rows.append(PlanRow(request, request.computed, count, count == request.remaining()))
            reserved += need
            budget -= count

        # 3. admissions: the head of the waiting queue only
        while self.waiting and len(plan.rows) < cfg.max_num_seqs and budget > 0:
            if len(self.running) >= cache.max_requests or not cache.free_slots:
                break
            request = self.waiting[0]
            tokens = request.tokens()
            cache.begin(request.request_id, tokens)
            request.computed = cache.length(request.request_id)
            count = self._chunk(request.remaining(), budget)
            need = cache.pages_needed(request.request_id, count) if count > 0 else 0
            if count <= 0 or reserved + need > cache.available_pages():
                cache.finish(request.request_id)      # roll back: nothing of it is held
                request.computed = 0
                break
            self.waiting.pop(0)
            self.running.append(request)
            self.admitted_requests += 1
            plan.rows.append(PlanRow(request, request.computed, count, count == request.remaining()))
            reserved += need
            budget -= count
        return plan

    def plan(self) -> StepPlan:
        """Decide the next step's batch. Never returns an empty plan while a request is
        live: it preempts (or, for a request no cache could hold, drops) until a row fits."""
        preempted, dropped = [], []
        while True:
            plan = self._plan_once()
            if plan.rows or not self.has_unfinished():
                break
            if self.running:
                victim = self.running.pop()           # the youngest
                self.cache.finish(victim.request_id)
                victim.computed = 0
                victim.preemptions += 1
                self.preemptions += 1
                self.waiting.insert(0, victim)
                preempted.append(victim.request_id)
                continue
            # nothing runs and the head still does not fit: no cache of this size can hold it
            victim = self.waiting.pop(0)
            victim.finished, victim.finish_reason = True, "capacity"
            self.finished[victim.request_id] = victim
            dropped.append(victim.request_id)
        plan.preempted, plan.dropped = preempted, dropped
        return plan

    # ------------------------------------------------------------ commit
    def commit(self, plan: StepPlan, sampled: Sequence[Optional[int]]) -> Dict[object, int]:
        """Apply a step's results: `sampled[i]` is the token of row i (ignored for rows that
        do not sample). Returns request id -> emitted token."""
        emitted: Dict[object, int] = {}
        for row, token in zip(plan.rows, sampled):
            request = row.request
            request.computed += row.count
            self.cache.publish(request.request_id, request.tokens()[:request.computed])
            if not row.sample:
                continue
            if token is None:
                raise ValueError(f"row of request {request.request_id!r} samples but got no token")
            emitted[request.request_id] = int(token)
            if request.record(int(token)):
                self.running.remove(request)
                self.cache.finish(request.request_id)
                self.finished[request.request_id] = request
        return emitted
