"""The engine: scheduler above the step function, with sampling. This is the Python
entry point.

    engine = Engine(model_dir, dtype="bfloat16", num_blocks=4096)
    engine.add_request(0, prompt_ids, max_tokens=8, eos_token_ids=[eos])
    while engine.has_unfinished():
        emitted = engine.step()            # {request id: token}
    # or
    outputs = engine.generate([prompt_ids, ...], max_tokens=8)

The surface is the reference's Rust API as its example drives it: `Engine::init`,
`try_add_request`, `step` -> emitted tokens (src/exec/engine.rs:2515, 2664, 2795;
examples/support/engine_serving.rs:211-219). One step is plan -> forward -> sample ->
publish completed pages -> commit (src/exec/engine.rs:2781-2782), with one device-to-host
copy for the sampled tokens and the device fault word. A request's sampler state
(temperature, seed, index of the next token) is written to its slot of fixed size on the
device when it takes the slot and advanced there by the sampling kernel
(src/boundary/sampler.rs:7-19: (state, logits) -> (state', token)). With `async_scheduling` the order
becomes plan -> launch the next step -> read the last step's tokens, and the commit is split
in two around the plan (`Scheduler.commit_ahead`, `Scheduler.resolve`).
"""
from __future__ import annotations

import json
import time
from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np
import torch

from ..sampling import sample_from_slots, sampler_state_words
from .batch import StepEntry
from .request import AdmissionStatus, Request
from .runner import DeviceFault, ModelRunner, _FAULTS
from .scheduler import Scheduler, SchedulerConfig, StepPlan


class _Launched:
    """A step that was launched: its plan, how many rows sample, and where its result lands."""

    __slots__ = ("plan", "count", "host", "event", "index")

    def __init__(self, plan: StepPlan, count: int, host: torch.Tensor, event: torch.cuda.Event, index: int):
        self.plan, self.count, self.host, self.event, self.index = plan, count, host, event, index


def _is_bfloat16(dtype) -> bool:
    return str(dtype).endswith("bfloat16")


class Engine:
    def __init__(self, model: Optional[str] = None, *, dtype="bfloat16", device: str = "cuda:0",
                 num_blocks: int = 32, block_size: int = 16, max_num_seqs: int = 1,
                 max_num_batched_tokens: int = 4096, prefill_chunk_size: int = 0,
                 enable_prefix_caching: bool = True, step_trace: Optional[str] = None,
                 cuda_graphs: bool = True, batch_invariant=False, async_scheduling: bool = False, spec=None,
                 tensors=None, consume_tensors: bool = False):
        """`num_blocks` pages of `block_size` tokens; `max_num_seqs` rows and
        `max_num_batched_tokens` tokens per step at most (the reference's VOSTI_NUM_BLOCKS,
        VOSTI_MAX_SEQS, VOSTI_MAX_BATCHED_TOKENS; its page size is fixed at 64).
        `batch_invariant` (bfloat16 only; ops.set_invariance, which this engine applies again
        before each of its steps, so two engines of one process may run in different modes):
        True or "full" computes every token in one order of arithmetic, so that its bits do not
        depend on how prompts are cut into portions, on reused prefixes or on the batch around
        it, at the price of slower decoding; "decode" only pins the decode attention's segment
        length, which makes decode steps of up to 64 rows independent of the batch and costs
        little; the default lets every launch cut its work to fit its shape.
        `async_scheduling`: `step` launches the next step before it reads the last one's tokens,
        so the GPU does not idle while the host plans; the tokens a call returns are then those
        of the step launched by the call before (one call later than without it).
        `cuda_graphs`: decode steps are recorded once per shape and replayed; it is switched
        off by itself for a model with a part that declares `capture_safe = False`."""
        from .. import ops
        self.invariance = ops.set_invariance(batch_invariant) if _is_bfloat16(dtype) else None
        self.runner = ModelRunner(model, dtype=dtype, device=device, num_pages=num_blocks, page_size=block_size,
                                  max_requests=max_num_seqs, prefix_reuse=enable_prefix_caching, spec=spec,
                                  tensors=tensors, consume_tensors=consume_tensors)
        spec = self.runner.spec
        self.scheduler = Scheduler(self.runner.cache, SchedulerConfig(
            max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens,
            prefill_chunk_size=prefill_chunk_size, vocab_size=spec.vocab_size, max_context=spec.max_positions))
        from .graphs import DecodeGraphs
        # a part that reads a step's host-side values cannot be replayed from a recording
        self.graphs = DecodeGraphs(self.runner) if cuda_graphs and self.runner.model.capture_safe else None
        self.async_scheduling = bool(async_scheduling)
        self._inflight: Optional[_Launched] = None
        rows = 1 + max(max_num_seqs, 1)
        self._host_results = [torch.zeros(rows, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._events = [torch.cuda.Event() for _ in range(2)]
        self._host_turn = 0
        self._slot_tenant: Dict[int, object] = {}      # request whose sampler state a slot holds
        self.step_trace = open(step_trace, "a") if step_trace else None
        self.step_index = 0
        self.last_plan: Optional[StepPlan] = None

    # ------------------------------------------------------------ requests
    def add_request(self, request_id, prompt_tokens: Sequence[int], max_tokens: int,
                    eos_token_ids: Optional[Sequence[int]] = None, ignore_eos: bool = False,
                    temperature: float = 0.0, seed: int = 0) -> AdmissionStatus:
        """Queue a request; pages are taken when a step first schedules it."""
        if eos_token_ids is None:
            eos_token_ids, ignore_eos = (), True
        request = Request(request_id, [int(t) for t in prompt_tokens], int(max_tokens),
                          tuple(int(t) for t in eos_token_ids), bool(ignore_eos), float(temperature), int(seed))
        return self.scheduler.add_request(request)

    def abort(self, request_id) -> bool:
        """End a queued or running request between steps; its pages and slot come back."""
        return self.scheduler.abort(request_id)

    def release(self, request_id) -> bool:
        """Drop the record of a finished request (`request(id)` no longer finds it). Records
        are also dropped by age: the scheduler keeps the newest `keep_finished` of them."""
        return self.scheduler.release(request_id)

    def has_unfinished(self) -> bool:
        return self._inflight is not None or self.scheduler.has_unfinished()

    def request(self, request_id) -> Optional[Request]:
        for r in self.scheduler.running + self.scheduler.waiting:
            if r.request_id == request_id:
                return r
        return self.scheduler.finished.get(request_id)

    # ------------------------------------------------------------ one step
    def step(self) -> Dict[object, int]:
        """Plan, run, sample and commit one step; returns the tokens emitted by it. With
        `async_scheduling` the step that is planned and launched is the next one, and the
        tokens returned are those of the step launched by the call before."""
        if self.async_scheduling:
            return self._step_ahead(launch=True)
        plan = self.scheduler.plan()
        self.last_plan = plan
        self.step_index += 1
        if not plan.rows:
            self._trace(plan, {})
            return {}
        launched = self._launch(plan, None)
        emitted = self.scheduler.commit(plan, self._collect(launched))
        self._trace(plan, emitted)
        return emitted

    def drain(self) -> Dict[object, int]:
        """Read the step that is still in flight, if any, without launching another."""
        return self._step_ahead(launch=False) if self._inflight is not None else {}

    def _step_ahead(self, launch: bool) -> Dict[object, int]:
        """Launch step n + 1 before step n's tokens are read, so that the GPU does not wait for
        the host between steps. The scheduler commits step n in two halves (what needs no token
        values now, the tokens and the end by EOS once they are read); a request's newest
        token, while the host does not have it, is fed to the next step on the device from
        where the sampler left it. A request that step n's tokens end still has a row in the
        step launched meanwhile: that row's result is dropped."""
        before = self._inflight
        if before is not None:
            self.scheduler.commit_ahead(before.plan)
        launched = None
        if launch:
            plan = self.scheduler.plan()
            self.last_plan = plan
            self.step_index += 1
            if plan.rows:
                launched = self._launch(plan, before)
            elif before is None:
                self._trace(plan, {})
        emitted: Dict[object, int] = {}
        if before is not None:
            emitted = self.scheduler.resolve(before.plan, self._collect(before))
            self._trace(before.plan, emitted, before.index)
        self._inflight = launched
        return emitted

    def _launch(self, plan: StepPlan, before: Optional["_Launched"]) -> "_Launched":
        """Lay out and launch the plan's step, sampling included, and start the copy of its
        result to the host. `before` is the step launched earlier whose tokens the host has not
        read: a row whose last token is one of them names its place in that step's result."""
        runner = self.runner
        if self.invariance is not None:
            from .. import ops
            ops.set_invariance(self.invariance)       # another engine of the process may have set its own
        entries, feedback, slots, positions = [], [], [], []
        slot_before = {}
        if before is not None:
            slot = 0
            for row in before.plan.rows:
                if row.sample:
                    slot_before[row.request.request_id] = slot
                    slot += 1
        table = runner.cache.request_state
        for row in plan.rows:
            request = row.request
            tokens = request.token_range(row.start, row.count)
            source = [-1] * row.count
            if tokens[-1] == Scheduler.PENDING:
                if request.request_id not in slot_before:
                    raise RuntimeError(f"request {request.request_id!r}: its newest token is neither known nor on the device")
                tokens[-1], source[-1] = 0, slot_before[request.request_id]
            feedback.extend(source)
            entries.append(StepEntry(request.request_id, tokens, [row.count - 1] if row.sample else []))
            # the sampler's state lives in the request's slot: written when the request takes the
            # slot (admission, re-admission after a preemption), advanced there by the kernel
            if self._slot_tenant.get(row.slot) != request.request_id:
                self._slot_tenant[row.slot] = request.request_id
                words = torch.tensor(sampler_state_words(request.temperature, request.seed, len(request.generated)),
                                     dtype=torch.int64).pin_memory()
                table[row.slot].copy_(words, non_blocking=True)
            if row.sample:
                slots.append(row.slot)
                positions.append(row.start + row.count - 1)
        count = len(slots)
        extras = {"sample_slots": np.asarray(slots, dtype=np.int32),
                  "sample_positions": np.asarray(positions, dtype=np.int32)} if count else {}
        if self.async_scheduling:
            extras["feedback"] = np.asarray(feedback, dtype=np.int32)
        if self.graphs is not None and all(row.count == 1 and row.sample for row in plan.rows):
            self.graphs.step(entries, extras, longest=max(row.start for row in plan.rows) + 1)
        else:
            ctx = runner.prepare(entries, extras=extras or None)
            logits = runner.run(ctx)
            if logits is not None:
                ex = ctx.extras
                sample_from_slots(logits, ex["sample_slots"], table, ex["sample_positions"], runner.status,
                                  out=runner.result[1:1 + count])
        self._host_turn ^= 1
        host = self._host_results[self._host_turn]
        host[:1 + count].copy_(runner.result[:1 + count], non_blocking=True)
        event = self._events[self._host_turn]
        event.record()
        if runner.cache.has_windows:
            for e in entries:
                runner.cache.trim(e.request_id)
        return _Launched(plan, count, host, event, self.step_index)

    def _collect(self, launched: "_Launched") -> List[Optional[int]]:
        """Wait for a launched step's result; returns the token of every row (None where the
        row does not sample)."""
        launched.event.synchronize()
        host = launched.host[:1 + launched.count].tolist()
        if host[0]:
            self.runner.status.zero_()
            raise DeviceFault("device reported: " + "; ".join(t for b, t in _FAULTS.items() if host[0] & b))
        it = iter(host[1:])
        return [next(it) if row.sample else None for row in launched.plan.rows]

    def _trace(self, plan: StepPlan, emitted: Dict[object, int], index: Optional[int] = None) -> None:
        """One JSON line per step, as the reference's VOSTI_ENGINE_STEP_TRACE
        (examples/support/engine_benchmark.rs:273-317)."""
        if self.step_trace is None:
            return
        self.step_trace.write(json.dumps({
            "step": self.step_index if index is None else index,
            "scheduled": [[str(r.request.request_id), r.start, r.count, r.sample] for r in plan.rows],
            "emitted": {str(k): v for k, v in emitted.items()},
            "preempted": [str(r) for r in plan.preempted], "dropped": [str(r) for r in plan.dropped],
            "free_pages": self.runner.cache.available_pages(),
        }) + "\n")
        self.step_trace.flush()

    # ------------------------------------------------------------ convenience
    def generate(self, prompts: Iterable[Sequence[int]], max_tokens: int = 8,
                 eos_token_ids: Optional[Sequence[int]] = None, ignore_eos: bool = False,
                 temperature: float = 0.0, seeds: Optional[Sequence[int]] = None,
                 arrival_steps: Optional[Sequence[int]] = None, first_id: Optional[int] = None) -> List[List[int]]:
        """Generate for token-id prompts and return the new tokens of each, in order.
        `arrival_steps[i]` delays prompt i until that many engine steps have passed."""
        prompts = list(prompts)
        base = first_id if first_id is not None else len(self.scheduler.accepted_ids)
        ids = [base + i for i in range(len(prompts))]
        pending = sorted(range(len(prompts)), key=lambda i: (arrival_steps[i] if arrival_steps else 0, i))
        outputs: Dict[object, List[int]] = {rid: [] for rid in ids}
        step = 0
        while pending or self.has_unfinished():
            while pending and (not arrival_steps or arrival_steps[pending[0]] <= step):
                i = pending.pop(0)
                status = self.add_request(ids[i], prompts[i], max_tokens, eos_token_ids, ignore_eos,
                                          temperature, seeds[i] if seeds else 0)
                if status is not AdmissionStatus.ACCEPTED:
                    raise ValueError(f"prompt {i} was not accepted: {status.value}")
            for rid, token in self.step().items():
                if rid in outputs:
                    outputs[rid].append(token)
            step += 1
        return [outputs[rid] for rid in ids]

    def cache_stats(self) -> dict:
        cache = self.runner.cache
        return {"admitted_requests": self.scheduler.admitted_requests,
                "requests_with_reuse": cache.requests_with_reuse,
                "reused_prefix_blocks": cache.reused_prefix_pages,
                "preemptions": self.scheduler.preemptions}
