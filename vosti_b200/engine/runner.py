"""The step function: run a batch of (request, its next tokens) from the cache and
return the logits at the wanted places.

A step holds portions of prompts beside single decoded tokens, cut anywhere; it runs
only the tokens it is given. The model, the cache manager and the kernels here are the
ones generation uses; trace replay drives this same object.

Order inside a step as in the reference (src/exec/engine.rs:2781-2782, 3315-3333;
src/exec/dense_swiglu_decoder.rs:253-320): every layer stores the step's keys and values
before its attention reads the cache.
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from ..cache import CacheManager, OutOfPages
from ..config import model_spec_from_dir, ModelSpec
from ..models import build_model
from ..weights import check_tensors, load_weights
from .batch import StagingBuffer, StepContext, StepEntry, build_context

_FAULTS = {
    1: "token id outside the vocabulary", 2: "cache slot outside the pool",
    4: "block-table entry outside the pool", 8: "position beyond the rotation table",
    16: "a bounded device wait gave up", 32: "gathered row outside the input",
}


class DeviceFault(RuntimeError):
    pass


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name in (torch.bfloat16, torch.float32):
            return name
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
             "fp32": torch.float32, "f32": torch.float32}
    if str(name) in table:
        return table[str(name)]
    raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}")


class ModelRunner:
    def __init__(self, model_dir: Optional[str | Path] = None, *, dtype="bfloat16", device="cuda:0",
                 num_pages: int, page_size: int = 16, max_requests: int = 64, prefix_reuse: bool = False,
                 spec: Optional[ModelSpec] = None, tensors: Optional[Dict[str, torch.Tensor]] = None,
                 consume_tensors: bool = False):
        """`tensors` (name -> tensor, already on the device) stands in for a model folder.
        With `consume_tensors` the dictionary is emptied once the parts have taken what they
        keep, before the cache is allocated, so that weights the parts re-packed do not stay in
        memory twice."""
        self.device = torch.device(device)
        self.dtype = parse_dtype(dtype)
        ops.require_device(self.device)
        ops.library()
        torch.cuda.set_device(self.device)
        if torch.backends.cuda.matmul.allow_tf32:
            torch.backends.cuda.matmul.allow_tf32 = False
        self.spec = spec if spec is not None else model_spec_from_dir(model_dir)
        self.model = build_model(self.spec)
        expected = self.model.expected_weights()
        if tensors is None:
            tensors = load_weights(model_dir, expected, device=self.device, dtype=self.dtype,
                                   ignore=self.model.ignorable_weights(), aliases=self.model.tied_weights())
        else:
            check_tensors(tensors, expected, ignore=self.model.ignorable_weights(),
                          aliases=self.model.tied_weights())
            if self.dtype == torch.float32:
                tensors = {k: (v.float() if v.is_floating_point() else v) for k, v in tensors.items()}
        self.model.load(tensors, self.dtype)
        if consume_tensors:
            tensors.clear()
            torch.cuda.empty_cache()
        cache_specs = [b.mixer.cache_spec() for b in self.model.blocks]
        state_specs = [b.mixer.state_spec() for b in self.model.blocks]
        self.cache = CacheManager(cache_specs, state_specs, num_pages=num_pages, page_size=page_size,
                                  max_requests=max_requests, device=self.device, dtype=self.dtype,
                                  prefix_reuse=prefix_reuse)
        self.staging = StagingBuffer(self.device)
        # word 0: device fault bits; the rest: sampled tokens of a step
        self.result = torch.zeros(1 + max(max_requests, 1), dtype=torch.int32, device=self.device)
        self.result_host = torch.zeros(1 + max(max_requests, 1), dtype=torch.int32, pin_memory=True)
        self.status = self.result[:1]
        self.sampled = self.result[1:]            # where the sampler leaves a step's tokens
        self.steps = 0
        self.kernel_launches = 0

    # ------------------------------------------------------------ requests
    def begin(self, request_id, prompt_for_reuse: Optional[Sequence[int]] = None):
        return self.cache.begin(request_id, prompt_for_reuse)

    def finish(self, request_id) -> None:
        self.cache.finish(request_id)

    # ------------------------------------------------------------ the step
    def prepare(self, entries: Sequence[StepEntry], extras: Optional[dict] = None, min_pages: int = 0,
                kv_bucket: int = 0) -> StepContext:
        """Reserve cache entries for the step's tokens (all requests or none) and copy the
        batch to the device."""
        self.cache.clear_fresh_state()       # slots the scheduler handed out since the last step
        ctx = build_context(self.staging, self.cache, entries, self.status, self.dtype, extras=extras,
                            min_pages=min_pages, kv_bucket=kv_bucket, position_limit=self.spec.max_positions)
        ctx.feedback_values = self.sampled
        return ctx

    def run(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """The model over the prepared batch; float32 logits [wanted, vocab] or None."""
        hidden, residual = self.model.forward(ctx, self.cache.layer_caches)
        self.steps += 1
        if ctx.want_rows.shape[0] == 0:
            return None
        return self.model.logits(ctx, hidden, residual, ctx.want_rows)

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        ctx = self.prepare(entries)
        logits = self.run(ctx)
        if self.cache.has_windows:
            for e in entries:
                self.cache.trim(e.request_id)
        return logits

    # ------------------------------------------------------------ status
    def check_status(self) -> None:
        """Read the device fault word (synchronises) and raise if a kernel set a bit."""
        bits = int(self.status.item())
        if bits:
            self.status.zero_()
            names = [text for bit, text in _FAULTS.items() if bits & bit]
            raise DeviceFault("device reported: " + "; ".join(names))
