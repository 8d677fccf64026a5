"""Trace replay over the engine's own step function (see bin/trace_run).

The reference has no tool that feeds given tokens portion by portion; its nearest
relatives are the prepared-request driver (examples/support/engine_benchmark.rs:79-88)
and the logits observer of its determinism suites (scripts/determinism_tests/). A request
is admitted when a step first names it and gives everything back when a step lists it
under `end`.
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Dict

import numpy as np

from .batch import StepEntry
from .runner import ModelRunner

MAX_LIVE = 8


class TraceReplayer:
    def __init__(self, model_dir, *, dtype: str, out_dir, max_tokens: int, page_size: int = 16,
                 device: str = "cuda:0", batch_invariant=False):
        if dtype == "bfloat16":
            from .. import ops
            ops.set_invariance(batch_invariant)
        self.out_dir = Path(out_dir)
        self.out_dir.mkdir(parents=True, exist_ok=True)
        num_pages = (max_tokens + page_size - 1) // page_size
        self.runner = ModelRunner(model_dir, dtype=dtype, device=device, num_pages=num_pages,
                                  page_size=page_size, max_requests=MAX_LIVE, prefix_reuse=False)

    def run_line(self, record: Dict) -> object:
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            rid = item["id"]
            if rid not in self.runner.cache.live:
                self.runner.begin(rid)
            entries.append(StepEntry(rid, [int(t) for t in item["tokens"]],
                                     [int(w) for w in item.get("want", [])]))
        if entries:
            logits = self.runner.step(entries)
            if logits is not None:
                host = logits.float().cpu().numpy().astype("<f4", copy=False)
                tmp = self.out_dir / f".{step}.f32.tmp"
                host.tofile(tmp)
                os.replace(tmp, self.out_dir / f"{step}.f32")
            self.runner.check_status()
        for rid in record.get("end", []):
            if rid in self.runner.cache.live:
                self.runner.finish(rid)
        return step
