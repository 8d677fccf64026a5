"""CUDA graphs for decode steps.

A decode step launches a few hundred small kernels; issuing them one by one from the host
takes longer than the GPU needs to run them. Steps in which every request brings exactly
one token are therefore captured once per shape and replayed: the shape is (requests,
per-step arrays present, block-table width bucket, key-length bucket), and everything else
a kernel needs (tokens, positions, slots, block tables) is read from the step's staging
buffer, whose address and layout are the same for every step of a shape; the sampler's
state is read from, and advanced in, the requests' slots.
The reference has the same remedy for its per-primitive host overhead
(python/vosti_kernels/graph_overlay.py; src/exec/engine.rs:1990-2027).

A shape is run eagerly the first two times it is seen (the second run also warms every
kernel variant), then captured. Graphs are dropped when a scratch buffer they point to
has moved.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, Optional, Sequence

import torch

from .. import ops
from ..sampling import sample_from_slots
from .batch import StepEntry

PAGES_BUCKET = 32      # block-table width is rounded up to this many pages
KV_BUCKET = 512        # the key length kernels size their grids for is rounded up to this


def _round_up(value: int, multiple: int) -> int:
    return (value + multiple - 1) // multiple * multiple


class DecodeGraphs:
    def __init__(self, runner, max_graphs: int = 12):
        if not runner.model.capture_safe:
            raise ValueError("this model has a part that declares capture_safe = False: its decode steps "
                             "cannot be replayed from a recorded CUDA graph")
        self.runner = runner
        self.max_graphs = max_graphs
        self.graphs: "OrderedDict[tuple, dict]" = OrderedDict()
        self.seen: Dict[tuple, int] = {}
        self.replays = 0
        self.captures = 0

    def _run(self, ctx, count: int) -> None:
        runner = self.runner
        logits = runner.run(ctx)
        ex = ctx.extras
        sample_from_slots(logits, ex["sample_slots"], runner.cache.request_state, ex["sample_positions"],
                          runner.status, out=runner.result[1:1 + count])

    def step(self, entries: Sequence[StepEntry], extras: Optional[dict], longest: Optional[int] = None) -> None:
        """Run a decode-only step; the sampled tokens are left in runner.result[1:1+B]."""
        runner, cache = self.runner, self.runner.cache
        count = len(entries)
        if longest is None:
            longest = max(cache.length(e.request_id) for e in entries) + 1
        pages = _round_up(cache.pages_for(longest), PAGES_BUCKET)
        kv_bucket = _round_up(longest, KV_BUCKET)
        key = (count, tuple(sorted(extras)) if extras else (), pages, kv_bucket)
        ctx = runner.prepare(entries, extras=extras, min_pages=pages, kv_bucket=kv_bucket)
        stamp = (ops.WORKSPACE_GENERATION, runner.staging.dev.data_ptr())
        entry = self.graphs.get(key)
        if entry is not None and entry["stamp"] != stamp:
            del self.graphs[key]
            entry = None
        if entry is not None:
            self.graphs.move_to_end(key)
            entry["graph"].replay()
            ops.LAUNCHES += entry["launches"]
            self.replays += 1
            return
        self._run(ctx, count)
        self.seen[key] = self.seen.get(key, 0) + 1
        if self.seen[key] < 2:
            return
        # capture for the steps to come (recording does not run anything)
        torch.cuda.current_stream().synchronize()
        stamp = (ops.WORKSPACE_GENERATION, runner.staging.dev.data_ptr())
        graph = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES
        with torch.cuda.graph(graph):
            self._run(ctx, count)
        launches = ops.LAUNCHES - before
        ops.LAUNCHES = before
        while len(self.graphs) >= self.max_graphs:
            self.graphs.popitem(last=False)
        self.graphs[key] = {"graph": graph, "stamp": stamp, "launches": launches, "ctx": ctx}
        self.captures += 1
