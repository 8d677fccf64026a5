"""Benchmark of the engine's decode step and prefill at Qwen3-8B layer sizes with random
weights, on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

A "step" is one decode step of a batch of 8 requests whose context is 2,048 prompt tokens
plus what they have generated. `value` is decoded tokens a second over K steps timed with
CUDA events; `e2e` is the same metric over K further steps by the wall clock through the
Python entry point (`Engine.step`: host token ids in, host token ids out, with the
host-to-device copy of the step's batch from pinned memory and the device-to-host read of
the sampled tokens inside the timed region). Also on the line: one 2,048-token prefill
with its share of the measured bf16 peak, the decode step's share of the measured HBM
bandwidth, and decode speed at batch 1 and 64. Weights (15 GB) are far larger than L2, so
nothing is flushed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
    vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
    max_position_embeddings=4096, hidden_act="silu", attention_bias=False, attention_dropout=0.0,
    use_sliding_window=False, sliding_window=None, rope_scaling=None,
)
CONTEXT, PAGE = 2048, 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as handle:
            return json.load(handle), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi in the background while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, top, reasons = [], 0.0, set()
        for line in self.file.read().splitlines():
            fields = [f.strip() for f in line.split(",")]
            if len(fields) != 6:
                continue
            try:
                sm.append(float(fields[0]))
                top = max(top, float(fields[1]))
            except ValueError:
                continue
            for name, value in zip(self.NAMES, fields[2:]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": top or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def random_prompts(count, length, vocab, seed):
    import torch
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=gen).tolist() for _ in range(count)]


def decode_run(engine, batch, steps, warmup, seed, sample_clocks=False):
    """Prefill `batch` requests of CONTEXT tokens, then time decode steps twice: with CUDA
    events (device) and by the wall clock through Engine.step (end to end)."""
    import torch
    from vosti_b200 import ops

    vocab = engine.runner.spec.vocab_size
    first = len(engine.scheduler.accepted_ids)
    budget = warmup + 2 * steps + batch + 8      # early requests decode while later ones are prefilled
    for i, prompt in enumerate(random_prompts(batch, CONTEXT, vocab, seed)):
        status = engine.add_request(first + i, prompt, budget, None, True)
        assert status.value == "accepted", status
    while any(not r.is_decoding() for r in engine.scheduler.running) or engine.scheduler.waiting:
        engine.step()
    assert len(engine.scheduler.running) == batch
    engine.step()                          # with async scheduling the first decode step's tokens come a call later
    for _ in range(warmup):
        assert len(engine.step()) == batch
    sampler = ClockSampler() if sample_clocks else None
    if sampler:
        sampler.start()
    context_start = engine.scheduler.running[0].computed
    launches_before = ops.LAUNCHES
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record()
    for _ in range(steps):
        emitted = engine.step()
    end.record()
    torch.cuda.synchronize()
    device_ms = begin.elapsed_time(end) / steps
    launches = ops.LAUNCHES - launches_before
    assert len(emitted) == batch
    torch.cuda.synchronize()
    wall = time.perf_counter()
    for _ in range(steps):
        emitted = engine.step()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - wall) * 1e3 / steps
    clocks = sampler.stop() if sampler else None
    h2d = engine.runner.staging.last_upload_bytes
    d2h = 4 * (1 + batch)
    context_mid = context_start + steps // 2
    for i in range(batch):
        engine.abort(first + i)
    engine.drain()
    assert not engine.has_unfinished()
    return {"device_ms": device_ms, "wall_ms": wall_ms, "launches": launches, "clocks": clocks,
            "h2d": h2d, "d2h": d2h, "context": context_mid}


def prefill_run(engine, repeats, seed):
    import torch

    vocab = engine.runner.spec.vocab_size
    times = []
    for r, prompt in enumerate(random_prompts(repeats, CONTEXT, vocab, seed)):
        rid = len(engine.scheduler.accepted_ids)
        engine.add_request(rid, prompt, 1, None, True)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        emitted = engine.step()
        end.record()
        torch.cuda.synchronize()
        emitted.update(engine.drain())
        assert rid in emitted and not engine.has_unfinished()
        times.append(begin.elapsed_time(end))
    return min(times[1:]) if len(times) > 1 else times[0]


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (both are reported)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    parser.add_argument("--no-prefill", action="store_true", help="skip the 2,048-token prefill measurement")
    parser.add_argument("--no-cuda-graphs", action="store_true", help="launch decode kernels one by one (for profilers)")
    parser.add_argument("--sync-scheduling", action="store_true",
                        help="read every step's tokens before the next step is planned (default: the engine's async scheduling)")
    parser.add_argument("--batch-invariant", default="off", choices=["off", "decode", "full"],
                        help="measure with the engine's bitwise-invariance modes (the default run has them off)")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference engine is a Rust crate driven by `cargo run --example verus_engine_qwen3`; "
                          "no cargo/rustc here and its crates need the network; the offline pip install yields an "
                          "empty wheel (pyproject declares no package)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from vosti_b200 import Engine, ops
    from vosti_b200.config import model_spec_from_config
    from vosti_b200.models import expected_weights
    from vosti_b200.weights import draw_tensors

    peaks, peak_kind = load_peaks()
    config = dict(QWEN3_8B)
    layers_full = config["num_hidden_layers"]
    if args.layers:
        config["num_hidden_layers"] = args.layers
    spec = model_spec_from_config(config)
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    tensors = draw_tensors(expected_weights(spec), seed=0, device=device, dtype=torch.bfloat16)
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    tokens_per_request = CONTEXT + args.warmup + 2 * args.steps + max_batch + 10 + PAGE
    num_blocks = max_batch * ((tokens_per_request + PAGE - 1) // PAGE) + 8
    engine = Engine(spec=spec, tensors=tensors, dtype="bfloat16", device="cuda:0", num_blocks=num_blocks,
                    block_size=PAGE, max_num_seqs=max_batch, max_num_batched_tokens=2 * CONTEXT,
                    enable_prefix_caching=False, cuda_graphs=not args.no_cuda_graphs,
                    batch_invariant=args.batch_invariant, async_scheduling=not args.sync_scheduling)
    del tensors
    torch.cuda.empty_cache()
    weight_bytes = engine.runner.model.weight_bytes() - spec.vocab_size * spec.hidden_size * 2  # embedding rows: not read whole
    kv_bytes_per_token = engine.runner.cache.bytes_per_token()

    prefill_ms = float("nan") if args.no_prefill else prefill_run(engine, 3, seed=11)
    main_run = decode_run(engine, args.batch, args.steps, args.warmup, seed=21, sample_clocks=True)
    points = {}
    if not args.no_points:
        for batch in (1, 64):
            run = decode_run(engine, batch, max(8, args.steps // 2), 3, seed=31 + batch)
            points[f"decode_b{batch}"] = round(batch * 1e3 / run["device_ms"], 1)

    L, H = config["num_hidden_layers"], config["hidden_size"]
    nq, nkv, d, I, V = (config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"],
                        config["intermediate_size"], config["vocab_size"])
    T = CONTEXT
    linear_flops = 2.0 * T * L * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I) + 2.0 * V * H
    attention_flops = L * nq * d * 4.0 * T * (T + 1) / 2
    prefill_tflops = (linear_flops + attention_flops) / (prefill_ms * 1e-3) / 1e12
    step_bytes = weight_bytes + args.batch * main_run["context"] * kv_bytes_per_token
    achieved_gbs = step_bytes / (main_run["device_ms"] * 1e-3) / 1e9

    value = args.batch * 1e3 / main_run["device_ms"]
    line = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B size, context 2048)", "value": round(value, 1),
        "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["device_ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random token ids, random-init weights",
        "impl": "ours",
        "config": {"model": "Qwen3-8B size", "layers": L, "layers_full": layers_full, "hidden": H, "heads": nq,
                   "kv_heads": nkv, "head_dim": d, "intermediate": I, "vocab": V, "global_batch": args.batch,
                   "seq_len": CONTEXT, "page_size": PAGE, "parallelism": "1 GPU", "invariance": args.batch_invariant,
                   "scheduling": "sync" if args.sync_scheduling else "async",
                   "l2": "inputs larger than L2 (weights read every step)", "peaks": peak_kind},
        "e2e": {"value": round(args.batch * 1e3 / main_run["wall_ms"], 1), "unit": "tok/s",
                "h2d_bytes_per_step": main_run["h2d"], "d2h_bytes_per_step": main_run["d2h"]},
        "gpu_launches": main_run["launches"],
        "clocks": main_run["clocks"],
        "prefill": {"value": round(T * 1e3 / prefill_ms, 1), "tokens": T, "ms": round(prefill_ms, 3),
                    "frac": round(prefill_tflops / peaks["bf16_tflops"], 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved_gbs / peaks["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
