"""Benchmark of the engine's decode step and prefill at Qwen3 layer sizes with random
weights, on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--size 8b|14b|32b] [--workload decode|mixed] [--layers L]

A "step" is one decode step of a batch of 8 requests whose context is 2,048 prompt tokens
plus what they have generated. The region of K steps is timed with CUDA events and repeated;
`value` is decoded tokens a second at the median repeat. `e2e` is the same metric over K
steps by the wall clock through the Python entry point (`Engine.step`: host token ids in,
host token ids out, with the host-to-device copy of the step's batch from pinned memory and
the device-to-host read of the sampled tokens inside the timed region), also the median of
the repeats. Also on the line: one 2,048-token prefill with its share of the measured bf16
peak, the decode step's share of the measured HBM bandwidth with the bytes it counts, and
decode speed at batch 1 and 64. Weights (15 GB and more) are far larger than L2, so nothing
is flushed between steps. SM clocks and throttle reasons are sampled over all repeats.

`--size` selects the layer sizes (8b is the headline; 14b and 32b are the further sizes of
the benchmark configuration list). `--workload mixed` runs a continuous batch instead: 32
requests, prompt lengths uniform in [64, 3072], 128 to 512 new tokens each, Poisson arrivals,
half of them sharing a 1,024-token prefix, and reports generated tokens a second.

`--impl reference` runs the unmodified reference through its own Python primitive API and
Triton kernels (baseline/reference_arm.py) on the same metric and configuration.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def qwen3(layers, hidden, heads, kv_heads, inter, context=4096):
    return dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=layers, hidden_size=hidden,
        num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=128, intermediate_size=inter,
        vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
        max_position_embeddings=context, hidden_act="silu", attention_bias=False, attention_dropout=0.0,
        use_sliding_window=False, sliding_window=None, rope_scaling=None,
    )


SIZES = {
    "8b": ("Qwen3-8B size", qwen3(36, 4096, 32, 8, 12288)),
    "14b": ("Qwen3-14B size", qwen3(40, 5120, 40, 8, 17408)),
    "32b": ("Qwen3-32B size", qwen3(64, 5120, 64, 8, 25600)),
}
CONTEXT, PAGE = 2048, 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
MIN_TIMED_MS = 1200.0     # repeats of the K-step region go on until this much was timed (clock samples)


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
                                          "--format=csv,noheader,nounits", "-lms", "50"],
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


def repeats_for(steps, ms_per_step, least, most):
    return max(1, min(most, max(least, math.ceil(MIN_TIMED_MS / max(steps * ms_per_step, 1e-3)))))


DECODE_STEPS = 256        # a request decodes this many tokens in the benchmark's workload


def decode_run(engine, batch, steps, warmup, seed, sample_clocks=False, least_repeats=5):
    """Prefill `batch` requests of CONTEXT tokens, then time regions of `steps` decode steps:
    with CUDA events (device) and by the wall clock through Engine.step (end to end). Each
    region is repeated (at most DECODE_STEPS steps in all, so the context stays near CONTEXT)
    and the median is reported."""
    import torch
    from vosti_b200 import ops

    vocab = engine.runner.spec.vocab_size
    first = len(engine.scheduler.accepted_ids)
    budget = engine.runner.spec.max_positions - CONTEXT
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
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    device_ms, launches, repeats = [], 0, max(1, min(least_repeats, DECODE_STEPS // steps))
    while len(device_ms) < repeats:
        launches_before = ops.LAUNCHES
        torch.cuda.synchronize()
        begin.record()
        for _ in range(steps):
            emitted = engine.step()
        end.record()
        torch.cuda.synchronize()
        device_ms.append(begin.elapsed_time(end) / steps)
        launches = ops.LAUNCHES - launches_before
        assert len(emitted) == batch
        if len(device_ms) == 1:
            repeats = repeats_for(steps, device_ms[0], least_repeats, max(1, DECODE_STEPS // steps))
    # the end-to-end regions stay inside the same key-length bucket of the decode graphs
    room = (CONTEXT // 512 + 1) * 512 - (context_start + repeats * steps) - 8
    wall_ms = []
    for _ in range(max(1, min(repeats, room // steps))):
        torch.cuda.synchronize()
        wall = time.perf_counter()
        for _ in range(steps):
            emitted = engine.step()
        torch.cuda.synchronize()
        wall_ms.append((time.perf_counter() - wall) * 1e3 / steps)
    clocks = sampler.stop() if sampler else None
    h2d = engine.runner.staging.last_upload_bytes
    d2h = 4 * (1 + batch)
    context_mid = context_start + repeats * steps // 2
    for i in range(batch):
        engine.abort(first + i)
    engine.drain()
    assert not engine.has_unfinished()
    return {"device_ms": statistics.median(device_ms), "wall_ms": statistics.median(wall_ms), "launches": launches,
            "clocks": clocks, "h2d": h2d, "d2h": d2h, "context": context_mid, "repeats": repeats}


def prefill_run(engine, repeats, seed):
    """One CONTEXT-token prompt in one step, timed with CUDA events; the median of `repeats`
    runs after one that is not counted."""
    import torch

    vocab = engine.runner.spec.vocab_size
    times = []
    for r, prompt in enumerate(random_prompts(repeats + 1, CONTEXT, vocab, seed)):
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
    return statistics.median(times[1:])


def flops_of_prefill(config, tokens):
    L, H = config["num_hidden_layers"], config["hidden_size"]
    nq, nkv, d, I, V = (config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"],
                        config["intermediate_size"], config["vocab_size"])
    linear = 2.0 * tokens * L * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I) + 2.0 * V * H
    attention = L * nq * d * 4.0 * tokens * (tokens + 1) / 2
    return linear + attention


def closed_form_weight_bytes(config):
    """bf16 bytes of every weight a decode step reads whole: per layer the four attention
    projections, two head norms, two norms, three feed-forward matrices; the final norm; the
    output head (the embedding table is read by rows, one per token)."""
    L, H = config["num_hidden_layers"], config["hidden_size"]
    nq, nkv, d, I, V = (config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"],
                        config["intermediate_size"], config["vocab_size"])
    per_layer = H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I + 2 * H + 2 * d
    return 2 * (L * per_layer + H + V * H)


def reference_main(args) -> int:
    """The reference arm: same metric, same configuration, the reference's own code."""
    name, config = SIZES[args.size]
    try:
        if args.size != "8b":
            raise RuntimeError(f"the reference has launch profiles for qwen3-0.6b and qwen3-8b only, not {args.size}")
        import torch
        from baseline import reference_arm as arm
        peaks, peak_kind = load_peaks()
        layers = args.layers or config["num_hidden_layers"]
        max_batch = args.batch if args.no_points else max(args.batch, 64)
        per_request = CONTEXT + 64 * 3
        model = arm.ReferenceModel("qwen3-8b", layers, max_batch * per_request + 128, seed=0)
        ref_config = dict(model.config)
        ref_config["num_hidden_layers"] = layers
        prefill_ms = float("nan") if args.no_prefill else arm.prefill_run(model, CONTEXT, 3, seed=11)
        sampler = ClockSampler()
        sampler.start()
        runs = [arm.decode_run(model, args.batch, CONTEXT, args.steps, args.warmup, seed=21)
                for _ in range(1 if args.steps * 2 + args.warmup + 2 > 60 else 3)]
        clocks = sampler.stop()
        main_run = sorted(runs, key=lambda r: r["device_ms"])[len(runs) // 2]
        points = {}
        if not args.no_points:
            for batch in (1, 64):
                run = arm.decode_run(model, batch, CONTEXT, max(8, min(args.steps // 2, 24)), 3, seed=31 + batch)
                points[f"decode_b{batch}"] = round(batch * 1e3 / run["device_ms"], 1)
        step_bytes = model.weight_bytes + args.batch * main_run["context"] * model.kv_bytes_per_token
        achieved = step_bytes / (main_run["device_ms"] * 1e-3) / 1e9
        tflops = flops_of_prefill(ref_config, CONTEXT) / (prefill_ms * 1e-3) / 1e12
        line = {
            "metric": f"decode tok/s at batch {args.batch} ({name}, context {CONTEXT})",
            "value": round(args.batch * 1e3 / main_run["device_ms"], 1), "unit": "tok/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(main_run["device_ms"], 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: random token ids, random-init weights", "impl": "reference",
            "config": {"model": name, "layers": layers, "layers_full": config["num_hidden_layers"],
                       "hidden": ref_config["hidden_size"], "heads": ref_config["num_attention_heads"],
                       "kv_heads": ref_config["num_key_value_heads"], "head_dim": ref_config["head_dim"],
                       "intermediate": ref_config["intermediate_size"], "vocab": ref_config["vocab_size"],
                       "global_batch": args.batch, "seq_len": CONTEXT, "page_size": arm.PAGE, "parallelism": "1 GPU",
                       "path": "vosti_kernels primitives + Triton kernels + CudaGraphOverlay, Python host loop",
                       "l2": "inputs larger than L2 (weights read every step)", "peaks": peak_kind},
            "e2e": {"value": round(args.batch * 1e3 / main_run["wall_ms"], 1), "unit": "tok/s",
                    "h2d_bytes_per_step": main_run["h2d"], "d2h_bytes_per_step": main_run["d2h"]},
            "clocks": clocks,
            "prefill": {"value": round(CONTEXT * 1e3 / prefill_ms, 1), "tokens": CONTEXT, "ms": round(prefill_ms, 3),
                        "frac": round(tflops / peaks["bf16_tflops"], 4),
                        "frac_of_sustained": round(tflops / peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]), 4)},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / peaks["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
            "points": points,
        }
        print(json.dumps(line))
    except Exception as error:  # the arm must report, not crash: the driver reads this line
        import traceback
        traceback.print_exc(file=sys.stderr)
        text = " ".join(f"{type(error).__name__}: {error}".split())
        print(json.dumps({"impl": "reference", "unavailable": text[:600]}))
    return 0


def mixed_run(engine, config, seed=5, requests=32, rate_per_s=16.0):
    """A continuous batch: `requests` prompts with lengths uniform in [64, 3072] and 128 to 512
    new tokens each, Poisson arrivals at `rate_per_s`, half of them starting with the same
    1,024 tokens. Returns generated tokens, wall seconds and what the cache reused."""
    import random
    import torch

    rng = random.Random(seed)
    vocab = config["vocab_size"]
    gen = torch.Generator().manual_seed(seed)
    draw = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()
    shared = draw(1024)
    plan, at = [], 0.0
    for i in range(requests):
        length = rng.randint(64, 3072)
        new_tokens = rng.randint(128, 512)
        prompt = (shared + draw(max(length - 1024, 1))) if i % 2 == 0 else draw(length)
        at += rng.expovariate(rate_per_s)
        plan.append((at, i, prompt, new_tokens))
    first = len(engine.scheduler.accepted_ids)
    generated, first_token_at, arrived_at = 0, {}, {}
    torch.cuda.synchronize()
    start = time.perf_counter()
    steps = 0
    while plan or engine.has_unfinished():
        now = time.perf_counter() - start
        while plan and plan[0][0] <= now:
            _, i, prompt, new_tokens = plan.pop(0)
            status = engine.add_request(first + i, prompt, new_tokens, None, True)
            assert status.value == "accepted", status
            arrived_at[first + i] = now
        if not engine.has_unfinished():
            time.sleep(max(0.0, plan[0][0] - now))
            continue
        emitted = engine.step()
        steps += 1
        generated += len(emitted)
        now = time.perf_counter() - start
        for rid in emitted:
            first_token_at.setdefault(rid, now)
    torch.cuda.synchronize()
    wall = time.perf_counter() - start
    ttft = sorted(first_token_at[r] - arrived_at[r] for r in first_token_at)
    return {"generated": generated, "wall_s": wall, "steps": steps, "ttft_median_s": ttft[len(ttft) // 2],
            "ttft_max_s": ttft[-1], **engine.cache_stats()}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--size", default="8b", choices=sorted(SIZES), help="layer sizes (8b is the headline)")
    parser.add_argument("--workload", default="decode", choices=["decode", "mixed"],
                        help="decode: the headline; mixed: a continuous batch with Poisson arrivals and a shared prefix")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (both are reported)")
    parser.add_argument("--context", type=int, default=2048,
                        help="prompt length of the decode requests and of the prefill (the headline is 2048)")
    parser.add_argument("--page", type=int, default=16, help="tokens per cache page")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    parser.add_argument("--no-prefill", action="store_true", help="skip the 2,048-token prefill measurement")
    parser.add_argument("--no-cuda-graphs", action="store_true", help="launch decode kernels one by one (for profilers)")
    parser.add_argument("--repeats", type=int, default=5, help="least number of repeats of the timed K-step region")
    parser.add_argument("--sync-scheduling", action="store_true",
                        help="read every step's tokens before the next step is planned (default: the engine's async scheduling)")
    parser.add_argument("--batch-invariant", default="off", choices=["off", "decode", "full"],
                        help="measure with the engine's bitwise-invariance modes (the default run has them off)")
    args = parser.parse_args()

    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    global CONTEXT, PAGE
    PAGE = args.page
    if args.context != CONTEXT:
        if args.context < 64 or args.context % 64:
            parser.error("--context must be a multiple of 64, at least 64")
        CONTEXT = args.context
        for _, config in SIZES.values():
            config["max_position_embeddings"] = max(config["max_position_embeddings"], CONTEXT + 2048)
    if args.impl == "reference":
        return reference_main(args)

    import torch
    from vosti_b200 import Engine
    from vosti_b200.config import model_spec_from_config
    from vosti_b200.models import expected_weights
    from vosti_b200.weights import draw_tensors

    peaks, peak_kind = load_peaks()
    name, config = SIZES[args.size]
    config = dict(config)
    layers_full = config["num_hidden_layers"]
    if args.layers:
        config["num_hidden_layers"] = args.layers
    spec = model_spec_from_config(config)
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    tensors = draw_tensors(expected_weights(spec), seed=0, device=device, dtype=torch.bfloat16)
    L, H = config["num_hidden_layers"], config["hidden_size"]
    nq, nkv, d, I, V = (config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"],
                        config["intermediate_size"], config["vocab_size"])
    shape = {"model": name, "layers": L, "layers_full": layers_full, "hidden": H, "heads": nq, "kv_heads": nkv,
             "head_dim": d, "intermediate": I, "vocab": V}

    if args.workload == "mixed":
        num_blocks = 32 * ((3072 + 512 + PAGE) // PAGE) + 8
        engine = Engine(spec=spec, tensors=tensors, dtype="bfloat16", device="cuda:0", num_blocks=num_blocks,
                        block_size=PAGE, max_num_seqs=32, max_num_batched_tokens=4096, enable_prefix_caching=True,
                        cuda_graphs=not args.no_cuda_graphs, batch_invariant=args.batch_invariant,
                        async_scheduling=not args.sync_scheduling, consume_tensors=True)
        del tensors
        torch.cuda.empty_cache()
        mixed_run(engine, config, seed=4, requests=4)            # warm the kernels and the graphs' first shapes
        sampler = ClockSampler()
        sampler.start()
        run = mixed_run(engine, config, seed=5)
        clocks = sampler.stop()
        line = {
            "metric": f"generated tok/s, mixed continuous batch ({name})", "value": round(run["generated"] / run["wall_s"], 1),
            "unit": "tok/s", "n_gpus": 1, "steps": run["steps"], "warmup": 0,
            "ms_per_step": round(run["wall_s"] * 1e3 / max(run["steps"], 1), 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: random token ids, random-init weights", "impl": "ours",
            "config": {**shape, "global_batch": 32, "seq_len": 3072, "page_size": PAGE, "parallelism": "1 GPU",
                       "workload": "32 requests, prompts U[64,3072], 128-512 new tokens, Poisson arrivals at 16/s, "
                                   "half share a 1,024-token prefix", "peaks": peak_kind},
            "mixed": {k: (round(v, 4) if isinstance(v, float) else v) for k, v in run.items()},
            "clocks": clocks,
        }
        print(json.dumps(line))
        return 0

    max_batch = args.batch if args.no_points else max(args.batch, 64)
    tokens_per_request = CONTEXT + 2 * DECODE_STEPS + 128     # prompt, both timed regions, warm-up and slack
    num_blocks = max_batch * ((tokens_per_request + PAGE - 1) // PAGE) + 8
    engine = Engine(spec=spec, tensors=tensors, dtype="bfloat16", device="cuda:0", num_blocks=num_blocks,
                    block_size=PAGE, max_num_seqs=max_batch, max_num_batched_tokens=2 * CONTEXT,
                    enable_prefix_caching=False, cuda_graphs=not args.no_cuda_graphs,
                    batch_invariant=args.batch_invariant, async_scheduling=not args.sync_scheduling,
                    consume_tensors=True)
    del tensors
    torch.cuda.empty_cache()
    weight_bytes = engine.runner.model.weight_bytes()
    assert abs(weight_bytes - closed_form_weight_bytes(config)) <= 0.002 * weight_bytes, \
        (weight_bytes, closed_form_weight_bytes(config))
    kv_bytes_per_token = engine.runner.cache.bytes_per_token()

    prefill_ms = float("nan") if args.no_prefill else prefill_run(engine, 5, seed=11)
    main_run = decode_run(engine, args.batch, args.steps, args.warmup, seed=21, sample_clocks=True,
                          least_repeats=args.repeats)
    points = {}
    if not args.no_points:
        for batch in (1, 64):
            run = decode_run(engine, batch, max(8, args.steps // 2), 3, seed=31 + batch, least_repeats=3)
            points[f"decode_b{batch}"] = round(batch * 1e3 / run["device_ms"], 1)

    prefill_tflops = flops_of_prefill(config, CONTEXT) / (prefill_ms * 1e-3) / 1e12
    step_bytes = weight_bytes + args.batch * main_run["context"] * kv_bytes_per_token
    achieved_gbs = step_bytes / (main_run["device_ms"] * 1e-3) / 1e9

    value = args.batch * 1e3 / main_run["device_ms"]
    line = {
        "metric": f"decode tok/s at batch {args.batch} ({name}, context {CONTEXT})", "value": round(value, 1),
        "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["device_ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random token ids, random-init weights",
        "impl": "ours",
        "config": {**shape, "global_batch": args.batch, "seq_len": CONTEXT, "page_size": PAGE, "parallelism": "1 GPU",
                   "invariance": args.batch_invariant, "scheduling": "sync" if args.sync_scheduling else "async",
                   "repeats": main_run["repeats"], "l2": "inputs larger than L2 (weights read every step)",
                   "peaks": peak_kind},
        "e2e": {"value": round(args.batch * 1e3 / main_run["wall_ms"], 1), "unit": "tok/s",
                "h2d_bytes_per_step": main_run["h2d"], "d2h_bytes_per_step": main_run["d2h"]},
        "gpu_launches": main_run["launches"],
        "clocks": main_run["clocks"],
        "prefill": {"value": round(CONTEXT * 1e3 / prefill_ms, 1), "tokens": CONTEXT, "ms": round(prefill_ms, 3),
                    "frac": round(prefill_tflops / peaks["bf16_tflops"], 4),
                    "frac_of_sustained": round(prefill_tflops / peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved_gbs / peaks["hbm_gbs"], 4), "bytes_per_step": int(step_bytes),
                     "weight_bytes": int(weight_bytes), "kv_bytes": int(step_bytes - weight_bytes)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
