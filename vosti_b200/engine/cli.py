"""Command line of the engine, in the manner of the reference's example driver
(examples/verus_engine_qwen3.rs, examples/support/engine_serving.rs:91-232,
engine_setup.rs:57-118, engine_benchmark.rs:44-88, output_tokens.rs:6-22).

The reference is configured by environment variables only; the same names keep their
meaning here, and every one also has a flag (the flag wins):

  MODEL_PATH                --model DIR        checkpoint folder (config.json + safetensors)
  CUDA_DEVICE               --device           default cuda:0
  VOSTI_PROMPT_IDS          --prompt-ids       comma-separated token ids (default "9707")
  VOSTI_MAX_TOKENS          --max-tokens       default 8
  VOSTI_IGNORE_EOS          --ignore-eos       presence switches EOS handling off
  VOSTI_NUM_BLOCKS          --num-blocks       cache pages, default 32
  VOSTI_MAX_SEQS            --max-seqs         rows per step, default: the batch
  VOSTI_MAX_BATCHED_TOKENS  --max-batched-tokens   default 4096
  VOSTI_OUTPUT_TOKENS       --output-tokens    file of "index<TAB>tok,tok,..." lines
  VOSTI_BENCH_INPUT         --bench-input      prepared requests: MAX_TOKENS<TAB>IDS[<TAB>ARRIVAL_STEP]
  VOSTI_BENCH_WARMUP_INPUT  --bench-warmup-input   a disjoint prepared workload run first
  VOSTI_ENGINE_STEP_TRACE   --step-trace       one JSON line per step
  VOSTI_CUDA_GRAPH          --cuda-graph       0/1: replay decode steps as CUDA graphs (default 1 here)

Added here: --dtype {bfloat16,float32} (VOSTI_DTYPE), --block-size (VOSTI_BLOCK_SIZE, the
reference's page size is the constant 64), --temperature, --seed, --chunk-size, and
--random-config FILE --random-seed N, which first writes a random-weights model folder to
--model. Prints MODEL_OUTPUT_TOKEN_IDS=[...] or, for a prepared workload, the BENCH and
CACHE_STATS lines.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path
from typing import List, Optional, Tuple


def _env(name: str, default=None):
    value = os.environ.get(name)
    return default if value is None else value


def parse_ids(text: str, what: str) -> List[int]:
    ids = []
    for part in text.split(","):
        part = part.strip()
        if part:
            if not part.lstrip("-").isdigit():
                raise SystemExit(f"{what} contains non-integer {part!r}")
            ids.append(int(part))
    if not ids:
        raise SystemExit(f"{what} must be nonempty")
    return ids


def read_prepared_requests(path: str) -> List[Tuple[int, List[int], int]]:
    """Lines MAX_TOKENS<TAB>IDS[<TAB>ARRIVAL_STEP]; blank lines and # comments are skipped."""
    requests = []
    for number, raw in enumerate(Path(path).read_text().splitlines(), 1):
        line = raw.strip()
        if not line or line.startswith("#"):
            continue
        fields = line.split("\t")
        if len(fields) not in (2, 3):
            raise SystemExit(f"{path}:{number}: expected MAX_TOKENS<TAB>IDS[<TAB>ARRIVAL_STEP]")
        max_tokens = int(fields[0])
        if max_tokens <= 0:
            raise SystemExit(f"{path}:{number}: MAX_TOKENS must be positive")
        arrival = int(fields[2]) if len(fields) == 3 else 0
        requests.append((max_tokens, parse_ids(fields[1], f"{path}:{number}"), arrival))
    if not requests:
        raise SystemExit(f"{path}: no requests")
    return requests


def write_outputs(path: str, outputs: List[List[int]]) -> None:
    with open(path, "w") as handle:
        for index, tokens in enumerate(outputs):
            handle.write(f"{index}\t{','.join(str(t) for t in tokens)}\n")


def checkpoint_eos_token_ids(model_dir: str) -> List[int]:
    """EOS ids of the checkpoint: generation_config.json's eos_token_id (an id or a list of
    up to three), else config.json's (python/vosti_kernels/serving_workload.py:78-110)."""
    for name in ("generation_config.json", "config.json"):
        path = Path(model_dir) / name
        if path.is_file():
            value = json.loads(path.read_text()).get("eos_token_id")
            if isinstance(value, int) and not isinstance(value, bool):
                return [value]
            if isinstance(value, list) and value and all(isinstance(v, int) for v in value):
                return value[:3]
    return []


def run_workload(engine, requests, eos, ignore_eos, temperature, seed, first_id):
    """Run prepared requests with their arrival steps; returns outputs and statistics."""
    import torch

    prompts = [ids for _, ids, _ in requests]
    arrivals = [a for _, _, a in requests]
    torch.cuda.synchronize()
    started = time.perf_counter()
    pending = sorted(range(len(requests)), key=lambda i: (arrivals[i], i))
    outputs = {first_id + i: [] for i in range(len(requests))}
    step = 0
    while pending or engine.has_unfinished():
        while pending and arrivals[pending[0]] <= step:
            i = pending.pop(0)
            status = engine.add_request(first_id + i, prompts[i], requests[i][0], eos or None,
                                        ignore_eos or not eos, temperature, seed + i)
            if status.value != "accepted":
                raise SystemExit(f"request {i} was not accepted: {status.value}")
        for rid, token in engine.step().items():
            outputs[rid].append(token)
        step += 1
    torch.cuda.synchronize()
    wall = time.perf_counter() - started
    outs = [outputs[first_id + i] for i in range(len(requests))]
    return outs, {"prompt_tokens": sum(len(p) for p in prompts), "output_tokens": sum(len(o) for o in outs),
                  "wall_s": wall}


def main(argv: Optional[List[str]] = None) -> int:
    parser = argparse.ArgumentParser(prog="vosti_engine_qwen3", description=__doc__,
                                     formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument("--model", default=_env("MODEL_PATH"))
    parser.add_argument("--device", default=_env("CUDA_DEVICE", "cuda:0"))
    parser.add_argument("--dtype", default=_env("VOSTI_DTYPE", "bfloat16"), choices=["bfloat16", "float32"])
    parser.add_argument("--prompt-ids", default=_env("VOSTI_PROMPT_IDS", "9707"))
    parser.add_argument("--max-tokens", type=int, default=int(_env("VOSTI_MAX_TOKENS", 8)))
    parser.add_argument("--ignore-eos", action="store_true", default="VOSTI_IGNORE_EOS" in os.environ)
    parser.add_argument("--num-blocks", type=int, default=int(_env("VOSTI_NUM_BLOCKS", 32)))
    parser.add_argument("--block-size", type=int, default=int(_env("VOSTI_BLOCK_SIZE", 16)))
    parser.add_argument("--max-seqs", type=int, default=int(_env("VOSTI_MAX_SEQS", 0)))
    parser.add_argument("--max-batched-tokens", type=int, default=int(_env("VOSTI_MAX_BATCHED_TOKENS", 4096)))
    parser.add_argument("--chunk-size", type=int, default=int(_env("VOSTI_CHUNK_SIZE", 0)))
    parser.add_argument("--temperature", type=float, default=float(_env("VOSTI_TEMPERATURE", 0.0)))
    parser.add_argument("--seed", type=int, default=int(_env("VOSTI_SEED", 0)))
    parser.add_argument("--output-tokens", default=_env("VOSTI_OUTPUT_TOKENS"))
    parser.add_argument("--bench-input", default=_env("VOSTI_BENCH_INPUT"))
    parser.add_argument("--bench-warmup-input", default=_env("VOSTI_BENCH_WARMUP_INPUT"))
    parser.add_argument("--step-trace", default=_env("VOSTI_ENGINE_STEP_TRACE"))
    parser.add_argument("--no-prefix-caching", action="store_true")
    parser.add_argument("--cuda-graph", type=int, choices=[0, 1], default=int(_env("VOSTI_CUDA_GRAPH", 1)))
    parser.add_argument("--async-scheduling", type=int, choices=[0, 1], default=int(_env("VOSTI_ASYNC_SCHEDULING", 1)),
                        help="launch the next step before the last one's tokens are read (1, default) or after (0)")
    parser.add_argument("--batch-invariant", nargs="?", const="full", choices=["off", "decode", "full"],
                        default={"0": "off", "1": "full"}.get(_env("VOSTI_BATCH_INVARIANT", "off"),
                                                              _env("VOSTI_BATCH_INVARIANT", "off")),
                        help="full: a token's bits do not depend on how the work is cut into steps and batches "
                             "(slower decoding); decode: decode steps of up to 64 rows do not depend on the batch")
    parser.add_argument("--random-config", help="config.json to draw a random-weights model from")
    parser.add_argument("--random-seed", type=int, default=0)
    args = parser.parse_args(argv)

    if not args.model or not args.model.strip():
        raise SystemExit("MODEL_PATH (or --model) must name a local model checkpoint directory")
    if args.max_tokens <= 0:
        raise SystemExit("VOSTI_MAX_TOKENS must be positive")
    if args.random_config:
        from ..weights import write_random_model
        write_random_model(args.model, json.loads(Path(args.random_config).read_text()), args.random_seed)

    from .engine import Engine

    prepared = read_prepared_requests(args.bench_input) if args.bench_input else None
    batch = len(prepared) if prepared else 1
    max_seqs = args.max_seqs or batch
    if max_seqs <= 0 or args.max_batched_tokens <= 0:
        raise SystemExit("VOSTI_MAX_SEQS and VOSTI_MAX_BATCHED_TOKENS must be positive")
    eos = checkpoint_eos_token_ids(args.model)
    engine = Engine(args.model, dtype=args.dtype, device=args.device, num_blocks=args.num_blocks,
                    block_size=args.block_size, max_num_seqs=max_seqs,
                    max_num_batched_tokens=args.max_batched_tokens, prefill_chunk_size=args.chunk_size,
                    enable_prefix_caching=not args.no_prefix_caching, step_trace=args.step_trace,
                    cuda_graphs=bool(args.cuda_graph), batch_invariant=args.batch_invariant,
                    async_scheduling=bool(args.async_scheduling))
    print(f"MODEL_RUNTIME architecture={engine.runner.spec.architecture} dtype={args.dtype} "
          f"device={args.device}", flush=True)

    if prepared:
        first_id = 0
        if args.bench_warmup_input:
            warmup = read_prepared_requests(args.bench_warmup_input)
            _, stats = run_workload(engine, warmup, eos, args.ignore_eos, args.temperature, args.seed, 0)
            print(f"WARMUP batch={len(warmup)} prompt_tokens={stats['prompt_tokens']} "
                  f"output_tokens={stats['output_tokens']} wall_s={stats['wall_s']:.9f}")
            print("WARMUP_CACHE_STATS " + json.dumps(engine.cache_stats(), separators=(",", ":")))
            first_id = len(warmup)
        before = engine.cache_stats()
        outputs, stats = run_workload(engine, prepared, eos, args.ignore_eos, args.temperature, args.seed, first_id)
        after = engine.cache_stats()
        if args.output_tokens:
            write_outputs(args.output_tokens, outputs)
        print(f"BENCH batch={len(prepared)} prompt_tokens={stats['prompt_tokens']} "
              f"output_tokens={stats['output_tokens']} wall_s={stats['wall_s']:.9f} "
              f"tok_s={stats['output_tokens'] / stats['wall_s']:.6f}")
        print("CACHE_STATS " + json.dumps({k: after[k] - before[k] for k in after}, separators=(",", ":")))
        return 0

    prompt = parse_ids(args.prompt_ids, "VOSTI_PROMPT_IDS")
    status = engine.add_request(0, prompt, args.max_tokens, eos or None, args.ignore_eos or not eos,
                                args.temperature, args.seed)
    if status.value != "accepted":
        raise SystemExit(f"invalid request: {status.value}")
    output: List[int] = []
    for _ in range(len(prompt) + args.max_tokens + 4):
        if not engine.has_unfinished():
            break
        emitted = engine.step()
        if 0 in emitted:
            output.append(emitted[0])
    if engine.has_unfinished():
        raise SystemExit("request did not finish within the conservative step limit")
    if args.output_tokens:
        write_outputs(args.output_tokens, [output])
    print(f"MODEL_OUTPUT_TOKEN_IDS={output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
