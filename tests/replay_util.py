"""Helpers of the replay tests: build traces, run them, compare with the plain model."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[1]

# Tolerances, fixed before the first GPU run. float32: summation order only.
# bfloat16: a few roundings to 8 bits per layer; the plain implementation with the
# reference's rounding points differs from its float32 self by about 0.3 % of the largest
# logit on these models, the bound is several times that.
TOLERANCE = {"float32": 2e-5, "bfloat16": 2e-2}


def random_tokens(vocab, length, seed):
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=gen).tolist()


def roundup64(n):
    return (n + 63) // 64 * 64


def whole_steps(requests):
    """Each request alone and whole: one step, every position wanted."""
    steps = []
    for rid, tokens in requests.items():
        steps.append({"entries": [{"id": rid, "tokens": tokens, "want": list(range(len(tokens)))}], "end": [rid]})
    return steps


def tail_steps(requests, tail=32):
    """Most of it in one step, the last `tail` tokens one by one."""
    steps = []
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"entries": [{"id": rid, "tokens": tokens[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(tokens)):
            steps.append({"entries": [{"id": rid, "tokens": [tokens[i]], "want": [0]}],
                          "end": [rid] if i == len(tokens) - 1 else []})
    return steps


def portion_steps(requests, sizes=(2, 7, 16, 3, 33, 2, 5, 17, 64, 2, 9)):
    """Portions of changing size, down to two tokens."""
    steps = []
    for n, (rid, tokens) in enumerate(requests.items()):
        at, k = 0, n
        while at < len(tokens):
            size = sizes[k % len(sizes)]
            k += 1
            left = len(tokens) - at
            if left - size == 1:        # never leave a single token as a "portion"
                size = left
            size = min(size, left)
            chunk = tokens[at:at + size]
            at += size
            steps.append({"entries": [{"id": rid, "tokens": chunk, "want": list(range(len(chunk)))}],
                          "end": [rid] if at == len(tokens) else []})
    return steps


def mixed_steps(requests, seed=0, max_live=4, prompt_share=0.6):
    """Up to `max_live` requests at a time: portions of some beside single decoded tokens
    of others; a request may sit a step out; finished requests give way to waiting ones."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live, steps = {}, []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, tokens = waiting.pop(0)
            live[rid] = {"tokens": tokens, "at": 0, "prompt": max(2, int(len(tokens) * prompt_share))}
        entries, ended = [], []
        for rid, st in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue
            left = len(st["tokens"]) - st["at"]
            if st["at"] < st["prompt"]:
                size = int(rng.integers(2, 24))
                size = min(size, st["prompt"] - st["at"], left)
                if st["prompt"] - st["at"] - size == 1:
                    size += 1
                size = min(size, left)
            else:
                size = 1
            chunk = st["tokens"][st["at"]:st["at"] + size]
            st["at"] += size
            entries.append({"id": rid, "tokens": chunk, "want": list(range(len(chunk)))})
            if st["at"] == len(st["tokens"]):
                ended.append(rid)
                del live[rid]
        if entries:
            steps.append({"entries": entries, "end": ended})
    return steps


def max_live_tokens(steps):
    """The --max-tokens a trace needs: the most that live requests hold at any time, each
    rounded up to a multiple of 64."""
    held, peak = {}, 0
    for step in steps:
        for e in step["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(roundup64(v) for v in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    return peak


def number(steps, start=0):
    return [dict(step=start + i, **s) for i, s in enumerate(steps)]


def run_in_process(model_dir, dtype, steps, max_tokens, page_size, out_dir, batch_invariant=False):
    """Replay through the package's TraceReplayer (what bin/trace_run wraps)."""
    from vosti_b200.engine.trace import TraceReplayer

    replayer = TraceReplayer(model_dir, dtype=dtype, out_dir=out_dir, max_tokens=max_tokens, page_size=page_size,
                             batch_invariant=batch_invariant)
    for record in steps:
        replayer.run_line(record)
    replayer.runner.cache.check()
    return replayer


def run_binary(model_dir, dtype, steps, max_tokens, out_dir, page_size=None, timeout=600):
    """Replay through bin/trace_run, one line at a time, waiting for each `done`."""
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens)]
    if page_size:
        cmd += ["--page-size", str(page_size)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for record in steps:
            proc.stdin.write(json.dumps(record) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {record['step']}", f"expected 'done {record['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=timeout) == 0
    finally:
        if proc.poll() is None:
            proc.kill()


def collect(steps, out_dir, vocab):
    """(request id, position) -> logits row, from the files a replay wrote."""
    rows, position = {}, {}
    for record in steps:
        wanted = sum(len(e["want"]) for e in record["entries"])
        path = Path(out_dir) / f"{record['step']}.f32"
        if wanted == 0:
            assert not path.exists()
            for e in record["entries"]:
                position[e["id"]] = position.get(e["id"], 0) + len(e["tokens"])
            continue
        data = np.fromfile(path, dtype="<f4")
        assert data.size == wanted * vocab, f"step {record['step']}: {data.size} floats for {wanted} rows"
        data = data.reshape(wanted, vocab)
        r = 0
        for e in record["entries"]:
            base = position.get(e["id"], 0)
            for w in e["want"]:
                rows[(e["id"], base + w)] = data[r]
                r += 1
            position[e["id"]] = base + len(e["tokens"])
        for rid in record["end"]:
            position.pop(rid, None)
    return rows


def compare_with_plain(rows, requests, plain_model, dtype, alias=None):
    """Every collected row against the plain implementation's logits of the whole sequence.
    Returns the largest error relative to the largest logit; on failure names the first
    wrong (request, position)."""
    import plain_qwen3 as plain

    config, W = plain_model
    worst = 0.0
    tol = TOLERANCE[dtype]
    reference = {}
    for (rid, pos), row in sorted(rows.items(), key=lambda kv: (str(kv[0][0]), kv[0][1])):
        base = alias(rid) if alias else rid
        if base not in reference:
            reference[base] = plain.forward_logits(config, W, requests[base]).numpy()
        ref = reference[base][pos]
        scale = max(1.0, float(np.abs(reference[base]).max()))
        err = float(np.abs(row - ref).max()) / scale
        assert np.isfinite(row).all(), f"request {rid} position {pos}: non-finite logits"
        assert err <= tol, (f"first wrong logits: request {rid} position {pos}: error {err:.3e} of the largest "
                            f"logit > {tol:.1e} ({dtype})")
        worst = max(worst, err)
    return worst
