"""Generation through the Python entry point and the command line, against the plain
implementation: greedy and temperature, alone and batched, portions beside decodes, long
decoding, the first tokens of a sequence, too few pages."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import replay_util as R

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def check_tokens(plain_model, prompt, generated, dtype, temperature=0.0, seed=0):
    """Each generated token is the plain model's choice given the same history. float32:
    greedy tokens are the argmax unless the two best logits are closer than float32
    round-off. bfloat16: the chosen token's logit is within the bfloat16 tolerance of the
    best. Temperature: the token's interval of the cumulative distribution holds u."""
    config, W = plain_model
    tol = R.TOLERANCE[dtype]
    history = list(prompt)
    for index, token in enumerate(generated):
        logits = plain.forward_logits(config, W, history)[-1].double()
        scale = max(1.0, float(logits.abs().max()))
        if temperature <= 0.0:
            assert float(logits.max() - logits[token]) <= 2 * tol * scale, (index, token, int(logits.argmax()))
        else:
            w = torch.exp((logits - logits.max()) / temperature)
            cdf = torch.cumsum(w, 0)
            u = plain.uniform(seed, index) * float(cdf[-1])
            low = float(cdf[token - 1]) if token > 0 else 0.0
            slack = 4 * tol * scale / temperature * float(cdf[-1])
            assert low - slack <= u <= float(cdf[token]) + slack, (index, token)
        history.append(token)


def engine_for(model_dirs, name, dtype, **kw):
    from vosti_b200 import Engine
    path, config, page = model_dirs[name]
    kw.setdefault("block_size", page)
    kw.setdefault("num_blocks", 256)
    kw.setdefault("max_num_seqs", 4)
    return Engine(path, dtype=dtype, **kw), config


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_config_a_workload_greedy(model_dirs, plain_models, dtype):
    """3 requests, prompts 5/17/33, 8 greedy tokens each."""
    engine, config = engine_for(model_dirs, "a", dtype)
    prompts = [R.random_tokens(config["vocab_size"], n, seed=n) for n in (5, 17, 33)]
    outputs = engine.generate(prompts, max_tokens=8)
    assert [len(o) for o in outputs] == [8, 8, 8]
    for prompt, out in zip(prompts, outputs):
        check_tokens(plain_models["a"], prompt, out, dtype)
    if dtype == "float32":
        config_, W = plain_models["a"]
        assert outputs == [plain.generate(config_, W, p, 8) for p in prompts]
    # one at a time gives the same tokens as batched
    for prompt, out in zip(prompts, outputs):
        alone, _ = engine_for(model_dirs, "a", dtype, max_num_seqs=1)
        assert alone.generate([prompt], max_tokens=8) == [out]
    assert engine.runner.cache.available_pages() == 256
    engine.runner.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_config_b_workload_temperature_in_portions(model_dirs, plain_models, dtype):
    """4 requests, prompts 1/9/40/70 prefilled in portions of 8 beside concurrent decodes,
    temperature 0.8 with seeds 0-3, 12 new tokens each."""
    engine, config = engine_for(model_dirs, "b", dtype, prefill_chunk_size=8)
    prompts = [R.random_tokens(config["vocab_size"], n, seed=40 + n) for n in (1, 9, 40, 70)]
    outputs = engine.generate(prompts, max_tokens=12, temperature=0.8, seeds=[0, 1, 2, 3], arrival_steps=[0, 0, 1, 3])
    assert [len(o) for o in outputs] == [12] * 4
    for i, (prompt, out) in enumerate(zip(prompts, outputs)):
        check_tokens(plain_models["b"], prompt, out, dtype, temperature=0.8, seed=i)
    # the same seeds alone and whole give the same tokens: sampling does not see the batch
    for i, prompt in enumerate(prompts):
        alone, _ = engine_for(model_dirs, "b", dtype, max_num_seqs=1)
        assert alone.generate([prompt], max_tokens=12, temperature=0.8, seeds=[i]) == [outputs[i]]
    other, _ = engine_for(model_dirs, "b", dtype, max_num_seqs=1)
    assert other.generate([prompts[2]], max_tokens=12, temperature=0.8, seeds=[99]) != [outputs[2]]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(model_dirs, plain_models, dtype):
    engine, config = engine_for(model_dirs, "c", dtype, max_num_seqs=3)
    prompts = [[7], [9, 200], R.random_tokens(config["vocab_size"], 40, seed=5)]
    outputs = engine.generate(prompts, max_tokens=150)
    for prompt, out in zip(prompts, outputs):
        assert len(out) == 150
        check_tokens(plain_models["c"], prompt, out, dtype)


def test_eos_stops_generation(model_dirs, plain_models):
    engine, config = engine_for(model_dirs, "b", "float32")
    prompt = R.random_tokens(config["vocab_size"], 12, seed=3)
    free_run = engine.generate([prompt], max_tokens=10)[0]
    stop = free_run[4]
    first = free_run.index(stop)
    again, _ = engine_for(model_dirs, "b", "float32")
    assert again.generate([prompt], max_tokens=10, eos_token_ids=[stop, 511])[0] == free_run[:first + 1]
    ignoring, _ = engine_for(model_dirs, "b", "float32")
    assert ignoring.generate([prompt], max_tokens=10, eos_token_ids=[stop], ignore_eos=True)[0] == free_run


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_too_few_pages_preempts_and_still_generates_the_same(model_dirs, plain_models, dtype):
    roomy, config = engine_for(model_dirs, "b", dtype, max_num_seqs=4)
    prompts = [R.random_tokens(config["vocab_size"], n, seed=70 + n) for n in (30, 41, 25, 38)]
    want = roomy.generate(prompts, max_tokens=40)
    tight, _ = engine_for(model_dirs, "b", dtype, max_num_seqs=4, num_blocks=26, enable_prefix_caching=False)
    got = tight.generate(prompts, max_tokens=40)
    assert tight.scheduler.preemptions > 0
    assert tight.runner.cache.available_pages() == 26
    if dtype == "float32":
        assert got == want
    for prompt, out in zip(prompts, got):
        check_tokens(plain_models["b"], prompt, out, dtype)


def test_prefix_reuse_gives_the_same_tokens(model_dirs):
    engine, config = engine_for(model_dirs, "b", "bfloat16", max_num_seqs=2)
    shared = R.random_tokens(config["vocab_size"], 48, seed=1)
    prompts = [shared + [5, 6, 7], shared + [9, 10]]
    cold = engine.generate([prompts[0]], max_tokens=6)
    warm = engine.generate([prompts[1]], max_tokens=6)
    stats = engine.cache_stats()
    assert stats["requests_with_reuse"] == 1 and stats["reused_prefix_blocks"] == 6
    fresh, _ = engine_for(model_dirs, "b", "bfloat16", max_num_seqs=2, enable_prefix_caching=False)
    assert fresh.generate([prompts[1]], max_tokens=6) == warm
    engine.runner.cache.check()


def test_command_line(model_dirs, plain_models, tmp_path):
    path, config, page = model_dirs["a"]
    prompt = R.random_tokens(config["vocab_size"], 9, seed=2)
    env = dict(os.environ, MODEL_PATH=path, VOSTI_PROMPT_IDS=",".join(map(str, prompt)), VOSTI_MAX_TOKENS="6",
               VOSTI_NUM_BLOCKS="8", VOSTI_DTYPE="float32", VOSTI_OUTPUT_TOKENS=str(tmp_path / "out.tsv"),
               VOSTI_ENGINE_STEP_TRACE=str(tmp_path / "trace.jsonl"))
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "vosti_engine_qwen3")], env=env, capture_output=True,
                          text=True, timeout=600)
    assert done.returncode == 0, done.stderr
    line = [l for l in done.stdout.splitlines() if l.startswith("MODEL_OUTPUT_TOKEN_IDS=")][0]
    tokens = [int(t) for t in line.split("=")[1].strip("[]").split(",")]
    cfg, W = plain_models["a"]
    assert tokens == plain.generate(cfg, W, prompt, 6)
    assert (tmp_path / "out.tsv").read_text() == "0\t" + ",".join(map(str, tokens)) + "\n"
    assert len((tmp_path / "trace.jsonl").read_text().splitlines()) == 6
    # a prepared workload with arrival steps
    (tmp_path / "bench.tsv").write_text("# max_tokens, ids, arrival\n4\t1,2,3\n3\t9,8,7,6,5\t2\n")
    (tmp_path / "warm.tsv").write_text("2\t4,4,4\n")
    env.update(VOSTI_BENCH_INPUT=str(tmp_path / "bench.tsv"), VOSTI_BENCH_WARMUP_INPUT=str(tmp_path / "warm.tsv"),
               VOSTI_NUM_BLOCKS="16")
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "vosti_engine_qwen3"), "--max-seqs", "2"], env=env,
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr
    assert "BENCH batch=2 prompt_tokens=8 output_tokens=7" in done.stdout and "CACHE_STATS" in done.stdout
    rows = (tmp_path / "out.tsv").read_text().splitlines()
    assert rows[0] == "0\t" + ",".join(map(str, plain.generate(cfg, W, [1, 2, 3], 4)))
    assert rows[1] == "1\t" + ",".join(map(str, plain.generate(cfg, W, [9, 8, 7, 6, 5], 3)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuda_graphs_change_nothing(model_dirs, dtype):
    """Decode steps replayed as CUDA graphs give the tokens of eager launches, across a
    change of batch size, temperature sampling and a growing block table."""
    path, config, page = model_dirs["c"]
    prompts = [R.random_tokens(config["vocab_size"], n, seed=200 + n) for n in (3, 50, 17)]
    outs = []
    for graphs in (False, True):
        from vosti_b200 import Engine
        engine = Engine(path, dtype=dtype, num_blocks=256, block_size=page, max_num_seqs=3, cuda_graphs=graphs)
        a = engine.generate(prompts, max_tokens=70, temperature=0.7, seeds=[1, 2, 3])
        b = engine.generate(prompts[:2], max_tokens=40)
        outs.append((a, b))
        if graphs:
            assert engine.graphs.captures >= 2 and engine.graphs.replays > 60
    assert outs[0] == outs[1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_async_scheduling_generates_the_same(model_dirs, plain_models, dtype):
    """Launching a step before the last one's tokens are read changes no token: prompts in
    portions beside decodes, temperature and greedy rows, staggered arrivals, CUDA graphs."""
    path, config, page = model_dirs["c"]
    from vosti_b200 import Engine
    prompts = [R.random_tokens(config["vocab_size"], n, seed=300 + n) for n in (3, 50, 17, 90, 33)]
    seeds = [4, 5, 6, 7, 8]
    outs = []
    for ahead in (False, True):
        engine = Engine(path, dtype=dtype, num_blocks=256, block_size=page, max_num_seqs=3, max_num_batched_tokens=48,
                        async_scheduling=ahead)
        a = engine.generate(prompts, max_tokens=50, temperature=0.7, seeds=seeds, arrival_steps=[0, 0, 3, 9, 30])
        b = engine.generate(prompts[:2], max_tokens=30)
        outs.append((a, b))
        assert not engine.has_unfinished()
        engine.runner.cache.check()
        if ahead:
            assert engine.graphs.replays > 20
    assert outs[0] == outs[1]
    for prompt, out in zip(prompts[:2], outs[1][1]):
        check_tokens(plain_models["c"], prompt, out, dtype)


def test_async_scheduling_with_eos_and_too_few_pages(model_dirs, plain_models):
    """The token that ends a request arrives after the next step is launched: the row the
    request still has there is dropped, and its pages come back. With so few pages that
    requests are preempted while their newest token is still on the device only."""
    from vosti_b200 import Engine
    path, config, page = model_dirs["b"]
    prompts = [R.random_tokens(config["vocab_size"], n, seed=70 + n) for n in (30, 41, 25, 38)]
    roomy = Engine(path, dtype="float32", num_blocks=256, block_size=page, max_num_seqs=4)
    free_run = roomy.generate(prompts, max_tokens=40)
    stops = [free_run[0][7], free_run[2][20]]
    want = roomy.generate(prompts, max_tokens=40, eos_token_ids=stops)
    assert any(len(out) < 40 for out in want)
    for blocks, reuse, eos, expected in ((256, True, stops, want), (40, False, stops, want), (26, False, None, free_run)):
        ahead = Engine(path, dtype="float32", num_blocks=blocks, block_size=page, max_num_seqs=4,
                       enable_prefix_caching=reuse, async_scheduling=True)
        got = ahead.generate(prompts, max_tokens=40, eos_token_ids=eos)
        assert got == expected, blocks
        assert not ahead.has_unfinished()
        ahead.runner.cache.check()
        assert reuse or ahead.runner.cache.available_pages() == blocks
        if blocks == 26:
            assert ahead.scheduler.preemptions > 0
    for prompt, out in zip(prompts, want):
        check_tokens(plain_models["b"], prompt, out, "float32")
