"""Schedules that need more than one mechanism at once: CUDA-graph replay across the
buckets its graphs are keyed by, prompts that start on published (reused) pages against the
plain logits, reuse together with portions, async scheduling, eviction and preemption, other
page sizes end to end, and a request that fills the model's last position."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import replay_util as R
from vosti_b200.engine.batch import StepEntry

pytestmark = pytest.mark.gpu


def check_greedy(plain_model, prompt, generated, dtype):
    """Every generated token is the plain model's best at its place, up to the dtype's
    rounding; the plain logits of the whole final sequence are computed once."""
    config, W = plain_model
    logits = plain.forward_logits(config, W, list(prompt) + list(generated)).double()
    tol = R.TOLERANCE[dtype]
    for index, token in enumerate(generated):
        row = logits[len(prompt) + index - 1]
        scale = max(1.0, float(row.abs().max()))
        assert float(row.max() - row[token]) <= 2 * tol * scale, (index, token, int(row.argmax()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuda_graphs_across_the_table_width_and_key_length_buckets(model_dirs, plain_models, dtype):
    """Decode graphs are keyed by the block-table width rounded up to 32 pages and the key
    length rounded up to 512: a 400-token prompt with 200 decoded tokens (pages of 16) crosses
    both, next to a short request that finishes meanwhile (the batch size changes too). Graphs
    on and off give the same tokens, and they are the plain model's."""
    from vosti_b200 import Engine
    from vosti_b200.engine import graphs as G
    path, config, page = model_dirs["c"]
    assert page * G.PAGES_BUCKET == 512 == G.KV_BUCKET and config["max_position_embeddings"] >= 600
    prompts = [R.random_tokens(config["vocab_size"], 400, seed=77), R.random_tokens(config["vocab_size"], 30, seed=78)]
    outs = []
    for graphs in (False, True):
        engine = Engine(path, dtype=dtype, num_blocks=64, block_size=page, max_num_seqs=2, max_num_batched_tokens=512,
                        cuda_graphs=graphs, async_scheduling=graphs)
        out = [[], []]
        engine.add_request(0, prompts[0], 200, None, True)
        engine.add_request(1, prompts[1], 60, None, True)
        while engine.has_unfinished():
            for rid, token in engine.step().items():
                out[rid].append(token)
        outs.append(out)
        if graphs:
            keys = set(engine.graphs.graphs)
            assert {k[2] for k in keys} == {32, 64} and {k[3] for k in keys} == {512, 1024}   # both buckets, both sides
            assert {k[0] for k in keys} == {1, 2} and engine.graphs.replays > 150
        engine.runner.cache.check()
    assert [len(o) for o in outs[1]] == [200, 60]
    assert outs[0] == outs[1]
    for prompt, out in zip(prompts, outs[1]):
        check_greedy(plain_models["c"], prompt, out, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_prompt_that_starts_on_published_pages_has_the_plain_logits(model_dirs, plain_models, dtype):
    """Prefix reuse against the plain implementation, logit by logit: the second prompt shares
    five pages with the first and computes only what follows them; after so many other pages
    were taken that the published ones were evicted, the same prompt is computed whole again.
    All three give the plain model's logits."""
    from vosti_b200.engine.runner import ModelRunner
    path, config, page = model_dirs["b"]
    cfg, W = plain_models["b"]
    vocab = config["vocab_size"]
    shared = R.random_tokens(vocab, 5 * page + 3, seed=21)
    first = shared + R.random_tokens(vocab, 20, seed=22)
    second = shared[:5 * page] + R.random_tokens(vocab, 27, seed=23)          # the same five pages, then its own
    runner = ModelRunner(path, dtype=dtype, num_pages=16, page_size=page, max_requests=2, prefix_reuse=True)
    tol = R.TOLERANCE[dtype]

    def run(rid, tokens, expect_reused):
        runner.begin(rid, tokens)
        start = runner.cache.length(rid)
        assert start == expect_reused * page
        logits = runner.step([StepEntry(rid, tokens[start:], list(range(len(tokens) - start)))]).cpu().numpy()
        want = plain.forward_logits(cfg, W, tokens).numpy()
        err = np.abs(logits - want[start:]).max() / max(1.0, np.abs(want).max())
        assert err <= tol, (rid, err)
        runner.cache.publish(rid, tokens)
        runner.finish(rid)
        runner.check_status()
        runner.cache.check()
        return err

    run("first", first, 0)
    run("second", second, 5)
    assert runner.cache.reused_prefix_pages == 5
    pool = runner.cache.groups[0].pool
    # a long stranger takes the whole pool: the published pages are evicted to make room
    run("stranger", R.random_tokens(vocab, 16 * page - 2, seed=24), 0)
    assert pool.evictions > 0
    run("second-again", second, 0)
    # ...and what it published is found again, its own pages too: all but the page of its last token
    run("second-thrice", second, (len(second) - 1) // page)


def test_reuse_with_portions_async_eviction_and_preemption_in_one_workload(model_dirs, plain_models):
    """Everything at once, float32 so that tokens must be equal: prompts that share a prefix
    arrive over time, are cut into portions of one page, run under async scheduling with CUDA
    graphs, in a pool so small that published pages are evicted and running requests are
    preempted and recomputed. The tokens are those of a roomy engine without any of it."""
    from vosti_b200 import Engine
    path, config, page = model_dirs["b"]
    vocab = config["vocab_size"]
    shared = R.random_tokens(vocab, 4 * page, seed=31)
    prompts = [shared + R.random_tokens(vocab, n, seed=32 + n) for n in (5, 13, 2, 21)]
    prompts += [R.random_tokens(vocab, 37, seed=40), shared[:2 * page] + R.random_tokens(vocab, 9, seed=41)]
    arrivals = [0, 0, 6, 14, 20, 45]
    roomy = Engine(path, dtype="float32", num_blocks=256, block_size=page, max_num_seqs=6, enable_prefix_caching=False)
    want = roomy.generate(prompts, max_tokens=30)
    tight = Engine(path, dtype="float32", num_blocks=22, block_size=page, max_num_seqs=3, max_num_batched_tokens=64,
                   prefill_chunk_size=page, enable_prefix_caching=True, cuda_graphs=True, async_scheduling=True)
    got = tight.generate(prompts, max_tokens=30, arrival_steps=arrivals)
    assert got == want
    stats = tight.cache_stats()
    pool = tight.runner.cache.groups[0].pool
    assert stats["requests_with_reuse"] >= 2 and stats["preemptions"] >= 1 and pool.evictions >= 1
    assert tight.graphs.replays > 0
    tight.runner.cache.check()
    assert tight.runner.cache.available_pages() == 22
    for prompt, out in zip(prompts, got):
        check_greedy(plain_models["b"], prompt, out, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page", [("a", 32), ("c", 64), ("b", 64), ("c", 48)])
def test_replay_with_other_page_sizes(name, page, dtype, model_dirs, plain_models, tmp_path):
    """Portions and a mixed batch on reused pages with pages of 32, 48 and 64 tokens (64 is the
    reference's fixed page size), plus one request that runs to the model's last position:
    most of it in one step, the last 32 tokens one by one."""
    path, config, _ = model_dirs[name]
    limit = config["max_position_embeddings"]
    lengths = [37, limit // 4 + 1, limit // 2 + 3, 64, 70]
    requests = {f"r{i}": R.random_tokens(config["vocab_size"], n, seed=500 + 13 * i + page) for i, n in enumerate(lengths)}
    full = {"full": R.random_tokens(config["vocab_size"], limit, seed=600 + page)}
    steps, alias = [], {}
    for kind, make, reqs in (("portion", R.portion_steps, requests), ("mixed", lambda r: R.mixed_steps(r, seed=page), requests),
                             ("tail", R.tail_steps, full)):
        alias.update({f"{kind}-{rid}": rid for rid in reqs})
        steps.extend(make({f"{kind}-{rid}": tokens for rid, tokens in reqs.items()}))
    steps = R.number(steps)
    held, pool_tokens = {}, 0          # the most that live requests hold at any time, in whole pages
    for step in steps:
        for e in step["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        pool_tokens = max(pool_tokens, sum(-(-v // page) * page for v in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    assert pool_tokens < sum(-(-len(t) // page) * page for t in requests.values()) + limit      # pages are used again
    replayer = R.run_in_process(path, dtype, steps, pool_tokens, page, tmp_path)
    rows = R.collect(steps, tmp_path, config["vocab_size"])
    assert len(rows) == 2 * sum(len(t) for t in requests.values()) + limit
    worst = R.compare_with_plain(rows, {**requests, **full}, plain_models[name], dtype, alias=lambda rid: alias[rid])
    pool = replayer.runner.cache.groups[0].pool
    assert pool.available() == pool.num_pages
    print(f"{name} page {page} {dtype}: worst error {worst:.3e} of the largest logit")
    # one token more than the model has positions for is refused, and nothing is lost by it
    replayer.run_line({"step": 10 ** 6, "entries": [{"id": "over", "tokens": full["full"][:limit - 1], "want": []}], "end": []})
    with pytest.raises(ValueError, match="limit"):
        replayer.run_line({"step": 10 ** 6 + 1, "entries": [{"id": "over", "tokens": [1, 2], "want": [1]}], "end": []})
    replayer.run_line({"step": 10 ** 6 + 2, "entries": [{"id": "over", "tokens": [3], "want": [0]}], "end": ["over"]})
    replayer.runner.cache.check()
    assert pool.available() == pool.num_pages


def test_two_engines_of_one_process_may_differ_in_their_invariance_mode(model_dirs):
    """An engine applies its own mode before each of its steps: stepped in turns with an engine in
    the default mode, an engine with one order of arithmetic still gives every request the bits
    (here: the tokens at temperature 0.9, which any changed bit of a logit would soon change) it
    gives that request alone, prompts cut into portions and decoded in a batch of three."""
    from vosti_b200 import Engine, ops
    path, config, page = model_dirs["c"]
    prompts = [R.random_tokens(config["vocab_size"], n, seed=900 + n) for n in (70, 33, 120)]
    try:
        fixed = Engine(path, dtype="bfloat16", num_blocks=128, block_size=page, max_num_seqs=3, max_num_batched_tokens=48,
                       batch_invariant="full")
        plain_mode = Engine(path, dtype="bfloat16", num_blocks=128, block_size=page, max_num_seqs=3)
        assert ops.INVARIANCE == "off"                        # the engine made last set the mode last
        for i, p in enumerate(prompts):
            fixed.add_request(i, p, 40, None, True, temperature=0.9, seed=i)
            plain_mode.add_request(i, p, 40, None, True, temperature=0.9, seed=i)
        together = {i: [] for i in range(3)}
        while fixed.has_unfinished() or plain_mode.has_unfinished():
            busy = fixed.has_unfinished()
            for rid, token in fixed.step().items():
                together[rid].append(token)
            assert not busy or ops.INVARIANCE == "full"
            busy = plain_mode.has_unfinished()
            plain_mode.step()
            assert not busy or ops.INVARIANCE == "off"
        for i, p in enumerate(prompts):
            alone = Engine(path, dtype="bfloat16", num_blocks=128, block_size=page, max_num_seqs=1, batch_invariant="full")
            plain_mode.add_request(100 + i, p, 3, None, True)
            plain_mode.step()                                   # the other engine keeps running in between
            assert alone.generate([p], max_tokens=40, temperature=0.9, seeds=[i]) == [together[i]]
    finally:
        ops.set_invariance("off")
