"""The engine at the benchmark model's layer sizes (hidden 4096, 32 query / 8 kv heads of
128, intermediate 12288) and at the next larger size of the family (hidden 5120, 40 query /
8 kv heads: five query heads per kv head, intermediate 17408), with two layers and a smaller
vocabulary that is no power of two, against the plain implementation: a whole prompt, a
decoded tail and portions, in float32 and bfloat16. This is where the kernels meet the tile
sizes they are tuned for, and sizes that divide none of them."""
import pytest
import torch

import plain_qwen3 as plain
import replay_util as R
from tiny_configs import _config

pytestmark = pytest.mark.gpu

WIDE = _config(num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=12288, vocab_size=20011, rope_theta=1000000.0, rms_norm_eps=1e-6,
               tie_word_embeddings=False, max_position_embeddings=4096)


WIDER = _config(num_hidden_layers=2, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
                intermediate_size=17408, vocab_size=10007, rope_theta=1000000.0, rms_norm_eps=1e-6,
                tie_word_embeddings=False, max_position_embeddings=4096)
CONFIGS = {"8b": WIDE, "14b": WIDER}


@pytest.fixture(scope="module", params=["8b", "14b"])
def wide_model(request, tmp_path_factory):
    from vosti_b200.weights import write_random_model
    config = CONFIGS[request.param]
    folder = tmp_path_factory.mktemp("wide_" + request.param)
    write_random_model(folder, config, seed=3)
    return str(folder), plain.load_model(folder), config


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_benchmark_layer_sizes(wide_model, dtype, tmp_path):
    path, plain_model, WIDE = wide_model
    requests = {"p": R.random_tokens(WIDE["vocab_size"], 333, seed=9), "q": R.random_tokens(WIDE["vocab_size"], 150, seed=10)}
    steps, alias = [], {}
    for kind, make in (("whole", R.whole_steps), ("tail", R.tail_steps),
                       ("portion", lambda reqs: R.portion_steps(reqs, sizes=(130, 2, 64, 7, 200))),
                       ("mixed", lambda reqs: R.mixed_steps(reqs, seed=5))):
        renamed = {f"{kind}-{rid}": tokens for rid, tokens in requests.items()}
        alias.update({f"{kind}-{rid}": rid for rid in requests})
        steps.extend(make(renamed))
    steps = R.number(steps)
    R.run_in_process(path, dtype, steps, R.max_live_tokens(steps), 16, tmp_path)
    rows = R.collect(steps, tmp_path, WIDE["vocab_size"])
    assert len(rows) == 4 * sum(len(t) for t in requests.values())
    worst = R.compare_with_plain(rows, requests, plain_model, dtype, alias=lambda rid: alias[rid])
    print(f"benchmark layer sizes, {dtype}: worst error {worst:.3e} of the largest logit")


def test_bfloat16_bits_do_not_depend_on_the_cut_in_fixed_order(wide_model, tmp_path):
    """At the benchmark layer sizes: with batch_invariant="full" a position's logits are the
    same bits for a whole prompt (the wide product kernel, 128-row attention tiles), a decoded
    tail (one-token steps), portions and a mixed batch."""
    import numpy as np
    from vosti_b200 import ops
    path, _, config = wide_model
    vocab = config["vocab_size"]
    requests = {"p": R.random_tokens(vocab, 333, seed=9), "q": R.random_tokens(vocab, 150, seed=10),
                "r": R.random_tokens(vocab, 70, seed=11)}
    kinds = {"whole": R.whole_steps, "tail": R.tail_steps,
             "portion": lambda reqs: R.portion_steps(reqs, sizes=(130, 2, 64, 7, 200)),
             "mixed": lambda reqs: R.mixed_steps(reqs, seed=5)}
    steps = []
    for kind, make in kinds.items():
        steps.extend(make({f"{kind}-{rid}": tokens for rid, tokens in requests.items()}))
    steps = R.number(steps)
    try:
        R.run_in_process(path, "bfloat16", steps, R.max_live_tokens(steps), 16, tmp_path, batch_invariant="full")
    finally:
        ops.set_invariance("off")
    rows = R.collect(steps, tmp_path, vocab)
    for rid, tokens in requests.items():
        for position in range(len(tokens)):
            whole = rows[(f"whole-{rid}", position)]
            for kind in ("tail", "portion", "mixed"):
                assert np.array_equal(whole, rows[(f"{kind}-{rid}", position)]), \
                    f"{rid} position {position}: {kind} differs from whole"
    # the comparison can fail: the default mode, which cuts every launch to fit its shape, agrees
    # across these cuts up to rounding only
    default_steps = [s for s in steps if s["entries"][0]["id"].startswith(("whole-", "tail-"))]
    R.run_in_process(path, "bfloat16", default_steps, R.max_live_tokens(default_steps), 16, tmp_path / "default")
    default_rows = R.collect(default_steps, tmp_path / "default", vocab)
    last = len(requests["p"]) - 1
    assert not np.array_equal(default_rows[("whole-p", last)], default_rows[("tail-p", last)])


def _decode_trace(requests, prompt_len, alone=None):
    """Prompts one by one (each whole, nothing wanted), then every request's remaining tokens
    one per step, all requests side by side; with `alone` only that request takes part."""
    names = [alone] if alone else list(requests)
    steps = [{"entries": [{"id": rid, "tokens": requests[rid][:prompt_len[rid]], "want": []}], "end": []} for rid in names]
    longest = max(len(requests[rid]) - prompt_len[rid] for rid in names)
    for i in range(longest):
        entries, ended = [], []
        for rid in names:
            at = prompt_len[rid] + i
            if at < len(requests[rid]):
                entries.append({"id": rid, "tokens": [requests[rid][at]], "want": [0]})
                if at == len(requests[rid]) - 1:
                    ended.append(rid)
        steps.append({"entries": entries, "end": ended})
    return R.number(steps)


def test_decode_bits_do_not_depend_on_the_batch_when_the_segment_length_is_pinned(wide_model, tmp_path):
    """With the decode attention's segment length fixed, a request decoded alone and decoded
    beside seven others (other lengths, another batch size, another table width) gives the same
    logits bit for bit: every other reduction order of a decode step depends on the weight's
    shape only."""
    import numpy as np
    path, _, config = wide_model
    vocab = config["vocab_size"]
    lengths = {"a": (300, 24), "b": (17, 30), "c": (129, 12), "d": (64, 24), "e": (500, 24), "f": (33, 8), "g": (260, 24),
               "h": (2, 20)}
    requests = {rid: R.random_tokens(vocab, p + n, seed=40 + i) for i, (rid, (p, n)) in enumerate(lengths.items())}
    prompt_len = {rid: p for rid, (p, n) in lengths.items()}
    together = _decode_trace(requests, prompt_len)
    alone = _decode_trace(requests, prompt_len, alone="a")
    R.run_in_process(path, "bfloat16", together, R.max_live_tokens(together), 16, tmp_path / "together", batch_invariant="decode")
    R.run_in_process(path, "bfloat16", alone, R.max_live_tokens(alone), 16, tmp_path / "alone", batch_invariant="decode")
    from vosti_b200 import ops
    ops.set_invariance("off")
    rows_together = R.collect(together, tmp_path / "together", vocab)
    rows_alone = R.collect(alone, tmp_path / "alone", vocab)
    assert len(rows_alone) == lengths["a"][1]
    for key, row in rows_alone.items():
        assert np.array_equal(row, rows_together[key]), f"position {key[1]} differs between the two batches"


def test_generation_does_not_depend_on_the_batch_with_batch_invariant(wide_model):
    """Through the entry point: the same prompt gives the same tokens, greedy and sampled,
    alone and among seven others (CUDA graphs on), with one order of arithmetic everywhere. The
    second run finds its prompt's pages in the prefix cache and computes only the last portion:
    in this mode that changes nothing either. The "decode" mode promises the same for decode
    steps only, so it is run with prefix reuse off."""
    from vosti_b200 import Engine, ops
    path, _, config = wide_model
    vocab = config["vocab_size"]
    prompts = [R.random_tokens(vocab, n, seed=70 + n) for n in (200, 3, 77, 130, 16, 301, 64, 9)]
    seeds = list(range(8))
    try:
        for mode, reuse in (("full", True), ("decode", False)):
            engine = Engine(path, dtype="bfloat16", num_blocks=400, block_size=16, max_num_seqs=8,
                            batch_invariant=mode, enable_prefix_caching=reuse)
            for temperature in (0.0, 0.8):
                together = engine.generate(prompts, max_tokens=40, temperature=temperature, seeds=seeds)
                alone = engine.generate(prompts[:1], max_tokens=40, temperature=temperature, seeds=seeds[:1])
                assert alone[0] == together[0], (mode, temperature)
            if reuse:
                assert engine.cache_stats()["requests_with_reuse"] >= 1
            engine.runner.cache.check()
            del engine
    finally:
        ops.set_invariance("off")
