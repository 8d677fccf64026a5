"""Two wider configurations through the engine against the plain implementation.

The tiny configurations have widths below 512 and head sizes 16, 32 and 48, so their products
never split K and their attention runs on the mma.sync kernels. These two are wide enough
that the engine takes the kernels a full-size model takes: split-K products whose unsummed
splits go to the add + norm kernel and to the decode attention (head norm, rotation and
cache store inside it), the split product with the SiLU epilogue, and the tensor-memory
prefill attention at head sizes 128 and 64. They differ in every size: layers, width, heads
and groups, head size, intermediate width, vocabulary, eps, theta, tied head, page size.
"""
import numpy as np
import pytest
import torch

import replay_util as R
from tiny_configs import _config

pytestmark = pytest.mark.gpu

WIDE = {
    "w": (_config(num_hidden_layers=2, hidden_size=1024, num_attention_heads=8, num_key_value_heads=2,
                  head_dim=128, intermediate_size=1536, vocab_size=1031, rope_theta=1000000.0,
                  rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=768), 5, 16),
    "x": (_config(num_hidden_layers=3, hidden_size=768, num_attention_heads=12, num_key_value_heads=4,
                  head_dim=64, intermediate_size=2048 + 64, vocab_size=2003, rope_theta=10000.0,
                  rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=512), 6, 32),
}
LENGTHS = {"w": [41, 150, 333, 64, 257], "x": [9, 129, 200, 77, 310]}


@pytest.fixture(scope="module")
def wide_dirs(tmp_path_factory):
    from vosti_b200.weights import write_random_model
    out = {}
    for name, (config, seed, page) in WIDE.items():
        folder = tmp_path_factory.mktemp(f"wide_{name}")
        write_random_model(folder, config, seed)
        out[name] = (str(folder), config, page)
    return out


@pytest.fixture(scope="module")
def wide_plain(wide_dirs):
    import plain_qwen3 as plain
    return {name: plain.load_model(path) for name, (path, _, _) in wide_dirs.items()}


def _requests(name, config):
    return {f"r{i}": R.random_tokens(config["vocab_size"], n, seed=4000 + 13 * i + ord(name))
            for i, n in enumerate(LENGTHS[name])}


def test_the_wide_configurations_reach_the_full_size_kernels(wide_dirs):
    """The premise of this file: at these widths a product of a few tokens splits K, and the
    head sizes are the ones the tensor-memory attention takes."""
    from vosti_b200 import ops
    lib = ops.library()
    for name, (_, config, page) in wide_dirs.items():
        hidden, d = config["hidden_size"], config["head_dim"]
        qkv = (config["num_attention_heads"] + 2 * config["num_key_value_heads"]) * d
        assert lib.vosti_gemm_tc_splits(4, qkv, hidden) > 1
        assert lib.vosti_gemm_tc_splits(4, hidden, config["num_attention_heads"] * d) > 1
        assert lib.vosti_gemm_tc_splits(4, hidden, config["intermediate_size"]) > 1
        assert lib.vosti_attention_prefill_tc_supported(d, page) == 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["w", "x"])
def test_wide_replay_all_cuts(name, dtype, wide_dirs, wide_plain, tmp_path):
    """Whole, with a decoded tail, in portions down to two tokens, and mixed on reused pages."""
    path, config, page = wide_dirs[name]
    requests = _requests(name, config)
    steps, alias = [], {}
    kinds = {"whole": R.whole_steps, "tail": R.tail_steps, "portion": R.portion_steps,
             "mixed": lambda reqs: R.mixed_steps(reqs, seed=5)}
    for kind, make in kinds.items():
        renamed = {f"{kind}-{rid}": tokens for rid, tokens in requests.items()}
        for rid in requests:
            alias[f"{kind}-{rid}"] = rid
        steps.extend(make(renamed))
    steps = R.number(steps)
    replayer = R.run_in_process(path, dtype, steps, R.max_live_tokens(steps), page, tmp_path)
    rows = R.collect(steps, tmp_path, config["vocab_size"])
    assert len(rows) == 4 * sum(len(t) for t in requests.values())
    worst = R.compare_with_plain(rows, requests, wide_plain[name], dtype, alias=lambda rid: alias[rid])
    pool = replayer.runner.cache.groups[0].pool
    assert pool.available() == pool.num_pages, "pages were lost"
    print(f"{name} {dtype}: worst error {worst:.3e} of the largest logit")
    if dtype == "bfloat16":
        # against the reference's own rounding points (every primitive's output stored in bfloat16,
        # emulated by the plain implementation): the engine must be about as close to the float32
        # model as that is
        import plain_qwen3 as plain
        cfg, W = wide_plain[name]
        emulated = 0.0
        for rid, tokens in requests.items():
            exact = plain.forward_logits(cfg, W, tokens).numpy()
            rounded = plain.forward_logits(cfg, W, tokens, round_to=torch.bfloat16).numpy()
            emulated = max(emulated, float(np.abs(rounded - exact).max()) / max(1.0, float(np.abs(exact).max())))
        print(f"{name}: the reference's rounding points give {emulated:.3e}")
        assert worst <= 1.5 * emulated


@pytest.mark.parametrize("name", ["w", "x"])
def test_wide_decode_steps_use_the_unsummed_splits(name, wide_dirs, monkeypatch):
    """A decode step of the wide model hands unsummed splits to the fused attention and to the
    add + norm kernel (counted here), and its greedy tokens are the plain implementation's
    float32 argmax wherever that argmax is clear (rounding may flip a near tie elsewhere)."""
    import plain_qwen3 as plain
    from vosti_b200 import Engine, ops
    path, config, page = wide_dirs[name]
    calls = {"fused": 0, "partial_norm": 0}
    fused, norm = ops.attention_decode_fused, ops.rmsnorm

    def counted_fused(*args, **kwargs):
        calls["fused"] += 1
        return fused(*args, **kwargs)

    def counted_norm(x, *args, **kwargs):
        if isinstance(x, ops.PartialSum):
            calls["partial_norm"] += 1
        return norm(x, *args, **kwargs)

    monkeypatch.setattr(ops, "attention_decode_fused", counted_fused)
    monkeypatch.setattr(ops, "rmsnorm", counted_norm)
    prompts = [R.random_tokens(config["vocab_size"], n, seed=77 + n) for n in (19, 64, 130)]
    new = 24
    engine = Engine(path, dtype="bfloat16", num_blocks=64, block_size=page, max_num_seqs=4, cuda_graphs=False)
    got = engine.generate(prompts, max_tokens=new)
    assert calls["fused"] >= config["num_hidden_layers"] * (new - 1)
    # every norm but the first layer's (it norms the embedding) and the final one (the last
    # product's splits are summed before the sampled rows are gathered)
    assert calls["partial_norm"] >= (2 * config["num_hidden_layers"] - 1) * (new - 1)
    cfg, W = plain.load_model(path)
    for prompt, tokens in zip(prompts, got):
        assert len(tokens) == new
        logits = plain.forward_logits(cfg, W, prompt + tokens[:-1])[len(prompt) - 1:]
        top = torch.topk(logits, 2, dim=-1)
        clear = (top.values[:, 0] - top.values[:, 1]) > 0.05 * logits.abs().max()
        want = top.indices[:, 0].tolist()
        for i, token in enumerate(tokens):
            if clear[i]:
                assert token == want[i], f"token {i}: {token} where the float32 model clearly says {want[i]}"
        assert clear.sum() >= new // 4, "the check would say nothing: no position has a clear argmax"


@pytest.mark.parametrize("name", ["w", "x"])
def test_wide_graph_replay_equals_eager(name, wide_dirs):
    """The same requests with and without CUDA graphs: the same tokens (the graphs replay the
    launches of the eager step, fused attention included)."""
    from vosti_b200 import Engine
    path, config, page = wide_dirs[name]
    prompts = [R.random_tokens(config["vocab_size"], n, seed=301 + n) for n in (33, 5, 190, 71)]
    out = {}
    for graphs in (False, True):
        engine = Engine(path, dtype="bfloat16", num_blocks=96, block_size=page, max_num_seqs=4, cuda_graphs=graphs)
        out[graphs] = engine.generate(prompts, max_tokens=20, temperature=0.7, seeds=[1, 2, 3, 4])
    assert out[True] == out[False]


@pytest.mark.parametrize("name", ["w", "x"])
def test_wide_bits_do_not_depend_on_the_cut_in_fixed_order(name, wide_dirs, tmp_path):
    """With one order of arithmetic everywhere the bfloat16 logits at a position are the same
    bits whole, with a decoded tail, in portions and mixed, also through the tensor-memory
    attention and the tensor-core products of these widths."""
    from vosti_b200 import ops
    path, config, page = wide_dirs[name]
    requests = _requests(name, config)
    kinds = {"whole": R.whole_steps, "tail": R.tail_steps, "portion": R.portion_steps,
             "mixed": lambda reqs: R.mixed_steps(reqs, seed=9)}
    steps = []
    for kind, make in kinds.items():
        steps.extend(make({f"{kind}-{rid}": tokens for rid, tokens in requests.items()}))
    steps = R.number(steps)
    try:
        R.run_in_process(path, "bfloat16", steps, R.max_live_tokens(steps), page, tmp_path, batch_invariant="full")
    finally:
        ops.set_invariance("off")
    rows = R.collect(steps, tmp_path, config["vocab_size"])
    for rid, tokens in requests.items():
        for position in range(len(tokens)):
            whole = rows[(f"whole-{rid}", position)]
            for kind in ("tail", "portion", "mixed"):
                assert np.array_equal(whole, rows[(f"{kind}-{rid}", position)]), \
                    f"{rid} position {position}: {kind} differs from whole"


@pytest.mark.parametrize("seed", [11, 12, 13])
@pytest.mark.parametrize("name", ["w", "x"])
def test_wide_random_mixes_in_the_default_mode(name, seed, wide_dirs, wide_plain, tmp_path):
    """Other random mixes of portions and decoded tokens of up to four live requests, in bfloat16
    with every fast path on (split products, fused decode attention with its clusters, graphs
    off in replay): every logit row against the plain implementation, within the bound the
    reference's own rounding points give."""
    import plain_qwen3 as plain
    path, config, page = wide_dirs[name]
    lengths = [LENGTHS[name][(seed + i) % len(LENGTHS[name])] + 3 * i + seed % 7 for i in range(5)]
    requests = {f"m{i}": R.random_tokens(config["vocab_size"], n, seed=seed * 100 + i) for i, n in enumerate(lengths)}
    steps = R.number(R.mixed_steps(requests, seed=seed))
    max_tokens = R.max_live_tokens(steps)
    assert max_tokens < sum(R.roundup64(len(t)) for t in requests.values())          # pages are used again
    R.run_in_process(path, "bfloat16", steps, max_tokens, page, tmp_path)
    rows = R.collect(steps, tmp_path, config["vocab_size"])
    assert len(rows) == sum(len(t) for t in requests.values())
    worst = R.compare_with_plain(rows, requests, wide_plain[name], "bfloat16")
    cfg, W = wide_plain[name]
    emulated = 0.0
    for tokens in requests.values():
        exact = plain.forward_logits(cfg, W, tokens).numpy()
        rounded = plain.forward_logits(cfg, W, tokens, round_to=torch.bfloat16).numpy()
        emulated = max(emulated, float(np.abs(rounded - exact).max()) / max(1.0, float(np.abs(exact).max())))
    print(f"{name} seed {seed}: worst {worst:.3e}, the reference's rounding points {emulated:.3e}")
    assert worst <= 1.5 * emulated
