"""Each part alone against the plain implementation, and the framework's generality: a toy
mixer with state of its own, a toy feed-forward with routing and a toy position encoding
(all defined here) are registered, built and stepped; a run order that names a layer twice;
a layer that reads another layer's cache; a windowed layer beside a full one, with pages of
their own."""
import pytest
import torch

import plain_qwen3 as plain
from gpu_util import Harness
from vosti_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry
from vosti_b200.engine.batch import StepEntry
from vosti_b200.parts import (FeedForward, Mixer, PositionEncoding, StateSpec, build_block, build_norm, register_part,
                              unregister_part)
from vosti_b200.parts.base import build_feed_forward, build_mixer
from vosti_b200.weights import WeightSpec, draw_tensors

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
DEV = "cuda:0"


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)


def load(part, seed, dtype, scale=1.0):
    tensors = {k: (v * scale if "norm" not in k else v).to(DEV, dtype)
               for k, v in draw_tensors(part.weight_specs(), seed, dtype=torch.float32).items()}
    part.load(tensors, dtype)
    part.setup(torch.device(DEV), dtype)
    return {k: v.float().cpu() for k, v in tensors.items()}


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    norm = build_norm(PartSpec.make("rmsnorm", eps=3e-6), 80)
    W = load(norm, 1, dtype)
    x = torch.randn(7, 80, device=DEV).to(dtype)
    r = torch.randn(7, 80, device=DEV).to(dtype)
    assert torch.allclose(norm.forward(None, x).float().cpu(), plain.rms_norm(x.float().cpu(), W["weight"], 3e-6), **tol(dtype))
    want_n, want_r = plain.add_rms_norm(x.float().cpu(), r.float().cpu(), W["weight"], 3e-6)
    got_n, got_r = norm.forward_add(None, x, r)
    assert torch.allclose(got_n.float().cpu(), want_n, **tol(dtype)) and torch.allclose(got_r.float().cpu(), want_r, **tol(dtype))


def test_position_part_tables():
    from vosti_b200.parts import build_position
    rope = build_position(PartSpec.make("rope", theta=50000.0, rotary_dim=48, max_positions=300), 80, 48)
    rope.setup(torch.device(DEV), torch.bfloat16)
    cos, sin = rope.rotation_tables()
    want_c, want_s = plain.rope_tables(torch.arange(300), 48, 50000.0)
    assert cos.dtype == torch.float32 and torch.equal(cos.cpu(), want_c) and torch.equal(sin.cpu(), want_s)
    for bad in (25, 64, 0 - 2):
        with pytest.raises(Exception):
            build_position(PartSpec.make("rope", theta=1e4, rotary_dim=bad, max_positions=8), 80, 48)
    part = build_position(PartSpec.make("rope", theta=1e4, rotary_dim=24, max_positions=8, interleaved=True), 80, 48)
    part.setup(torch.device(DEV), torch.bfloat16)
    assert part.rotary_dim == 24 and part.interleaved and part.rotation_tables()[0].shape == (8, 12)


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    ffn = build_feed_forward(PartSpec.make("swiglu", intermediate_size=208), 96)
    W = load(ffn, 2, dtype, scale=5.0)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ctx = type("Ctx", (), {"status": status})()          # the feed-forward reads nothing else of a step
    x = torch.randn(9, 96, device=DEV).to(dtype)
    got = ffn.forward(ctx, x)
    want = plain.swiglu(x.float().cpu(), W["gate_proj.weight"], W["up_proj.weight"], W["down_proj.weight"])
    assert torch.allclose(got.float().cpu(), want, **tol(dtype))
    assert status.item() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 11])
def test_attention_part_in_portions(dtype, window):
    """The mixer alone over the paged cache: a sequence fed in portions equals the plain
    whole-sequence attention block."""
    cfg = dict(num_attention_heads=6, num_key_value_heads=2, head_dim=32, rms_norm_eps=2e-6, rope_theta=30000.0)
    spec = PartSpec.make("attention", num_heads=6, num_kv_heads=2, head_dim=32, head_norm_eps=2e-6, window=window,
                         scale=32 ** -0.5)
    position = PartSpec.make("rope", theta=30000.0, rotary_dim=32, max_positions=128)
    mixer = build_mixer(spec, 80, position)
    W = load(mixer, 3, dtype, scale=4.0)
    harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=16, page_size=8)
    x = torch.randn(70, 80).to(dtype)
    outs, at = [], 0
    for size in (5, 1, 30, 2, 1, 31):
        ctx = harness.context([StepEntry("s", [0] * size)])
        outs.append(mixer.forward(ctx, x[at:at + size].to(DEV), harness.cache.layer_caches[0]).float().cpu())
        harness.cache.trim("s")
        at += size
    want = plain.attention_block(x.float(), torch.arange(70), {("p." + k): v for k, v in W.items()}, "p.", cfg,
                                 window=window)
    assert torch.allclose(torch.cat(outs), want, **tol(dtype))
    assert harness.status.item() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part(dtype):
    layer = LayerSpec(mixer=PartSpec.make("attention", num_heads=4, num_kv_heads=4, head_dim=16, head_norm_eps=1e-6,
                                          window=0, scale=0.25),
                      feed_forward=PartSpec.make("swiglu", intermediate_size=96), norm=PartSpec.make("rmsnorm", eps=1e-6),
                      position=PartSpec.make("rope", theta=1e4, rotary_dim=16, max_positions=64),
                      names=(("input_norm", "n1"), ("post_norm", "n2"), ("mixer", "att"), ("feed_forward", "ff")))
    block = build_block(layer, 64)
    assert set(k.split(".")[0] for k in block.weight_specs()) == {"n1", "n2", "att", "ff"}
    tensors = {k: v.to(DEV, dtype) for k, v in draw_tensors(block.weight_specs(), 4, dtype=torch.float32).items()}
    block.load(tensors, dtype)
    block.setup(torch.device(DEV), dtype)
    harness = Harness([block.mixer.cache_spec()], [None], dtype)
    ctx = harness.context([StepEntry("s", [0] * 12)])
    hidden = torch.randn(12, 64).to(dtype)
    residual = torch.randn(12, 64).to(dtype)
    out, new_res = block.forward(ctx, hidden.to(DEV), residual.clone().to(DEV), harness.cache.layer_caches[0])
    W = {k: v.float().cpu() for k, v in tensors.items()}
    cfg = dict(num_attention_heads=4, num_key_value_heads=4, head_dim=16, rms_norm_eps=1e-6, rope_theta=1e4)
    normed, res = plain.add_rms_norm(hidden.float(), residual.float(), W["n1.weight"], 1e-6)
    proj = plain.attention_block(normed, torch.arange(12), W, "att.", cfg)
    normed2, res = plain.add_rms_norm(proj, res, W["n2.weight"], 1e-6)
    want = plain.swiglu(normed2, W["ff.gate_proj.weight"], W["ff.up_proj.weight"], W["ff.down_proj.weight"])
    assert torch.allclose(new_res.float().cpu(), res, **tol(dtype))
    assert torch.allclose(out.float().cpu(), want, **tol(dtype))


# ---------------------------------------------------------------- a toy mixer with state
class DecayMixer(Mixer):
    """A toy recurrent mixer: per request a state s of the hidden width, s <- decay * s + x_t,
    y_t = (s W^T). Its state lives in the per-request slot the cache manager gives out."""

    def __init__(self, spec, hidden_size, position):
        super().__init__(spec, hidden_size, position)
        self.decay = float(spec["decay"])
        self.w = None

    def weight_specs(self):
        return {"mix.weight": WeightSpec((self.hidden_size, self.hidden_size), std=0.1)}

    def load(self, tensors, dtype):
        self.w = tensors["mix.weight"]

    def state_spec(self):
        return StateSpec((self.hidden_size,), torch.float32)

    def forward(self, ctx, x, cache, writes_cache=True):
        out = torch.empty_like(x)
        at = 0
        for n, slot in zip(ctx.host_q_lens, ctx.host_state_slots):
            state = cache.state[slot]
            for i in range(at, at + n):
                state.mul_(self.decay).add_(x[i].float())
                out[i] = (state @ self.w.float().T).to(x.dtype)
            at += n
        return out


def toy_spec(layers, run_order, hidden=32, vocab=50):
    return ModelSpec(architecture="Toy", hidden_size=hidden, vocab_size=vocab, max_positions=256, layers=tuple(layers),
                     run_order=tuple(run_order), final_norm=PartSpec.make("rmsnorm", eps=1e-5), tie_word_embeddings=True)


def attention_layer(window=0, ffn=True):
    return LayerSpec(mixer=PartSpec.make("attention", num_heads=2, num_kv_heads=1, head_dim=16, head_norm_eps=None,
                                         window=window, scale=0.25),
                     feed_forward=PartSpec.make("swiglu", intermediate_size=48) if ffn else None,
                     norm=PartSpec.make("rmsnorm", eps=1e-5),
                     position=PartSpec.make("rope", theta=1e4, rotary_dim=16, max_positions=256))


def run_whole_and_cut(spec, tokens, dtype="float32", page_size=4, num_pages=64):
    """Logits of the sequence fed whole and fed in portions with a second request beside it."""
    from vosti_b200.engine.runner import ModelRunner
    from vosti_b200.models import expected_weights
    tensors = {k: v.to(DEV) for k, v in draw_tensors(expected_weights(spec), 5).items()}
    results = []
    for cuts in ([len(tokens)], [3, 1, 9, 2, 1, len(tokens) - 16]):
        runner = ModelRunner(spec=spec, tensors=dict(tensors), dtype=dtype, num_pages=num_pages, page_size=page_size,
                             max_requests=3)
        runner.begin("x"), runner.begin("other")
        rows, at = [], 0
        for n in cuts:
            entries = [StepEntry("x", tokens[at:at + n], list(range(n)))]
            if len(cuts) > 1:
                entries.insert(0, StepEntry("other", [7, 8], [1]))
            logits = runner.step(entries)
            rows.append(logits[-n:].cpu())
            at += n
        runner.check_status()
        runner.finish("x"), runner.finish("other")
        runner.cache.check()
        results.append((torch.cat(rows), runner))
    return results


def test_toy_mixer_with_state_registers_builds_and_steps():
    register_part("mixer", "decay", DecayMixer, replace=True)
    try:
        toy = LayerSpec(mixer=PartSpec.make("decay", decay=0.5), feed_forward=PartSpec.make("swiglu", intermediate_size=48),
                        norm=PartSpec.make("rmsnorm", eps=1e-5), position=None)
        spec = toy_spec([attention_layer(), toy], [RunEntry(0), RunEntry(1)])
        tokens = torch.randint(0, 50, (40,), generator=torch.Generator().manual_seed(1)).tolist()
        (whole, runner), (cut, _) = run_whole_and_cut(spec, tokens)
        assert runner.cache.has_state and not runner.cache.prefix_reuse
        assert runner.cache.layer_caches[1].state.shape == (3, 32) and runner.cache.layer_caches[1].group == -1
        assert "model.layers.1.mixer.mix.weight" in runner.model.expected_weights()
        assert torch.allclose(whole, cut, atol=1e-4, rtol=1e-4)
        # the state matters: a different history gives different logits at the same token
        (other, _), _ = run_whole_and_cut(spec, [tokens[0] + 1] + tokens[1:])
        assert (other[-1] - whole[-1]).abs().max() > 1e-4
    finally:
        unregister_part("mixer", "decay")


# ------------------------------------------------- a toy feed-forward that routes its tokens
class RoutedToy(FeedForward):
    """Every token goes to the one expert its router row scores highest (scores in 32-bit);
    an expert is one square matrix."""

    def __init__(self, spec, hidden_size):
        super().__init__(spec, hidden_size)
        self.experts = int(spec["experts"])
        self.router = self.w = None

    def weight_specs(self):
        specs = {"router.weight": WeightSpec((self.experts, self.hidden_size), std=1.0)}
        for e in range(self.experts):
            specs[f"experts.{e}.weight"] = WeightSpec((self.hidden_size, self.hidden_size), std=0.2)
        return specs

    def load(self, tensors, dtype):
        self.router = tensors["router.weight"].float()
        self.w = torch.stack([tensors[f"experts.{e}.weight"] for e in range(self.experts)])

    def forward(self, ctx, x):
        choice = (x.float() @ self.router.T).argmax(-1)
        return torch.bmm(x[:, None, :], self.w[choice].transpose(1, 2))[:, 0, :]


def test_toy_feed_forward_with_routing_registers_builds_and_steps():
    register_part("feed_forward", "routed_toy", RoutedToy, replace=True)
    try:
        base = attention_layer()
        routed = LayerSpec(mixer=base.mixer, feed_forward=PartSpec.make("routed_toy", experts=3), norm=base.norm,
                           position=base.position)
        spec = toy_spec([routed, attention_layer()], [RunEntry(0), RunEntry(1)])
        tokens = torch.randint(0, 50, (40,), generator=torch.Generator().manual_seed(4)).tolist()
        (whole, runner), (cut, _) = run_whole_and_cut(spec, tokens)
        names = runner.model.expected_weights()
        assert "model.layers.0.feed_forward.router.weight" in names and "model.layers.0.feed_forward.experts.2.weight" in names
        assert torch.allclose(whole, cut, atol=1e-4, rtol=1e-4)
        # the routing is per token: every expert gets some of these tokens
        ffn = runner.model.blocks[0].feed_forward
        hidden = torch.randn(64, 32, device=DEV)
        assert len(set((hidden @ ffn.router.T).argmax(-1).tolist())) == 3
    finally:
        unregister_part("feed_forward", "routed_toy")


# --------------------------------------------------------- a toy position encoding
class SlowRotation(PositionEncoding):
    """A rotation whose angle grows `slowdown` times slower than the position."""

    def __init__(self, spec, hidden_size, head_dim):
        super().__init__(spec, hidden_size, head_dim)
        self.cos = self.sin = None

    def setup(self, device, dtype):
        positions = torch.arange(int(self.spec["max_positions"]), dtype=torch.float32) / float(self.spec["slowdown"])
        self.cos, self.sin = (t.to(device).contiguous()
                              for t in plain.rope_tables(positions, self.head_dim, self.spec["theta"]))

    def rotation_tables(self):
        return self.cos, self.sin


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_position_encoding_registers_and_reaches_the_kernels(dtype):
    register_part("position", "slow_rotation", SlowRotation, replace=True)
    try:
        cfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-5, rope_theta=500.0)
        spec = PartSpec.make("attention", num_heads=4, num_kv_heads=2, head_dim=16, head_norm_eps=1e-5, window=0,
                             scale=0.25)
        mixer = build_mixer(spec, 48, PartSpec.make("slow_rotation", theta=500.0, slowdown=4.0, max_positions=64))
        assert isinstance(mixer.position, SlowRotation)
        W = load(mixer, 6, dtype, scale=4.0)
        harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=8, page_size=8)
        x = torch.randn(50, 48).to(dtype)
        outs, at = [], 0
        for size in (7, 1, 40, 2):
            ctx = harness.context([StepEntry("s", [0] * size)])
            outs.append(mixer.forward(ctx, x[at:at + size].to(DEV), harness.cache.layer_caches[0]).float().cpu())
            harness.cache.trim("s")
            at += size
        weights = {("p." + k): v for k, v in W.items()}
        want = plain.attention_block(x.float(), torch.arange(50) / 4.0, weights, "p.", cfg)
        assert torch.allclose(torch.cat(outs), want, **tol(dtype))
        plain_rope = plain.attention_block(x.float(), torch.arange(50), weights, "p.", cfg)
        assert (plain_rope - want).abs().max() > 0.05       # the slowdown is not a no-op
        assert harness.status.item() == 0
    finally:
        unregister_part("position", "slow_rotation")


def test_run_order_may_name_a_layer_twice_and_share_a_cache():
    layers = [attention_layer(), attention_layer(ffn=False)]
    tokens = torch.randint(0, 50, (40,), generator=torch.Generator().manual_seed(2)).tolist()
    plain_order = toy_spec(layers, [RunEntry(0), RunEntry(1)])
    twice = toy_spec(layers, [RunEntry(0), RunEntry(1), RunEntry(1, cache_from=0)])
    (a_whole, _), (a_cut, _) = run_whole_and_cut(plain_order, tokens)
    (b_whole, runner), (b_cut, _) = run_whole_and_cut(twice, tokens)
    assert torch.allclose(a_whole, a_cut, atol=1e-4, rtol=1e-4) and torch.allclose(b_whole, b_cut, atol=1e-4, rtol=1e-4)
    assert (a_whole - b_whole).abs().max() > 1e-3               # the third entry did run
    # the repeated entry brings no weights and no cache of its own
    from vosti_b200.models import expected_weights
    assert set(expected_weights(twice)) == set(expected_weights(plain_order))
    assert len(runner.cache.layer_caches) == 2 and len(runner.cache.groups) == 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_layer_beside_a_full_one_has_pages_of_its_own(dtype):
    spec = toy_spec([attention_layer(), attention_layer(window=6)], [RunEntry(0), RunEntry(1)])
    tokens = torch.randint(0, 50, (60,), generator=torch.Generator().manual_seed(3)).tolist()
    (whole, _), (cut, runner) = run_whole_and_cut(spec, tokens, dtype=dtype, num_pages=40)
    bound = dict(atol=1e-4, rtol=1e-4) if dtype == "float32" else dict(atol=3e-2, rtol=3e-2)
    assert torch.allclose(whole, cut, **bound)
    assert [g.window for g in runner.cache.groups] == [0, 6] and len(runner.cache.groups) == 2
    # the windowed group gives pages back while the request lives
    from vosti_b200.engine.runner import ModelRunner
    from vosti_b200.models import expected_weights
    tensors = {k: v.to(DEV) for k, v in draw_tensors(expected_weights(spec), 5).items()}
    small = ModelRunner(spec=spec, tensors=tensors, dtype=dtype, num_pages=15, page_size=4, max_requests=1)
    small.begin("x")
    for start in range(0, 60, 5):
        small.step([StepEntry("x", tokens[start:start + 5], [4])])
    full_pool, window_pool = (g.pool for g in small.cache.groups)
    assert full_pool.held() == 15 and window_pool.held() <= 3
    small.check_status()


def rotate_reference(x, positions, rotary_dim, theta, interleaved):
    """x: [T, heads, d]; the first rotary_dim elements of every head rotated by angle position *
    theta^(-2i/rotary_dim), pairs (i, i + rotary_dim/2) or (2i, 2i + 1); the rest unchanged."""
    cos, sin = plain.rope_tables(positions, rotary_dim, theta)
    c, s = cos[:, None, :].double(), sin[:, None, :].double()
    out = x.double().clone()
    half = rotary_dim // 2
    ia = torch.arange(half) * 2 if interleaved else torch.arange(half)
    ib = ia + 1 if interleaved else ia + half
    a, b = x.double()[..., ia], x.double()[..., ib]
    out[..., ia] = a * c - b * s
    out[..., ib] = b * c + a * s
    return out.float()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rotary_dim,interleaved", [(16, False), (32, True), (8, True)])
def test_partial_and_interleaved_rotations_through_the_attention_part(dtype, rotary_dim, interleaved):
    """A rotation of only the first elements of a head, or of neighbouring pairs, as a parameter of
    the built-in position encoding: the attention part fed in portions and single tokens equals a
    plain attention over queries and keys rotated by the formula."""
    nq, nkv, d, hidden = 4, 2, 32, 80
    spec = PartSpec.make("attention", num_heads=nq, num_kv_heads=nkv, head_dim=d, head_norm_eps=1e-5, window=0, scale=d ** -0.5)
    mixer = build_mixer(spec, hidden, PartSpec.make("rope", theta=3e4, rotary_dim=rotary_dim, max_positions=128,
                                                    interleaved=interleaved))
    W = load(mixer, 7, dtype, scale=4.0)
    harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=16, page_size=8)
    T = 45
    x = torch.randn(T, hidden).to(dtype)
    outs, at = [], 0
    for size in (9, 1, 1, 30, 2, 1, 1):
        ctx = harness.context([StepEntry("s", [0] * size)])
        outs.append(mixer.forward(ctx, x[at:at + size].to(DEV), harness.cache.layer_caches[0]).float().cpu())
        at += size
    xf = x.float()
    q = plain.head_rms_norm((xf @ W["q_proj.weight"].T).view(T, nq, d), W["q_norm.weight"], 1e-5)
    k = plain.head_rms_norm((xf @ W["k_proj.weight"].T).view(T, nkv, d), W["k_norm.weight"], 1e-5)
    v = (xf @ W["v_proj.weight"].T).view(T, nkv, d)
    positions = torch.arange(T)
    q, k = (rotate_reference(t, positions, rotary_dim, 3e4, interleaved) for t in (q, k))
    want = plain.causal_attention(q, k, v, d ** -0.5).reshape(T, nq * d) @ W["o_proj.weight"].T
    assert torch.allclose(torch.cat(outs), want, **tol(dtype))
    full = plain.attention_block(xf, positions, {("p." + n): t for n, t in W.items()}, "p.",
                                 dict(num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d, rms_norm_eps=1e-5, rope_theta=3e4))
    assert (full - want).abs().max() > 0.05                      # not the whole-head half-split rotation
    assert harness.status.item() == 0


def test_a_part_can_ask_for_index_arrays_of_its_own_in_every_step():
    """A step-layout provider registered from outside the framework: its arrays travel with the
    step's one copy and reach the parts through the context, beside the attention's own lists."""
    from vosti_b200.parts import register_step_layout
    from vosti_b200.parts.base import step_layout_providers

    def starts_and_longest(q_lens):
        starts, at = [], 0
        for n in q_lens:
            starts.append(at)
            at += n
        return {"starts": starts, "nothing": []}, {"longest": max(q_lens)}

    register_step_layout("toy_lists", starts_and_longest)
    try:
        harness = Harness([attention_layer().mixer and build_mixer(attention_layer().mixer, 32, attention_layer().position).cache_spec()],
                          [None], torch.bfloat16)
        ctx = harness.context([StepEntry("a", [1] * 7), StepEntry("b", [2]), StepEntry("c", [3] * 5)])
        assert ctx.extras["toy_lists.starts"].tolist() == [0, 7, 8] and ctx.layout["toy_lists"] == {"longest": 7}
        assert ctx.extras["toy_lists.nothing"].numel() == 0
        assert ctx.layout["attention"] == {"num_short_tokens": 1, "num_long_rows": 2, "max_long_q_len": 7}
        assert ctx.extras["attention.short_tokens"].tolist() == [7] and ctx.extras["attention.long_rows"].tolist() == [0, 2]
    finally:
        step_layout_providers().pop("toy_lists")
