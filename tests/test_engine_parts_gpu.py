"""Toy architectures through the whole engine: scheduler, state slots, CUDA graphs, async
scheduling, preemption. The parts are defined here (a recurrent mixer whose state lives in
the per-request slot, in a host-looping and in a device-only form; a feed-forward that routes
its tokens) together with the engine's own options for an embedding scale, a projection bias
and a head with bias, scale and soft cap. Nothing in the framework's files knows them.

What is compared: greedy generation through `Engine` (several requests at once, so few pages
that requests are preempted and recomputed, slots used again by later requests) against the
same model stepped alone through a fresh `ModelRunner`: whole prompt, then token by token.
"""
import pytest
import torch

import plain_qwen3 as plain
from vosti_b200 import Engine
from vosti_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry
from vosti_b200.engine.batch import StepEntry
from vosti_b200.engine.runner import ModelRunner
from vosti_b200.models import expected_weights
from vosti_b200.parts import FeedForward, Mixer, StateSpec, register_part, unregister_part
from vosti_b200.weights import WeightSpec, draw_tensors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class DecayMixer(Mixer):
    """s <- decay * s + x_t per request, y_t = s W^T; the host walks the requests of the step,
    so a recorded step cannot be replayed: it says so."""

    capture_safe = False

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


class DecayMixerOnDevice(DecayMixer):
    """The same mixer, but a step in which every request brings one token touches nothing on
    the host: the slots come from the step's device arrays. Such steps may be replayed."""

    capture_safe = True

    def forward(self, ctx, x, cache, writes_cache=True):
        if not ctx.all_decode:
            return super().forward(ctx, x, cache, writes_cache)
        slots = ctx.state_slots.long()
        state = cache.state.index_select(0, slots) * self.decay + x.float()
        cache.state.index_copy_(0, slots, state)
        return (state @ self.w.float().T).to(x.dtype)


class RoutedToy(FeedForward):
    """Every token goes to the expert its router row scores highest (32-bit scores)."""

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


@pytest.fixture
def toy_parts():
    register_part("mixer", "decay", DecayMixer, replace=True)
    register_part("mixer", "decay_on_device", DecayMixerOnDevice, replace=True)
    register_part("feed_forward", "routed_toy", RoutedToy, replace=True)
    yield
    unregister_part("mixer", "decay")
    unregister_part("mixer", "decay_on_device")
    unregister_part("feed_forward", "routed_toy")


def toy_spec(mixer_kind, hidden=32, vocab=61):
    norm = PartSpec.make("rmsnorm", eps=1e-5)
    attention = LayerSpec(
        mixer=PartSpec.make("attention", num_heads=2, num_kv_heads=1, head_dim=16, head_norm_eps=None, window=0,
                            scale=0.25, qkv_bias=True),
        feed_forward=PartSpec.make("routed_toy", experts=3), norm=norm,
        position=PartSpec.make("rope", theta=1e4, rotary_dim=16, max_positions=256))
    recurrent = LayerSpec(mixer=PartSpec.make(mixer_kind, decay=0.5),
                          feed_forward=PartSpec.make("swiglu", intermediate_size=48), norm=norm, position=None)
    return ModelSpec(architecture="Toy", hidden_size=hidden, vocab_size=vocab, max_positions=256,
                     layers=(attention, recurrent), run_order=(RunEntry(0), RunEntry(1)), final_norm=norm,
                     tie_word_embeddings=False, embedding=PartSpec.make("table", scale=hidden ** 0.5),
                     head=PartSpec.make("linear", bias=True, scale=0.5, softcap=7.0))


def toy_tensors(spec, seed=9):
    tensors = draw_tensors(expected_weights(spec), seed)
    # make the parts matter: a bias of visible size, an embedding of unit size
    tensors["lm_head.bias"] = torch.randn(spec.vocab_size, generator=torch.Generator().manual_seed(3)) * 0.5
    tensors["model.embed_tokens.weight"] = tensors["model.embed_tokens.weight"] * 20
    return {k: v.to(DEV) for k, v in tensors.items()}


def alone(spec, tensors, prompt, new_tokens):
    """Greedy generation of one request on a fresh runner: the whole prompt, then one token a step."""
    runner = ModelRunner(spec=spec, tensors=dict(tensors), dtype="float32", num_pages=64, page_size=4, max_requests=1)
    runner.begin("r")
    logits = runner.step([StepEntry("r", prompt, [len(prompt) - 1])])
    out = [int(logits[0].argmax())]
    while len(out) < new_tokens:
        logits = runner.step([StepEntry("r", [out[-1]], [0])])
        out.append(int(logits[0].argmax()))
    runner.check_status()
    return out


def prompts_for(spec, count, seed):
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, spec.vocab_size, (int(torch.randint(3, 14, (1,), generator=gen)),), generator=gen).tolist()
            for _ in range(count)]


@pytest.mark.parametrize("mixer_kind,async_scheduling", [("decay", False), ("decay", True),
                                                         ("decay_on_device", False), ("decay_on_device", True)])
def test_stateful_toy_model_through_the_engine_with_preemption_and_slot_reuse(toy_parts, mixer_kind, async_scheduling):
    spec = toy_spec(mixer_kind)
    tensors = toy_tensors(spec)
    prompts = prompts_for(spec, 6, seed=5)
    want = [alone(spec, tensors, p, 12) for p in prompts]
    # 2 slots for 6 requests (every slot is used again), 9 pages of 4 tokens for two requests
    # that grow to 6 or 7 pages each (the younger one is preempted and recomputed)
    engine = Engine(spec=spec, tensors=dict(tensors), dtype="float32", num_blocks=9, block_size=4, max_num_seqs=2,
                    max_num_batched_tokens=16, prefill_chunk_size=8, cuda_graphs=True,
                    async_scheduling=async_scheduling)
    assert engine.runner.cache.has_state and not engine.runner.cache.prefix_reuse
    assert (engine.graphs is not None) == (mixer_kind == "decay_on_device")
    got = engine.generate(prompts, max_tokens=12, arrival_steps=[0, 0, 1, 5, 9, 30])
    assert got == want
    assert engine.scheduler.preemptions > 0
    if engine.graphs is not None:
        assert engine.graphs.replays > 0
    engine.runner.cache.check()
    assert engine.runner.cache.available_pages() == 9 and len(engine.runner.cache.free_slots) == 2


def test_a_slot_is_cleared_for_its_next_tenant(toy_parts):
    """max_num_seqs=1: the second request takes the slot the first one left its state in."""
    spec = toy_spec("decay")
    tensors = toy_tensors(spec)
    prompts = prompts_for(spec, 3, seed=8)
    want = [alone(spec, tensors, p, 5) for p in prompts]
    engine = Engine(spec=spec, tensors=dict(tensors), dtype="float32", num_blocks=16, block_size=4, max_num_seqs=1)
    assert engine.generate(prompts, max_tokens=5) == want
    state = engine.runner.cache.layer_caches[1].state
    assert state.shape[0] == 1 and state.abs().max() > 0            # the last tenant's state is still there...
    engine.add_request("late", prompts[0], 5, None, True)
    out = []
    while engine.has_unfinished():
        out += list(engine.step().values())
    assert out == want[0]                                            # ...and does not reach the next one


def test_graphs_are_refused_for_a_model_that_cannot_be_replayed(toy_parts):
    from vosti_b200.engine.graphs import DecodeGraphs
    spec = toy_spec("decay")
    runner = ModelRunner(spec=spec, tensors=toy_tensors(spec), dtype="float32", num_pages=8, page_size=4, max_requests=1)
    assert not runner.model.capture_safe
    with pytest.raises(ValueError, match="capture_safe"):
        DecodeGraphs(runner)
    spec = toy_spec("decay_on_device")
    runner = ModelRunner(spec=spec, tensors=toy_tensors(spec), dtype="float32", num_pages=8, page_size=4, max_requests=1)
    assert runner.model.capture_safe


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_scale_and_head_transform_against_plain_formulas(toy_parts, dtype):
    """hidden = table[id] * scale; logits = cap * tanh((x W^T * scale + bias) / cap), float32."""
    from vosti_b200.parts import build_embedding, build_head
    H, V = 80, 331
    gen = torch.Generator().manual_seed(0)
    table = (torch.randn(V, H, generator=gen)).to(dtype).to(DEV)
    embed = build_embedding(PartSpec.make("table", scale=H ** 0.5), H, V)
    embed.load({"weight": table}, dtype)
    ids = torch.randint(0, V, (9,), generator=gen).int().to(DEV)
    ctx = type("Ctx", (), {"status": torch.zeros(1, dtype=torch.int32, device=DEV)})()
    got = embed.forward(ctx, ids)
    want = (plain.embedding(ids.cpu(), table.float().cpu()) * (H ** 0.5)).to(dtype)
    assert got.dtype == dtype and torch.equal(got.cpu(), want)
    plain_copy = build_embedding(PartSpec.make("table"), H, V)
    plain_copy.load({"weight": table}, dtype)
    assert torch.equal(plain_copy.forward(ctx, ids).cpu(), table[ids.long()].cpu())

    w = (torch.randn(V, H, generator=gen) * 0.3).to(dtype).to(DEV)
    bias = torch.randn(V, generator=gen).to(DEV)
    x = torch.randn(5, H, generator=gen).to(dtype).to(DEV)
    for tied in (False, True):
        head = build_head(PartSpec.make("linear", bias=True, scale=0.25, softcap=3.0), H, V, tied)
        assert ("weight" in head.weight_specs()) == (not tied) and "bias" in head.weight_specs()
        head.load({"bias": bias} if tied else {"weight": w, "bias": bias}, dtype, tied=w if tied else None)
        logits = head.forward(ctx, x)
        exact = 3.0 * torch.tanh((x.double().cpu() @ w.double().cpu().T * 0.25 + bias.double().cpu()) / 3.0)
        assert logits.dtype == torch.float32
        assert torch.allclose(logits.double().cpu(), exact, atol=1e-5 if dtype == torch.float32 else 2e-2)
        assert logits.abs().max() <= 3.0
    assert ctx.status.item() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_projection_bias_against_plain_attention(dtype):
    """The attention part with q/k/v and output biases, fed in portions, against the plain block."""
    from gpu_util import Harness
    from vosti_b200.parts.base import build_mixer
    cfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-5, rope_theta=1e4)
    spec = PartSpec.make("attention", num_heads=4, num_kv_heads=2, head_dim=32, head_norm_eps=1e-5, window=0,
                         scale=32 ** -0.5, qkv_bias=True, o_bias=True)
    mixer = build_mixer(spec, 96, PartSpec.make("rope", theta=1e4, rotary_dim=32, max_positions=128))
    names = mixer.weight_specs()
    assert {"q_proj.bias", "k_proj.bias", "v_proj.bias", "o_proj.bias"} <= set(names)
    tensors = draw_tensors(names, 3, dtype=torch.float32)
    for k in tensors:
        if k.endswith("proj.weight"):
            tensors[k] = tensors[k] * 4
        if k.endswith(".bias"):
            tensors[k] = torch.randn(tensors[k].shape, generator=torch.Generator().manual_seed(len(k))) * 0.5
    tensors = {k: v.to(DEV, dtype) for k, v in tensors.items()}
    mixer.load(tensors, dtype)
    mixer.setup(torch.device(DEV), dtype)
    harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=16, page_size=8)
    x = torch.randn(40, 96).to(dtype)
    outs, at = [], 0
    for size in (6, 1, 30, 1, 2):
        ctx = harness.context([StepEntry("s", [0] * size)])
        outs.append(mixer.forward(ctx, x[at:at + size].to(DEV), harness.cache.layer_caches[0]).float().cpu())
        at += size
    W = {("p." + k): v.float().cpu() for k, v in tensors.items()}
    want = plain.attention_block(x.float(), torch.arange(40), W, "p.", cfg)
    no_bias = plain.attention_block(x.float(), torch.arange(40), {k: v for k, v in W.items() if not k.endswith("bias")},
                                    "p.", cfg)
    assert (want - no_bias).abs().max() > 0.1                    # the biases are not a no-op
    bound = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    assert torch.allclose(torch.cat(outs), want, **bound)
    assert harness.status.item() == 0
