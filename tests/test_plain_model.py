"""The plain implementation: against the logits the reference's own CPU code produced
(tests/golden/), and its parts against direct formulas."""
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from tiny_configs import ALL

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("name", ["a", "b"])
def test_plain_matches_reference_golden(name, plain_models):
    data = np.load(GOLDEN / f"qwen3_tiny_{name}.npz")
    config, W = plain_models[name]
    logits = plain.forward_logits(config, W, data["tokens"].tolist()).numpy()
    assert logits.shape == data["logits"].shape
    assert np.abs(logits - data["logits"]).max() < 2e-6


def test_rope_is_half_split_and_norm_preserving():
    x = torch.randn(5, 3, 8)
    cos, sin = plain.rope_tables(torch.arange(5), 8, 10000.0)
    y = plain.apply_rope(x, cos, sin)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    assert torch.equal(y[0], x[0])                                  # position 0 rotates nothing
    # pair (i, i + d/2) rotates by angle pos * theta^(-2i/d)
    pos, i = 3, 1
    angle = pos * 10000.0 ** (-2 * i / 8)
    want = x[pos, 0, i] * np.cos(angle) - x[pos, 0, i + 4] * np.sin(angle)
    assert abs(y[pos, 0, i].item() - want.item()) < 1e-5


def test_attention_is_causal_and_grouped():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    out = plain.causal_attention(q, k, v, 8 ** -0.5)
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -7.0                                     # the future does not matter
    assert torch.allclose(plain.causal_attention(q, k2, v2, 8 ** -0.5)[:4], out[:4])
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])   # heads 0,1 -> kv 0; 2,3 -> kv 1
    windowed = plain.causal_attention(q, k, v, 8 ** -0.5, window=2)
    k3, v3 = k.clone(), v.clone()
    k3[:3], v3[:3] = 5.0, 5.0                                      # outside the window of query 5 (keys 4, 5)
    assert torch.allclose(plain.causal_attention(q, k3, v3, 8 ** -0.5, window=2)[5], windowed[5])


def test_rms_norm_and_residual():
    x, r, w = torch.randn(3, 10), torch.randn(3, 10), torch.rand(10) + 0.5
    normed, new_r = plain.add_rms_norm(x, r, w, 1e-5)
    h = x + r
    assert torch.allclose(new_r, h)
    assert torch.allclose(normed, h / torch.sqrt((h * h).mean(-1, keepdim=True) + 1e-5) * w, atol=1e-6)


def test_sampler_is_greedy_at_zero_and_seeded_otherwise():
    row = torch.tensor([0.1, 2.0, 2.0, -1.0])
    assert plain.sample(row) == 1                                   # lowest index on ties
    draws = [plain.sample(row, 1.0, seed=5, index=i) for i in range(200)]
    assert draws == [plain.sample(row, 1.0, seed=5, index=i) for i in range(200)]
    assert set(draws) <= {0, 1, 2, 3} and draws.count(1) + draws.count(2) > 120
    assert all(0.0 <= plain.uniform(s, i) < 1.0 for s in range(5) for i in range(50))
    from vosti_b200.sampling import uniform
    assert all(uniform(s, i) == plain.uniform(s, i) for s in (0, 3, 2 ** 40 + 1) for i in range(20))


def test_generate_depends_on_weights(plain_models):
    config, W = plain_models["b"]
    out = plain.generate(config, W, [5, 9, 200, 17], 6)
    assert len(out) == 6 and all(0 <= t < config["vocab_size"] for t in out)
