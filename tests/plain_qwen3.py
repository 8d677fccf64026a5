"""Plain, slow Qwen3 dense implementation: whole sequences, no cache, one
function per part. It shares no code with the package (it reads config.json and
the safetensors file through the `safetensors` library, not through
`vosti_b200.weights`). Written from the reference's formulas; each function
cites the file and lines it restates. `tests/golden/make_golden.py` compares it
once with the reference's own CPU primitives on a tiny random model.

All paths are by the reference project's layout (QDelta/Vosti).
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def load_model(model_dir, dtype=torch.float32):
    """config.json as a dict and all tensors widened to `dtype` (exact for bf16 -> f32)."""
    from safetensors import safe_open

    root = Path(model_dir)
    config = json.loads((root / "config.json").read_text())
    tensors = {}
    with safe_open(str(root / "model.safetensors"), framework="pt", device="cpu") as handle:
        for name in handle.keys():
            tensors[name] = handle.get_tensor(name).to(dtype)
    return config, tensors


def _round(x, round_to):
    """Optional emulation of the reference's rounding points: it stores every
    primitive's output in bf16 (each of its kernels ends in
    `.to(o.dtype.element_ty)`, e.g. kernels/triton_kernels/rmsnorm.py:93)."""
    return x if round_to is None else x.to(round_to).to(x.dtype)


def embedding(ids, table):
    """o[m,:] = W[ids[m],:], a row copy without scaling
    (kernels/triton_kernels/embedding.py:62-84)."""
    return table[ids.long()]


def rms_norm(x, weight, eps):
    """var = sum(x^2)/N; o = x * rsqrt(var + eps) * w with a plain weight, all in
    float32 (kernels/triton_kernels/rmsnorm.py:63-93)."""
    xf = x.float()
    var = (xf * xf).sum(-1, keepdim=True) / xf.shape[-1]
    return ((xf * torch.rsqrt(var + eps)) * weight.float()).to(x.dtype)


def add_rms_norm(x, residual, weight, eps, round_to=None):
    """hidden = x + residual (stored as the new residual); the norm is taken of
    the unrounded sum (kernels/triton_kernels/rmsnorm_residual.py:86-125)."""
    hidden = x.float() + residual.float()
    var = (hidden * hidden).sum(-1, keepdim=True) / hidden.shape[-1]
    normed = hidden * torch.rsqrt(var + eps) * weight.float()
    return _round(normed.to(x.dtype), round_to), _round(hidden.to(x.dtype), round_to)


def head_rms_norm(x, weight, eps):
    """Per-head RMSNorm over head_dim with one (head_dim,) weight shared by all
    heads (kernels/triton_kernels/qk_norm.py:40-95). x: [T, heads, d]."""
    xf = x.float()
    var = (xf * xf).sum(-1, keepdim=True) / xf.shape[-1]
    return (xf * torch.rsqrt(var + eps) * weight.float()).to(x.dtype)


def rope_tables(positions, head_dim, theta, table_dtype=torch.float32):
    """inv_freq[i] = 1 / theta^(2i/d) in float32 from an integer arange; angle =
    inv_freq * float(position); cos/sin cast to the table dtype
    (python/vosti_kernels/rotary.py:80-88, 137-160)."""
    exponent = torch.arange(0, head_dim, 2, dtype=torch.int64).to(torch.float32) / head_dim
    inv_freq = 1.0 / (float(theta) ** exponent)
    angles = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    return angles.cos().to(table_dtype), angles.sin().to(table_dtype)


def apply_rope(x, cos, sin):
    """Half-split rotation: x1 = x[..., :d/2], x2 = x[..., d/2:];
    y1 = x1*cos - x2*sin; y2 = x2*cos + x1*sin
    (kernels/triton_kernels/rope.py:78-101). x: [T, heads, d]; cos/sin: [T, d/2]."""
    half = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:]
    c, s = cos.float()[:, None, :], sin.float()[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def causal_attention(q, k, v, scale, window=0, round_p_to=None):
    """Whole-sequence causal GQA attention. Query j sees keys 0..j (and, with a
    window w > 0, only keys > j - w); query head h uses kv head h*nkv/nq by
    integer division; softmax in float32; out = softmax(q k^T * scale) v
    (kernels/triton_kernels/fattn_paged.py:176-179, 220-252; oracle :716-763).
    q: [T, nq, d]; k, v: [T, nkv, d]. `round_p_to` emulates the reference rounding
    the probabilities to bf16 before P.V (:246)."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    out = torch.zeros(T, nq, d, dtype=torch.float32)
    idx = torch.arange(T)
    visible = idx[None, :] <= idx[:, None]
    if window and window > 0:
        visible &= idx[None, :] > (idx[:, None] - window)
    for h in range(nq):
        g = h * nkv // nq
        scores = (q[:, h, :].float() @ k[:, g, :].float().T) * scale
        scores = scores.masked_fill(~visible, float("-inf"))
        m = scores.max(-1, keepdim=True).values
        p = torch.exp(scores - m)
        l = p.sum(-1, keepdim=True)
        if round_p_to is not None:
            p = p.to(round_p_to).float()
        out[:, h, :] = (p @ v[:, g, :].float()) / l
    return out.to(q.dtype)


def swiglu(x, w_gate, w_up, w_down, round_to=None):
    """gate = x Wg^T, up = x Wu^T, mlp = gate*sigmoid(gate)*up in float32, out = mlp Wd^T;
    gate first, then up (kernels/triton_kernels/silu_mul.py:66-87;
    python/vosti_kernels/model_families/qwen3/loader.py:55-58)."""
    gate = _round(x @ w_gate.T, round_to)
    up = _round(x @ w_up.T, round_to)
    mlp = _round((gate.float() * torch.sigmoid(gate.float()) * up.float()).to(x.dtype), round_to)
    return _round(mlp @ w_down.T, round_to)


def attention_block(x, positions, W, prefix, cfg, round_to=None, window=0):
    """q,k,v projections (without bias in Qwen3; a `*_proj.bias` in W is added, for the
    tests of the projection bias other architectures have); per-head q/k norm before RoPE; v
    neither normed nor rotated; attention; output projection
    (src/exec/dense_swiglu_decoder.rs:171-367)."""
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    T = x.shape[0]

    def project(name, inp):
        y = inp @ W[prefix + name + ".weight"].T
        bias = W.get(prefix + name + ".bias")
        return _round(y if bias is None else y + bias.to(y.dtype), round_to)

    q = project("q_proj", x).view(T, nq, d)
    k = project("k_proj", x).view(T, nkv, d)
    v = project("v_proj", x).view(T, nkv, d)
    q = _round(head_rms_norm(q, W[prefix + "q_norm.weight"], eps), round_to)
    k = _round(head_rms_norm(k, W[prefix + "k_norm.weight"], eps), round_to)
    table_dtype = torch.float32 if round_to is None else round_to
    cos, sin = rope_tables(positions, d, cfg["rope_theta"], table_dtype)
    q = _round(apply_rope(q, cos, sin), round_to)
    k = _round(apply_rope(k, cos, sin), round_to)
    attn = causal_attention(q, k, v, float(d) ** -0.5, window=window, round_p_to=round_to)
    attn = _round(attn, round_to).reshape(T, nq * d)
    return project("o_proj", attn)


def forward_hidden(config, W, tokens, round_to=None):
    """Embedding, then every layer with the deferred residual add: a layer gets
    (hidden, residual), norms hidden+residual, runs attention, norms the sum again,
    runs the feed-forward and returns (mlp_out, residual); layer 0 starts with
    residual = embedding and no add; after the last layer one more add and the
    final norm (src/exec/dense_swiglu_decoder.rs:556-615, 740-813, 370-383;
    src/exec/dense_swiglu_model.rs:897-903)."""
    ids = torch.as_tensor(tokens, dtype=torch.int64)
    positions = torch.arange(ids.shape[0])
    eps = config["rms_norm_eps"]
    hidden = embedding(ids, W["model.embed_tokens.weight"])
    residual = None
    for i in range(config["num_hidden_layers"]):
        p = f"model.layers.{i}."
        if residual is None:
            residual = hidden
            normed = _round(rms_norm(hidden, W[p + "input_layernorm.weight"], eps), round_to)
        else:
            normed, residual = add_rms_norm(hidden, residual, W[p + "input_layernorm.weight"],
                                            eps, round_to)
        proj = attention_block(normed, positions, W, p + "self_attn.", config, round_to)
        normed2, residual = add_rms_norm(proj, residual, W[p + "post_attention_layernorm.weight"],
                                         eps, round_to)
        hidden = swiglu(normed2, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                        W[p + "mlp.down_proj.weight"], round_to)
    if residual is None:
        return _round(rms_norm(hidden, W["model.norm.weight"], eps), round_to)
    final, _ = add_rms_norm(hidden, residual, W["model.norm.weight"], eps, round_to)
    return final


def forward_logits(config, W, tokens, round_to=None):
    """Logits at every position of one whole sequence, [T, vocab] in float32. The
    head is the embedding table when tie_word_embeddings is set
    (python/vosti_kernels/model_families/qwen3/physical.py:131-134;
    src/exec/dense_swiglu_model.rs:976-984)."""
    final = forward_hidden(config, W, tokens, round_to)
    head = W["model.embed_tokens.weight"] if config["tie_word_embeddings"] else W["lm_head.weight"]
    return (final @ head.T).float()


def uniform(seed, index):
    """The sampler's counter-based uniform in [0,1) with 24 bits, keyed by the
    request's seed and the index of the token being drawn (ours; the reference
    samples greedily only, python/vosti_kernels/kernels.py:1088-1104)."""
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + (index + 1) * 0xBF58476D1CE4E5B9) & mask
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & mask
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & mask
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


def sample(logits_row, temperature=0.0, seed=0, index=0):
    """Greedy: the lowest index of the maximum (torch.argmax over the row,
    python/vosti_kernels/kernels.py:1103). Temperature: p = softmax(logits/T);
    the token is the first whose inclusive cumulative weight exceeds u * total."""
    row = logits_row.double()
    if temperature <= 0.0:
        return int(torch.argmax(row))
    w = torch.exp((row - row.max()) / temperature)
    cdf = torch.cumsum(w, 0)
    u = uniform(seed, index)
    token = int(torch.searchsorted(cdf, torch.tensor(u * float(cdf[-1]), dtype=cdf.dtype),
                                   right=True))
    return min(token, row.shape[0] - 1)


def generate(config, W, prompt, max_tokens, temperature=0.0, seed=0, eos=()):
    """Token-by-token generation by recomputing the whole sequence every time."""
    tokens, out = list(prompt), []
    for index in range(max_tokens):
        logits = forward_logits(config, W, tokens)[-1]
        token = sample(logits, temperature, seed, index)
        out.append(token)
        tokens.append(token)
        if token in eos:
            break
    return out
