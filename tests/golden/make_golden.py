"""Compare the plain implementation (tests/plain_qwen3.py) once with the reference's own
CPU code, and store the reference's logits.

The reference's engine is Rust and cannot be built offline, but its Python primitives run
on the CPU in float32 (`runtime_for_tests`, python/vosti_kernels/model_families/qwen3/
runtime.py:81-110) and its attention oracle `_sdpa_reference`
(kernels/triton_kernels/fattn_paged.py:716-763) runs on the CPU with any page size. This
script composes those primitives in the order of src/exec/dense_swiglu_decoder.rs:43-441
and src/exec/dense_swiglu_model.rs:131-1041 on the tiny random models A and B, writes the
resulting logits to tests/golden/qwen3_tiny_{a,b}.npz and prints the difference to the
plain implementation.

Run from the repository root with the reference checkout given:
    python tests/golden/make_golden.py /path/to/reference
"""
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def reference_logits(ref, config, W, tokens, page_size):
    import vosti_kernels as vk
    from vosti_kernels.model_families.qwen3.runtime import runtime_for_tests
    from triton_kernels.fattn_paged import _sdpa_reference

    nq, nkv, d = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    rt = runtime_for_tests(hidden_size=config["hidden_size"], num_heads=nq, num_kv_heads=nkv, head_dim=d,
                           intermediate_size=config["intermediate_size"],
                           rms_norm_eps=config["rms_norm_eps"], rope_theta=config["rope_theta"])
    T = len(tokens)
    ids = torch.tensor(tokens, dtype=torch.int32)
    positions = torch.arange(T, dtype=torch.int64)
    pages = (T + page_size - 1) // page_size
    order = list(reversed(range(pages)))                  # pages deliberately out of order
    block_table = torch.tensor([order], dtype=torch.int32)
    slots = torch.tensor([order[t // page_size] * page_size + t % page_size for t in range(T)], dtype=torch.int32)
    cu_q = torch.tensor([0, T], dtype=torch.int32)
    hidden = vk.embed(ids, W["model.embed_tokens.weight"], rt)
    residual = None
    for i in range(config["num_hidden_layers"]):
        p = f"model.layers.{i}."
        if residual is None:
            residual = hidden
            normed = vk.rms_norm(hidden, W[p + "input_layernorm.weight"], rt)
        else:
            normed, residual = vk.add_rms_norm(hidden, residual, W[p + "input_layernorm.weight"], rt)
        q, k, v = vk.qkv_linear(normed, W[p + "self_attn.q_proj.weight"], W[p + "self_attn.k_proj.weight"],
                                W[p + "self_attn.v_proj.weight"], rt)
        vv = vk.view_as_kv(v, rt)
        nq_, nk_ = vk.qk_norm(q, k, W[p + "self_attn.q_norm.weight"], W[p + "self_attn.k_norm.weight"], rt)
        rq, rk = vk.rotary_embed(positions, nq_, nk_, rt)
        k_cache = torch.full((pages, page_size, nkv, d), float("nan"))
        v_cache = torch.full((pages, page_size, nkv, d), float("nan"))
        k_cache.view(-1, nkv, d)[slots.long()] = rk.reshape(T, nkv, d)
        v_cache.view(-1, nkv, d)[slots.long()] = vv.reshape(T, nkv, d)
        attn = _sdpa_reference(rq.reshape(T, nq, d), k_cache, v_cache, cu_q, cu_q, T, T, block_table=block_table)
        proj = vk.linear(attn.reshape(T, nq * d), W[p + "self_attn.o_proj.weight"], rt)
        normed2, residual = vk.add_rms_norm(proj, residual, W[p + "post_attention_layernorm.weight"], rt)
        gate_up_w = torch.cat([W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"]], dim=0)
        mlp = vk.silu_and_mul(vk.linear(normed2, gate_up_w, rt), rt)
        hidden = vk.linear(mlp, W[p + "mlp.down_proj.weight"], rt)
    final, _ = vk.add_rms_norm(hidden, residual, W["model.norm.weight"], rt)
    head = W["model.embed_tokens.weight"] if config["tie_word_embeddings"] else W["lm_head.weight"]
    return vk.linear(final, head, rt).float()


def main():
    ref = Path(sys.argv[1])
    for sub in ("python", "", "kernels"):
        sys.path.insert(0, str(ref / sub))
    import plain_qwen3 as plain
    from tiny_configs import ALL
    from vosti_b200.weights import write_random_model

    for name in ("a", "b"):
        config, seed, page = ALL[name]
        with tempfile.TemporaryDirectory() as folder:
            write_random_model(folder, config, seed)
            cfg, W = plain.load_model(folder)
        gen = torch.Generator().manual_seed(100 + seed)
        tokens = torch.randint(0, config["vocab_size"], (37,), generator=gen).tolist()
        ours = plain.forward_logits(cfg, W, tokens)
        theirs = reference_logits(ref, cfg, W, tokens, page)
        diff = (ours - theirs).abs().max().item()
        print(f"tiny {name}: max |plain - reference| = {diff:.3e} (max |logit| {theirs.abs().max().item():.3f})")
        np.savez_compressed(Path(__file__).parent / f"qwen3_tiny_{name}.npz",
                            tokens=np.asarray(tokens, dtype=np.int32), logits=theirs.numpy().astype(np.float32))


if __name__ == "__main__":
    main()
