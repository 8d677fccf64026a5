"""The reference arm of bench.py: the unmodified reference (QDelta/Vosti) measured on the same
metric and configuration, through its own public Python API and stock code path.

The reference's engine is a Rust crate that calls the Python package `vosti_kernels` through
pyo3 for every tensor operation; the crate cannot be built offline (no cargo, crates from the
network), but the package is the reference's documented primitive surface
(python/vosti_kernels/__init__.py) and runs as it is: `load_runtime` loads the reference's
Triton kernels with its own source attestation and binds the launch tiles of its `qwen3-8b`
profile (python/vosti_kernels/model_families/qwen3/scope.json). This module only does what
the Rust side does around those calls: it keeps the page tables, builds a step's index
tensors with the reference's materializers (`token_tensor`, `position_tensor`, `slot_tensor`,
`block_tables_tensor`, `seq_lens_tensor`), calls the primitives in the order of
src/exec/dense_swiglu_model.rs:271-319 and src/exec/dense_swiglu_decoder.rs:171-427 (the
`*_from_verified_caller` forms the Rust boundary uses, src/boundary/tensor_runtime.rs:4625,
4766), samples with `sample_tokens_rows`, and replays decode steps through the reference's
`CudaGraphOverlay` with its probe / capture / replay protocol
(src/boundary/model_forward_graph.rs). Nothing of vosti_b200 is imported here.

The reference tree is looked for under baseline/_ref/reference (the offline "install": a
copy of the checkout's python/ and kernels/ folders, because the project declares no
installable Python package).
"""
from __future__ import annotations

import os
import shutil
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref", "reference")
PAGE = 64          # the reference's fixed page size (python/vosti_kernels/physical.py)


def install(source: str = "") -> str:
    """Copy the parts of the reference checkout that run (python/, kernels/) under
    baseline/_ref/reference, unmodified, from `source` or the folder VOSTI_REFERENCE_CHECKOUT
    names. Returns the root; does nothing if the copy is there already."""
    if os.path.isdir(os.path.join(REF_ROOT, "python", "vosti_kernels")):
        return REF_ROOT
    source = source or os.environ.get("VOSTI_REFERENCE_CHECKOUT", "")
    if not source or not os.path.isdir(os.path.join(source, "python", "vosti_kernels")):
        raise FileNotFoundError(f"the reference is not installed under {REF_ROOT}; name its checkout in "
                                f"VOSTI_REFERENCE_CHECKOUT and call baseline.reference_arm.install()")
    os.makedirs(REF_ROOT, exist_ok=True)
    for sub in ("python", "kernels"):
        shutil.copytree(os.path.join(source, sub), os.path.join(REF_ROOT, sub), dirs_exist_ok=True,
                        ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return REF_ROOT


class ReferenceModel:
    """Random Qwen3 weights and KV caches for the reference's runtime, and one `forward`
    that is the reference's model_forward."""

    def __init__(self, profile: str, layers: int, token_capacity: int, seed: int = 0):
        import torch
        root = install()
        # the checkout's root (for `kernels.triton_kernels`) and its python/ folder (for `vosti_kernels`)
        for folder in (root, os.path.join(root, "python")):
            if folder not in sys.path:
                sys.path.insert(0, folder)
        import vosti_kernels as vk
        from vosti_kernels.graph_overlay import CudaGraphOverlay
        from vosti_kernels.model_families.qwen3 import runtime as qwen3_runtime

        self.torch, self.vk = torch, vk
        self.config = qwen3_runtime.config_for_profile(profile)
        self.runtime = qwen3_runtime.load_runtime(
            self.config, kernel_root=os.path.join(root, "kernels"), framework_root=root, device="cuda:0",
            dtype=torch.bfloat16)
        self.overlay = CudaGraphOverlay()
        c = self.config
        self.layers = layers or c["num_hidden_layers"]
        H, I, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
        nq, nkv, d = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        gen = torch.Generator(device="cuda:0").manual_seed(seed)
        dev = "cuda:0"

        def linear(rows, cols):
            return (torch.randn(rows, cols, device=dev, generator=gen, dtype=torch.float32) * 0.02).bfloat16()

        def norm(width):
            return (1.0 + 0.1 * torch.randn(width, device=dev, generator=gen, dtype=torch.float32)).bfloat16()

        self.embed = linear(V, H)
        self.head = self.embed if c["tie_word_embeddings"] else linear(V, H)
        self.final_norm = norm(H)
        self.blocks = []
        for _ in range(self.layers):
            self.blocks.append(dict(
                input_norm=norm(H), post_norm=norm(H), q=linear(nq * d, H), k=linear(nkv * d, H), v=linear(nkv * d, H),
                o=linear(H, nq * d), q_norm=norm(d), k_norm=norm(d),
                gate_up=linear(2 * I, H),      # gate rows, then up rows (model_families/qwen3/loader.py:55-58)
                down=linear(H, I)))
        self.caches = vk.init_kv_caches(self.layers, token_capacity, self.runtime)
        self.num_pages = int(self.caches[0][0].shape[0])
        self.free_pages = list(range(self.num_pages - 1, 0, -1))     # page 0 stays the padding sentinel
        self.weight_bytes = sum(t.numel() * 2 for b in self.blocks for t in b.values()) + self.final_norm.numel() * 2 \
            + self.head.numel() * 2
        self.kv_bytes_per_token = self.layers * 2 * nkv * d * 2

    # ---- the model forward (src/exec/dense_swiglu_model.rs:271-319)
    def forward(self, input_ids, positions, slot_mapping, cu_q, cu_k, max_q, max_k, block_table):
        vk, rt = self.vk, self.runtime
        hidden = vk.embed(input_ids, self.embed, rt)
        residual = None
        for w, (k_cache, v_cache) in zip(self.blocks, self.caches):
            if residual is None:
                residual = hidden
                normed = vk.rms_norm(hidden, w["input_norm"], rt)
            else:
                normed, residual = vk.add_rms_norm(hidden, residual, w["input_norm"], rt)
            q, k, v = vk.qkv_linear(normed, w["q"], w["k"], w["v"], rt)
            vv = vk.view_as_kv(v, rt)
            nq, nk = vk.qk_norm(q, k, w["q_norm"], w["k_norm"], rt)
            rq, rk = vk.rotary_embed(positions, nq, nk, rt)
            vk.store_kv_cache_from_verified_caller(rk, vv, k_cache, v_cache, slot_mapping, rt)
            attn = vk.paged_attention_from_verified_caller(rq, k_cache, v_cache, cu_q, cu_k, max_q, max_k,
                                                           block_table, rt)
            projected = vk.linear(attn, w["o"], rt)
            normed2, residual = vk.add_rms_norm(projected, residual, w["post_norm"], rt)
            mlp = vk.silu_and_mul(vk.linear(normed2, w["gate_up"], rt), rt)
            hidden = vk.linear(mlp, w["down"], rt)
        final, _ = vk.add_rms_norm(hidden, residual, self.final_norm, rt)
        selected = vk.select_rows_for_sampling(final, cu_q)
        return vk.linear(selected, self.head, rt)

    # ---- a step as the engine runs it: host lists in, host tokens out
    def step(self, requests, tokens_of, decode: bool):
        """`requests`: dicts with 'pages' and 'length'; `tokens_of[i]`: the tokens request i
        brings. Extends the page tables, materializes the index tensors, runs the forward
        (through the graph overlay for decode steps) and returns the sampled tokens."""
        vk, rt = self.vk, self.runtime
        ids, positions, slots, cu_q, cu_k = [], [], [], [0], [0]
        for request, tokens in zip(requests, tokens_of):
            start = request["length"]
            need = (start + len(tokens) + PAGE - 1) // PAGE
            while len(request["pages"]) < need:
                request["pages"].append(self.free_pages.pop())
            for j, token in enumerate(tokens):
                pos = start + j
                ids.append(int(token))
                positions.append(pos)
                slots.append(request["pages"][pos // PAGE] * PAGE + pos % PAGE)
            request["length"] = start + len(tokens)
            cu_q.append(cu_q[-1] + len(tokens))
            cu_k.append(cu_k[-1] + request["length"])
        max_q = max(len(t) for t in tokens_of)
        max_k = max(r["length"] for r in requests)
        tensors = (vk.token_tensor(ids, runtime=rt), vk.position_tensor(positions, runtime=rt),
                   vk.slot_tensor(slots, runtime=rt), vk.seq_lens_tensor(cu_q, runtime=rt),
                   vk.seq_lens_tensor(cu_k, runtime=rt),
                   vk.block_tables_tensor([r["pages"] for r in requests], runtime=rt))
        input_ids, pos_t, slot_t, cu_q_t, cu_k_t, table = tensors
        if not decode:
            logits = self.forward(input_ids, pos_t, slot_t, cu_q_t, cu_k_t, max_q, max_k, table)
        else:
            overlay = self.overlay
            signature = (1, len(ids), len(requests), max_q, int(table.shape[1]))
            action = overlay.probe(*signature)
            if action == overlay.REPLAY:
                logits = overlay.replay(1, max_q, input_ids, pos_t, slot_t, cu_q_t, cu_k_t, table)
            elif action == overlay.CAPTURE:
                overlay.capture_begin(*signature, input_ids)
                logits = self.forward(input_ids, pos_t, slot_t, cu_q_t, cu_k_t, max_q, max_k, table)
                logits = overlay.capture_end_and_replay(input_ids, pos_t, slot_t, cu_q_t, cu_k_t, table, logits)
            else:
                logits = self.forward(input_ids, pos_t, slot_t, cu_q_t, cu_k_t, max_q, max_k, table)
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in tensors)
        return vk.sample_tokens_rows(logits)

    def release(self, requests):
        for request in requests:
            self.free_pages.extend(reversed(request["pages"]))
            request["pages"], request["length"] = [], 0


def _prompts(count, length, vocab, seed):
    import torch
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=gen).tolist() for _ in range(count)]


def decode_run(model, batch, context, steps, warmup, seed):
    """Prefill `batch` requests of `context` tokens one by one, then time decode steps: with
    CUDA events, and by the wall clock (host tokens in, host tokens out, both inside)."""
    torch = model.torch
    vocab = model.config["vocab_size"]
    requests = [{"pages": [], "length": 0} for _ in range(batch)]
    last = []
    for request, prompt in zip(requests, _prompts(batch, context, vocab, seed)):
        last.append(model.step([request], [prompt], decode=False)[0])
    # (a graph is captured per block-table width, so a run that crosses into a new 64-token page
    # pays one eager step and one capture there, as the reference's engine does)
    for _ in range(warmup + 2):                       # eager, capture, then replays
        last = model.step(requests, [[t] for t in last], decode=True)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record()
    for _ in range(steps):
        last = model.step(requests, [[t] for t in last], decode=True)
    end.record()
    torch.cuda.synchronize()
    device_ms = begin.elapsed_time(end) / steps
    wall = time.perf_counter()
    for _ in range(steps):
        last = model.step(requests, [[t] for t in last], decode=True)
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - wall) * 1e3 / steps
    length = requests[0]["length"]
    h2d = model.h2d_bytes
    model.release(requests)
    return {"device_ms": device_ms, "wall_ms": wall_ms, "h2d": h2d, "d2h": 8 * batch, "context": length - steps}


def prefill_run(model, context, repeats, seed):
    torch = model.torch
    times = []
    for prompt in _prompts(repeats, context, model.config["vocab_size"], seed):
        request = {"pages": [], "length": 0}
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        model.step([request], [prompt], decode=False)
        end.record()
        torch.cuda.synchronize()
        times.append(begin.elapsed_time(end))
        model.release([request])
    return sorted(times[1:])[len(times[1:]) // 2] if len(times) > 1 else times[0]
