"""Grouped-query attention over the paged cache, with optional per-head q/k RMSNorm
and an optional rotation, as one mixer.

Order of operations (src/exec/dense_swiglu_decoder.rs:171-367): q, k, v projections
without bias; per-head norm of q and k (not v) before the rotation; keys (normed and
rotated) and values are stored in the cache before the layer's attention, so a query
reads its own key through the cache; attention with scale `scale`, causal, optionally
limited to a window; output projection. Sizes and constants are parameters of the spec:
num_heads, num_kv_heads, head_dim, scale, window (0 = all keys), head_norm_eps (None =
no head norm), qkv_bias and o_bias (false for Qwen3, whose configuration must say
attention_bias=false; true adds `{q,k,v}_proj.bias` / `o_proj.bias` to the tensors the part
asks for, added to the float32 products before they are rounded).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec
from .base import Mixer, PagedCacheSpec, PositionEncoding, register_part, register_step_layout
from .linear import linear, prepare_weight


class Attention(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int, position: Optional[PositionEncoding]):
        super().__init__(spec, hidden_size, position)
        self.nq = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        self.scale = float(spec["scale"])
        self.window = int(spec.get("window", 0) or 0)
        eps = spec.get("head_norm_eps")
        self.head_norm_eps = None if eps is None else float(eps)
        if self.nq <= 0 or self.nkv <= 0 or self.nq % self.nkv:
            raise ConfigError(f"attention: num_heads {self.nq} must be a positive multiple of "
                              f"num_kv_heads {self.nkv}")
        if self.d <= 0 or self.d % 16 or self.d > 256:
            raise ConfigError(f"attention: head_dim {self.d} must be a multiple of 16, at most 256")
        if self.window < 0:
            raise ConfigError("attention: window must be >= 0")
        self.qkv_bias, self.o_bias = bool(spec.get("qkv_bias", False)), bool(spec.get("o_bias", False))
        self.w_qkv = self.w_q = self.w_o = self.q_norm = self.k_norm = self.b_qkv = self.b_o = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h, nq, nkv, d = self.hidden_size, self.nq, self.nkv, self.d
        specs = {
            "q_proj.weight": WeightSpec((nq * d, h)), "k_proj.weight": WeightSpec((nkv * d, h)),
            "v_proj.weight": WeightSpec((nkv * d, h)), "o_proj.weight": WeightSpec((h, nq * d)),
        }
        if self.head_norm_eps is not None:
            specs["q_norm.weight"] = WeightSpec((d,), init="norm", std=0.1)
            specs["k_norm.weight"] = WeightSpec((d,), init="norm", std=0.1)
        if self.qkv_bias:
            specs.update({"q_proj.bias": WeightSpec((nq * d,)), "k_proj.bias": WeightSpec((nkv * d,)),
                          "v_proj.bias": WeightSpec((nkv * d,))})
        if self.o_bias:
            specs["o_proj.bias"] = WeightSpec((h,))
        return specs

    def load(self, tensors, dtype):
        parts = [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]]
        common = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        # one [ (nq + 2 nkv) d, hidden ] matrix: the projection is a single product
        w_qkv = torch.cat([p.to(common) for p in parts], dim=0).contiguous()
        self.w_qkv = prepare_weight(w_qkv, dtype)
        # a layer that reads another layer's cache needs q only: the first rows of the matrix,
        # or (tile-packed weight) the whole product, whose k and v are then dropped
        self.w_q = w_qkv[: self.nq * self.d] if self.w_qkv is w_qkv else None
        self.w_o = prepare_weight(tensors["o_proj.weight"], dtype)
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors[f"{p}_proj.bias"].float() for p in "qkv"]).contiguous()
        if self.o_bias:
            self.b_o = tensors["o_proj.bias"]
        if self.head_norm_eps is not None:
            self.q_norm, self.k_norm = tensors["q_norm.weight"], tensors["k_norm.weight"]
            if self.q_norm.dtype != self.k_norm.dtype:
                self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()

    def setup(self, device, dtype):
        if self.position is not None:
            self.position.setup(device, dtype)

    def first_weight(self):
        return self.w_qkv

    def cache_spec(self) -> PagedCacheSpec:
        return PagedCacheSpec(entries=2, heads=self.nkv, width=self.d, window=self.window)

    def forward(self, ctx, x, cache, writes_cache: bool = True):
        group = ctx.group(cache.group)
        tables = self.position.rotation_tables() if self.position is not None else None
        cos, sin = tables if tables is not None else (None, None)
        eps = self.head_norm_eps if self.head_norm_eps is not None else 1.0
        rotary_dim = getattr(self.position, "rotary_dim", None) or self.d
        interleaved = bool(getattr(self.position, "interleaved", False))
        common = dict(nq=self.nq, head_dim=self.d, page_size=group.page_size, q_norm_w=self.q_norm, eps=eps, cos=cos, sin=sin,
                      positions=ctx.positions, status=ctx.status, rotary_dim=rotary_dim, interleaved=interleaved)
        if writes_cache:
            qkv = linear(ctx, x, self.w_qkv, allow_partial=True, bias=self.b_qkv)   # summed inside qkv_post
            if (ops.DECODE_FUSION and isinstance(qkv, ops.PartialSum) and qkv.dtype == torch.bfloat16
                    and ctx.layout["attention"]["num_short_tokens"] == ctx.num_tokens == ctx.num_requests
                    and self.nq // self.nkv <= 16 and cache.k.dtype == torch.bfloat16
                    and (cos is None or (rotary_dim == self.d and not interleaved))):
                # every request brings one token: head norm, rotation, cache store and attention in
                # one kernel, straight from the projection's partial sums
                attn = ops.attention_decode_fused(
                    qkv, cache.k, cache.v, positions=ctx.positions, request_of=ctx.request_of,
                    block_table=group.block_table, slot_mapping=group.slot_mapping, page_size=group.page_size,
                    nq=self.nq, nkv=self.nkv, head_dim=self.d, max_kv_len=ctx.max_kv_len, scale=self.scale,
                    window=self.window, q_norm_w=self.q_norm, k_norm_w=self.k_norm, eps=eps, cos=cos, sin=sin,
                    status=ctx.status)
                return linear(ctx, attn, self.w_o, allow_partial=True, bias=self.b_o)
            q = ops.qkv_post(qkv, cache.k, cache.v, nkv=self.nkv, k_norm_w=self.k_norm,
                             slot_mapping=group.slot_mapping, **common)
        elif self.w_q is not None:
            bias = None if self.b_qkv is None else self.b_qkv[: self.nq * self.d]
            q = ops.qkv_post(linear(ctx, x, self.w_q, bias=bias), None, None, nkv=0, k_norm_w=None,
                             slot_mapping=None, **common)
        else:
            q = ops.qkv_post(linear(ctx, x, self.w_qkv, allow_partial=True, bias=self.b_qkv), None, None, nkv=self.nkv,
                             k_norm_w=self.k_norm, slot_mapping=None, **common)
        attn = ops.attention(ctx, q, cache.k, cache.v, group, nq=self.nq, nkv=self.nkv, head_dim=self.d,
                             scale=self.scale, window=self.window)
        return linear(ctx, attn, self.w_o, allow_partial=True, bias=self.b_o)   # summed by the norm that follows


register_part("mixer", "attention", Attention, replace=True)
# the attention kernels' work lists are made with every step's layout
register_step_layout("attention", ops.attention_step_layout)
