"""Matrix product y = x @ w.T for the parts, choosing the kernel by operand types.

bfloat16 x bfloat16 goes to the tensor-core kernel when it takes the sizes; every
other combination (the float32 path, a 32-bit weight under bfloat16 serving, sizes
the tensor-core kernel refuses) goes to the CUDA-core kernel with float32 arithmetic.
The choice depends on types and on (N, K) only, never on the number of rows.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import ops

# VOSTI_PACK_WEIGHTS=0 keeps weights row-major (for comparisons; the results are the same bits).
PACK_WEIGHTS = os.environ.get("VOSTI_PACK_WEIGHTS", "1") != "0"


def uses_tensor_cores(x_dtype: torch.dtype, w) -> bool:
    return (x_dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_cuda
            and ops.gemm_tc_supported(w.shape[0], w.shape[1]))


def prepare_weight(w: torch.Tensor, serving_dtype: torch.dtype):
    """What a part keeps of a [features, k] weight it only ever multiplies with: the
    tile-packed copy if the tensor-core product will read it, else the tensor itself. A
    weight that is also read by rows (a tied embedding table) must stay a tensor."""
    if PACK_WEIGHTS and isinstance(w, torch.Tensor) and uses_tensor_cores(serving_dtype, w):
        return ops.PackedWeight(w)
    return w


def linear(ctx, x: torch.Tensor, w: torch.Tensor, *, out_dtype: Optional[torch.dtype] = None,
           row_index: Optional[torch.Tensor] = None, allow_partial: bool = False,
           bias: Optional[torch.Tensor] = None):
    """y = x @ w.T (+ bias). With `allow_partial` the result may come back as an `ops.PartialSum`
    (the K splits not yet summed) for a consumer that adds them itself; the caller must hand it
    to such a consumer, or to `ops.materialize`, before any other product runs. With a `bias`
    (a vector of w's row count, float32 or bfloat16) the product is taken in float32, the bias
    is added there and the sum is rounded once; such a result is never partial."""
    x = ops.materialize(x)
    if bias is not None:
        if bias.dim() != 1 or bias.shape[0] != w.shape[0]:
            raise ops.KernelError(f"linear: bias has shape {tuple(bias.shape)}, the weight has {w.shape[0]} rows")
        product = linear(ctx, x, w, out_dtype=torch.float32, row_index=row_index)
        return ops.affine_rows(product, bias=bias, out_dtype=out_dtype or x.dtype)
    if isinstance(w, ops.PackedWeight) and x.dtype != torch.bfloat16:
        raise ops.KernelError("a tile-packed weight serves bfloat16 activations only")
    if uses_tensor_cores(x.dtype, w):
        if row_index is not None:
            x = ops.gather_rows(x, row_index, ctx.status)
        return ops.gemm_tc(x, w, ctx.status, out_dtype=out_dtype, allow_partial=allow_partial)
    return ops.gemm_simt(x, w, ctx.status, out_dtype=out_dtype, row_index=row_index)
