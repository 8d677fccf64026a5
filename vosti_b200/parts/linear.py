"""Matrix product y = x @ w.T for the parts, choosing the kernel by operand types.

bfloat16 x bfloat16 goes to the tensor-core kernel when it takes the sizes; every
other combination (the float32 path, a 32-bit weight under bfloat16 serving, sizes
the tensor-core kernel refuses) goes to the CUDA-core kernel with float32 arithmetic.
The choice depends on types and on (N, K) only, never on the number of rows.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops


def uses_tensor_cores(x_dtype: torch.dtype, w: torch.Tensor) -> bool:
    return (x_dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_cuda
            and ops.gemm_tc_supported(w.shape[0], w.shape[1]))


def linear(ctx, x: torch.Tensor, w: torch.Tensor, *, out_dtype: Optional[torch.dtype] = None,
           row_index: Optional[torch.Tensor] = None, allow_partial: bool = False):
    """y = x @ w.T. With `allow_partial` the result may come back as an `ops.PartialSum` (the
    K splits not yet summed) for a consumer that adds them itself; the caller must hand it to
    such a consumer, or to `ops.materialize`, before any other product runs."""
    x = ops.materialize(x)
    if uses_tensor_cores(x.dtype, w):
        if row_index is not None:
            x = ops.gather_rows(x, row_index, ctx.status)
        return ops.gemm_tc(x, w, ctx.status, out_dtype=out_dtype, allow_partial=allow_partial)
    return ops.gemm_simt(x, w, ctx.status, out_dtype=out_dtype, row_index=row_index)
