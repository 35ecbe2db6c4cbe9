"""Choosing the matrix-product kernel for ``y[n, o] = sum_k x[n, k] w[o, k]``.

The result is returned as partials ``[S, N, O]`` that the consumer sums (S = 1 unless a
split-K kernel ran).  float32 operands always take the CUDA-core kernel (true 32-bit).
"""
from __future__ import annotations

import torch

from . import ops


def linear(ctx, x: torch.Tensor, w: torch.Tensor, name: str, out_dtype: torch.dtype,
           out: torch.Tensor = None) -> torch.Tensor:
    """``out`` (a ``[1, N, O]`` view) makes the product write there instead of into the named buffer."""
    n, k = x.shape
    o = w.shape[0]
    if out is None:
        out = ctx.buffer(name, (1, n, o), out_dtype)
    ctx.ops.gemm_simt(x, w, out[0])
    return out
