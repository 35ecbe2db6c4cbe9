"""Choosing the matrix-product kernel for ``y[n, o] = sum_k x[n, k] w[o, k]``.

The result is returned as partials ``[S, N, O]`` that the consumer sums.  bfloat16 operands go to
the tensor-core kernel (tcgen05 + TMA, csrc/gemm_tc.cu); with few rows it splits K so that the
weight stream is spread over every SM.  float32 operands always take the CUDA-core kernel: the
true 32-bit path uses no tensor cores.
"""
from __future__ import annotations

import torch

_SMS = 148


def plan_splits(n: int, o: int, k: int) -> int:
    """Split-K wish for a product with few rows.

    ``tiles`` output tiles, each with ``nkb`` k-blocks of 64, are cut into ``s`` splits; the blocks run
    in ``ceil(tiles * s / resident)`` rounds (two blocks are resident per SM for token tiles up to 64)
    of ``ceil(nkb / s)`` k-blocks plus a fixed cost each.  The cheapest ``s`` wins, the smallest on
    ties: a last round with a few stragglers costs as much as a full one."""
    if n > 64:
        return 1
    tile_n = 16 if n <= 16 else 32 if n <= 32 else 64
    tiles = -(-o // 128) * -(-n // tile_n)
    nkb = -(-k // 64)
    resident = 2 * _SMS
    best, best_cost = 1, None
    for s in range(1, max(1, min(nkb // 4, 32)) + 1):
        cost = -(-tiles * s // resident) * (-(-nkb // s) + 3)
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


def linear(ctx, x: torch.Tensor, w: torch.Tensor, name: str, out_dtype: torch.dtype,
           out: torch.Tensor = None) -> torch.Tensor:
    """``out`` (a ``[1, N, O]`` view) makes the product write there instead of into the named buffer."""
    ops = ctx.ops
    n, k = x.shape
    o = w.shape[0]
    tc = getattr(ops, "gemm_tc_supported", None)
    if tc is not None and tc(x, w):
        splits = 1
        if out is None and out_dtype == torch.float32:
            splits = ops.gemm_tc_splits(k, plan_splits(n, o, k))
        if out is None:
            out = ctx.buffer(name, (splits, n, o), out_dtype)
        ops.gemm_tc(x, w, out)
        return out
    if out is None:
        out = ctx.buffer(name, (1, n, o), out_dtype)
    ops.gemm_simt(x, w, out[0])
    return out
