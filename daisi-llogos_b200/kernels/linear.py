"""Choosing the matrix-product kernel for ``y[n, o] = sum_k x[n, k] w[o, k]``.

The result is returned as partials ``[S, N, O]`` that the consumer sums.  bfloat16 operands go to
the tensor-core kernel (tcgen05 + TMA, csrc/gemm_tc.cu); with few rows it splits K so that the
weight stream is spread over every SM.  float32 operands always take the CUDA-core kernel: the
true 32-bit path uses no tensor cores.
"""
from __future__ import annotations

import torch

_plan_cache = {}

# What one block of the small-tile product streams when it runs alone on its multiprocessor: a ring of
# five 18 KB stages (about 80 KB in flight) against a memory latency near 1.8 us, measured on a B200 as
# 43-47 GB/s per block (one o-projection tile column timed alone).  Only ratios of costs matter below.
_BLOCK_BYTES_PER_US = 45e3
# Rate at which split-K partials are written and read back by the consumer kernel: L2-resident float32
# traffic, measured near 4 TB/s for the [S, N, O] buffers of a decode step.
_PARTIAL_BYTES_PER_US = 4e6


def plan_splits(n: int, o: int, k: int, n_sms: int) -> int:
    s = _plan_cache.get((n, o, k, n_sms))
    if s is None:
        s = _plan_cache[(n, o, k, n_sms)] = _plan_splits(n, o, k, n_sms)
    return s


def _plan_splits(n: int, o: int, k: int, n_sms: int) -> int:
    """Split-K wish for a product with few enough rows that streaming the weights is what takes the time.

    ``tiles`` output tiles, each with ``nkb`` k-blocks of 64, are cut into ``s`` splits; the blocks run
    in ``ceil(tiles * s / resident)`` rounds of ``ceil(nkb / s)`` k-blocks plus a fixed cost each, and
    the ``s`` partial results are written and read once more.  The cheapest ``s`` wins, the smallest on
    ties: a last round with a few stragglers costs as much as a full one.  The tile shapes and the
    blocks per SM are those the kernel takes for ``n`` rows (csrc/gemm_tc.cu)."""
    if n > SPLIT_ROWS_MAX:
        return 1
    nkb = -(-k // 64)
    if n >= 256:                  # tokens are the MMA rows: 128 tokens x 256 features per tile, one block per SM
        tiles, tile_bytes, resident = -(-n // 128) * -(-o // 256), (128 + 256) * 128, n_sms
    else:                         # weights are the MMA rows: 128 features x a token tile
        tile_n = 16 if n <= 16 else 32 if n <= 32 else 64 if n <= 64 else 128 if n <= 128 else 256
        tiles, tile_bytes = -(-o // 128) * -(-n // tile_n), (128 + tile_n) * 128
        resident = 2 * n_sms if tile_n <= 64 else n_sms
    unit_us = tile_bytes / _BLOCK_BYTES_PER_US
    best, best_cost = 1, None
    for s in range(1, max(1, min(nkb // 4, 32)) + 1):
        cost = -(-tiles * s // resident) * (-(-nkb // s) + 3) * unit_us
        if s > 1:
            cost += s * n * o * 8 / _PARTIAL_BYTES_PER_US      # the partials, out and in again
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


SPLIT_ROWS_MAX = 512    # with more rows the products are bound by arithmetic and one split is right


def linear(ctx, x: torch.Tensor, w: torch.Tensor, name: str, out_dtype: torch.dtype,
           out: torch.Tensor = None, split_k: bool = True, row_scale=None) -> torch.Tensor:
    """``out`` (a ``[1, N, O]`` view) makes the product write there instead of into the named buffer.
    ``split_k=False`` is for a caller that does not sum partials: the result is ``[1, N, O]``.
    ``row_scale``: what a norm left for the rows of ``x`` (``ops.RowScale``); the product's rows are multiplied by it."""
    ops = ctx.ops
    n, k = x.shape
    o = w.shape[0]
    tc = getattr(ops, "gemm_tc_supported", None)
    if tc is not None and tc(x, w):
        splits = 1
        if out is None and out_dtype == torch.float32 and split_k:
            splits = ops.gemm_tc_splits(k, plan_splits(n, o, k, ops.sm_count()))
        if out is None:
            out = ctx.buffer(name, (splits, n, o), out_dtype)
        if row_scale is not None:
            ops.gemm_tc(x, w, out, row_scale=row_scale)
        else:
            ops.gemm_tc(x, w, out)
        return out
    if out is None:
        out = ctx.buffer(name, (1, n, o), out_dtype)
    if row_scale is not None:
        ops.gemm_simt(x, w, out[0], row_scale=row_scale)
    else:
        ops.gemm_simt(x, w, out[0])
    return out


_GATED_CHUNK = 16384   # rows per pass of the two-kernel path, bounds its [rows, 2I] scratch


def gated_layout(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """One matrix ``[2 P, hidden]``, P = the feature count rounded up to a multiple of 128: the gate rows,
    zero rows up to P, then the up rows in the same way."""
    inter, hidden = gate.shape
    pad = -(-inter // 128) * 128
    out = torch.zeros((2, pad, hidden), dtype=gate.dtype, device=gate.device)
    out[0, :inter] = gate
    out[1, :inter] = up
    return out.view(2 * pad, hidden)


def gated_linear(ctx, x: torch.Tensor, w_gated: torch.Tensor, out: torch.Tensor, row_scale=None) -> None:
    """out[n, i] = silu(x . gate_i) * (x . up_i) for a gate/up matrix in ``gated_layout``.

    On the tensor cores the gating is the epilogue of the product; otherwise the product writes
    gate and up values and the gating kernel follows.  ``row_scale`` as in ``linear``: both products' rows are
    multiplied by it before the gating."""
    ops = ctx.ops
    n = x.shape[0]
    rows = w_gated.shape[0]
    tc = getattr(ops, "gemm_tc_supported", None)
    if tc is not None and tc(x, w_gated) and out.dtype == torch.bfloat16:
        if row_scale is not None:
            ops.gemm_tc(x, w_gated, out.unsqueeze(0), gated_features=out.shape[1], row_scale=row_scale)
        else:
            ops.gemm_tc(x, w_gated, out.unsqueeze(0), gated_features=out.shape[1])
        return
    for r0 in range(0, n, _GATED_CHUNK):
        r1 = min(n, r0 + _GATED_CHUNK)
        gu = ctx.buffer("ffn.gate_up", (1, r1 - r0, rows), x.dtype)
        if row_scale is not None:
            ops.gemm_simt(x[r0:r1], w_gated, gu[0], row_scale=row_scale.slice(r0, r1))
        else:
            ops.gemm_simt(x[r0:r1], w_gated, gu[0])
        ops.silu_mul(gu, out[r0:r1])
