"""RMSNorm fused with the residual add.

``out = v / sqrt(mean(v^2) + eps) * weight`` with ``v = residual + branch``; eps is added to
the mean inside the root and the weight multiplies after normalisation
(Daisi.Llogos.Cpu/RmsNorm.cs:14-65; fused forms IComputeBackend.cs:417-438).  The residual
stream and the statistics are float32.

For a consumer that takes a row scale, bfloat16 models write ``v * weight`` and hand the division on as the
row's sum of squares (whole, or in parts that add up to it): a product is linear in its rows, so the consumer's
first product scales its result instead.  Nothing then has to see a whole row, and the few rows of a decode
step are spread over many blocks, each adding up the partial sums of its own columns.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import Branch, Norm, TensorDecl, register_part


class RmsNorm(Norm):
    """params: size, eps."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        if self.eps <= 0:
            raise ValueError("RMSNorm eps must be positive")
        self.weight: Optional[torch.Tensor] = None

    def tensors(self):
        return {"weight": TensorDecl((self.size,), "norm")}

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, residual, branch: Optional[Branch], ctx, rows=None):
        m = residual.shape[0] if rows is None else rows.numel()
        out = ctx.buffer("norm.out", (m, self.size))
        ctx.ops.add_rmsnorm(residual, branch.data if branch is not None else None, self.weight, self.eps, out, rows)
        return out

    def forward_unscaled(self, residual, branch: Optional[Branch], ctx, rows=None):
        ops = ctx.ops
        make_scale = getattr(ops, "RowScale", None)
        if make_scale is None or ctx.dtype != torch.bfloat16:
            return self.forward(residual, branch, ctx, rows), None
        m = residual.shape[0] if rows is None else rows.numel()
        out = ctx.buffer("norm.out", (m, self.size))
        ss = ctx.buffer("norm.ss", (m, ops.norm_ss_parts(m, self.size)), torch.float32)
        ops.add_rmsnorm(residual, branch.data if branch is not None else None, self.weight, self.eps, out, rows, ss_out=ss)
        return out, make_scale(ss, self.size, self.eps)


register_part("norm", "rmsnorm", RmsNorm)
