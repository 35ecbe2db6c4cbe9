"""RMSNorm fused with the residual add.

``out = v / sqrt(mean(v^2) + eps) * weight`` with ``v = residual + branch``; eps is added to
the mean inside the root and the weight multiplies after normalisation
(Daisi.Llogos.Cpu/RmsNorm.cs:14-65; fused forms IComputeBackend.cs:417-438).  The residual
stream and the statistics are float32.
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


register_part("norm", "rmsnorm", RmsNorm)
