"""Feed-forward parts.

``SwiGLU``: ``down( silu(gate(x)) * up(x) )`` without biases
(Inference/ForwardPass.cs:242-246; silu(g) = g / (1 + exp(-g)), Daisi.Llogos.Cpu/Silu.cs:9-16).
The gate and up matrices are stored as one matrix (gate rows, then up rows, each part filled up to a
multiple of 128 rows), so that the gating is the epilogue of one product.
"""
from __future__ import annotations

import torch

from ..kernels.linear import gated_layout, gated_linear, linear
from .base import Branch, FeedForward, TensorDecl, register_part


class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size."""

    TAKES_ROW_SCALE = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.w_gate_up = None
        self.w_down = None

    def tensors(self):
        return {
            "gate_proj.weight": TensorDecl((self.inter, self.hidden)),
            "up_proj.weight": TensorDecl((self.inter, self.hidden)),
            "down_proj.weight": TensorDecl((self.hidden, self.inter)),
        }

    def bind(self, tensors):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            raise ValueError(f"{self.prefix}: gate_proj and up_proj are stored with different types")
        self.w_gate_up = gated_layout(g, u)
        self.w_down = tensors["down_proj.weight"]

    def forward(self, x, ctx, row_scale=None) -> Branch:
        act = ctx.buffer("ffn.act", (x.shape[0], self.inter))
        gated_linear(ctx, x, self.w_gate_up, act, row_scale)
        return Branch(linear(ctx, act, self.w_down, "ffn.out", torch.float32))


register_part("ffn", "swiglu", SwiGLU)
