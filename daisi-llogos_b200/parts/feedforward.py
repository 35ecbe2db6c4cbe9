"""Feed-forward parts.

``SwiGLU``: ``down( silu(gate(x)) * up(x) )`` without biases
(Inference/ForwardPass.cs:242-246; silu(g) = g / (1 + exp(-g)), Daisi.Llogos.Cpu/Silu.cs:9-16).
The gate and up matrices are stored as one ``[2I, H]`` matrix so that one product feeds the
gating kernel.
"""
from __future__ import annotations

import torch

from ..kernels.linear import linear
from .base import Branch, FeedForward, TensorDecl, register_part

_CHUNK_TOKENS = 16384   # rows per pass, bounds the [tokens, 2I] scratch of long prompt steps


class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size."""

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
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"]

    def forward(self, x, ctx) -> Branch:
        n = x.shape[0]
        small = ctx.decode or n <= 64
        mid_dtype = torch.float32 if small else ctx.dtype
        if n <= _CHUNK_TOKENS:
            gu = linear(ctx, x, self.w_gate_up, "ffn.gate_up", mid_dtype)
            act = ctx.buffer("ffn.act", (n, self.inter))
            ctx.ops.silu_mul(gu, act)
            return Branch(linear(ctx, act, self.w_down, "ffn.out", torch.float32))
        out = ctx.buffer("ffn.out", (1, n, self.hidden), torch.float32)
        for r0 in range(0, n, _CHUNK_TOKENS):
            r1 = min(n, r0 + _CHUNK_TOKENS)
            gu = linear(ctx, x[r0:r1], self.w_gate_up, "ffn.gate_up", mid_dtype)
            act = ctx.buffer("ffn.act", (r1 - r0, self.inter))
            ctx.ops.silu_mul(gu, act)
            linear(ctx, act, self.w_down, "ffn.out.chunk", torch.float32, out=out[:, r0:r1])
        return Branch(out)


register_part("ffn", "swiglu", SwiGLU)
