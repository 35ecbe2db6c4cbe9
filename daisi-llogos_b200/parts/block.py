"""Arrangements of norms, a mixer and a feed-forward around the residual stream.

``PreNormBlock`` is the reference's order (Inference/ForwardPass.cs:215-250): the output of the
previous feed-forward is added to the residual inside this block's first norm; the attention
output is added inside the second norm; the block returns its feed-forward output still to
be added (by the next block's first norm, or by the model's final norm).
"""
from __future__ import annotations

from typing import Optional

from .base import Block, Branch, register_part


class PreNormBlock(Block):
    """roles: norm1, mixer, norm2, ffn."""

    ROLES = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "ffn": "ffn"}

    def forward(self, residual, pending: Optional[Branch], ctx, cache) -> Optional[Branch]:
        p = self.parts
        h, kw = normed_for(p["norm1"], p["mixer"], residual, pending, ctx)
        a = p["mixer"].forward(h, ctx, cache, **kw)
        h, kw = normed_for(p["norm2"], p["ffn"], residual, a, ctx)
        return p["ffn"].forward(h, ctx, **kw)


def normed_for(norm, consumer, residual, pending, ctx, rows=None):
    """``(x, keyword arguments)`` for ``consumer.forward``: a consumer that takes a row scale lets the norm leave
    its division to the consumer's first product."""
    if getattr(consumer, "TAKES_ROW_SCALE", False):
        x, scale = norm.forward_unscaled(residual, pending, ctx, rows)
        return x, {"row_scale": scale}
    return norm.forward(residual, pending, ctx, rows), {}


register_part("block", "prenorm", PreNormBlock)
