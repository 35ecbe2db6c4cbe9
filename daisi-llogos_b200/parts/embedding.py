"""Token embedding and output head.

The embedding copies one table row per token, unscaled, into the float32 residual stream
(Inference/ForwardPass.cs:205).  The head is a matrix product of the final norm's output with
the vocabulary matrix, which is the embedding table itself when the model ties them
(Model/ModelWeights.cs:29); logits are float32.
"""
from __future__ import annotations

import torch

from ..kernels.linear import linear
from .base import Part, TensorDecl, register_part


class TokenEmbedding(Part):
    """params: vocab_size, hidden_size."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.vocab, self.hidden), "table")}

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx) -> torch.Tensor:
        residual = ctx.buffer("residual", (ctx.n_tokens, self.hidden), torch.float32)
        ctx.ops.embed_rows(self.weight, ctx.token_ids, residual)
        return residual


class LinearHead(Part):
    """params: vocab_size, hidden_size, tied_to (full name of the tensor to share, or None)."""

    TAKES_ROW_SCALE = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.tied_to = params.get("tied_to")
        self.weight = None

    def tensors(self):
        if self.tied_to:
            return {}
        return {"weight": TensorDecl((self.vocab, self.hidden))}

    def bind(self, tensors):
        self.weight = tensors["weight"]
        if tuple(self.weight.shape) != (self.vocab, self.hidden):
            raise ValueError(f"output head: shared tensor has shape {tuple(self.weight.shape)}, "
                             f"expected {(self.vocab, self.hidden)}")

    def forward(self, x, ctx, row_scale=None) -> torch.Tensor:
        # the logits go to samplers and callers as they are: one product, no partial sums to add up
        return linear(ctx, x, self.weight, "head.logits", torch.float32, split_k=False, row_scale=row_scale)[0]


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "linear_head", LinearHead)
