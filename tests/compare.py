"""How the GPU tests judge logits against the plain implementation.

float32: every logit within 2e-5 of the request's largest |logit| of the plain model.
bfloat16: two lines.  Against the plain model that rounds to bfloat16 where the engine does
(``plain_model.forward(..., rounded=True)``) the bound is 1e-2 of the largest |logit|: what remains
between the two is the order of the sums and a softmax weight rounded on the other side of a tie.
Against the exact plain model the looser 4e-2 holds as well, which bounds the rounding noise itself.
The reference compares its backends' logits with 0.001 absolute in float32
(tests/Daisi.Llogos.Tests/Chat/LayerByLayerCompareTest.cs:110) and below 1.0 for a 16-bit cache
(tests/Daisi.Llogos.Tests/Inference/LongContextTests.cs:40).
"""
import torch

import plain_model as P

TOL_F32 = 2e-5
TOL_BF16_ROUNDED = 1e-2
TOL_BF16_EXACT = 4e-2


_kept = {}


def reference(key, weights, cfg, tokens):
    """A ``Reference`` that is worked out once per (key, tokens); ``key`` stands for the weights (a model
    folder's path), so that the float32 and the bfloat16 run of a test share the plain model's work."""
    k = (key, tuple(tokens))
    if k not in _kept:
        if len(_kept) > 400:
            _kept.clear()
        _kept[k] = Reference(weights, cfg, tokens)
    return _kept[k]


class Reference:
    """Plain logits of one whole request: ``exact`` always, ``rounded`` when a bfloat16 check first asks."""

    def __init__(self, weights, cfg, tokens):
        self.weights, self.cfg, self.tokens = weights, cfg, list(tokens)
        self.exact = P.forward(weights, cfg, self.tokens)
        self.scale = float(self.exact.abs().max())
        self._rounded = None

    @property
    def rounded(self):
        if self._rounded is None:
            self._rounded = P.forward(self.weights, self.cfg, self.tokens, rounded=True)
        return self._rounded

    def errors(self, got, positions, dtype):
        """(error against the line that decides, its bound), both relative to the request's scale."""
        got = got.detach().to("cpu", torch.float64).reshape(-1, self.exact.shape[1])
        idx = torch.as_tensor(list(positions), dtype=torch.long)
        assert got.shape[0] == idx.numel(), (got.shape, idx.numel())
        exact = float((got - self.exact[idx]).abs().max()) / self.scale
        if dtype == torch.float32:
            return exact, TOL_F32
        rounded = float((got - self.rounded[idx]).abs().max()) / self.scale
        if exact > TOL_BF16_EXACT:
            return exact, TOL_BF16_EXACT
        return rounded, TOL_BF16_ROUNDED

    def check(self, got, positions, dtype, what=()):
        err, tol = self.errors(got, positions, dtype)
        assert err <= tol, (*what, "error", err, "bound", tol)
        return err
