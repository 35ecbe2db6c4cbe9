"""How the GPU tests judge logits against the plain implementation.

float32: every logit within 2e-5 of the request's largest |logit| of the plain model.

bfloat16: against the exact plain model every logit within 4e-2 of the largest |logit| (this bounds the
rounding noise itself: measured 0.007 to 0.026 on the tiny configurations), and against the plain model
that rounds to bfloat16 where the engine does (``plain_model.forward(..., rounded=True)``):

* every logit within 1.5e-2 of the largest |logit| (measured: at most 0.0082), and
* where a check covers 16 positions or more, the root-mean-square error within 8e-3 of the reference's
  root mean square (measured: at most 0.0054), so that an error of one percent in every logit shows.

What remains between the engine and the rounding plain model is not a rounding that the plain model leaves
out (one layer of the smallest configuration agrees bit for bit in every intermediate tensor): it is the
order of the float32 sums.  The tensor cores add with truncation (a product over 4,096 terms is 4e-6 low,
relative, against 6e-7 for a chain of fused multiply-adds), a value that lies within that distance of a
bfloat16 tie rounds the other way, and one such value makes a few percent of the values downstream of it
round the other way too.  Per layer that adds about 1e-3 (root mean square, relative) to the logits.
The reference compares its backends' logits with 0.001 absolute in float32
(tests/Daisi.Llogos.Tests/Chat/LayerByLayerCompareTest.cs:110) and below 1.0 for a 16-bit cache
(tests/Daisi.Llogos.Tests/Inference/LongContextTests.cs:40).
"""
import torch

import plain_model as P

TOL_F32 = 2e-5
TOL_BF16_ROUNDED = 1.5e-2
TOL_BF16_ROUNDED_RMS = 8e-3
TOL_BF16_EXACT = 4e-2
RMS_ROWS = 16


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
        if exact > TOL_BF16_EXACT:
            return exact, TOL_BF16_EXACT
        ref = self.rounded[idx]
        if idx.numel() >= RMS_ROWS:
            rms = float((got - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt())
            if rms > TOL_BF16_ROUNDED_RMS:
                return rms, TOL_BF16_ROUNDED_RMS
        return float((got - ref).abs().max()) / self.scale, TOL_BF16_ROUNDED

    def check(self, got, positions, dtype, what=()):
        err, tol = self.errors(got, positions, dtype)
        assert err <= tol, (*what, "error", err, "bound", tol)
        return err
