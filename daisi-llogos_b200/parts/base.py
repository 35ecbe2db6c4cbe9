"""Interfaces of the parts a model is put together from, and their registries.

A part knows its own sizes and constants (its ``params``), declares the tensors
it needs under its name prefix, and runs on packed tokens.  It does not know
which model it is in, which layer it is, or what the other parts are.  The five
kinds:

* ``Norm``             - ``forward(residual, branch, ctx, rows=None) -> x``: adds the pending
  branch output into the float32 residual stream and returns the normalised rows.
* ``Mixer``            - ``forward(x, ctx, cache) -> Branch``: mixes tokens of one sequence
  (attention here); may keep keys/values or fixed-size state per sequence.
* ``FeedForward``      - ``forward(x, ctx) -> Branch``: per-token transformation.

One optional refinement: a consumer that sets ``TAKES_ROW_SCALE`` gets ``row_scale=`` beside ``x``, and the norm
may then leave its division by the root mean square to the consumer's first product (``Norm.forward_unscaled``): a
product is linear in its rows.  A norm that does so needs no whole row in one place, so the few rows of a decode
step can be spread over many blocks that never wait for one another.
* ``PositionEncoding`` - gives mixers a rotation table and/or adds to the embeddings.
* ``Block``            - arranges norms, a mixer and a feed-forward around the residual stream.

The reference has one hard-wired arrangement (Inference/ForwardPass.cs:199-267);
its fused ops ``AddRmsNormResidual`` / ``AddRmsNorm`` (IComputeBackend.cs:417-438)
are the ``Norm.forward`` contract here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class TensorDecl:
    """A tensor a part needs: its shape and what it is (decides random initialisation)."""

    shape: Tuple[int, ...]
    role: str = "matrix"       # "matrix" | "norm" | "bias" | "table"
    optional: bool = False


@dataclass
class Branch:
    """Output of a mixer or feed-forward that has not been added to the residual stream yet.

    ``data`` is ``[n_partials, n_tokens, hidden]``; the partials (split-K slices of a
    matrix product, in float32) are summed by whoever consumes the branch.
    """

    data: torch.Tensor

    @property
    def n_partials(self) -> int:
        return self.data.shape[0]


@dataclass(frozen=True)
class KvNeed:
    """A mixer keeps keys and values per position: ``window`` = 0 for all of them."""

    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """A mixer keeps a fixed-size state per sequence, zeroed when a sequence starts."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Base of all parts.  ``params`` holds every size and constant; ``prefix`` the tensor names."""

    def __init__(self, params: Dict[str, Any], prefix: str, env: "BuildEnv"):
        self.params = dict(params)
        self.prefix = prefix
        self.env = env

    def tensors(self) -> Dict[str, TensorDecl]:
        """Tensor name (relative to the prefix) -> declaration."""
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receive the loaded tensors (same relative names); fuse or re-lay-out here."""

    def cache_need(self):
        return None


class Norm(Part):
    def forward(self, residual, branch: Optional[Branch], ctx, rows=None) -> torch.Tensor:
        raise NotImplementedError

    def forward_unscaled(self, residual, branch: Optional[Branch], ctx, rows=None):
        """``(x, row_scale)``: like ``forward``, but the norm may leave a per-row factor to the consumer
        (``row_scale``, a ``kernels.ops.RowScale``, or ``None`` when ``x`` is finished).  Called instead of
        ``forward`` for a consumer that sets ``TAKES_ROW_SCALE``."""
        return self.forward(residual, branch, ctx, rows), None


class Mixer(Part):
    TAKES_ROW_SCALE = False     # True: ``forward`` accepts ``row_scale=`` and applies it to the rows of ``x``

    def forward(self, x, ctx, cache) -> Branch:
        raise NotImplementedError

    def check_borrowed(self, need) -> None:
        """Called when the model is built for a mixer whose schedule entry reads another entry's cache
        (``cache_of``): ``need`` is what the owner keeps.  Raise ``ValueError`` if this mixer cannot read it."""


class FeedForward(Part):
    TAKES_ROW_SCALE = False     # as for ``Mixer``

    def forward(self, x, ctx) -> Branch:
        raise NotImplementedError


class PositionEncoding(Part):
    def prepare(self, max_positions: int) -> None:
        """Build tables for positions ``[0, max_positions)``.  May be called again with another number (a
        second engine on the same model): tables only grow, and one that a step may still read stays alive."""

    def limit(self) -> Optional[int]:
        """Positions the tables built so far cover (``None``: no limit)."""
        return None

    def rotation(self):
        """``None`` or a ``Rotation`` that a mixer applies to its queries and keys."""
        return None

    def on_embeddings(self, residual, ctx) -> None:
        """Hook for encodings that are added to the embeddings (default: nothing)."""


class Block(Part):
    """``ROLES`` names the roles this arrangement has and the family each role's part is looked up in
    (``{"norm1": "norm", "mixer": "mixer", ...}``).  A layer's ``PartSpec`` may also carry its family
    itself; that wins, and lets a spec give a block a role that its class did not list."""

    ROLES: Dict[str, str] = {}

    def __init__(self, params, prefix, env, parts: Dict[str, Part]):
        super().__init__(params, prefix, env)
        self.parts = parts

    def forward(self, residual, pending: Optional[Branch], ctx, cache) -> Optional[Branch]:
        raise NotImplementedError

    def cache_parts(self):
        """The parts of this block that keep something per sequence (at most one: an entry of the run order
        has one cache unit)."""
        keepers = [p for p in self.parts.values() if p.cache_need() is not None]
        if len(keepers) > 1:
            raise ValueError("a block may hold only one part that keeps a cache or a state per sequence")
        return keepers

    def cache_need(self):
        keepers = self.cache_parts()
        return keepers[0].cache_need() if keepers else None


@dataclass
class BuildEnv:
    """What a part gets at construction: the compute dtype, the device, the kernels, shared encodings."""

    dtype: torch.dtype
    device: torch.device
    ops: Any
    encodings: Dict[str, PositionEncoding]


_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "norm": {}, "mixer": {}, "ffn": {}, "position": {}, "block": {}, "embedding": {}, "head": {},
}


def register_part(family: str, kind: str, cls, *, replace: bool = False) -> None:
    """Make ``kind`` available to model specs; ``family`` is one of the registry names."""
    reg = _REGISTRIES[family]
    if kind in reg and not replace:
        raise ValueError(f"{family} part '{kind}' is already registered")
    reg[kind] = cls


def unregister_part(family: str, kind: str) -> None:
    _REGISTRIES[family].pop(kind, None)


def part_class(family: str, kind: str):
    reg = _REGISTRIES[family]
    if kind not in reg:
        raise KeyError(f"no {family} part named '{kind}' (known: {', '.join(sorted(reg)) or 'none'})")
    return reg[kind]


def part_families():
    return tuple(_REGISTRIES)
