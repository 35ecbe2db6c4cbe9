"""Position encodings.

``RotaryEncoding`` owns the cos/sin tables of rotary position encoding.  Frequencies
and angles are computed in float64 on the host, as the reference does
(Daisi.Llogos.Cpu/Rope.cs:131-162: ``freq_i = 1 / theta^(2i/rotary_dim)``,
``angle = position * freq_i``), and stored as float32.  The rotation itself happens
inside the mixer's fused query/key kernel; ``pairing`` says which elements form a
pair: "half" pairs ``(i, i + rotary_dim/2)`` (Rope.cs:42-63, the layout of
safetensors checkpoints), "adjacent" pairs ``(2i, 2i+1)`` (Rope.cs:150-161, the layout
of converted GGUF files).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .base import PositionEncoding, register_part


@dataclass
class Rotation:
    cos: torch.Tensor        # [positions, rotary_dim / 2] float32, on the device
    sin: torch.Tensor
    rotary_dim: int
    pairing: int             # 0 = half, 1 = adjacent


def rotary_inverse_frequencies(rotary_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """float64 ``[rotary_dim / 2]``; ``scaling`` is a llama3 ``rope_scaling`` dict or None.

    llama3: with wavelength ``lam = 2 pi / f`` and ``L`` the original context length,
    ``f`` is kept where ``lam < L / high_freq_factor``, divided by ``factor`` where
    ``lam > L / low_freq_factor``, and interpolated between:
    ``s = (L / lam - low) / (high - low)``, ``f' = (1 - s) f / factor + s f``.
    """
    half = rotary_dim // 2
    i = torch.arange(half, dtype=torch.float64)
    inv = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float64), 2.0 * i / rotary_dim)
    if scaling:
        if scaling.get("rope_type") != "llama3":
            raise ValueError(f"rotary scaling '{scaling.get('rope_type')}' is not supported")
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position_embeddings"])
        lam = 2.0 * math.pi / inv
        smooth = (orig / lam - low) / (high - low)
        mid = (1.0 - smooth) * inv / factor + smooth * inv
        inv = torch.where(lam < orig / high, inv, torch.where(lam > orig / low, inv / factor, mid))
    return inv


class RotaryEncoding(PositionEncoding):
    """params: head_dim, rotary_dim (<= head_dim, even), theta, scaling (dict or None), pairing."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.rotary_dim = int(params["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2 or self.rotary_dim > int(params["head_dim"]):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {params['head_dim']}")
        pairing = params.get("pairing", "half")
        if pairing not in ("half", "adjacent"):
            raise ValueError(f"rotary pairing '{pairing}' is not known (half, adjacent)")
        self.pairing = 0 if pairing == "half" else 1
        self._rotation: Optional[Rotation] = None
        self._retired = []        # smaller tables that were replaced: a recorded CUDA graph may still read them

    def limit(self) -> Optional[int]:
        return None if self._rotation is None else int(self._rotation.cos.shape[0])

    def prepare(self, max_positions: int) -> None:
        if self._rotation is not None:
            if self._rotation.cos.shape[0] >= max_positions:
                return
            self._retired.append(self._rotation)
        inv = rotary_inverse_frequencies(self.rotary_dim, self.params["theta"], self.params.get("scaling"))
        pos = torch.arange(max_positions, dtype=torch.float64)
        ang = pos[:, None] * inv[None, :]
        cos = torch.cos(ang).to(torch.float32).to(self.env.device).contiguous()
        sin = torch.sin(ang).to(torch.float32).to(self.env.device).contiguous()
        self._rotation = Rotation(cos, sin, self.rotary_dim, self.pairing)

    def rotation(self) -> Rotation:
        if self._rotation is None:
            raise RuntimeError("RotaryEncoding.prepare() has not run")
        return self._rotation


class NoEncoding(PositionEncoding):
    """No position information (mixers then skip the rotation)."""


register_part("position", "rotary", RotaryEncoding)
register_part("position", "none", NoEncoding)
