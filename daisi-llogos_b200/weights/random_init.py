"""Counter-based random initialisation: every element of every tensor is a pure function of
(seed, tensor name, element index).

The same values come out of plain integer and double arithmetic on the host (here, with numpy) and of
the device kernel ``llg_fill_normal`` (csrc/init.cu), so a model initialised on the GPU holds exactly the
weights that ``write_random_model`` puts into a file for the same configuration and seed, and a plain CPU
implementation can be given the very weights a GPU run used without shipping files.  The reference's only
random model is a test fixture filled from ``System.Random``
(tests/Daisi.Llogos.Tests/Training/TrainingForwardPassTests.cs:342-360).

    key = splitmix64(splitmix64(seed) ^ fnv1a64(name))
    h1, h2 = splitmix64(key + 2 i), splitmix64(key + 2 i + 1)             (64-bit wrap-around)
    u1 = ((h1 >> 11) + 1) / 2^53,  u2 = (h2 >> 11) / 2^53
    z = sqrt(-2 ln u1) cos(2 pi u2)                                        (Box-Muller, double)
    value = float32(mean + std z), then rounded to the tensor's type
"""
from __future__ import annotations

import numpy as np
import torch

_M64 = (1 << 64) - 1
TWO_PI = 6.283185307179586476925286766559


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def fnv1a64(text: str) -> int:
    h = 0xCBF29CE484222325
    for byte in text.encode("utf-8"):
        h = ((h ^ byte) * 0x100000001B3) & _M64
    return h


def tensor_key(seed: int, name: str) -> int:
    return splitmix64(splitmix64(seed & _M64) ^ fnv1a64(name))


def _splitmix64_array(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = x + np.uint64(0x9E3779B97F4A7C15)
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return x ^ (x >> np.uint64(31))


def normal_values(key: int, n: int, mean: float, std: float, start: int = 0) -> np.ndarray:
    """float32 values of elements ``start .. start + n`` of the tensor with this key."""
    out = np.empty(n, dtype=np.float32)
    chunk = 1 << 20
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        with np.errstate(over="ignore"):
            idx = np.arange(start + lo, start + hi, dtype=np.uint64) * np.uint64(2) + np.uint64(key)
            h1 = _splitmix64_array(idx)
            h2 = _splitmix64_array(idx + np.uint64(1))
        u1 = ((h1 >> np.uint64(11)) + np.uint64(1)).astype(np.float64) * (1.0 / 9007199254740992.0)
        u2 = (h2 >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)
        z = np.sqrt(-2.0 * np.log(u1)) * np.cos(TWO_PI * u2)
        out[lo:hi] = (mean + std * z).astype(np.float32)
    return out


def fill_normal(out: torch.Tensor, key: int, mean: float, std: float, ops=None) -> None:
    """Fills ``out`` (float32 or bfloat16, contiguous) in place: on the GPU by the kernel, on the CPU by numpy."""
    if out.is_cuda:
        ops.fill_normal(out, key, mean, std)
        return
    vals = torch.from_numpy(normal_values(key, out.numel(), mean, std)).view(out.shape)
    out.copy_(vals)          # float32 -> bfloat16 rounds to nearest even, as the kernel does
