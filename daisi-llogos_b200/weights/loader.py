"""From a model folder to a bound model: tensors are read by name, checked against what the
parts declare, and kept in bfloat16.

Storage rule: with compute type bfloat16, tensors stored as BF16 stay as they are, F16 is
converted to bfloat16, a tensor stored in 32 bits stays float32, integer tables become int32.
With compute type float32 every floating tensor becomes float32 (the bfloat16 values exactly).
All problems of a checkpoint are reported in ONE error that lists missing tensors, unexpected
tensors and wrong shapes.  The reference looks tensors up by name and fails on the first
missing one (Model/ModelLoader.cs:95-113, :144-145; optional ones :152-162).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Mapping, Optional

import torch

from ..config.dense import read_config_json
from ..config.registry import architecture_of
from ..engine.model import DecoderModel
from .safetensors_io import ModelFiles, write_safetensors


class WeightsError(ValueError):
    pass


def _ops_for(device: torch.device):
    from ..kernels import ops
    if device.type == "cuda":
        ops.require_gpu()
    return ops


def _stored_as(t: torch.Tensor, compute: torch.dtype) -> torch.dtype:
    if t.dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8):
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if t.dtype in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def check_tensors(decls, available: Mapping[str, Any], where: str) -> None:
    """``available`` maps name -> shape.  Raises one WeightsError that lists everything wrong."""
    missing = sorted(n for n, d in decls.items() if not d.optional and n not in available)
    unexpected = sorted(n for n in available if n not in decls)
    wrong = sorted((n, tuple(available[n]), tuple(decls[n].shape)) for n in available
                   if n in decls and tuple(available[n]) != tuple(decls[n].shape))
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where}: the tensors do not fit the model that config.json describes"]
    if missing:
        lines.append(f"  missing ({len(missing)}):")
        lines += [f"    {n}  expected shape {tuple(decls[n].shape)}" for n in missing]
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}):")
        lines += [f"    {n}  shape {tuple(available[n])}" for n in unexpected]
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}):")
        lines += [f"    {n}  has {got}, expected {exp}" for n, got, exp in wrong]
    raise WeightsError("\n".join(lines))


def build_model(config_dict: Mapping[str, Any], *, dtype: torch.dtype, device, ops=None) -> DecoderModel:
    """An unbound model (parts built, no tensors yet) for the architecture ``config_dict`` names."""
    device = torch.device(device)
    arch = architecture_of(config_dict)
    cfg = arch.read_config(config_dict)
    spec = arch.build_spec(cfg)
    model = DecoderModel(spec, dtype=dtype, device=device, ops=ops)
    model.config = cfg
    return model


def load_model(model_dir: str, *, dtype: torch.dtype = torch.bfloat16, device="cuda:0", ops=None) -> DecoderModel:
    """Reads ``config.json`` and the safetensors of ``model_dir``; returns a model ready to step."""
    device = torch.device(device)
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"compute type must be bfloat16 or float32, got {dtype}")
    if ops is None:
        ops = _ops_for(device)
    config_dict = read_config_json(model_dir)
    model = build_model(config_dict, dtype=dtype, device=device, ops=ops)
    decls = model.tensor_decls()
    files = ModelFiles(model_dir)
    try:
        check_tensors(decls, {n: files.info(n)[1] for n in files.names()}, model_dir)
        tensors: Dict[str, torch.Tensor] = {}
        for name in decls:
            if name not in files.names():
                continue
            t = files.tensor(name)
            tensors[name] = t.to(device=device, dtype=_stored_as(t, dtype)).contiguous()
        model.bind(tensors)
    finally:
        files.close()
    return model


# ---- random weights -----------------------------------------------------------------------

def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensors(decls, seed: int, *, std: float = 0.02, norm_std: float = 0.0, bias_std: float = 0.02,
                   dtype: torch.dtype = torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    """One tensor per declaration: matrices and tables N(0, std), norm weights 1 + N(0, norm_std),
    biases N(0, bias_std); each tensor's generator is seeded by (seed, its name)."""
    device = torch.device(device)
    out = {}
    for name, d in decls.items():
        g = torch.Generator(device=device)
        g.manual_seed(_tensor_seed(seed, name))
        x = torch.randn(d.shape, generator=g, device=device, dtype=torch.float32)
        if d.role == "norm":
            x = 1.0 + norm_std * x
        elif d.role == "bias":
            x = bias_std * x
        else:
            x = std * x
        out[name] = x.to(dtype)
    return out


def write_random_model(model_dir: str, config_dict: Mapping[str, Any], seed: int, *, std: float = 0.02,
                       norm_std: float = 0.0, bias_std: float = 0.02,
                       dtype: torch.dtype = torch.bfloat16) -> None:
    """Writes ``config.json`` and ``model.safetensors`` of a randomly initialised model."""
    os.makedirs(model_dir, exist_ok=True)
    model = build_model(config_dict, dtype=torch.float32, device="cpu")
    tensors = random_tensors(model.tensor_decls(), seed, std=std, norm_std=norm_std, bias_std=bias_std, dtype=dtype)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(config_dict), f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      {"format": "pt", "seed": str(seed)})


def random_model(config_dict: Mapping[str, Any], seed: int, *, dtype: torch.dtype = torch.bfloat16,
                 device="cuda:0", std: float = 0.02, norm_std: float = 0.0, bias_std: float = 0.02,
                 ops=None) -> DecoderModel:
    """A bound model with random bfloat16-valued weights generated on the device (no files)."""
    device = torch.device(device)
    if ops is None:
        ops = _ops_for(device)
    model = build_model(config_dict, dtype=dtype, device=device, ops=ops)
    store = torch.bfloat16
    tensors = random_tensors(model.tensor_decls(), seed, std=std, norm_std=norm_std, bias_std=bias_std,
                             dtype=store, device=device)
    if dtype == torch.float32:
        tensors = {n: t.to(torch.float32) for n, t in tensors.items()}
    model.bind(tensors)
    return model
