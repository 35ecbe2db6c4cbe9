"""From a model folder to a bound model: tensors are read by name, checked against what the
parts declare, and kept in bfloat16.

Storage rule: with compute type bfloat16, tensors stored as BF16 stay as they are, F16 is
converted to bfloat16, a tensor stored in 32 bits stays float32, integer tables become int32.
With compute type float32 every floating tensor becomes float32 (the bfloat16 values exactly).
All problems of a checkpoint are reported in ONE error that lists missing tensors, unexpected
tensors and wrong shapes.  Tensors that the architecture declares harmless (buffers that exporters
write beside the weights, a second copy of a tied matrix) are not an error: they are skipped and
named in the model's ``load_warnings``.  The reference looks tensors up by name and fails on the
first missing one (Model/ModelLoader.cs:95-113, :144-145; optional ones :152-162) and never looks at
the names it does not ask for.
"""
from __future__ import annotations

import json
import os
import re
from typing import Any, Dict, List, Mapping, Optional, Sequence

import torch

from ..config.dense import read_config_json
from ..config.registry import architecture_of
from ..engine.model import DecoderModel
from .random_init import fill_normal, tensor_key
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


def check_tensors(decls, available: Mapping[str, Any], where: str, ignorable: Sequence[str] = ()) -> List[str]:
    """``available`` maps name -> shape.  Raises one WeightsError that lists everything wrong; returns the
    names of tensors that were found, are not part of the model, and match one of the ``ignorable``
    patterns (regular expressions on the whole name)."""
    missing = sorted(n for n, d in decls.items() if not d.optional and n not in available)
    extra = sorted(n for n in available if n not in decls)
    skipped = [n for n in extra if any(re.fullmatch(p, n) for p in ignorable)]
    unexpected = [n for n in extra if n not in skipped]
    wrong = sorted((n, tuple(available[n]), tuple(decls[n].shape)) for n in available
                   if n in decls and tuple(available[n]) != tuple(decls[n].shape))
    if not (missing or unexpected or wrong):
        return skipped
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
        skipped = check_tensors(decls, {n: files.info(n)[1] for n in files.names()}, model_dir,
                                model.spec.ignorable_tensors)
        model.load_warnings = [f"{model_dir}: tensor '{n}' is not part of the model and was skipped" for n in skipped]
        tensors: Dict[str, torch.Tensor] = {}
        for name in decls:
            if name not in files.names():
                continue
            tensors[name] = _to_device(files.tensor(name), device, dtype, ops)
        model.bind(tensors)
    finally:
        files.close()
    return model


def _to_device(t: torch.Tensor, device: torch.device, compute: torch.dtype, ops) -> torch.Tensor:
    """The tensor on ``device`` in the type the storage rule gives it.  On the GPU float32 <-> bfloat16 is
    converted by the library's own kernel after the copy; what the kernel does not take (float16, float64,
    integers) is converted on the host first."""
    want = _stored_as(t, compute)
    if device.type != "cuda" or want == torch.int32:
        return t.to(device=device, dtype=want).contiguous()
    if t.dtype not in (torch.float32, torch.bfloat16):
        t = t.to(torch.float32)
    src = t.contiguous().to(device)
    if src.dtype == want:
        return src
    dst = torch.empty(src.shape, dtype=want, device=device)
    ops.cast(src, dst)
    return dst


# ---- random weights -----------------------------------------------------------------------

def random_tensors(decls, seed: int, *, std: float = 0.02, norm_std: float = 0.0, bias_std: float = 0.02,
                   dtype: torch.dtype = torch.bfloat16, device="cpu", ops=None) -> Dict[str, torch.Tensor]:
    """One tensor per declaration: matrices and tables N(0, std), norm weights 1 + N(0, norm_std),
    biases N(0, bias_std).  Every element is a function of (seed, tensor name, element index) alone
    (weights/random_init.py), so the values do not depend on the device that makes them: on the GPU the
    library's fill kernel writes them, on the CPU numpy does."""
    device = torch.device(device)
    if device.type == "cuda" and ops is None:
        ops = _ops_for(device)
    out = {}
    for name, d in decls.items():
        mean, spread = (1.0, norm_std) if d.role == "norm" else (0.0, bias_std) if d.role == "bias" else (0.0, std)
        t = torch.empty(d.shape, dtype=dtype, device=device)
        fill_normal(t, tensor_key(seed, name), mean, spread, ops)
        out[name] = t
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
                             dtype=store, device=device, ops=ops)
    if dtype == torch.float32:
        wide = {}
        for n, t in tensors.items():                  # the bfloat16 values exactly, stored in 32 bits
            wide[n] = torch.empty(t.shape, dtype=torch.float32, device=device)
            if device.type == "cuda":
                ops.cast(t, wide[n])
            else:
                wide[n].copy_(t)
        tensors = wide
    model.bind(tensors)
    return model
