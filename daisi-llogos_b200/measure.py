"""What a step has to read and to compute, and the peaks to hold it against.

The reference's ``--bench`` prints tokens per second only (Daisi.Llogos.Cli/Program.cs:283-297,
Inference/TextGenerator.cs:126-186); this module adds the two numbers that say how far a step is from the
hardware: the bytes a decode step must read (every weight matrix it uses once, and the keys and values of the
live sequences) and the floating-point operations of a prompt step, each with the measured peak it is a
fraction of.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Optional, Sequence

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# An earlier measurement of a B200's copy bandwidth and bfloat16 matrix throughput, used when no file of
# measured peaks is found.
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks(path: Optional[str] = None) -> Dict[str, object]:
    """``{"hbm_gbs", "bf16_tflops", ["bf16_tflops_sustained"], "source"}``: from the JSON file at ``path``, at
    ``$LLOGOS_PEAKS`` or ``MEASURED_PEAKS.json`` beside the package (keys of the same names), else the fallback."""
    for cand in (path, os.environ.get("LLOGOS_PEAKS"), os.path.join(_ROOT, "MEASURED_PEAKS.json")):
        if not cand or not os.path.isfile(cand):
            continue
        try:
            with open(cand) as f:
                d = json.load(f)
        except (ValueError, OSError):
            continue
        if d.get("hbm_gbs") and d.get("bf16_tflops"):
            out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
            if d.get("bf16_tflops_sustained"):
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            return out
    return dict(FALLBACK_PEAKS)


@dataclass(frozen=True)
class ModelCosts:
    matrix_params: int          # elements of the matrices every token passes through (the layers' products)
    head_params: int            # elements of the output matrix (the embedding table when tied)
    bytes_per_param: int
    kv_units: Sequence[tuple]   # per cache unit: (bytes per token, window or 0)
    attn_flops_per_pair: int    # flops per (query, key) pair summed over the layers: 4 * heads * head size each

    def decode_step_bytes(self, lengths: Sequence[int], hidden_size: int = 0) -> float:
        """Bytes one decode step must read: every matrix once, the head once, and the keys and values that the
        new token of each sequence looks at (``lengths``: keys per sequence, the new one included)."""
        cache = 0.0
        for per_token, window in self.kv_units:
            for n in lengths:
                cache += per_token * (min(n, window) if window > 0 else n)
        return (self.matrix_params + self.head_params) * self.bytes_per_param + cache

    def prompt_step_flops(self, counts: Sequence[int], before: Optional[Sequence[int]] = None, wanted_rows: int = 1) -> float:
        """Flops of a step that brings ``counts[i]`` tokens to a sequence of ``before[i]`` tokens: 2 per matrix
        element and token, the causal score and value products, and the head on the wanted rows."""
        before = before or [0] * len(counts)
        pairs = sum(c * b + c * (c + 1) / 2 for c, b in zip(counts, before))
        return 2.0 * sum(counts) * self.matrix_params + 2.0 * wanted_rows * self.head_params + self.attn_flops_per_pair * pairs


def model_costs(model) -> ModelCosts:
    """Read off a built model: matrices by their declarations, cache bytes by what the mixers keep."""
    import torch
    from .parts.base import KvNeed
    elem = 2 if model.dtype == torch.bfloat16 else 4
    head = 0
    matrix = 0
    decls = model.tensor_decls()
    head_prefix = model.head.prefix
    for name, d in decls.items():
        if d.role != "matrix":
            continue
        n = 1
        for s in d.shape:
            n *= int(s)
        if name.startswith(head_prefix):
            head += n
        else:
            matrix += n
    if head == 0:                                        # tied: the embedding table serves as the output matrix
        head = int(model.spec.vocab_size) * int(model.spec.hidden_size)
    # a layer that the run order names twice runs twice
    per_layer = {}
    for name, d in decls.items():
        if d.role == "matrix" and name.startswith("model.layers."):
            idx = int(name.split(".")[2])
            n = 1
            for s in d.shape:
                n *= int(s)
            per_layer[idx] = per_layer.get(idx, 0) + n
    if per_layer:
        counted = sum(per_layer.values())
        scheduled = sum(per_layer.get(e.layer, 0) for e in model.spec.schedule)
        matrix += scheduled - counted
    kv, attn = [], 0
    for e_i, e in enumerate(model.spec.schedule):
        block = model.blocks[e.layer]
        need = block.cache_need()
        if isinstance(need, KvNeed):
            kv.append((2 * need.num_kv_heads * need.head_dim * elem, need.window))
        for part in block.parts.values():
            nh, hd = getattr(part, "nh", None), getattr(part, "hd", None)
            if nh and hd:
                attn += 4 * nh * hd
    return ModelCosts(matrix, head, elem, tuple(kv), attn)


def decode_bytes_of_run(costs: ModelCosts, prompt_lengths: Sequence[int], generated: Sequence[int]):
    """(bytes, steps) that the decode steps of one generation call had to read: sequence i (prompt of
    ``prompt_lengths[i]`` tokens, ``generated[i]`` tokens made) takes part in ``generated[i] - 1`` decode steps, at
    lengths ``prompt + 1 ... prompt + generated - 1`` (its first token comes out of the prompt step)."""
    by_step: Dict[int, list] = {}
    for n, m in zip(prompt_lengths, generated):
        for k in range(1, m):
            by_step.setdefault(k, []).append(n + k)
    return sum(costs.decode_step_bytes(v) for v in by_step.values()), len(by_step)
