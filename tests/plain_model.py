"""A plain, slow implementation of the dense Llama / Qwen decoder, for tests only.

It rests on the reference's formulas (cited per function as file:line of MjrTom/daisi-llogos),
not on a run of the reference: its C# cannot be compiled here (no dotnet), so there is no
golden output of the reference itself.  Whole sequences, no cache, one function per part,
float64 arithmetic, and no code shared with the library under test: it parses config.json's
keys and looks tensors up by name on its own.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

F64 = torch.float64


# ---- parts ------------------------------------------------------------------------------------

def embedding(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """Row copy, no scaling.  Inference/ForwardPass.cs:205; Daisi.Llogos.Cpu/CpuBackend.cs:327-370."""
    return table.to(F64)[torch.as_tensor(list(tokens), dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, rnd=None) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w: eps inside the root, weight after.
    Daisi.Llogos.Cpu/RmsNorm.cs:14-65 (sum of squares in double, :19-41).

    ``rnd``: a rounding applied to ``x * w`` before the division by the root: what an engine stores when it
    leaves that division to the product that consumes the norm (a product is linear in its rows)."""
    x = x.to(F64)
    ms = (x * x).mean(dim=-1, keepdim=True)
    if rnd is not None:
        return rnd(x * weight.to(F64)) * (1.0 / torch.sqrt(ms + eps))
    return x * (1.0 / torch.sqrt(ms + eps)) * weight.to(F64)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T with W stored [out, in], each output's row contiguous.
    Daisi.Llogos.Cuda/kernels/dequant_matmul.cu:4-6, :593-619; Daisi.Llogos.Cpu/MatMul.cs:50-56."""
    y = x.to(F64) @ weight.to(F64).t()
    if bias is not None:
        y = y + bias.to(F64)
    return y


def per_head_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over each head's slice; one weight vector [head_dim] for all heads.
    x is [T, heads, head_dim].  Daisi.Llogos.Cpu/CpuBackend.cs:406-421;
    Daisi.Llogos.Cuda/kernels/composite_ops.cu:106-136."""
    return rms_norm(x, weight, eps)


def rope_inverse_frequencies(rotary_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """freq_i = 1 / theta^(2 i / rotary_dim), in double.  Daisi.Llogos.Cpu/Rope.cs:131-146.
    The reference has no frequency scaling; the llama3 rule is this build's own: wavelengths
    below L/high are kept, above L/low divided by factor, between interpolated linearly in
    L/wavelength."""
    freqs = []
    for i in range(rotary_dim // 2):
        f = 1.0 / math.pow(theta, 2.0 * i / rotary_dim)
        if scaling is not None:
            factor = scaling["factor"]
            low, high = scaling["low_freq_factor"], scaling["high_freq_factor"]
            orig = scaling["original_max_position_embeddings"]
            wavelen = 2.0 * math.pi / f
            if wavelen < orig / high:
                pass
            elif wavelen > orig / low:
                f = f / factor
            else:
                s = (orig / wavelen - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        freqs.append(f)
    return torch.tensor(freqs, dtype=F64)


def rope_rotate(x: torch.Tensor, positions: Sequence[int], inv_freq: torch.Tensor, pairing: str) -> torch.Tensor:
    """x is [T, heads, head_dim]; angle = position * freq_i;
    (a, b) -> (a cos - b sin, a sin + b cos).  Pairs are (2i, 2i+1) in
    Daisi.Llogos.Cpu/Rope.cs:148-162 ("adjacent") and (i, i + half) in Rope.cs:115-129 ("half");
    dimensions beyond rotary_dim pass through (Rope.cs:15-19)."""
    x = x.to(F64).clone()
    half = inv_freq.numel()
    pos = torch.as_tensor(list(positions), dtype=F64)
    ang = pos[:, None] * inv_freq[None, :]                  # [T, half]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    if pairing == "half":
        a, b = x[..., :half].clone(), x[..., half:2 * half].clone()
        x[..., :half] = a * cos - b * sin
        x[..., half:2 * half] = a * sin + b * cos
    elif pairing == "adjacent":
        a, b = x[..., 0:2 * half:2].clone(), x[..., 1:2 * half:2].clone()
        x[..., 0:2 * half:2] = a * cos - b * sin
        x[..., 1:2 * half:2] = a * sin + b * cos
    else:
        raise ValueError(pairing)
    return x


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int = 0,
              round_weights=None) -> torch.Tensor:
    """Causal softmax attention of one whole sequence.  q [T, nH, hd], k/v [T, nKV, hd];
    query head h uses key/value head h // (nH / nKV); score = (q . k) * scale, applied after the
    dot product; query t sees keys j <= t, and with a window W only j > t - W.
    Daisi.Llogos.Cpu/CpuBackend.cs:476-590 (scores :527-537, softmax :540-553, values :556-571);
    window: Inference/AttentionStrategy.cs:64-71.
    ``round_weights``: a rounding applied to the unnormalised softmax weights as they enter the
    product with the values (the sum that normalises them stays unrounded).  The weights are then taken
    as 2^(x - M) with x = score * log2(e) and M the row's largest x rounded up to a whole number: a
    floating-point rounding gives the same digits for any whole M, so this pins the rounded weights
    without saying in which order or in how many pieces an engine visits the keys."""
    t, nh, hd = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    out = torch.zeros((t, nh, hd), dtype=F64)
    idx = torch.arange(t)
    visible = idx[None, :] <= idx[:, None]
    if window > 0:
        visible &= idx[None, :] > (idx[:, None] - window)
    for h in range(nh):
        kh = h // g
        s = (q[:, h, :].to(F64) @ k[:, kh, :].to(F64).t()) * scale
        s = s.masked_fill(~visible, float("-inf"))
        if round_weights is None:
            p = torch.exp(s - s.max(dim=-1, keepdim=True).values)
            p = p / p.sum(dim=-1, keepdim=True)
            out[:, h, :] = p @ v[:, kh, :].to(F64)
        else:
            x = s * math.log2(math.e)
            p = torch.exp2(x - torch.ceil(x.max(dim=-1, keepdim=True).values))
            out[:, h, :] = (round_weights(p) @ v[:, kh, :].to(F64)) / p.sum(dim=-1, keepdim=True)
    return out


def swiglu(x: torch.Tensor, w_gate, w_up, w_down, rnd=None) -> torch.Tensor:
    """down( silu(gate(x)) * up(x) ), silu(g) = g / (1 + exp(-g)).
    Inference/ForwardPass.cs:242-246; Daisi.Llogos.Cpu/Silu.cs:9-16.
    ``rnd``: a rounding applied to the gated values before the last product."""
    g = linear(x, w_gate)
    u = linear(x, w_up)
    m = g / (1.0 + torch.exp(-g)) * u
    return linear(m if rnd is None else rnd(m), w_down)


# ---- the model --------------------------------------------------------------------------------

def layer_windows(cfg: dict) -> List[int]:
    n = cfg["num_hidden_layers"]
    w = cfg.get("sliding_window") or 0
    if cfg.get("layer_types") is not None:
        return [w if t == "sliding_attention" else 0 for t in cfg["layer_types"]]
    if cfg.get("use_sliding_window"):
        first = cfg.get("max_window_layers", 0)
        return [w if i >= first else 0 for i in range(n)]
    return [0] * n


def round_bfloat16(t: torch.Tensor) -> torch.Tensor:
    """The nearest bfloat16 value (ties to even), as float64."""
    return t.to(torch.float32).to(torch.bfloat16).to(F64)


def forward(weights: Dict[str, torch.Tensor], cfg: dict, tokens: Sequence[int], rounded: bool = False) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  Order as Inference/ForwardPass.cs:199-267 (layers)
    and :174-184 (final norm, head): norm, q/k/v, per-head norm, bias, rotation, attention, output
    projection, residual, norm, SwiGLU, residual (ForwardPass.cs:368-404 for the attention part).

    ``rounded``: values that a bfloat16 engine keeps in bfloat16 between its kernels are rounded to
    bfloat16 here as well: the input of every norm times the norm's weight (the division by the root mean
    square follows the rounding, see ``rms_norm``), q, k and v after the rotation, the softmax weights
    as they enter the product with the values, the attention output and the gated feed-forward values.
    Sums, statistics, the residual stream and the logits stay unrounded.  The reference keeps every
    activation in 32 bits (Inference/ForwardPass.cs:1046-1047), so this form has no counterpart there;
    it tells a bfloat16 engine's rounding from a fault."""
    r = round_bfloat16 if rounded else (lambda t: t)
    rnd = round_bfloat16 if rounded else None
    arch = cfg["architectures"][0]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    eps = cfg.get("rms_norm_eps", 1e-6)
    qk_norm = cfg.get("qk_norm", arch == "Qwen3ForCausalLM")
    bias = cfg.get("attention_bias", arch == "Qwen2ForCausalLM")
    scaling = cfg.get("rope_scaling")
    if scaling is not None and scaling.get("rope_type", scaling.get("type")) in (None, "default"):
        scaling = None
    rotary_dim = int(hd * cfg.get("partial_rotary_factor", 1.0))      # the rest of a head passes through
    inv_freq = rope_inverse_frequencies(rotary_dim, cfg.get("rope_theta", 10000.0), scaling)
    windows = layer_windows(cfg)
    t = len(tokens)
    positions = list(range(t))
    h = embedding(weights["model.embed_tokens.weight"], tokens)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        x = rms_norm(h, weights[p + "input_layernorm.weight"], eps, rnd)
        a = p + "self_attn."
        q = linear(x, weights[a + "q_proj.weight"]).view(t, nh, hd)
        k = linear(x, weights[a + "k_proj.weight"]).view(t, nkv, hd)
        v = linear(x, weights[a + "v_proj.weight"]).view(t, nkv, hd)
        if qk_norm:
            q = per_head_rms_norm(q, weights[a + "q_norm.weight"], eps)
            k = per_head_rms_norm(k, weights[a + "k_norm.weight"], eps)
        if bias:
            q = q + weights[a + "q_proj.bias"].to(F64).view(nh, hd)
            k = k + weights[a + "k_proj.bias"].to(F64).view(nkv, hd)
            v = v + weights[a + "v_proj.bias"].to(F64).view(nkv, hd)
        q = r(rope_rotate(q, positions, inv_freq, "half"))
        k = r(rope_rotate(k, positions, inv_freq, "half"))
        v = r(v)
        o = r(attention(q, k, v, 1.0 / math.sqrt(hd), windows[i], r if rounded else None).reshape(t, nh * hd))
        h = h + linear(o, weights[a + "o_proj.weight"])
        x = rms_norm(h, weights[p + "post_attention_layernorm.weight"], eps, rnd)
        m = p + "mlp."
        h = h + swiglu(x, weights[m + "gate_proj.weight"], weights[m + "up_proj.weight"], weights[m + "down_proj.weight"],
                       r if rounded else None)
    x = rms_norm(h, weights["model.norm.weight"], eps, rnd)
    head = weights["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else weights["lm_head.weight"]
    return linear(x, head)


# ---- sampling ---------------------------------------------------------------------------------

def splitmix64(x: int) -> int:
    m = (1 << 64) - 1
    x = (x + 0x9E3779B97F4A7C15) & m
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & m
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & m
    return x ^ (x >> 31)


def uniform_of(seed: int, seq_id: int, step: int) -> float:
    """The library's counter-based uniform number (its own design; the reference draws from
    System.Random, Inference/Sampler.cs:334-336)."""
    m = (1 << 64) - 1
    h = splitmix64(seed & m)
    h = splitmix64(h ^ ((0xD1B54A32D192ED03 * (seq_id + 1)) & m))
    h = splitmix64(h ^ ((0x8CB92BA72F3D8DD7 * (step + 1)) & m))
    return (h >> 40) / 16777216.0


def sampling_distribution(logits: Sequence[float], *, temperature: float, top_k: int = 0, top_p: float = 1.0,
                          min_p: float = 0.0, typical_p: float = 1.0, min_keep: int = 1,
                          repetition_penalty: float = 1.0, frequency_penalty: float = 0.0,
                          presence_penalty: float = 0.0, penalize_newline: bool = False,
                          previous: Sequence[int] = (), banned: Sequence[int] = ()) -> torch.Tensor:
    """The probability of every token after the reference's pipeline (Inference/Sampler.cs:26-85):
    penalties (:89-143, the repetition penalty once per occurrence in the window), banned tokens
    (:49-53), temperature (:60-62), top-k (:65-66, :249-276), min-p on the scaled logits (:150-170),
    softmax over candidates (:278-295), typical-p (:178-230), top-p (:297-332)."""
    w = [float(x) for x in logits]
    n = len(w)
    if repetition_penalty != 1.0 or frequency_penalty != 0 or presence_penalty != 0:
        counts: Dict[int, int] = {}
        for t in previous:
            counts[t] = counts.get(t, 0) + 1
        if repetition_penalty != 1.0:
            for t in previous:
                if not 0 <= t < n or (not penalize_newline and t in (10, 13)):
                    continue
                w[t] = w[t] / repetition_penalty if w[t] > 0 else w[t] * repetition_penalty
        for t, c in counts.items():
            if not 0 <= t < n or (not penalize_newline and t in (10, 13)):
                continue
            w[t] -= frequency_penalty * c
            w[t] -= presence_penalty
    for t in banned:
        if 0 <= t < n:
            w[t] = float("-inf")
    probs = torch.zeros(n, dtype=F64)
    if temperature == 0:
        best = max(range(n), key=lambda i: (w[i], -i))
        probs[best] = 1.0
        return probs
    w = [x / temperature for x in w]
    k = top_k if 0 < top_k < n else n
    cand = sorted(range(n), key=lambda i: (-w[i], i))[:k]
    min_keep = max(min_keep, 1)
    if 0 < min_p < 1 and len(cand) > min_keep:
        thr = max(w[c] for c in cand) + math.log(min_p)
        kept = []
        for c in cand:
            if w[c] >= thr or len(kept) < min_keep:
                kept.append(c)
        cand = kept
    mx = max(w[c] for c in cand)
    e = {c: math.exp(w[c] - mx) for c in cand}
    z = sum(e.values())
    p = {c: e[c] / z for c in cand}
    if 0 < typical_p < 1 and len(cand) > min_keep:
        ent = -sum(pc * math.log(pc) for pc in p.values() if pc > 0)
        scored = sorted(cand, key=lambda c: abs((-math.log(p[c]) if p[c] > 0 else float("inf")) - ent))
        kept, cum = [], 0.0
        for c in scored:
            kept.append(c)
            cum += p[c]
            if cum >= typical_p and len(kept) >= min_keep:
                break
        s = sum(p[c] for c in kept)
        p = {c: p[c] / s for c in kept}
        cand = kept
    if 0 < top_p < 1:
        order = sorted(cand, key=lambda c: -p[c])
        cum, cutoff = 0.0, len(order)
        for i, c in enumerate(order):
            cum += p[c]
            if cum > top_p and i + 1 >= min_keep:
                cutoff = i + 1
                break
        kept = order[:cutoff]
        s = sum(p[c] for c in kept)
        p = {c: p[c] / s for c in kept}
    for c, pc in p.items():
        probs[c] = pc
    return probs


def draw(probs: torch.Tensor, u: float) -> int:
    """Inverse CDF in index order: the first token whose cumulative probability exceeds u * total
    (the reference walks its candidates the same way, in their sorted order: Sampler.cs:337-344)."""
    total = float(probs.sum())
    target = u * total
    c = 0.0
    last = 0
    for i, p in enumerate(probs.tolist()):
        if p > 0:
            c += p
            last = i
            if target < c:
                return i
    return last
