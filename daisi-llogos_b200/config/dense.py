"""Typed configuration of the dense Llama / Qwen2 / Qwen3 decoder.

Every size and constant of the model is read from the architecture's own
``config.json`` keys; nothing here hard-codes a model size.  The reference reads
the same quantities from GGUF metadata (Model/ModelConfig.cs:124-201: block
count, embedding length, feed-forward length, head counts, key length, RMS
epsilon with default 1e-6 at :170, rope base with default 10000 at :179).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A config.json key is missing, has the wrong type or an unsupported value."""


@dataclass(frozen=True)
class RopeScaling:
    """Frequency rescaling of rotary position encoding (``rope_scaling`` key).

    Only ``rope_type == "llama3"`` is known: wavelengths longer than
    ``original_max_position_embeddings / low_freq_factor`` are stretched by
    ``factor``, wavelengths shorter than ``original / high_freq_factor`` are
    kept, and the band between is interpolated.
    """

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def to_dict(self) -> dict:
        return {
            "rope_type": self.rope_type,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


def _need(d: Mapping[str, Any], key: str, typ, *, default=None, required=True):
    if key not in d or d[key] is None:
        if required:
            raise ConfigError(f"config.json: missing key '{key}'")
        return default
    v = d[key]
    if typ is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if typ is int and isinstance(v, bool):
        raise ConfigError(f"config.json: key '{key}' must be an integer, got {v!r}")
    if not isinstance(v, typ):
        raise ConfigError(
            f"config.json: key '{key}' must be {typ.__name__}, got {type(v).__name__} ({v!r})")
    return v


def _parse_rope_scaling(raw: Any) -> Optional[RopeScaling]:
    if raw is None:
        return None
    if not isinstance(raw, Mapping):
        raise ConfigError("config.json: 'rope_scaling' must be an object or null")
    rope_type = raw.get("rope_type", raw.get("type"))
    if rope_type in (None, "default"):
        return None
    if rope_type != "llama3":
        raise ConfigError(
            f"config.json: rope_scaling.rope_type '{rope_type}' is not supported (known: 'llama3')")
    return RopeScaling(
        rope_type="llama3",
        factor=_need(raw, "factor", float),
        low_freq_factor=_need(raw, "low_freq_factor", float),
        high_freq_factor=_need(raw, "high_freq_factor", float),
        original_max_position_embeddings=_need(raw, "original_max_position_embeddings", int),
    )


@dataclass(frozen=True)
class DenseDecoderConfig:
    """Hyper-parameters of one dense decoder, as config.json gives them."""

    architecture: str
    num_hidden_layers: int
    hidden_size: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: Optional[int]      # None: the file gives no limit, the cache's size is the limit
    rms_norm_eps: float
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rope_theta: float
    rope_scaling: Optional[RopeScaling] = None
    rotary_dim: Optional[int] = None            # dimensions of a head that are rotated; None = all of them
    attention_bias: bool = False
    qk_norm: bool = False
    tie_word_embeddings: bool = False
    # one entry per layer: 0 = all keys, W > 0 = the last W keys (the query's own included)
    layer_windows: Tuple[int, ...] = ()
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False, hash=False)

    # ---- derived -----------------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def window_of(self, layer: int) -> int:
        return self.layer_windows[layer] if self.layer_windows else 0

    # ---- construction ------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any], *, qk_norm: Optional[bool] = None,
                  force_attention_bias: Optional[bool] = None) -> "DenseDecoderConfig":
        """Build from the parsed config.json.

        ``qk_norm`` and ``force_attention_bias`` are what the registry entry of an
        architecture name fixes (Qwen3 normalises q and k per head; Qwen2 always
        has q/k/v biases); config keys of the same name win when present.
        """
        archs = d.get("architectures")
        if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
            raise ConfigError("config.json: missing key 'architectures' (a non-empty list of names)")
        n_layers = _need(d, "num_hidden_layers", int)
        hidden = _need(d, "hidden_size", int)
        inter = _need(d, "intermediate_size", int)
        vocab = _need(d, "vocab_size", int)
        n_heads = _need(d, "num_attention_heads", int)
        n_kv = _need(d, "num_key_value_heads", int, default=n_heads, required=False)
        max_pos = _need(d, "max_position_embeddings", int, default=None, required=False)
        eps = _need(d, "rms_norm_eps", float, default=1e-6, required=False)
        for name, v in (("num_hidden_layers", n_layers), ("hidden_size", hidden),
                        ("intermediate_size", inter), ("vocab_size", vocab),
                        ("num_attention_heads", n_heads), ("num_key_value_heads", n_kv),
                        ("max_position_embeddings", max_pos)):
            if v is not None and v <= 0:
                raise ConfigError(f"config.json: key '{name}' must be positive, got {v}")
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = _need(d, "head_dim", int)
        else:
            if hidden % n_heads:
                raise ConfigError(
                    f"config.json: no 'head_dim' and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {n_heads}")
            head_dim = hidden // n_heads
        if head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"config.json: head_dim must be a positive even number, got {head_dim}")
        if n_heads % n_kv:
            raise ConfigError(
                f"config.json: num_attention_heads {n_heads} is not a multiple of "
                f"num_key_value_heads {n_kv}")
        if eps <= 0:
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {eps}")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported (known: 'silu')")
        if d.get("mlp_bias", False):
            raise ConfigError("config.json: mlp_bias=true is not supported by this architecture")

        rope_params = d.get("rope_parameters") if isinstance(d.get("rope_parameters"), Mapping) else {}
        theta = _need(d, "rope_theta", float, default=None, required=False)
        if theta is None:
            theta = _need(rope_params, "rope_theta", float, default=10000.0, required=False)
        scaling_raw = d.get("rope_scaling")
        if scaling_raw is None and rope_params.get("rope_type") not in (None, "default"):
            scaling_raw = rope_params
        scaling = _parse_rope_scaling(scaling_raw)
        # the first head_dim * partial_rotary_factor dimensions of a head are rotated, the rest pass through
        factor = _need(d, "partial_rotary_factor", float, default=None, required=False)
        if factor is None:
            factor = _need(rope_params, "partial_rotary_factor", float, default=1.0, required=False)
        rotary_dim = int(head_dim * factor)
        if not 0 < factor <= 1 or rotary_dim <= 0 or rotary_dim % 2:
            raise ConfigError(f"config.json: partial_rotary_factor {factor} of head_dim {head_dim} must give a "
                              f"positive even number of rotated dimensions, got {rotary_dim}")

        bias = _need(d, "attention_bias", bool, default=None, required=False)
        if bias is None:
            bias = bool(force_attention_bias)
        qkn = _need(d, "qk_norm", bool, default=None, required=False)
        if qkn is None:
            qkn = bool(qk_norm)
        tied = _need(d, "tie_word_embeddings", bool, default=False, required=False)

        windows = cls._windows(d, n_layers)

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError("config.json: 'eos_token_id' must be an integer or a list of integers")
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"config.json: eos_token_id {e} is outside the vocabulary [0, {vocab})")
        bos = _need(d, "bos_token_id", int, default=None, required=False)

        return cls(
            architecture=archs[0], num_hidden_layers=n_layers, hidden_size=hidden,
            intermediate_size=inter, vocab_size=vocab, max_position_embeddings=max_pos,
            rms_norm_eps=eps, num_attention_heads=n_heads, num_key_value_heads=n_kv,
            head_dim=head_dim, rope_theta=theta, rope_scaling=scaling,
            rotary_dim=None if rotary_dim == head_dim else rotary_dim, attention_bias=bias,
            qk_norm=qkn, tie_word_embeddings=tied, layer_windows=windows,
            eos_token_ids=eos_ids, bos_token_id=bos, extra=dict(d))

    @staticmethod
    def _windows(d: Mapping[str, Any], n_layers: int) -> Tuple[int, ...]:
        """Per-layer window from ``layer_types`` or ``use_sliding_window``.

        ``layer_types`` (a list of "full_attention" / "sliding_attention") decides
        layer by layer.  Without it, ``use_sliding_window=true`` gives the window
        ``sliding_window`` to the layers from ``max_window_layers`` upward.  The
        reference's window is a ring of the last W positions
        (Inference/AttentionStrategy.cs:46-71: EffectiveSeqLen = min(pos+1, W)).
        """
        window = _need(d, "sliding_window", int, default=0, required=False) or 0
        types = d.get("layer_types")
        if types is not None:
            if not isinstance(types, (list, tuple)) or len(types) != n_layers:
                raise ConfigError(
                    f"config.json: 'layer_types' must list one entry per layer ({n_layers})")
            out = []
            for i, t in enumerate(types):
                if t == "full_attention":
                    out.append(0)
                elif t == "sliding_attention":
                    if window <= 0:
                        raise ConfigError(
                            "config.json: layer_types names a sliding layer but 'sliding_window' "
                            "is missing or not positive")
                    out.append(window)
                else:
                    raise ConfigError(
                        f"config.json: layer_types[{i}] = {t!r} is not supported "
                        "(known: 'full_attention', 'sliding_attention')")
            return tuple(out)
        use = _need(d, "use_sliding_window", bool, default=False, required=False)
        if not use:
            return tuple([0] * n_layers)
        if window <= 0:
            raise ConfigError("config.json: use_sliding_window=true needs a positive 'sliding_window'")
        # which layers slide must be said: checkpoints disagree on what a missing key would mean
        if d.get("max_window_layers") is None:
            raise ConfigError("config.json: use_sliding_window=true needs 'max_window_layers' (the first layer with "
                              "a window) or 'layer_types'")
        first = _need(d, "max_window_layers", int)
        return tuple(window if i >= first else 0 for i in range(n_layers))

    @classmethod
    def from_json_file(cls, path: str, **kw) -> "DenseDecoderConfig":
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f), **kw)

    def to_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        d = {
            "architectures": [self.architecture],
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "attention_bias": self.attention_bias,
            "qk_norm": self.qk_norm,
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": "bfloat16",
        }
        if self.rotary_dim is not None:
            d["partial_rotary_factor"] = self.rotary_dim / self.head_dim
        if any(self.layer_windows):
            d["sliding_window"] = max(self.layer_windows)
            d["layer_types"] = ["sliding_attention" if w else "full_attention"
                                for w in self.layer_windows]
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json in this folder")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d
