"""One registry from an architecture's name to its configuration reader and model builder.

The reference dispatches on the GGUF architecture string in its command line
(Daisi.Llogos.Cli/Program.cs:54-101) and infers optional tensors from their
presence (Model/ModelLoader.cs:106-110).  Here a name maps to two functions:
``read_config(dict) -> typed config`` and ``build_spec(config) -> ModelSpec``;
options come from the configuration, never from tensor shapes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .dense import ConfigError, DenseDecoderConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    read_config: Callable[[Mapping[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, read_config, build_spec, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = Architecture(name, read_config, build_spec)


def known_architectures():
    return sorted(_ARCHITECTURES)


def architecture_of(config_dict: Mapping[str, Any]) -> Architecture:
    archs = config_dict.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs:
        raise ConfigError("config.json: missing key 'architectures' (a non-empty list of names)")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"config.json: architecture '{name}' is not registered (known: {', '.join(known_architectures())})")
    return _ARCHITECTURES[name]


# ---- the dense decoder ------------------------------------------------------------

def dense_decoder_spec(cfg: DenseDecoderConfig) -> ModelSpec:
    """Pre-norm decoder of RMSNorm, rotary GQA attention and SwiGLU.

    Layer order as the reference runs it (Inference/ForwardPass.cs:199-267):
    norm, attention, residual, norm, feed-forward, residual; then the final norm
    and the output head (:174-184), which falls back to the embedding table when
    the model ties them (Model/ModelWeights.cs:29).
    """
    norm = {"eps": cfg.rms_norm_eps, "size": cfg.hidden_size}
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = PartSpec("attention", {
            "hidden_size": cfg.hidden_size,
            "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "qkv_bias": cfg.attention_bias,
            "qk_norm": cfg.qk_norm,
            "qk_norm_eps": cfg.rms_norm_eps,
            "window": cfg.window_of(i),
            "position": "rope",
            "softmax_scale": None,          # None = 1/sqrt(head_dim), Inference/ForwardPass.cs:336
        }, p + "self_attn.")
        ffn = PartSpec("swiglu", {
            "hidden_size": cfg.hidden_size,
            "intermediate_size": cfg.intermediate_size,
        }, p + "mlp.")
        layers.append(LayerSpec("prenorm", {
            "norm1": PartSpec("rmsnorm", dict(norm), p + "input_layernorm."),
            "mixer": mixer,
            "norm2": PartSpec("rmsnorm", dict(norm), p + "post_attention_layernorm."),
            "ffn": ffn,
        }))
    rope = PartSpec("rotary", {
        "head_dim": cfg.head_dim,
        "rotary_dim": cfg.rotary_dim or cfg.head_dim,
        "theta": cfg.rope_theta,
        "scaling": cfg.rope_scaling.to_dict() if cfg.rope_scaling else None,
        "pairing": "half",                  # safetensors rows are not permuted: pair (i, i + d/2)
    })
    spec = ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding",
                           {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size},
                           "model.embed_tokens."),
        encodings={"rope": rope},
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", dict(norm), "model.norm."),
        head=PartSpec("linear_head",
                      {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                       "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None},
                      "lm_head."),
        stop_token_ids=cfg.eos_token_ids,
        # exporters write the rotation's frequency buffers beside the weights, and some write the output
        # matrix again although it is tied to the embedding table
        ignorable_tensors=(r".*\.rotary_emb\.inv_freq",) + ((r"lm_head\.weight",) if cfg.tie_word_embeddings else ()),
    )
    spec.validate()
    return spec


def _dense_reader(*, qk_norm: bool, force_bias: bool):
    def read(d: Mapping[str, Any]) -> DenseDecoderConfig:
        return DenseDecoderConfig.from_dict(d, qk_norm=qk_norm, force_attention_bias=force_bias)
    return read


register_architecture("LlamaForCausalLM", _dense_reader(qk_norm=False, force_bias=False), dense_decoder_spec)
register_architecture("Qwen2ForCausalLM", _dense_reader(qk_norm=False, force_bias=True), dense_decoder_spec)
register_architecture("Qwen3ForCausalLM", _dense_reader(qk_norm=True, force_bias=False), dense_decoder_spec)
