"""Configuration and registry (no GPU)."""
import copy
import json

import pytest

from conftest import TINY, TINY_LLAMA, TINY_QWEN2, TINY_QWEN3


def test_reads_every_key(llogos):
    C = llogos.config
    for cfg in TINY.values():
        arch = C.architecture_of(cfg)
        c = arch.read_config(cfg)
        assert c.num_hidden_layers == cfg["num_hidden_layers"]
        assert c.hidden_size == cfg["hidden_size"]
        assert c.intermediate_size == cfg["intermediate_size"]
        assert c.vocab_size == cfg["vocab_size"]
        assert c.num_attention_heads == cfg["num_attention_heads"]
        assert c.num_key_value_heads == cfg["num_key_value_heads"]
        assert c.head_dim == cfg["head_dim"]
        assert c.rms_norm_eps == cfg["rms_norm_eps"]
        assert c.rope_theta == cfg["rope_theta"]
        assert c.max_position_embeddings == cfg["max_position_embeddings"]


def test_architecture_options(llogos):
    C = llogos.config
    llama = C.architecture_of(TINY_LLAMA).read_config(TINY_LLAMA)
    assert (llama.qk_norm, llama.attention_bias, llama.tie_word_embeddings) == (False, False, False)
    assert llama.eos_token_ids == (2,) and llama.layer_windows == (0, 0)
    q3 = C.architecture_of(TINY_QWEN3).read_config(TINY_QWEN3)
    assert (q3.qk_norm, q3.attention_bias, q3.tie_word_embeddings) == (True, True, True)
    assert q3.layer_windows == (0, 24, 0) and q3.eos_token_ids == (5, 7)
    q2 = C.architecture_of(TINY_QWEN2).read_config(TINY_QWEN2)
    assert (q2.qk_norm, q2.attention_bias) == (False, True)
    assert q2.layer_windows == (0, 0, 70, 70)
    assert q2.rope_scaling.factor == 4.0 and q2.rope_scaling.original_max_position_embeddings == 64


def test_defaults(llogos):
    cfg = {k: v for k, v in TINY_LLAMA.items() if k not in ("head_dim", "num_key_value_heads", "rms_norm_eps", "rope_theta")}
    c = llogos.config.architecture_of(cfg).read_config(cfg)
    assert c.head_dim == 16 and c.num_key_value_heads == 4
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0      # the reference's defaults
    assert c.rotary_dim is None                                      # every dimension of a head is rotated


def test_without_a_position_limit_the_cache_is_the_limit(llogos):
    cfg = {k: v for k, v in TINY_LLAMA.items() if k != "max_position_embeddings"}
    c = llogos.config.architecture_of(cfg).read_config(cfg)
    assert c.max_position_embeddings is None
    assert llogos.config.dense_decoder_spec(c).max_positions is None


def test_partial_rotary_factor(llogos):
    cfg = dict(TINY_LLAMA, partial_rotary_factor=0.5)
    c = llogos.config.architecture_of(cfg).read_config(cfg)
    assert c.rotary_dim == 8
    spec = llogos.config.dense_decoder_spec(c)
    assert spec.encodings["rope"].params["rotary_dim"] == 8 and spec.encodings["rope"].params["head_dim"] == 16
    full = dict(TINY_LLAMA, partial_rotary_factor=1.0)
    assert llogos.config.architecture_of(full).read_config(full).rotary_dim is None


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "intermediate_size", "vocab_size",
                                 "num_attention_heads", "architectures"])
def test_missing_key_is_named(llogos, key):
    cfg = copy.deepcopy(TINY_LLAMA)
    del cfg[key]
    with pytest.raises(llogos.config.ConfigError, match=key):
        llogos.config.architecture_of(cfg).read_config(cfg)


@pytest.mark.parametrize("patch, word", [
    ({"hidden_size": "64"}, "hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "head_dim"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"use_sliding_window": True}, "sliding_window"),
    ({"use_sliding_window": True, "sliding_window": 32}, "max_window_layers"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"eos_token_id": 100000}, "eos_token_id"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"partial_rotary_factor": 0.45}, "partial_rotary_factor"),
    ({"partial_rotary_factor": 1.5}, "partial_rotary_factor"),
    ({"max_position_embeddings": 0}, "max_position_embeddings"),
])
def test_bad_values(llogos, patch, word):
    cfg = copy.deepcopy(TINY_LLAMA)
    cfg.update(patch)
    with pytest.raises(llogos.config.ConfigError, match=word):
        llogos.config.architecture_of(cfg).read_config(cfg)


def test_unknown_architecture_lists_known(llogos):
    cfg = dict(TINY_LLAMA, architectures=["GemmaForCausalLM"])
    with pytest.raises(llogos.config.ConfigError) as e:
        llogos.config.architecture_of(cfg)
    assert "LlamaForCausalLM" in str(e.value) and "Qwen3ForCausalLM" in str(e.value)


def test_round_trip_through_json(llogos):
    for cfg in TINY.values():
        arch = llogos.config.architecture_of(cfg)
        c = arch.read_config(cfg)
        again = arch.read_config(json.loads(json.dumps(c.to_dict())))
        assert again == c


def test_spec_is_data(llogos):
    """Layers differ by configuration: the sliding layer of the Qwen3 config gets a window."""
    C = llogos.config
    spec = C.dense_decoder_spec(C.architecture_of(TINY_QWEN3).read_config(TINY_QWEN3))
    windows = [l.parts["mixer"].params["window"] for l in spec.layers]
    assert windows == [0, 24, 0]
    assert [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.head.params["tied_to"] == "model.embed_tokens.weight"
    assert spec.stop_token_ids == (5, 7)


def test_register_architecture(llogos):
    C = llogos.config
    C.register_architecture("ToyForCausalLM", C.architecture_of(TINY_LLAMA).read_config, C.dense_decoder_spec)
    try:
        assert "ToyForCausalLM" in C.known_architectures()
        with pytest.raises(ValueError):
            C.register_architecture("ToyForCausalLM", None, None)
    finally:
        importlib = __import__("importlib")
        importlib.import_module("daisi-llogos_b200.config.registry")._ARCHITECTURES.pop("ToyForCausalLM")


def test_plugin_modules_register_architectures_for_the_command_line(tmp_path):
    """A module named in LLOGOS_PLUGINS is imported with the library, so what it registers is known wherever a
    model is chosen by its config.json; a name that cannot be imported is an error that says so."""
    import os
    import subprocess
    import sys
    from conftest import ROOT
    (tmp_path / "toy_plugin.py").write_text(
        "import importlib\n"
        "C = importlib.import_module('daisi-llogos_b200.config')\n"
        "R = importlib.import_module('daisi-llogos_b200.config.registry')\n"
        "C.register_architecture('PluginToyLM', R._dense_reader(qk_norm=False, force_bias=False), C.dense_decoder_spec)\n")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([str(tmp_path), ROOT]), LLOGOS_PLUGINS="toy_plugin")
    code = "import llogos_b200 as L; print('PluginToyLM' in L.config.known_architectures())"
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=str(tmp_path))
    assert p.returncode == 0 and p.stdout.strip() == "True", p.stderr
    env["LLOGOS_PLUGINS"] = "toy_plugin, no_such_module_here"
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=str(tmp_path))
    assert p.returncode != 0 and "LLOGOS_PLUGINS" in p.stderr and "no_such_module_here" in p.stderr
