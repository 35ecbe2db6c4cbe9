"""Shared fixtures: the library under its import name, tiny configurations, model folders."""
import importlib
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def llogos():
    return importlib.import_module("daisi-llogos_b200")


# Tiny configurations that differ in every size and option.
TINY_LLAMA = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 176,
    "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 512,
    "tie_word_embeddings": False, "eos_token_id": 2,
}
TINY_QWEN3 = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 3, "hidden_size": 96,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 32, "intermediate_size": 256,
    "vocab_size": 384, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 1024,
    "tie_word_embeddings": True, "attention_bias": True, "sliding_window": 24,
    "layer_types": ["full_attention", "sliding_attention", "full_attention"], "eos_token_id": [5, 7],
}
TINY_QWEN2 = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 4, "hidden_size": 80,
    "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 48, "intermediate_size": 112,
    "vocab_size": 301, "rope_theta": 50000.0, "rms_norm_eps": 3e-5, "max_position_embeddings": 2048,
    "tie_word_embeddings": False, "use_sliding_window": True, "sliding_window": 70, "max_window_layers": 2,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
}
# head size 128: the geometry the tcgen05 attention and the register-resident q/k kernel are written for
TINY_WIDE = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 192,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 320,
    "vocab_size": 500, "rope_theta": 20000.0, "rms_norm_eps": 2e-6, "max_position_embeddings": 1024,
    "tie_word_embeddings": False, "sliding_window": 90,
    "layer_types": ["sliding_attention", "full_attention"],
}
# sums long enough (k = 576 and 1096) that the tensor-core products split them: the q/k/v kernel and the
# norms add up partial results, and the output head must not hand out half a sum
TINY_DEEP = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 576,
    "num_attention_heads": 9, "num_key_value_heads": 3, "head_dim": 64, "intermediate_size": 1096,
    "vocab_size": 1003, "rope_theta": 300000.0, "rms_norm_eps": 4e-6, "max_position_embeddings": 1024,
    "tie_word_embeddings": True, "attention_bias": True, "partial_rotary_factor": 0.5,
}
TINY = {"llama": TINY_LLAMA, "qwen3": TINY_QWEN3, "qwen2": TINY_QWEN2, "wide": TINY_WIDE, "deep": TINY_DEEP}
INIT = dict(std=0.15, norm_std=0.1, bias_std=0.1)
INIT_OF = {"deep": dict(std=0.05, norm_std=0.1, bias_std=0.1)}     # spread follows the width


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory, llogos):
    """Folders with config.json and model.safetensors of the tiny configurations (random weights)."""
    out = {}
    for i, (name, cfg) in enumerate(TINY.items()):
        d = str(tmp_path_factory.mktemp(f"model_{name}"))
        llogos.weights.write_random_model(d, cfg, seed=100 + i, **INIT_OF.get(name, INIT))
        out[name] = d
    return out


def read_weights(llogos, model_dir):
    files = llogos.weights.ModelFiles(model_dir)
    return {n: files.tensor(n).clone() for n in files.names()}


def random_tokens(vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
