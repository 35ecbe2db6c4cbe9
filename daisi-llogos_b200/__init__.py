"""A small B200-native library for the dense Llama / Qwen2 / Qwen3 decoder: typed configuration,
safetensors weights, composable parts, a paged cache with slots, one step function, generation
and sampling, all on hand-written CUDA kernels for sm_100a.
"""
from . import cache, config, engine, parts, weights  # noqa: F401

__version__ = "0.1.0"
