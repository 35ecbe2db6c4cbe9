"""A small B200-native library for the dense Llama / Qwen2 / Qwen3 decoder: typed configuration,
safetensors weights, composable parts, a paged cache with slots, one step function, generation
and sampling, all on hand-written CUDA kernels for sm_100a.

``LLOGOS_PLUGINS`` (module names separated by commas) names modules that are imported once the library is:
a module that registers parts or an architecture of its own (``parts.register_part``,
``config.register_architecture``) is so known to the command line and to ``bin/trace_run`` as well, which choose
the model class by config.json like everything else.
"""
import importlib as _importlib
import os as _os

from . import cache, config, engine, parts, weights  # noqa: F401

__version__ = "0.1.0"


def _load_plugins() -> None:
    for name in (n.strip() for n in _os.environ.get("LLOGOS_PLUGINS", "").split(",")):
        if not name:
            continue
        try:
            _importlib.import_module(name)
        except ImportError as e:
            raise ImportError(f"LLOGOS_PLUGINS names the module '{name}', which cannot be imported: {e}") from e


_load_plugins()
