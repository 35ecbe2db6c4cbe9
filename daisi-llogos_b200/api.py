"""The Python entry point: load (or randomly initialise) a model and generate from token ids.

    model = LlogosModel.load("path/to/folder", dtype="bfloat16", max_context=2048, max_batch=8)
    out = model.generate([[1, 2, 3], [4, 5]], GenerationParams(max_tokens=32, temperature=0))
    out.tokens        # generated ids per prompt

The reference's counterparts are its text backend and chat session
(Chat/DaisiLlogosTextBackend.cs:39,171) and ``TextGenerator.Generate`` / ``Benchmark``
(Inference/TextGenerator.cs:26,126); text and tokenizers are not part of this library.
"""
from __future__ import annotations

from typing import Any, List, Mapping, Optional, Sequence, Union

import torch

from .engine.engine import Engine
from .sampling.generate import GenerationResult, generate
from .sampling.params import GenerationParams
from .sampling.sampler import DeviceSampler
from .weights.loader import load_model, random_model

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def _dtype(d) -> torch.dtype:
    if isinstance(d, torch.dtype):
        return d
    try:
        return _DTYPES[str(d).lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {d!r}") from None


class LlogosModel:
    """A loaded model with its cache, step function, sampler and generation loop."""

    def __init__(self, model, *, max_context: int = 2048, max_batch: int = 8, max_tokens: Optional[int] = None,
                 use_graphs: bool = True):
        self.model = model
        self.max_batch = max_batch
        if max_tokens is None:
            max_tokens = max_batch * ((max_context + 63) // 64) * 64
        self.engine = Engine(model, max_tokens=max_tokens, max_seq_len=max_context, n_slots=max(max_batch, 1),
                             use_graphs=use_graphs)
        self.sampler = DeviceSampler(model.env.ops, model.device, model.spec.vocab_size)

    # ---- construction --------------------------------------------------------------------
    @classmethod
    def load(cls, model_dir: str, *, dtype="bfloat16", device="cuda:0", **kw) -> "LlogosModel":
        return cls(load_model(model_dir, dtype=_dtype(dtype), device=device), **kw)

    @classmethod
    def random(cls, config: Mapping[str, Any], seed: int = 0, *, dtype="bfloat16", device="cuda:0",
               std: float = 0.02, norm_std: float = 0.0, bias_std: float = 0.02, **kw) -> "LlogosModel":
        return cls(random_model(config, seed, dtype=_dtype(dtype), device=device, std=std, norm_std=norm_std,
                                bias_std=bias_std), **kw)

    # ---- use -------------------------------------------------------------------------------
    @property
    def config(self):
        return self.model.config

    @property
    def stop_token_ids(self):
        return tuple(self.model.spec.stop_token_ids)

    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]],
                 params: Optional[GenerationParams] = None, **kw) -> GenerationResult:
        """Generates for one prompt (a list of ids) or several (a list of lists), host ids in and out.

        Without ``params.stop_tokens`` the model's end-of-sequence ids stop a sequence.
        """
        params = params or GenerationParams()
        single = len(prompts) > 0 and not isinstance(prompts[0], (list, tuple))
        batch = [list(prompts)] if single else [list(p) for p in prompts]
        stop = params.stop_tokens if params.stop_tokens is not None else self.stop_token_ids
        sync = (lambda: torch.cuda.synchronize(self.model.device)) if self.model.device.type == "cuda" else None
        return generate(self.engine, self.sampler, batch, params, stop_tokens=stop, max_batch=self.max_batch,
                        sync=sync, **kw)

    def open(self) -> int:
        return self.engine.open()

    def close(self, slot: int) -> None:
        self.engine.close(slot)

    def step(self, entries, want=None) -> torch.Tensor:
        """See ``Engine.step``."""
        return self.engine.step(entries, want)
