"""The Python entry point: load (or randomly initialise) a model and generate from token ids.

    model = LlogosModel.load("path/to/folder", dtype="bfloat16", max_context=2048, max_batch=8)
    out = model.generate([[1, 2, 3], [4, 5]], GenerationParams(max_tokens=32, temperature=0))
    out.tokens        # generated ids per prompt

The reference's counterparts are its text backend and chat session
(Chat/DaisiLlogosTextBackend.cs:39,171) and ``TextGenerator.Generate`` / ``Benchmark``
(Inference/TextGenerator.cs:26,126); text and tokenizers are not part of this library.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Sequence, Union

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


@dataclass
class BenchmarkResult:
    """What ``LlogosModel.benchmark`` measured: the reference's fields (Inference/TextGenerator.cs:176-184) and, beyond
    them, the bytes a decode step had to read and the flops of the prompt step with the fractions of the peaks."""

    prompt_tokens: int
    generated_tokens: int
    prefill_seconds: float
    decode_seconds: float
    prefill_tokens_per_second: float
    decode_tokens_per_second: float
    batch: int
    prompt_lengths: List[int]
    final_lengths: List[int]
    decode_steps: int
    decode_bytes_per_step: float
    decode_gb_per_second: float
    decode_fraction_of_copy_bandwidth: float
    prompt_step_flops: float
    prompt_tflops: float
    prompt_fraction_of_matrix_peak: float
    peaks: Dict[str, Any]


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

    def benchmark(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]], max_tokens: int = 128, *,
                  peaks_file: Optional[str] = None) -> "BenchmarkResult":
        """Warm-up, then the prompts in one timed step and ``max_tokens`` greedy tokens per sequence, timed (the
        reference's ``TextGenerator.Benchmark``, Inference/TextGenerator.cs:126-186: prompt tokens, generated tokens,
        the two times and rates).  Unlike the reference it takes a batch, ignores stop tokens (every sequence makes
        ``max_tokens`` tokens unless the cache's limit ends it), and adds what the steps had to move and compute,
        against the measured peaks (``measure.peaks(peaks_file)``)."""
        from .measure import decode_bytes_of_run, model_costs, peaks
        single = len(prompts) > 0 and not isinstance(prompts[0], (list, tuple))
        batch = [list(prompts)] if single else [list(p) for p in prompts]
        self.generate([p[:64] for p in batch], GenerationParams.greedy_params(min(4, max_tokens), stop_tokens=()))   # warm-up
        r = self.generate(batch, GenerationParams.greedy_params(max_tokens, stop_tokens=()))
        pk = peaks(peaks_file)
        costs = model_costs(self.model)
        lens, made = [len(p) for p in batch], [len(t) for t in r.tokens]
        decode_bytes, n_steps = decode_bytes_of_run(costs, lens, made)
        flops = costs.prompt_step_flops(lens, wanted_rows=len(lens))
        gbs = decode_bytes / r.decode_seconds / 1e9 if r.decode_seconds > 0 and n_steps else 0.0
        tflops = flops / r.prefill_seconds / 1e12 if r.prefill_seconds > 0 else 0.0
        return BenchmarkResult(
            prompt_tokens=r.prompt_tokens, generated_tokens=r.generated_tokens, prefill_seconds=r.prefill_seconds,
            decode_seconds=r.decode_seconds, prefill_tokens_per_second=r.prefill_tokens_per_second,
            decode_tokens_per_second=r.decode_tokens_per_second, batch=len(batch), prompt_lengths=lens,
            final_lengths=[n + m for n, m in zip(lens, made)], decode_steps=n_steps,
            decode_bytes_per_step=decode_bytes / max(1, n_steps), decode_gb_per_second=gbs,
            decode_fraction_of_copy_bandwidth=gbs / pk["hbm_gbs"], prompt_step_flops=flops, prompt_tflops=tflops,
            prompt_fraction_of_matrix_peak=tflops / pk["bf16_tflops"], peaks=pk)

    def truncate(self, slot: int, n_tokens: int) -> None:
        """Rolls a sequence back to its first ``n_tokens`` tokens (the reference's ``KvCache.SetLength``,
        Inference/KvCache.cs); see ``Engine.truncate`` for when that is refused."""
        self.engine.truncate(slot, n_tokens)

    def open(self) -> int:
        return self.engine.open()

    def close(self, slot: int) -> None:
        self.engine.close(slot)

    def step(self, entries, want=None) -> torch.Tensor:
        """See ``Engine.step``."""
        return self.engine.step(entries, want)
