"""Sampling parameters and stop conditions, with the reference's names and defaults
(Inference/GenerationParams.cs:6-60).  Anti-prompt strings and grammars are not carried."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class GenerationParams:
    max_tokens: int = 256                 # most tokens to generate per sequence
    temperature: float = 0.8              # 0 = greedy (lowest index among the maxima)
    top_k: int = 40                       # 0 = off
    top_p: float = 0.95                   # 1.0 = off
    repetition_penalty: float = 1.1       # 1.0 = off
    stop_tokens: Optional[Tuple[int, ...]] = None   # None = the model's end-of-sequence ids
    seed: Optional[int] = None            # None = a fresh seed per call
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    min_p: float = 0.0                    # 0 = off
    typical_p: float = 1.0                # 1.0 = off
    penalize_newline: bool = False
    penalty_count: int = 64               # recent tokens the penalties look at; 0 = all
    min_keep: int = 1
    prevent_eos: bool = False             # stop tokens can never be drawn

    def validate(self) -> None:
        if self.max_tokens < 0:
            raise ValueError("max_tokens must not be negative")
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")
        if self.top_k < 0 or self.penalty_count < 0 or self.min_keep < 0:
            raise ValueError("top_k, penalty_count and min_keep must not be negative")

    @property
    def greedy(self) -> bool:
        """No penalties and temperature 0: the plain argmax (Inference/Sampler.cs:32-34)."""
        return (self.temperature == 0 and self.repetition_penalty == 1.0
                and self.frequency_penalty == 0 and self.presence_penalty == 0)

    @property
    def uses_history(self) -> bool:
        return self.repetition_penalty != 1.0 or self.frequency_penalty != 0 or self.presence_penalty != 0

    @classmethod
    def greedy_params(cls, max_tokens: int = 256, **kw) -> "GenerationParams":
        return cls(max_tokens=max_tokens, temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.0, **kw)
