"""What a step hands to the parts: the packed token layout, the batch's cache bookkeeping
on the device, and scratch memory.

Tokens of all sequences of a step are packed without padding: sequence ``b`` of the batch
owns tokens ``cu_tokens[b] .. cu_tokens[b+1]``; ``positions[n]`` is a token's position in its
sequence and ``seq_of_token[n]`` its sequence's index in the batch.  The reference runs one
sequence at a time with a start position (Inference/IForwardPass.cs:8-45); the packed layout
is what lets unequal prompts share one step.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch


class Workspace:
    """Named scratch buffers that only grow; a name is reused by every layer in turn."""

    def __init__(self, device: torch.device):
        self.device = device
        self._flat: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._views: Dict[Tuple[str, torch.dtype, Tuple[int, ...]], torch.Tensor] = {}
        self.frozen = False   # set while a CUDA graph that uses these buffers exists

    def get(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """``zero``: the buffer is zero when it is first handed out (and whenever it had to grow)."""
        view = self._views.get((name, dtype, shape))
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        flat = self._flat.get(key)
        if flat is None or flat.numel() < n:
            if self.frozen:
                raise RuntimeError(f"workspace buffer '{name}' would have to grow after graph capture")
            flat = (torch.zeros if zero else torch.empty)(max(n, 1), dtype=dtype, device=self.device)
            self._flat[key] = flat
            for k in [k for k in self._views if k[0] == name and k[1] == dtype]:
                del self._views[k]          # views of the buffer that was replaced
        if len(self._views) > 4096:
            self._views.clear()
        view = self._views[(name, dtype, shape)] = flat[:n].view(shape)
        return view

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._flat.values())


@dataclass
class StepContext:
    n_tokens: int
    n_seqs: int
    decode: bool                      # every sequence brings exactly one token
    counts: List[int]                 # tokens per sequence (host)
    max_count: int
    # device int32 tensors
    token_ids: torch.Tensor           # [N]
    positions: torch.Tensor           # [N]
    seq_of_token: torch.Tensor        # [N]
    slots: torch.Tensor               # [B]
    cu_tokens: torch.Tensor           # [B + 1]
    len_before: torch.Tensor          # [B] tokens each sequence held before this step
    prefill_tiles: Optional[Dict[int, torch.Tensor]]   # queries per tile -> [n_tiles, 2] (sequence, first query)
    dtype: torch.dtype = torch.float32
    device: torch.device = None
    ops: Any = None
    workspace: Workspace = None
    max_len_after: int = 0            # host upper bound of len_before + count over the batch
    extras: Dict[str, Any] = field(default_factory=dict)

    def buffer(self, name: str, shape, dtype=None, zero: bool = False) -> torch.Tensor:
        return self.workspace.get(name, tuple(shape), dtype or self.dtype, zero)
