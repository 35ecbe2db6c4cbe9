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
from typing import Any, Callable, Dict, List, Optional, Tuple

import numpy as np
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
    dtype: torch.dtype = torch.float32
    device: torch.device = None
    ops: Any = None
    workspace: Workspace = None
    max_len_after: int = 0            # host upper bound of len_before + count over the batch
    len_before_host: Optional[List[int]] = None   # the same lengths on the host (None in a decode step, where
                                                  # the launches are recorded once and replayed)
    upload: Optional[Callable[[np.ndarray, torch.Tensor], None]] = None   # host int32 array -> device buffer
    extras: Dict[str, Any] = field(default_factory=dict)

    def buffer(self, name: str, shape, dtype=None, zero: bool = False) -> torch.Tensor:
        return self.workspace.get(name, tuple(shape), dtype or self.dtype, zero)

    def query_tiles(self, tile_queries: int) -> torch.Tensor:
        """The step's queries cut into tiles of ``tile_queries`` per sequence: int32 ``[n_tiles, 2]`` (sequence,
        first query among its step tokens), the tiles that see the most keys first (a mixer's blocks start in
        list order, and the long ones should not be the last to start).  Worked out when a mixer first asks
        for a tile size and kept for the rest of the step; a step with one token per sequence has none."""
        key = ("query_tiles", int(tile_queries))
        tiles = self.extras.get(key)
        if tiles is None:
            if self.len_before_host is None:
                raise RuntimeError("query_tiles: this step's lengths are not known on the host")
            tq = int(tile_queries)
            lb, counts = self.len_before_host, self.counts
            order = sorted(((i, q0) for i, c in enumerate(counts) for q0 in range(0, c, tq)),
                           key=lambda t: -(lb[t[0]] + min(counts[t[0]], t[1] + tq)))
            host = np.asarray(order, dtype=np.int32).reshape(-1)
            dev = self.buffer(f"query_tiles.{tq}", (host.size,), torch.int32)
            if self.upload is not None:
                self.upload(host, dev)
            else:
                dev.copy_(torch.from_numpy(host))
            tiles = self.extras[key] = dev.view(-1, 2)
        return tiles
