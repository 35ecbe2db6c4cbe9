"""The sampler that generation uses: one kernel launch per step for the whole batch."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .params import GenerationParams


class DeviceSampler:
    """Draws one token per row of the logits on the GPU (csrc/sampling.cu).

    ``seq_ids`` identify sequences across batches, so that with a seed a sequence's tokens do not
    depend on which other sequences share its batch.
    """

    def __init__(self, ops, device: torch.device, vocab_size: int):
        self.ops = ops
        self.device = device
        self.vocab = vocab_size
        self._work: Optional[torch.Tensor] = None
        self._out: Optional[torch.Tensor] = None
        self._banned = None
        self._banned_key = None

    def _buffers(self, b: int):
        if self._work is None or self._work.numel() < b * self.vocab:
            self._work = torch.empty(b * self.vocab, dtype=torch.float32, device=self.device)
            self._out = torch.empty(b, dtype=torch.int32, device=self.device)
        return self._work, self._out[:b]

    def sample(self, logits: torch.Tensor, params: GenerationParams, *, seed: int, step: int,
               seq_ids: Sequence[int], histories: Optional[Sequence[Sequence[int]]] = None,
               stop_tokens: Sequence[int] = ()) -> List[int]:
        return self.sample_device(logits, params, seed=seed, step=step, seq_ids=seq_ids, histories=histories,
                                  stop_tokens=stop_tokens).cpu().tolist()

    def fetch(self, picked: torch.Tensor) -> "PendingTokens":
        """Starts the copy of ``picked`` (what ``sample_device`` returned) to pinned host memory and returns
        at once; ``result()`` of the returned object waits for the copy and gives the ids."""
        b = picked.numel()
        self._fetch_i = (getattr(self, "_fetch_i", 0) + 1) % 4
        bufs = self.__dict__.setdefault("_fetch_bufs", [None] * 4)
        buf = bufs[self._fetch_i]
        if buf is None or buf.numel() < b:
            buf = bufs[self._fetch_i] = torch.empty(max(b, 64), dtype=torch.int32, pin_memory=self.device.type == "cuda")
        buf[:b].copy_(picked, non_blocking=True)
        event = None
        if self.device.type == "cuda":
            event = torch.cuda.Event()
            event.record()
        return PendingTokens(buf[:b], event)

    def sample_device(self, logits: torch.Tensor, params: GenerationParams, *, seed: int, step: int,
                      seq_ids: Sequence[int], histories: Optional[Sequence[Sequence[int]]] = None,
                      stop_tokens: Sequence[int] = ()) -> torch.Tensor:
        """As ``sample``, but the ids stay on the device (int32 ``[rows]``, valid until the next call)."""
        b = logits.shape[0]
        work, out = self._buffers(b)
        if params.greedy and not (params.prevent_eos and stop_tokens):
            self.ops.argmax(logits, out)
            return out
        hist = hist_len = None
        if params.uses_history and histories is not None:
            win = [list(h[-params.penalty_count:]) if params.penalty_count > 0 else list(h) for h in histories]
            width = max(1, max(len(w) for w in win))
            arr = np.zeros((b, width), dtype=np.int32)
            for i, w in enumerate(win):
                arr[i, :len(w)] = w
            hist = torch.from_numpy(arr).to(self.device)
            hist_len = torch.tensor([len(w) for w in win], dtype=torch.int32, device=self.device)
        banned = None
        if params.prevent_eos and stop_tokens:
            key = tuple(stop_tokens)
            if self._banned_key != key:
                self._banned = torch.tensor(list(key), dtype=torch.int32, device=self.device)
                self._banned_key = key
            banned = self._banned
        ids = torch.tensor(list(seq_ids), dtype=torch.int32, device=self.device)
        self.ops.sample(logits, work, out, temperature=params.temperature, top_k=params.top_k, top_p=params.top_p,
                        min_p=params.min_p, typical_p=params.typical_p, min_keep=params.min_keep,
                        repetition_penalty=params.repetition_penalty, frequency_penalty=params.frequency_penalty,
                        presence_penalty=params.presence_penalty, penalize_newline=params.penalize_newline,
                        seed=seed, step=step, seq_ids=ids, history=hist, history_len=hist_len, banned=banned)
        return out


class PendingTokens:
    """Token ids on their way to the host."""

    def __init__(self, host: torch.Tensor, event):
        self._host = host
        self._event = event

    def result(self) -> List[int]:
        if self._event is not None:
            self._event.synchronize()
        return self._host.tolist()
