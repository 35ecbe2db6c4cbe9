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

    RING_MAX = 256       # recent tokens per sequence that the kernels can keep on the device

    def begin(self, histories: Sequence[Sequence[int]], params: GenerationParams) -> bool:
        """Puts the recent tokens of a batch's sequences on the device, one ring per sequence (row = position
        in ``histories``); from then on ``sample_device(..., ring_rows=...)`` reads and extends them itself.
        False when the penalties look further back than the kernels keep."""
        self._ring = None
        if not params.uses_history:
            return True
        width = params.penalty_count
        if not 0 < width <= self.RING_MAX:
            return False
        arr = np.zeros((len(histories), width), dtype=np.int32)
        for r, h in enumerate(histories):
            for j in range(max(0, len(h) - width), len(h)):
                arr[r, j % width] = h[j]
        self._ring = torch.from_numpy(arr).to(self.device)
        self._ring_len = torch.tensor([len(h) for h in histories], dtype=torch.int32, device=self.device)
        return True

    def _ints(self, values: Sequence[int]) -> torch.Tensor:
        """A small int32 device tensor, kept for the next step that asks for the same values."""
        key = tuple(int(v) for v in values)
        cache = self.__dict__.setdefault("_int_cache", {})
        t = cache.get(key)
        if t is None:
            if len(cache) > 256:
                cache.clear()
            t = cache[key] = torch.tensor(list(key), dtype=torch.int32, device=self.device)
        return t

    def sample_device(self, logits: torch.Tensor, params: GenerationParams, *, seed: int, step: int,
                      seq_ids: Sequence[int], histories: Optional[Sequence[Sequence[int]]] = None,
                      stop_tokens: Sequence[int] = (), ring_rows: Optional[Sequence[int]] = None) -> torch.Tensor:
        """As ``sample``, but the ids stay on the device (int32 ``[rows]``, valid until the next call).
        ``ring_rows``: the rows of the rings that ``begin`` made, instead of ``histories``."""
        b = logits.shape[0]
        work, out = self._buffers(b)
        if params.greedy and not (params.prevent_eos and stop_tokens) and not params.uses_history:
            self.ops.argmax(logits, out)
            return out
        hist = hist_len = rows = None
        if params.uses_history and ring_rows is not None and getattr(self, "_ring", None) is not None:
            hist, hist_len, rows = self._ring, self._ring_len, self._ints(ring_rows)
        elif params.uses_history and histories is not None:
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
        ids = self._ints(seq_ids)
        self.ops.sample(logits, work, out, temperature=params.temperature, top_k=params.top_k, top_p=params.top_p,
                        min_p=params.min_p, typical_p=params.typical_p, min_keep=params.min_keep,
                        repetition_penalty=params.repetition_penalty, frequency_penalty=params.frequency_penalty,
                        presence_penalty=params.presence_penalty, penalize_newline=params.penalize_newline,
                        seed=seed, step=step, seq_ids=ids, history=hist, history_len=hist_len, banned=banned,
                        history_rows=rows, history_append=rows is not None)
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
