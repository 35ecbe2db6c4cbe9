"""The generation loop above the step function.

Requests (lists of token ids) are served in batches, one batch after another: a batch's
prompts, unequal in length, run in one step; then every live sequence gets one token per step.
A sequence ends at a stop token (which is not emitted, Inference/TextGenerator.cs:78-79), at
``max_tokens`` (:73) or when the cache cannot hold a longer sequence; it then leaves the
batch, which goes on smaller.  When the batch is over, its slots go back to the cache and the
next batch uses them again.  The loop decides; the engine and the sampler do the arithmetic, so
the decisions can be tested with stand-ins for both.

When the sampler can leave its tokens on the device and the engine can take them from there
(``sample_device`` / ``fetch`` / ``step_fed``; with penalties also ``begin``, which puts the recent
tokens on the device where the sampler extends them itself), the loop runs one step ahead of what it
has read: it queues the step that consumes the tokens of sample k before it
reads them, and reads them while that step runs.  A stop token is then seen one step late; the
sequence has run one step too many, whose token is thrown away.  The tokens that come out are the same.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from .params import GenerationParams


@dataclass
class GenerationResult:
    tokens: List[List[int]]                 # generated ids per request, in request order
    finish_reasons: List[str]               # "stop" | "length" | "context" per request
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    batches: int = 0
    decode_steps: int = 0

    @property
    def prefill_tokens_per_second(self) -> float:
        return self.prompt_tokens / self.prefill_seconds if self.prefill_seconds > 0 else 0.0

    @property
    def decode_tokens_per_second(self) -> float:
        return self.generated_tokens / self.decode_seconds if self.decode_seconds > 0 else 0.0


def plan_batches(prompt_lengths: Sequence[int], max_new: int, *, max_batch: int, free_pages: int,
                 page: int, max_seq_len: int) -> List[List[int]]:
    """Splits request indices, in order, into batches that fit the slots and the pages.

    A request is charged the pages of its prompt plus ``max_new`` tokens (capped by the longest
    sequence the cache holds).  A request that cannot fit even alone raises ``ValueError``.
    """
    batches: List[List[int]] = []
    cur: List[int] = []
    cur_pages = 0
    for i, n in enumerate(prompt_lengths):
        if n <= 0:
            raise ValueError(f"request {i}: empty prompt")
        if n > max_seq_len:
            raise ValueError(f"request {i}: prompt of {n} tokens exceeds the longest sequence ({max_seq_len})")
        need = (min(n + max_new, max_seq_len) + page - 1) // page
        if need > free_pages:
            raise ValueError(f"request {i}: needs {need} cache pages, only {free_pages} exist")
        if cur and (len(cur) >= max_batch or cur_pages + need > free_pages):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(i)
        cur_pages += need
    if cur:
        batches.append(cur)
    return batches


def generate(engine, sampler, prompts: Sequence[Sequence[int]], params: GenerationParams, *,
             stop_tokens: Optional[Sequence[int]] = None, max_batch: int = 64,
             on_token: Optional[Callable[[int, int], None]] = None,
             clock: Callable[[], float] = time.perf_counter,
             sync: Optional[Callable[[], None]] = None, run_ahead: bool = True) -> GenerationResult:
    """Generates for every prompt; ``on_token(request index, token)`` is called as tokens appear.

    ``engine`` needs ``open()``, ``close(slot)``, ``step(entries, want=None)`` and a ``cache`` with
    ``n_pages`` (or ``free_pages()``) / ``max_seq_len`` / ``slots.free_count``; ``sampler.sample(logits, params, seed=, step=,
    seq_ids=, histories=, stop_tokens=)`` returns one token per row.
    """
    params.validate()
    if stop_tokens is None:
        stop_tokens = params.stop_tokens if params.stop_tokens is not None else ()
    stop = frozenset(int(t) for t in stop_tokens)
    seed = params.seed if params.seed is not None else int.from_bytes(os.urandom(8), "little")
    sync = sync or (lambda: None)
    n_req = len(prompts)
    result = GenerationResult(tokens=[[] for _ in range(n_req)], finish_reasons=["length"] * n_req)
    if n_req == 0:
        return result
    cache = engine.cache
    page = getattr(cache, "page", 64)
    # what is free now: sequences that the caller holds open keep their pages while this call runs
    free_pages = cache.free_pages() if hasattr(cache, "free_pages") else cache.n_pages
    batches = plan_batches([len(p) for p in prompts], params.max_tokens, max_batch=min(max_batch, cache.slots.free_count),
                           free_pages=free_pages, page=page, max_seq_len=cache.max_seq_len)
    for batch in batches:
        result.batches += 1
        slots = {i: engine.open() for i in batch}
        try:
            histories = {i: list(prompts[i]) for i in batch}
            active = list(batch)
            sync()
            t0 = clock()
            logits = engine.step([(slots[i], list(prompts[i])) for i in active]) if params.max_tokens > 0 else None
            sync()
            result.prefill_seconds += clock() - t0
            result.prompt_tokens += sum(len(prompts[i]) for i in active)
            t0 = clock()
            step_no = 0
            if (run_ahead and params.max_tokens > 0 and hasattr(sampler, "sample_device")
                    and hasattr(sampler, "fetch") and hasattr(engine, "step_fed")
                    and (not params.uses_history
                         or (hasattr(sampler, "begin") and sampler.begin([histories[i] for i in active], params)))):
                _decode_ahead(engine, sampler, params, seed, sorted(stop), stop, slots, histories, active, logits,
                              result, on_token, cache.max_seq_len)
                active = []
            while active and params.max_tokens > 0:
                picked = sampler.sample(logits, params, seed=seed, step=step_no, seq_ids=active,
                                        histories=[histories[i] for i in active], stop_tokens=sorted(stop))
                nxt = []
                for i, tok in zip(active, picked):
                    tok = int(tok)
                    if tok in stop:
                        result.finish_reasons[i] = "stop"
                        continue
                    result.tokens[i].append(tok)
                    histories[i].append(tok)
                    result.generated_tokens += 1
                    if on_token is not None:
                        on_token(i, tok)
                    if len(result.tokens[i]) >= params.max_tokens:
                        result.finish_reasons[i] = "length"
                    elif len(histories[i]) >= cache.max_seq_len:
                        result.finish_reasons[i] = "context"
                    else:
                        nxt.append(i)
                active = nxt
                step_no += 1
                if not active:
                    break
                logits = engine.step([(slots[i], [histories[i][-1]]) for i in active])
                result.decode_steps += 1
            sync()
            result.decode_seconds += clock() - t0
        finally:
            for s in slots.values():
                engine.close(s)
    return result


def _decode_ahead(engine, sampler, params, seed, stop_list, stop, slots, histories, active, logits, result,
                  on_token, max_seq_len) -> None:
    """The decode loop of one batch, one step ahead of the tokens it has read (see the module's text)."""
    alive = {i: True for i in active}
    length = {i: len(histories[i]) for i in active}      # tokens of the sequence counting samples not yet read
    unread = []                                         # (pending tokens, their sequences), oldest first

    def read(pending, seqs):
        for i, tok in zip(seqs, pending.result()):
            if not alive[i]:
                continue                                # the step too many of a sequence that had stopped
            tok = int(tok)
            if tok in stop:
                result.finish_reasons[i] = "stop"
                alive[i] = False
                continue
            result.tokens[i].append(tok)
            histories[i].append(tok)
            result.generated_tokens += 1
            if on_token is not None:
                on_token(i, tok)
            if len(result.tokens[i]) >= params.max_tokens:
                result.finish_reasons[i] = "length"
                alive[i] = False
            elif len(histories[i]) >= max_seq_len:
                result.finish_reasons[i] = "context"
                alive[i] = False

    rows = list(active)
    ring_row = {i: r for r, i in enumerate(active)}     # where the sampler keeps a sequence's recent tokens
    extra = {"ring_rows": None} if params.uses_history else {}
    step_no = 0
    while rows:
        if params.uses_history:
            extra["ring_rows"] = [ring_row[i] for i in rows]
        picked = sampler.sample_device(logits, params, seed=seed, step=step_no, seq_ids=rows, stop_tokens=stop_list,
                                       **extra)
        unread.append((sampler.fetch(picked), rows))
        for i in rows:
            length[i] += 1
        while len(unread) > 1:                          # everything but the sample just queued
            read(*unread.pop(0))
        # who goes on: not known to have ended, and not ending by count or context with the sample just queued
        nxt = [(r, i) for r, i in enumerate(rows)
               if alive[i] and length[i] - len(histories[i]) + len(result.tokens[i]) < params.max_tokens
               and length[i] < max_seq_len]
        step_no += 1
        if not nxt:
            break
        logits = engine.step_fed([slots[i] for _, i in nxt], picked, [r for r, _ in nxt])
        result.decode_steps += 1
        rows = [i for _, i in nxt]
    while unread:
        read(*unread.pop(0))
