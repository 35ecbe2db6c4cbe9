"""The step function: a batch of sequences, the tokens each brings now, logits where wanted.

One call runs exactly the tokens it is given, as one packed batch, against the cache that
earlier calls left; it never re-runs old tokens and never pads.  A step in which every
sequence brings one token takes the decode kernels (and, once a batch size has been seen, a
CUDA graph of the whole step); any other step takes the prompt kernels.  The reference has
four entry points for one sequence (Inference/IForwardPass.cs:8-50) and replays its token step
as a CUDA graph (Daisi.Llogos.Cuda/CudaBackend.cs:99-141); here there is one entry point for
a batch.

All checks happen on the host before anything is launched: unknown or repeated slots, empty
token lists, token ids outside the vocabulary, wanted positions outside the step, no room in
the cache.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.slots import CacheError
from ..cache.store import PAGE, SequenceCache
from .context import StepContext, Workspace
from .model import DecoderModel


class StepError(ValueError):
    """A step was asked for that cannot run; nothing was launched and the cache is unchanged."""


class _Staging:
    """Pinned host buffers that alternate, so that filling one never races a copy still in flight."""

    def __init__(self, device: torch.device, depth: int = 3):
        self.device = device
        self.cuda = device.type == "cuda"
        self.bufs: List[Optional[torch.Tensor]] = [None] * depth
        self.events: List[Optional[torch.cuda.Event]] = [None] * depth
        self.i = 0

    def upload(self, host: np.ndarray, dst: torch.Tensor) -> None:
        n = host.size
        self.i = (self.i + 1) % len(self.bufs)
        buf = self.bufs[self.i]
        if self.events[self.i] is not None:
            self.events[self.i].synchronize()
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 256), dtype=torch.int32, pin_memory=self.cuda)
            self.bufs[self.i] = buf
        buf[:n].numpy()[:] = host
        dst[:n].copy_(buf[:n], non_blocking=True)
        if self.cuda:
            ev = self.events[self.i] or torch.cuda.Event()
            ev.record()
            self.events[self.i] = ev


_BUCKETS = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512, 768, 1024)


def length_bucket(n: int) -> int:
    """Upper bound on the lengths of a decode step that its recorded launches are planned for: the next power
    of two from 1,024 on.  A batch whose sequences grow past it moves on to the next bound's graph."""
    x = 1024
    while x < n:
        x *= 2
    return x


def decode_bucket(b: int) -> int:
    """Batch size a decode step of ``b`` sequences runs at: the next of a short list of sizes (at most a
    third more rows), so that a batch that shrinks as sequences end reuses a few CUDA graphs instead of
    recording one per size.  The extra rows are parked on the cache's padding slot."""
    for x in _BUCKETS:
        if x >= b:
            return x
    return -(-b // 256) * 256


class _DecodeState:
    """Static buffers (and later the CUDA graph) of decode steps of one batch size."""

    def __init__(self, b: int, device: torch.device):
        self.b = b
        self.meta = torch.zeros(6 * b + 1, dtype=torch.int32, device=device)
        self.workspace = Workspace(device)
        self.rows = torch.arange(b, dtype=torch.int32, device=device)
        self.graph = None
        self.kernels = 0
        self.logits: Optional[torch.Tensor] = None
        self.eager_runs = 0


class Engine:
    """A model, its cache and the step function.

    ``max_tokens``: tokens that live sequences may hold together, each rounded up to whole pages
    of 64.  ``max_seq_len``: longest single sequence (default: the smaller of the model's
    position limit and ``max_tokens``).  ``n_slots``: most sequences alive at once.
    """

    def __init__(self, model: DecoderModel, *, max_tokens: int, max_seq_len: Optional[int] = None,
                 n_slots: Optional[int] = None, use_graphs: bool = True):
        self.model = model
        self.device = model.device
        self.dtype = model.dtype
        self.ops = model.env.ops
        n_pages = (max_tokens + PAGE - 1) // PAGE
        if max_seq_len is None:
            max_seq_len = n_pages * PAGE
            if model.spec.max_positions is not None:
                max_seq_len = min(model.spec.max_positions, max_seq_len)
        elif model.spec.max_positions is not None and max_seq_len > model.spec.max_positions:
            raise ValueError(f"max_seq_len {max_seq_len} exceeds the model's position limit "
                             f"(max_position_embeddings = {model.spec.max_positions})")
        if n_slots is None:
            n_slots = max(1, min(n_pages, 1024))
        self.cache = SequenceCache(model.cache_needs(), max_tokens=max_tokens, max_seq_len=max_seq_len,
                                   n_slots=n_slots, dtype=self.dtype, device=self.device)
        model.prepare(self.cache.max_seq_len)
        # the stock blocks' launch chain in native code, where the model is made of nothing else
        self._runner = None
        if self.device.type == "cuda":
            from .runner import BlockRunner
            self._runner = BlockRunner.build(model, self.cache)
        self.vocab = model.spec.vocab_size
        self.use_graphs = use_graphs and self.device.type == "cuda"
        self._staging = _Staging(self.device)
        self._meta = torch.zeros(1024, dtype=torch.int32, device=self.device)
        self._workspace = Workspace(self.device)
        self._decode: Dict[Tuple[int, int], _DecodeState] = {}     # (batch size, length bound) -> buffers and graph
        self.graph_kernels = 0      # kernels inside CUDA graphs replayed by step(), for reporting

    # ---- sequences -----------------------------------------------------------------------
    def open(self) -> int:
        """Starts a sequence: returns its slot (length 0)."""
        return self.cache.acquire()

    def close(self, slot: int) -> None:
        """Ends a sequence: its slot and pages go back to the free lists."""
        self.cache.release(slot)

    def truncate(self, slot: int, length: int) -> None:
        """Forgets a sequence's tokens from position ``length`` on; the next step continues there."""
        try:
            self.cache.truncate(slot, length)
        except CacheError as e:
            raise StepError(str(e)) from None

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def assume(self, slot: int, n_tokens: int) -> None:
        """Declares ``n_tokens`` more tokens of ``slot`` as present without running them: pages are
        reserved and the length advances, the keys and values are whatever the pages hold.  For
        measurements of a step at a given context length; results after it mean nothing."""
        growth = [(int(slot), int(n_tokens))]
        try:
            self.cache.check_room(growth)
        except CacheError as e:
            raise StepError(str(e)) from None
        host: List[np.ndarray] = []
        plan = self._apply_updates(self.cache.grow(growth), host)
        if plan:
            block = np.concatenate(host)
            meta = self._ensure_meta(block.size)
            self._staging.upload(block, meta)
            for g, off, k in plan:
                self.ops.scatter_i32(g.page_table, meta[off:off + k], meta[off + k:off + 2 * k])
        self.cache.commit(growth)

    # ---- the step ------------------------------------------------------------------------
    def step(self, entries: Sequence[Tuple[int, Sequence[int]]],
             want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """Runs ``tokens`` of every ``(slot, tokens)`` entry; returns float32 logits ``[n_wanted, vocab]``.

        ``want[i]`` lists positions among entry i's tokens (0-based) whose logits are returned, in
        the order of the entries and of ``want``; ``None`` means the last token of every entry.
        The returned tensor is valid until the next call of ``step``.
        """
        if len(entries) == 0:
            raise StepError("a step needs at least one sequence")
        slots = [int(s) for s, _ in entries]
        toks = [np.asarray(t, dtype=np.int64).reshape(-1) for _, t in entries]
        counts = [int(t.size) for t in toks]
        if want is None:
            want = [[c - 1] for c in counts]
        if len(want) != len(entries):
            raise StepError("want must have one list per entry")
        for i, (t, c) in enumerate(zip(toks, counts)):
            if c == 0:
                raise StepError(f"entry {i} (slot {slots[i]}) brings no tokens")
            if t.min() < 0 or t.max() >= self.vocab:
                bad = int(t[(t < 0) | (t >= self.vocab)][0])
                raise StepError(f"entry {i} (slot {slots[i]}): token id {bad} is outside the vocabulary [0, {self.vocab})")
            for w in want[i]:
                if not 0 <= int(w) < c:
                    raise StepError(f"entry {i} (slot {slots[i]}): wanted position {w} is outside its {c} tokens")
        return self._run(slots, toks, counts, want, None)

    def step_fed(self, slots: Sequence[int], source: torch.Tensor, rows: Sequence[int],
                 want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """A step of one token per sequence whose ids are still on the device: sequence ``slots[i]`` gets
        ``source[rows[i]]`` (``source``: int32, what a sampler wrote).  The host never sees the ids, so the
        step can be queued before the sampler's result has been read; an id outside the vocabulary is read
        as token 0.  Everything else is as in ``step``."""
        if len(slots) == 0:
            raise StepError("a step needs at least one sequence")
        if len(rows) != len(slots):
            raise StepError("step_fed needs one source row per slot")
        if source.dtype != torch.int32 or source.device != self.device:
            raise StepError("step_fed: the token source must be an int32 tensor on the engine's device")
        for r in rows:
            if not 0 <= int(r) < source.numel():
                raise StepError(f"step_fed: source row {r} is outside the source's {source.numel()} entries")
        slots = [int(s) for s in slots]
        if want is None:
            want = [[0]] * len(slots)
        if len(want) != len(slots):
            raise StepError("want must have one list per entry")
        for i, w_ in enumerate(want):
            for w in w_:
                if int(w) != 0:
                    raise StepError(f"entry {i} (slot {slots[i]}): wanted position {w} is outside its 1 tokens")
        toks = [np.zeros(1, dtype=np.int64) for _ in slots]
        return self._run(slots, toks, [1] * len(slots), want, (source, [int(r) for r in rows]))

    def _run(self, slots, toks, counts, want, fed) -> torch.Tensor:
        growth = list(zip(slots, counts))
        try:
            self.cache.check_room(growth)
        except CacheError as e:
            raise StepError(str(e)) from None

        len_before = [self.cache.length(s) for s in slots]
        longest = max(lb + c for lb, c in zip(len_before, counts))
        limit = self.model.position_limit()
        if limit is not None and longest > limit:
            raise StepError(f"a sequence would reach {longest} tokens, the position tables hold {limit}")
        updates = self.cache.grow(growth)
        b = len(slots)
        decode = all(c == 1 for c in counts)
        if decode:
            logits = self._decode_step(b, slots, toks, len_before, updates, want, fed)
        else:
            logits = self._prompt_step(b, slots, toks, counts, len_before, updates, want)
        self.cache.commit(growth)
        return logits

    # ---- page-table updates ----------------------------------------------------------------
    def _apply_updates(self, updates, extra_host: List[np.ndarray]) -> List[Tuple[object, int, int]]:
        """Appends (index, value) lists to the host block; returns (group, offset, n) per group."""
        plan = []
        off = sum(a.size for a in extra_host)
        for g, ups in updates:
            if not ups:
                continue
            idx = np.fromiter((u[0] for u in ups), dtype=np.int32, count=len(ups))
            val = np.fromiter((u[1] for u in ups), dtype=np.int32, count=len(ups))
            extra_host.append(idx)
            extra_host.append(val)
            plan.append((g, off, len(ups)))
            off += 2 * len(ups)
        return plan

    def _ensure_meta(self, n: int) -> torch.Tensor:
        if self._meta.numel() < n:
            self._meta = torch.zeros(max(n, 2 * self._meta.numel()), dtype=torch.int32, device=self.device)
        return self._meta

    # ---- prompt step -----------------------------------------------------------------------
    def _prompt_step(self, b, slots, toks, counts, len_before, updates, want) -> torch.Tensor:
        n = sum(counts)
        cu = np.zeros(b + 1, dtype=np.int32)
        np.cumsum(counts, out=cu[1:])
        token_ids = np.concatenate(toks).astype(np.int32)
        positions = np.concatenate([np.arange(lb, lb + c, dtype=np.int32) for lb, c in zip(len_before, counts)])
        seq_of = np.repeat(np.arange(b, dtype=np.int32), counts)
        rows = np.array([cu[i] + int(w) for i in range(b) for w in want[i]], dtype=np.int32)
        host = [token_ids, positions, seq_of, np.asarray(slots, dtype=np.int32), cu,
                np.asarray(len_before, dtype=np.int32), rows]
        plan = self._apply_updates(updates, host)
        block = np.concatenate(host)
        meta = self._ensure_meta(block.size)
        self._staging.upload(block, meta)
        o = 0

        def take(k):
            nonlocal o
            v = meta[o:o + k]
            o += k
            return v

        ctx = StepContext(
            n_tokens=n, n_seqs=b, decode=False, counts=counts, max_count=max(counts),
            token_ids=take(n), positions=take(n), seq_of_token=take(n), slots=take(b), cu_tokens=take(b + 1),
            len_before=take(b), dtype=self.dtype, device=self.device,
            ops=self.ops, workspace=self._workspace,
            max_len_after=max(lb + c for lb, c in zip(len_before, counts)),
            len_before_host=list(len_before), upload=self._staging.upload)
        rows_dev = take(rows.size)
        for g, off, k in plan:
            self.ops.scatter_i32(g.page_table, meta[off:off + k], meta[off + k:off + 2 * k])
        return self.model.forward(ctx, self.cache, rows_dev, self._runner)

    # ---- decode step -----------------------------------------------------------------------
    def _decode_step(self, n_real, slots, toks, len_before, updates, want, fed=None) -> torch.Tensor:
        b = decode_bucket(n_real) if self.use_graphs else n_real
        # the launches are planned for lengths up to a bound that the batch's own longest sequence decides
        # (not the cache's limit), so that short sequences in a cache sized for long ones are not over-split
        bound = min(self.cache.max_seq_len, length_bucket(max(len_before) + 1))
        st = self._decode.get((b, bound))
        if st is None:
            st = self._decode[(b, bound)] = _DecodeState(b, self.device)
        pad = b - n_real
        token_ids = np.concatenate(toks + [np.zeros(pad, dtype=np.int64)]).astype(np.int32)
        ar = np.arange(b, dtype=np.int32)
        # padding rows: token 0 at position 0 of the padding slot (its one page is never anyone else's)
        lb = np.asarray(list(len_before) + [0] * pad, dtype=np.int32)
        all_slots = np.asarray(list(slots) + [self.cache.pad_slot] * pad, dtype=np.int32)
        # layout: token_ids | positions | seq_of_token | slots | cu_tokens (b + 1) | len_before
        host = [token_ids, lb, ar, all_slots, np.arange(b + 1, dtype=np.int32), lb]
        fixed = 6 * b + 1
        if fed is not None:
            host.append(np.asarray(fed[1], dtype=np.int32))      # source rows, right after the fixed part
        plan = self._apply_updates(updates, host)
        block = np.concatenate(host)
        if plan or fed is not None:
            # page-table updates and source rows travel through the general buffer, the fixed part through the static one
            meta2 = self._ensure_meta(block.size)
            self._staging.upload(block, meta2)
            for g, off, k in plan:
                self.ops.scatter_i32(g.page_table, meta2[off:off + k], meta2[off + k:off + 2 * k])
            st.meta.copy_(meta2[:fixed], non_blocking=True)
            if fed is not None:
                self.ops.gather_i32(st.meta[:n_real], fed[0], meta2[fixed:fixed + n_real])
        else:
            self._staging.upload(block, st.meta)
        m = st.meta
        if st.graph is not None:
            st.graph.replay()
            self.graph_kernels += st.kernels
            logits = st.logits
        else:
            ctx = StepContext(
                n_tokens=b, n_seqs=b, decode=True, counts=[1] * b, max_count=1,
                token_ids=m[0:b], positions=m[b:2 * b], seq_of_token=m[2 * b:3 * b], slots=m[3 * b:4 * b],
                cu_tokens=m[4 * b:5 * b + 1], len_before=m[5 * b + 1:6 * b + 1],
                dtype=self.dtype, device=self.device, ops=self.ops, workspace=st.workspace,
                max_len_after=bound)
            if self.use_graphs and st.eager_runs >= 1:
                # the buffers exist since the eager run; record the same launches and replay them
                graph = torch.cuda.CUDAGraph()
                st.workspace.frozen = True
                before = getattr(self.ops, "launches", lambda: 0)()
                with torch.cuda.graph(graph):
                    st.logits = self.model.forward(ctx, self.cache, st.rows, self._runner)
                st.kernels = getattr(self.ops, "launches", lambda: 0)() - before
                st.graph = graph
                graph.replay()
                self.graph_kernels += st.kernels
                logits = st.logits
            else:
                logits = self.model.forward(ctx, self.cache, st.rows, self._runner)
                st.eager_runs += 1
        flat_want = [(i, int(w)) for i in range(n_real) for w in want[i]]
        if len(flat_want) == n_real and all(i == j for j, (i, _) in enumerate(flat_want)):
            return logits[:n_real]
        if not flat_want:
            return logits[:0]
        idx = torch.tensor([i for i, _ in flat_want], dtype=torch.long, device=self.device)
        return logits.index_select(0, idx)
