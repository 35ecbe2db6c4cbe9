"""The cache of live sequences: paged keys/values per storage group, and fixed-size state.

Layers are put into groups by what they need.  A key/value group is defined by
(key/value heads, head size, window): all its layers share one page table per sequence and
one pool of pages, and each layer has its own key and value pages
``[n_pages, n_kv, 64, head_dim]``.  A group with a window keeps a ring of
``ceil(window / 64) + 1`` pages per sequence; a group without keeps every page.  Besides,
every layer that declares a fixed-size state gets ``[n_slots, *shape]``, zeroed when a
sequence starts (the reference keeps such state for its recurrent layers, one sequence only:
Inference/DeltaNetState.cs:78-87, :110-114).

The reference stores ``[n_kv, max_seq, head_dim]`` per layer for its single sequence
(Inference/KvCache.cs:35-71) and maps a position to a ring index for windows
(Inference/AttentionStrategy.cs:46-62).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import KvNeed, StateNeed
from .slots import CacheError, FreeList, SlotTable

PAGE = 64


def pages_for(tokens: int) -> int:
    return (tokens + PAGE - 1) // PAGE


@dataclass
class KvView:
    """What an attention-like mixer sees of its cache unit during a step."""

    k_pages: torch.Tensor
    v_pages: torch.Tensor
    page_table: torch.Tensor         # [n_slots, table_width] int32 (device)
    ring_pages: int
    window: int
    unit: int
    owner: bool = True               # False: this entry reads the unit, another entry writes it
    keep_step_kv: bool = False       # the unit is read by later entries: keep this step's packed k/v
    shared: Dict = field(default_factory=dict)   # owner leaves {"k_new", "v_new"} here for readers


@dataclass
class StateView:
    state: torch.Tensor              # [n_slots, *shape]
    unit: int
    owner: bool = True


class KvGroup:
    """Host bookkeeping and device storage of one key/value group."""

    def __init__(self, need: KvNeed, units: List[int], n_pages: int, n_slots: int, max_seq_pages: int,
                 dtype: torch.dtype, device: torch.device):
        self.need = need
        self.units = list(units)
        self.window = need.window
        full = max(1, max_seq_pages)
        self.ring_pages = min(full, pages_for(need.window) + 1) if need.window > 0 else full
        self.table_width = self.ring_pages
        # a sequence never holds more than its ring: a windowed group needs no more pages than that
        n_pages = min(n_pages, n_slots * self.ring_pages)
        self.n_pages = n_pages
        self.pool = FreeList(n_pages, "page")
        self.pages_of: Dict[int, List[int]] = {}
        # One row and one page beyond what sequences can get: the padding slot (row n_slots) owns page
        # n_pages for good.  Steps that are padded up to a graph's batch size park their extra rows there.
        self.page_table = torch.zeros((n_slots + 1, self.table_width), dtype=torch.int32, device=device)
        self.page_table[n_slots, :] = n_pages
        shape = (n_pages + 1, need.num_kv_heads, PAGE, need.head_dim)
        self.k = {u: torch.zeros(shape, dtype=dtype, device=device) for u in units}
        self.v = {u: torch.zeros(shape, dtype=dtype, device=device) for u in units}

    def pages_needed(self, length: int) -> int:
        return min(pages_for(length), self.ring_pages)

    def reserve(self, slot: int, new_len: int) -> List[Tuple[int, int]]:
        """Makes room for ``new_len`` tokens; returns new page-table entries (flat index, page)."""
        have = self.pages_of.setdefault(slot, [])
        want = self.pages_needed(new_len)
        if want <= len(have):
            return []
        fresh = self.pool.take(want - len(have))
        updates = []
        for p in fresh:
            updates.append((slot * self.table_width + len(have), p))
            have.append(p)
        return updates

    def can_shrink(self, old_len: int, new_len: int) -> bool:
        """True when the keys that a token at position ``new_len`` looks at are still in the pages.  A ring
        that has gone round has overwritten the oldest ones."""
        if self.window <= 0 or pages_for(old_len) <= self.ring_pages:
            return True
        oldest_needed = max(0, new_len - self.window + 1) // PAGE
        oldest_kept = (old_len - 1) // PAGE - self.ring_pages + 1
        return oldest_needed >= oldest_kept

    def shrink(self, slot: int, old_len: int, new_len: int) -> None:
        """Gives back the pages beyond ``new_len`` tokens.  A ring that has gone round keeps all of its pages:
        their order in the table is no longer their age."""
        if pages_for(old_len) > self.ring_pages:
            return
        have = self.pages_of.get(slot, [])
        keep = self.pages_needed(new_len)
        if len(have) > keep:
            self.pool.give(have[keep:])
            del have[keep:]

    def extra_pages(self, slot: int, new_len: int) -> int:
        return max(0, self.pages_needed(new_len) - len(self.pages_of.get(slot, [])))

    def release(self, slot: int) -> None:
        pages = self.pages_of.pop(slot, [])
        self.pool.give(pages)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in list(self.k.values()) + list(self.v.values()))


class SequenceCache:
    """All cache storage of one model instance.

    ``unit_needs`` maps a cache unit (one per schedule entry that keeps a cache) to what its
    mixer declared.  ``max_tokens`` is the number of tokens live sequences may hold together,
    each sequence rounded up to whole pages; ``max_seq_len`` bounds one sequence.
    """

    def __init__(self, unit_needs: Dict[int, object], *, max_tokens: int, max_seq_len: int,
                 n_slots: int, dtype: torch.dtype, device: torch.device):
        if max_tokens <= 0 or max_seq_len <= 0 or n_slots <= 0:
            raise ValueError("max_tokens, max_seq_len and n_slots must be positive")
        self.dtype = dtype
        self.device = device
        self.page = PAGE
        self.n_pages = pages_for(max_tokens)
        self.max_seq_len = min(max_seq_len, self.n_pages * PAGE)
        self.slots = SlotTable(n_slots)
        self.pad_slot = n_slots          # never handed out; see KvGroup
        self.kv_groups: List[KvGroup] = []
        self._group_of_unit: Dict[int, KvGroup] = {}
        self.state: Dict[int, torch.Tensor] = {}
        self._longest: Dict[int, int] = {}       # slots that were truncated: the most tokens they ever held
        by_need: Dict[KvNeed, List[int]] = {}
        for unit, need in unit_needs.items():
            if need is None:
                continue
            if isinstance(need, KvNeed):
                by_need.setdefault(need, []).append(unit)
            elif isinstance(need, StateNeed):
                self.state[unit] = torch.zeros((n_slots + 1, *need.shape), dtype=need.dtype, device=device)
            else:
                raise TypeError(f"cache unit {unit}: unknown need {need!r}")
        for need, units in by_need.items():
            g = KvGroup(need, units, self.n_pages, n_slots, pages_for(self.max_seq_len), dtype, device)
            self.kv_groups.append(g)
            for u in units:
                self._group_of_unit[u] = g

    # ---- sequences ---------------------------------------------------------------------
    def acquire(self) -> int:
        """A fresh slot: length 0, no pages, state zeroed."""
        slot = self.slots.acquire()
        self._longest.pop(slot, None)
        for t in self.state.values():
            t[slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        self.slots.check_live(slot)
        for g in self.kv_groups:
            g.release(slot)
        self.slots.release(slot)

    def length(self, slot: int) -> int:
        self.slots.check_live(slot)
        return self.slots.length[slot]

    def truncate(self, slot: int, new_len: int) -> None:
        """Forgets the tokens of ``slot`` from position ``new_len`` on (the reference's rollback,
        Inference/KvCache.cs:135); pages that hold none of the rest go back to the pool.  Refused, with
        nothing changed, where the past cannot be restored: fixed-size state, or a window whose older
        keys the ring has overwritten."""
        self.slots.check_live(slot)
        old = self.slots.length[slot]
        if not 0 <= new_len <= old:
            raise CacheError(f"slot {slot}: cannot truncate {old} tokens to {new_len}")
        if new_len == old:
            return
        if self.state:
            raise CacheError(f"slot {slot}: fixed-size state cannot be rolled back")
        # what a ring has overwritten follows from the longest the sequence has ever been
        written = max(old, self._longest.get(slot, 0))
        for g in self.kv_groups:
            if not g.can_shrink(written, new_len):
                raise CacheError(f"slot {slot}: the window of {g.window} keys before position {new_len} has been "
                                 f"overwritten (the sequence has held {written} tokens)")
        for g in self.kv_groups:
            g.shrink(slot, written, new_len)
        self._longest[slot] = written
        self.slots.length[slot] = new_len

    def check_room(self, growth: Sequence[Tuple[int, int]]) -> None:
        """``growth`` = (slot, tokens to add) for a whole step; raises before anything changes."""
        seen = set()
        for slot, add in growth:
            self.slots.check_live(slot)
            if slot in seen:
                raise CacheError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if add <= 0:
                raise CacheError(f"slot {slot}: a step must bring at least one token")
            new_len = self.slots.length[slot] + add
            if new_len > self.max_seq_len:
                raise CacheError(
                    f"slot {slot}: {new_len} tokens exceed the longest sequence the cache holds ({self.max_seq_len})")
        for g in self.kv_groups:
            extra = sum(g.extra_pages(s, self.slots.length[s] + add) for s, add in growth)
            if extra > g.pool.free_count:
                raise CacheError(
                    f"cache full: the step needs {extra} more pages of {PAGE} tokens, {g.pool.free_count} are free")

    def grow(self, growth: Sequence[Tuple[int, int]]) -> List[Tuple[KvGroup, List[Tuple[int, int]]]]:
        """Reserves pages for a step (after ``check_room``); lengths advance in ``commit``."""
        out = []
        for g in self.kv_groups:
            ups: List[Tuple[int, int]] = []
            for slot, add in growth:
                ups.extend(g.reserve(slot, self.slots.length[slot] + add))
            out.append((g, ups))
        return out

    def commit(self, growth: Sequence[Tuple[int, int]]) -> None:
        for slot, add in growth:
            self.slots.length[slot] += add

    # ---- views -------------------------------------------------------------------------
    def view(self, unit: int, *, owner: bool = True, keep_step_kv: bool = False, shared: Optional[Dict] = None):
        g = self._group_of_unit.get(unit)
        if g is not None:
            return KvView(g.k[unit], g.v[unit], g.page_table, g.ring_pages, g.window, unit, owner,
                          keep_step_kv, shared if shared is not None else {})
        if unit in self.state:
            return StateView(self.state[unit], unit, owner)
        return None

    def free_pages(self) -> int:
        """Pages that new sequences can still get: the scarcest group decides, among those whose pool can run
        out before the slots do (a group that owns a full ring for every slot never does)."""
        n_slots = self.slots.n_slots
        scarce = [g.pool.free_count for g in self.kv_groups if g.n_pages < n_slots * g.ring_pages]
        return min(scarce, default=self.n_pages)

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.kv_groups) + sum(t.numel() * t.element_size() for t in self.state.values())

    def audit(self) -> None:
        """Checks that every page is either free or held by exactly one live sequence."""
        live = self.slots.live()
        for g in self.kv_groups:
            held = []
            for slot, pages in g.pages_of.items():
                if slot not in live and pages:
                    raise CacheError(f"pages held by slot {slot}, which is not live")
                held.extend(pages)
            if len(held) != len(set(held)):
                raise CacheError("a page is held twice")
            if set(held) != set(g.pool.held):
                raise CacheError("the pool's held pages differ from the pages of live sequences")
            if len(held) + g.pool.free_count != g.pool.n:
                raise CacheError("pages were lost")
