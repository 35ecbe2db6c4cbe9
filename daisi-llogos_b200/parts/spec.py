"""Plain-data description of a model: which parts, with which sizes, in which order.

An architecture's builder turns its typed configuration into a ``ModelSpec``.
The engine builds parts from the spec through the part registries and never
looks at the architecture's name again.  The reference chooses per layer between
mixers with ``IsStandardAttention(layer)`` (Model/ModelConfig.cs:92-94) and
lets late layers read an earlier layer's keys and values
(Model/ModelConfig.cs:121-122); here both are data: every layer names its own
parts, and the run order is a list of entries.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered kind, its parameters, the prefix of its tensor names.  ``family`` (norm,
    mixer, ffn, position, ...) is needed only where the part fills a block role whose family the block's
    class does not declare."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""
    family: Optional[str] = None


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement and the parts it arranges."""

    block: str                     # registered block kind, e.g. "prenorm"
    parts: Dict[str, PartSpec]     # role in the block -> part (the block's class names its roles)


@dataclass(frozen=True)
class ScheduleEntry:
    """One application of a layer.

    ``layer`` indexes ``ModelSpec.layers``; a layer may appear in several entries
    (its weights are then shared, each entry keeps its own cache).  ``cache_of``
    names an EARLIER entry whose cache this entry reads instead of keeping one.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: Optional[int]      # None: no limit besides the cache's size
    embedding: PartSpec
    encodings: Dict[str, PartSpec]          # position encodings by name; mixers refer to them by name
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: Tuple[int, ...] = ()
    # Regular expressions (matched against whole names) of tensors that a checkpoint of this architecture
    # may hold although the model has no use for them; the loader skips them with a warning.
    ignorable_tensors: Tuple[str, ...] = ()

    def validate(self) -> None:
        for e_i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule[{e_i}] names layer {e.layer}, but there are {len(self.layers)}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < e_i:
                    raise ValueError(
                        f"schedule[{e_i}].cache_of = {e.cache_of} must name an earlier entry")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(
                        f"schedule[{e_i}].cache_of = {e.cache_of} names an entry that itself borrows a cache")
        for l_i, layer in enumerate(self.layers):
            for role, part in layer.parts.items():
                enc = part.params.get("position")
                if enc is not None and enc not in self.encodings:
                    raise ValueError(f"layers[{l_i}].{role} names position encoding {enc!r}, which is not defined")
