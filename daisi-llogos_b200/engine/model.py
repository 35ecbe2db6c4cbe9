"""A model put together from a ``ModelSpec``: parts built through the registries, the tensors
they declare, and the forward pass over the run order.

The forward pass is the reference's (Inference/ForwardPass.cs:174-184, :199-267): embedding,
the layers in order, final norm and output head on the rows whose logits are wanted.  Which
parts a layer has and in which order layers run is data of the spec.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..parts.base import Branch, BuildEnv, Part, TensorDecl, part_class, part_families
from ..parts.spec import ModelSpec

# importing the modules registers the stock parts
from ..parts import attention as _attention  # noqa: F401
from ..parts.block import normed_for
from ..parts import embedding as _embedding  # noqa: F401
from ..parts import feedforward as _feedforward  # noqa: F401
from ..parts import norm as _norm  # noqa: F401
from ..parts import position as _position  # noqa: F401


class DecoderModel:
    def __init__(self, spec: ModelSpec, *, dtype: torch.dtype, device: torch.device, ops):
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.encodings = {}
        self.env = BuildEnv(dtype=dtype, device=device, ops=ops, encodings=self.encodings)
        for name, ps in spec.encodings.items():
            self.encodings[name] = part_class("position", ps.kind)(ps.params, ps.prefix, self.env)
        self.embedding = part_class("embedding", spec.embedding.kind)(spec.embedding.params, spec.embedding.prefix, self.env)
        self.blocks = []
        for l_i, ls in enumerate(spec.layers):
            block_cls = part_class("block", ls.block)
            roles = dict(getattr(block_cls, "ROLES", {}))
            parts: Dict[str, Part] = {}
            for role, ps in ls.parts.items():
                family = ps.family or roles.get(role)
                if family is None:
                    raise ValueError(f"layers[{l_i}]: block '{ls.block}' declares no role '{role}' "
                                     f"({', '.join(roles) or 'none'}) and the part names no family")
                if family not in part_families():
                    raise ValueError(f"layers[{l_i}].{role}: '{family}' is not a part family ({', '.join(part_families())})")
                parts[role] = part_class(family, ps.kind)(ps.params, ps.prefix, self.env)
            self.blocks.append(block_cls({}, "", self.env, parts))
        # an entry that reads another entry's cache: its mixer must be able to read what the owner keeps
        self._last_reader: Dict[int, int] = {}
        for e_i, e in enumerate(spec.schedule):
            if e.cache_of is None:
                continue
            self._last_reader[e.cache_of] = e_i
            need = self.blocks[spec.schedule[e.cache_of].layer].cache_need()
            if need is None:
                raise ValueError(f"schedule[{e_i}].cache_of = {e.cache_of}: that entry keeps no cache")
            for part in self.blocks[e.layer].parts.values():
                check = getattr(part, "check_borrowed", None)
                if check is not None:
                    try:
                        check(need)
                    except ValueError as err:
                        raise ValueError(f"schedule[{e_i}].cache_of = {e.cache_of}: {err}") from None
        self.final_norm = part_class("norm", spec.final_norm.kind)(spec.final_norm.params, spec.final_norm.prefix, self.env)
        self.head = part_class("head", spec.head.kind)(spec.head.params, spec.head.prefix, self.env)
        self._bound = False

    # ---- tensors -------------------------------------------------------------------------
    def _all_parts(self) -> List[Part]:
        out: List[Part] = list(self.encodings.values()) + [self.embedding]
        for b in self.blocks:
            out.extend(b.parts.values())
        out += [self.final_norm, self.head]
        return out

    def tensor_decls(self) -> Dict[str, TensorDecl]:
        """Full tensor name -> declaration, for the loader and the random initialiser."""
        decls: Dict[str, TensorDecl] = {}
        for p in self._all_parts():
            for rel, d in p.tensors().items():
                name = p.prefix + rel
                if name in decls:
                    raise ValueError(f"tensor '{name}' is declared by two parts")
                decls[name] = d
        return decls

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self._all_parts():
            mine = {rel: tensors[p.prefix + rel] for rel in p.tensors() if (p.prefix + rel) in tensors}
            tied = getattr(p, "tied_to", None)
            if tied:
                mine["weight"] = tensors[tied]
            p.bind(mine)
        self._bound = True

    def prepare(self, max_positions: int) -> None:
        for e in self.encodings.values():
            e.prepare(max_positions)

    def position_limit(self) -> Optional[int]:
        """The most positions every position encoding has tables for (``None``: no limit)."""
        limits = [e.limit() for e in self.encodings.values()]
        limits = [x for x in limits if x is not None]
        return min(limits) if limits else None

    # ---- cache units ---------------------------------------------------------------------
    def cache_needs(self) -> Dict[int, object]:
        """Schedule entry -> what its mixer keeps (entries that borrow a cache keep nothing)."""
        needs = {}
        for e_i, e in enumerate(self.spec.schedule):
            if e.cache_of is not None:
                continue
            need = self.blocks[e.layer].cache_need()
            if need is not None:
                needs[e_i] = need
        return needs

    # ---- forward -------------------------------------------------------------------------
    def forward(self, ctx, cache, rows: Optional[torch.Tensor], runner=None) -> torch.Tensor:
        """Runs the step's tokens; returns float32 logits of ``rows`` (token indices), [len(rows), vocab].
        ``runner``: an ``engine.runner.BlockRunner`` built for this model and cache; it then runs the layers."""
        residual = self.embedding.forward(ctx)
        for enc in self.encodings.values():
            enc.on_embeddings(residual, ctx)
        pending: Optional[Branch] = None
        if runner is not None:
            pending = runner.run(ctx, residual)
        borrowed = {e.cache_of for e in self.spec.schedule if e.cache_of is not None}
        shared: Dict[int, Dict] = {}
        for e_i, e in enumerate(self.spec.schedule if runner is None else ()):
            unit = e.cache_of if e.cache_of is not None else e_i
            view = cache.view(unit, owner=e.cache_of is None, keep_step_kv=e_i in borrowed,
                              shared=shared.setdefault(unit, {}))
            pending = self.blocks[e.layer].forward(residual, pending, ctx, view)
            # what an owner put off until its cache's last reader has run (a ring's writes would
            # overwrite keys that a reader of the same step still needs)
            for unit in [u for u, last in self._last_reader.items() if last == e_i]:
                for finish in shared.get(unit, {}).pop("after_last_reader", []):
                    finish()
        if rows is None or rows.numel() == 0:
            # nothing wanted: the residual need not be finished, the cache already is
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        x, kw = normed_for(self.final_norm, self.head, residual, pending, ctx, rows)
        return self.head.forward(x, ctx, **kw)
