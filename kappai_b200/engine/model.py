"""A model put together from parts, as a :class:`ModelSpec` describes it.

The reference builds, once at load, a per-layer list of ops from the model's
metadata (src/recipe/build.c:186-246, src/models/lfm.c:155-162) and runs
"pre ops, layers, post ops" every step (src/recipe/exec.c:704-758).  Here the
spec names parts; this class builds them through the part registry, binds
their weights, and runs embedding -> schedule -> selected rows -> final norm ->
head.  It holds no request state: caches come in with each call.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..config.schema import ModelSpec, PartSpec
from ..parts.base import BuildEnv, Part, WeightSpec, make_part


class Model:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        spec.validate()
        self.spec, self.env = spec, env
        self._table: Dict[str, Tuple[Part, str, WeightSpec]] = {}
        self._bound: Dict[int, Dict[str, torch.Tensor]] = {}

        self.embedding = self._make("embedding", spec.embedding)
        self.blocks = []
        for ls in spec.layers:
            mixer = self._make("mixer", ls.mixer)
            ffn = self._make("feed_forward", ls.ffn) if ls.ffn is not None else None
            n1 = self._make("norm", ls.mixer_norm) if ls.mixer_norm is not None else None
            n2 = self._make("norm", ls.ffn_norm) if ls.ffn_norm is not None else None
            block = make_part("block", PartSpec(ls.block), env)
            self.blocks.append(block.assemble(mixer, ffn, n1, n2))
        self.final_norm = self._make("norm", spec.final_norm) if spec.final_norm is not None else None
        self.head = self._make("head", spec.head)
        self.schedule = list(spec.schedule)
        parts = [self.embedding, self.final_norm, self.head]
        for b in self.blocks:
            parts += [b, b.mixer, b.ffn, b.mixer_norm, b.ffn_norm]
        # a decode step may be captured in a CUDA graph only if every part reads its tables from the device
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in parts if p is not None)
        # parts that build tables of their own for every step, one builder per key
        self.table_builders: Dict[object, Part] = {}
        for p in parts:
            for q in (p, getattr(p, "position", None)):
                key = getattr(q, "step_tables_key", None)
                if key is not None and key not in self.table_builders:
                    self.table_builders[key] = q

    def _make(self, category: str, ps: PartSpec) -> Part:
        part = make_part(category, ps, self.env)
        for local, ws in part.weight_specs().items():
            name = ps.prefix + ps.rename.get(local, local)
            if name in self._table:
                raise ValueError(f"two parts claim the tensor '{name}'")
            self._table[name] = (part, local, ws)
        return part

    # -- weights
    def weight_table(self) -> Dict[str, WeightSpec]:
        """Tensor name in the weight file -> what is expected there."""
        return {n: ws for n, (_, _, ws) in self._table.items()}

    def bind_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        """``tensors``: name -> device tensor, already checked against the table."""
        per_part: Dict[int, Tuple[Part, Dict[str, torch.Tensor]]] = {}
        for name, (part, local, _) in self._table.items():
            if name in tensors:
                per_part.setdefault(id(part), (part, {}))[1][local] = tensors[name]
        for part, w in per_part.values():
            part.bind(w)
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding)

    # -- caches
    def cache_specs(self) -> List[Optional[object]]:
        """Per schedule entry: what its mixer keeps (None if nothing or borrowed)."""
        out = []
        for e in self.schedule:
            out.append(None if e.cache_of is not None else self.blocks[e.layer].mixer.cache_spec())
        return out

    def cache_borrowing(self) -> List[Optional[int]]:
        return [e.cache_of for e in self.schedule]

    # -- the forward pass of one step
    def forward(self, ctx, cache_views, observer=None) -> Optional[torch.Tensor]:
        """Run the rows of ``ctx`` through every schedule entry; return float32
        logits [n_out, vocab] of the wanted rows (None if none are wanted).
        ``observer(where, x)``, if given, is shown the float32 residual behind
        the embedding (where = -1) and behind every schedule entry (its index)."""
        x = self.embedding.forward(ctx.token_ids)
        if observer is not None:
            observer(-1, x)
        for i, e in enumerate(self.schedule):
            self.blocks[e.layer].forward(x, ctx, cache_views[i])
            if observer is not None:
                observer(i, x)
        if ctx.n_out == 0:
            return None
        if self.final_norm is not None:
            h = self.final_norm.forward(x, rows=ctx.logit_rows)
        else:
            h = x.index_select(0, ctx.logit_rows.long()).to(self.env.dtype)
        return self.head.forward(h)
