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
            side = self._make("side", ls.side) if ls.side is not None else None
            p1 = self._make("norm", ls.mixer_post_norm) if ls.mixer_post_norm is not None else None
            p2 = self._make("norm", ls.ffn_post_norm) if ls.ffn_post_norm is not None else None
            block = make_part("block", PartSpec(ls.block, dict(ls.block_params)), env)
            # (an arrangement registered from outside may not know of side parts or of norms behind the sublayers: it is
            # asked only where there is one)
            if p1 is not None or p2 is not None:
                self.blocks.append(block.assemble(mixer, ffn, n1, n2, side, post_norms=(p1, p2)))
            else:
                self.blocks.append(block.assemble(mixer, ffn, n1, n2, side) if side is not None else block.assemble(mixer, ffn, n1, n2))
        self.final_norm = self._make("norm", spec.final_norm) if spec.final_norm is not None else None
        self.head = self._make("head", spec.head)
        self.schedule = list(spec.schedule)
        self.entry = self._make("entry", spec.entry) if spec.entry is not None else None
        self.token_table = self._make("embedding", spec.token_table) if spec.token_table is not None else None
        parts = [self.embedding, self.final_norm, self.head, self.entry, self.token_table]
        for b in self.blocks:
            parts += [b, b.mixer, b.ffn, b.mixer_norm, b.ffn_norm, getattr(b, "side", None),
                      getattr(b, "mixer_post_norm", None), getattr(b, "ffn_post_norm", None)]
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
        if self.token_table is not None:
            for b in self.blocks:
                if getattr(b, "side", None) is not None:
                    b.side.attach(self.token_table)

    # -- caches
    def cache_specs(self) -> List[Optional[object]]:
        """Per schedule entry: what its mixer keeps (None if nothing or borrowed)."""
        out = []
        for i, e in enumerate(self.schedule):
            own = self.blocks[e.layer].mixer.cache_spec()
            if e.cache_of is not None:
                lent = self.blocks[self.schedule[e.cache_of].layer].mixer.cache_spec()
                if own != lent:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which keeps {lent}, "
                                     f"but its mixer works on {own}")
            out.append(None if e.cache_of is not None else own)
        return out

    def cache_borrowing(self) -> List[Optional[int]]:
        return [e.cache_of for e in self.schedule]

    # -- the forward pass of one step
    def forward(self, ctx, cache_views, observer=None) -> Optional[torch.Tensor]:
        """Run the rows of ``ctx`` through every schedule entry; return float32
        logits [n_out, vocab] of the wanted rows (None if none are wanted).
        ``observer(where, x)``, if given, is shown the float32 residual behind
        the embedding (where = -1) and behind every schedule entry (its index)."""
        if getattr(self.embedding, "pos_weight", None) is not None:
            x = self.embedding.forward(ctx.token_ids, ctx.positions)
        else:
            x = self.embedding.forward(ctx.token_ids)
        if observer is not None:
            observer(-1, x)
        h0 = None
        if self.entry is not None:
            # the embedding output as the entry part's second operand, kept for every pass
            from ..ops import kernels as K
            h0 = torch.empty(x.shape, dtype=self.env.dtype, device=x.device)
            if self.env.dtype == torch.float32:
                K.scale_cast(x, None, h0, 1.0)
            else:
                K.cast(x, h0)
        for i, e in enumerate(self.schedule):
            if e.enter:
                x = self.entry.forward(x, h0)
            # (the block that runs next on this residual, for arrangements that prepare its input in their last kernel)
            nxt = self.schedule[i + 1] if i + 1 < len(self.schedule) else None
            ctx.next_block = self.blocks[nxt.layer] if nxt is not None and not nxt.enter else None
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
