"""Token embedding and the output head.

``x[r,:] = E[token[r],:]`` (times ``scale`` if the architecture has one;
src/recipe/scratch.c:195-235), into the float32 residual.  With ``positions``
(a number of positions) the embedding also owns a table of learned position
vectors and adds the row of the token's position, unscaled.  The head computes
``logits = h W^T`` in float32 output (times ``scale`` if the architecture has
one); when tied, W is the embedding table (src/model.c:2562-2572).  With
``softcap`` (a positive number c) the logits are then bounded smoothly:
``logits <- c tanh(logits / c)``.

``token_table``: a second table by token id that other parts read columns of
(a per-layer token input); it has no forward of its own.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels as K
from ..ops.linear import linear
from .base import Part, WeightSpec, register_part


class TokenEmbedding(Part):
    category = "embedding"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.V = int(self._p("vocab_size"))
        self.d = int(self._p("hidden_size"))
        s = self._p("scale", None)
        self.scale = 1.0 if s is None else float(s)
        n_pos = self._p("positions", None)
        self.n_positions = None if n_pos is None else int(n_pos)
        self.pos_weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {"weight": WeightSpec((self.V, self.d), "embedding")}
        if self.n_positions is not None:
            s["positions.weight"] = WeightSpec((self.n_positions, self.d), "embedding")
        return s

    def bind(self, w):
        self.weight = w["weight"].contiguous()
        if self.n_positions is not None:
            self.pos_weight = w["positions.weight"].contiguous()

    def forward(self, token_ids: torch.Tensor, positions: torch.Tensor = None) -> torch.Tensor:
        x = torch.empty((token_ids.numel(), self.d), dtype=torch.float32, device=token_ids.device)
        if self.pos_weight is not None:
            return K.embed_rows(self.weight, token_ids, x, self.scale, self.pos_weight, positions)
        return K.embed_rows(self.weight, token_ids, x, self.scale)


class TokenTable(Part):
    """A table [vocab_size, width] by token id, kept for the parts that read stretches of its rows."""

    category = "embedding"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.V = int(self._p("vocab_size"))
        self.width = int(self._p("width"))
        self.weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.V, self.width), "embedding")}

    def bind(self, w):
        self.weight = w["weight"].contiguous()


class LMHead(Part):
    category = "head"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.V = int(self._p("vocab_size"))
        self.d = int(self._p("hidden_size"))
        self.tied = bool(self._p("tied", True))
        s = self._p("scale", None)
        self.scale = 1.0 if s is None else float(s)
        c = self._p("softcap", None)
        self.softcap = None if c is None else float(c)
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError(f"lm_head: softcap={self.softcap} must be positive")
        self.weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {} if self.tied else {"weight": WeightSpec((self.V, self.d), "matrix")}

    def bind(self, w):
        if not self.tied:
            self.weight = w["weight"].contiguous()

    def tie(self, embedding: TokenEmbedding) -> None:
        self.weight = embedding.weight

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = linear(h, self.weight, out_dtype=torch.float32)
        if self.scale != 1.0:
            K.scale_cast(logits, None, logits, self.scale)
        if self.softcap is not None:
            K.softcap(logits, self.softcap)
        return logits


register_part("embedding", "embedding", TokenEmbedding)
register_part("embedding", "token_table", TokenTable)
register_part("head", "lm_head", LMHead)
