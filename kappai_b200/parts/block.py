"""Arrangements of a mixer, a feed-forward and their norms around the residual.

``prenorm_residual``: ``x += mixer(norm1(x)); x += ffn(norm2(x))``
(src/models/lfm.c:7-53 followed by src/recipe/builders.c:378-388).  The
residual ``x`` is float32 and is updated in place.  A ``side`` part, if the
layer has one, then changes the residual once more (``side.forward(x, ctx)``).

``postnorm_residual``: ``x <- norm1(alpha x + mixer(x)); x <- norm2(alpha x + ffn(x))``:
the sublayers read ``x`` itself (in the compute type), the norm comes after the
sum, and ``alpha`` (parameter, default 1) weighs the residual branch.  A layer
without a feed-forward has the first half only.  The sum and the norm are
float32; one kernel norms a sum and writes what the next sublayer needs (its
input in the compute type and ``alpha`` times the new residual to add into), so
a layer costs two row-wise launches, as a pre-norm layer does.

``parallel_residual``: ``h = norm1(x); x += mixer(h); x += ffn(h)``: one norm a
layer, and both sublayers read its output.  Each sublayer adds its float32
output into the float32 residual, so the layer's sum is
``(x + mixer(h)) + ffn(h)``.

``sandwich_residual``: ``x += norm1b(mixer(norm1(x))); x += norm2b(ffn(norm2(x)))``:
a norm in front of every sublayer and one behind it, before its output joins the
residual.  The sublayer adds its float32 output into a zeroed float32 branch;
one kernel norms the branch, adds it to the residual, clears the branch for
its next use and, where another norm follows at once (the feed-forward's, or
the first norm of the layer that runs next), norms the new residual for it in
the same pass.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import Part, register_part


class PreNormResidualBlock(Part):
    category = "block"
    graph_safe = True

    def assemble(self, mixer, ffn, mixer_norm, ffn_norm, side=None):
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm, self.side = mixer, ffn, mixer_norm, ffn_norm, side
        return self

    def forward(self, x, ctx, cache):
        self.mixer.forward(self.mixer_norm.forward(x) if self.mixer_norm is not None else x, x, ctx, cache)
        if self.ffn is not None:
            self.ffn.forward(self.ffn_norm.forward(x) if self.ffn_norm is not None else x, x, ctx)
        if self.side is not None:
            self.side.forward(x, ctx)


class PostNormResidualBlock(Part):
    category = "block"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.alpha = float(self._p("alpha", 1.0))

    def assemble(self, mixer, ffn, mixer_norm, ffn_norm, side=None):
        if mixer_norm is None or (ffn is not None and ffn_norm is None):
            raise ValueError("postnorm_residual: every sublayer needs the norm that follows its sum")
        if side is not None:
            raise ValueError("postnorm_residual: no side part in this arrangement")
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm, self.side = mixer, ffn, mixer_norm, ffn_norm, None
        return self

    def _enter(self, x, ctx):
        """The sublayer input (x in the compute type) and alpha * x: left by the block before this one for
        this very residual, or made here."""
        carry = getattr(ctx, "postnorm_carry", None)
        ctx.postnorm_carry = None
        if carry is not None and carry[0] is x and carry[1] == self.alpha:
            return carry[2], carry[3]
        acc = torch.empty_like(x)
        if self.env.dtype == torch.float32:
            K.scale_cast(x, None, acc, self.alpha)
            return x, acc
        h = torch.empty(x.shape, dtype=self.env.dtype, device=x.device)
        K.scale_cast(x, h, acc, self.alpha)
        return h, acc

    def forward(self, x, ctx, cache):
        f32 = self.env.dtype == torch.float32
        h, acc = self._enter(x, ctx)
        self.mixer.forward(h, acc, ctx, cache)
        # what the sublayer after this norm reads and adds into; in 32-bit its input is the residual itself
        h2 = x if f32 else (h if h is not x else torch.empty(x.shape, dtype=self.env.dtype, device=x.device))
        if self.ffn is not None:
            n1 = self.mixer_norm
            K.postnorm_rows(acc, n1.weight, n1.eps, x_out=x if f32 else None, h_out=None if f32 else h2,
                            scaled_out=acc, alpha=self.alpha)
            self.ffn.forward(h2, acc, ctx)
            last = self.ffn_norm
        else:
            last = self.mixer_norm
        # the new residual, and with it the entry of a post-norm block that may follow
        K.postnorm_rows(acc, last.weight, last.eps, x_out=x, h_out=None if f32 else h2, scaled_out=acc, alpha=self.alpha)
        ctx.postnorm_carry = (x, self.alpha, x if f32 else h2, acc)


class ParallelResidualBlock(Part):
    category = "block"
    graph_safe = True

    def assemble(self, mixer, ffn, mixer_norm, ffn_norm, side=None):
        if ffn_norm is not None:
            raise ValueError("parallel_residual: the sublayers share one norm")
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm, self.side = mixer, ffn, mixer_norm, None, side
        return self

    def forward(self, x, ctx, cache):
        if self.mixer_norm is not None:
            h = self.mixer_norm.forward(x)
        elif self.env.dtype == torch.float32:
            h = x.clone()                      # the sublayers add into x while the second still has to read its input
        else:
            h = K.cast(x, torch.empty(x.shape, dtype=self.env.dtype, device=x.device))
        self.mixer.forward(h, x, ctx, cache)
        if self.ffn is not None:
            self.ffn.forward(h, x, ctx)
        if self.side is not None:
            self.side.forward(x, ctx)


class SandwichResidualBlock(Part):
    category = "block"
    graph_safe = True

    def assemble(self, mixer, ffn, mixer_norm, ffn_norm, side=None, post_norms=(None, None)):
        p1, p2 = post_norms
        if mixer_norm is None or p1 is None or (ffn is not None and (ffn_norm is None or p2 is None)):
            raise ValueError("sandwich_residual: every sublayer needs a norm in front and a norm behind")
        if any(type(n).__name__ != "RMSNorm" for n in (mixer_norm, p1, ffn_norm, p2) if n is not None):
            raise ValueError("sandwich_residual: the norms are RMS norms")
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm, self.side = mixer, ffn, mixer_norm, ffn_norm, side
        self.mixer_post_norm, self.ffn_post_norm = p1, p2
        return self

    @staticmethod
    def _branch(x, ctx):
        """The float32 rows a sublayer adds its output into: one zeroed buffer a step, shared by the layers (the
        kernel that reads a branch clears it)."""
        y = getattr(ctx, "sandwich_branch", None)
        if y is None or y.shape != x.shape:
            y = torch.zeros_like(x)
            ctx.sandwich_branch = y
        return y

    def forward(self, x, ctx, cache):
        y = self._branch(x, ctx)
        # the input of this layer's mixer: left by the layer before for this very residual, or made here
        carry = getattr(ctx, "sandwich_carry", None)
        ctx.sandwich_carry = None
        n1 = self.mixer_norm
        if carry is not None and carry[0] is x and carry[1] is n1:
            h = carry[2]
        else:
            h = n1.forward(x)
        self.mixer.forward(h, y, ctx, cache)
        if self.ffn is not None:
            n2, pn = self.ffn_norm, self.mixer_post_norm
            h2 = torch.empty(x.shape, dtype=self.env.dtype, device=x.device)
            K.rmsnorm_add_norm_rows(y, pn.weight, pn.eps, x, n2.weight, n2.eps, h2)
            self.ffn.forward(h2, y, ctx)
            last = self.ffn_post_norm
        else:
            last = self.mixer_post_norm
        nxt = getattr(ctx, "next_block", None)
        if isinstance(nxt, SandwichResidualBlock) and self.side is None:
            nn = nxt.mixer_norm
            h_next = torch.empty(x.shape, dtype=self.env.dtype, device=x.device)
            K.rmsnorm_add_norm_rows(y, last.weight, last.eps, x, nn.weight, nn.eps, h_next)
            ctx.sandwich_carry = (x, nn, h_next)
        else:
            K.rmsnorm_add_norm_rows(y, last.weight, last.eps, x)
        if self.side is not None:
            self.side.forward(x, ctx)


register_part("block", "sandwich_residual", SandwichResidualBlock)
register_part("block", "prenorm_residual", PreNormResidualBlock)
register_part("block", "parallel_residual", ParallelResidualBlock)
register_part("block", "postnorm_residual", PostNormResidualBlock)
