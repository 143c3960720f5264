"""Grouped-query attention over the paged cache.

``q,k,v = h Wq^T, h Wk^T, h Wv^T`` (run as one product against the rows
[Wq; Wk; Wv], as the reference does with ``--fuse qkv``, src/model.c:1440-1448);
optional per-head RMSNorm of q and k with one weight [head_dim] shared by the
heads, before the rotation (src/models/lfm.c:36-39); position encoding; keys and
values into the cache; causal softmax attention with ``scale`` over the keys
``max(0, p - window + 1) .. p`` (src/backend/cpu/scalar/core.c:383-433);
``out = attn Wo^T`` added to the residual (src/models/lfm.c:51,
src/recipe/builders.c:381).

Variants, each a parameter: ``values`` = ``"keys"`` leaves the value matrix out
and takes as values the key projections as they leave the product, before the
key norm and the rotation; ``block`` (a number of positions) lets a row read no
key from before the start of its own block, blocks being counted from position
0 of the sequence, whatever the portions a prompt is run in; ``gate`` =
``"sigmoid"`` multiplies the concatenated heads, element by element, with
``sigmoid(h Wg^T)`` in front of the output matrix (Wg rides in the same product
as q and k).  ``softmax_weights`` = ``"float32"`` keeps the softmax weights
whole where they are multiplied with the values (the general and scalar kernels
always do; the ``mma.sync`` kernels then take them as three bfloat16 parts, and
the tcgen05 prompt kernel, which rounds them to one bfloat16 operand, is left
out); the default ``"operand"`` rounds them to bfloat16 as a matrix operand.

More variants: ``qk_norm`` = ``"projection"`` norms q, and k, each as one row
over all its heads at once, with weights as long as the projections (the
default ``"per_head"`` is the norm above); ``gate`` = ``"head_sigmoid"`` is a
gate of one number a head, ``sigmoid(h Wg^T)`` with Wg [num_heads, hidden];
``value_dim`` (default head_dim) is the width of a value head: where it differs
from head_dim a cache head is as wide as the wider of the two rounded up to a
multiple of 16, and the matrices get zero rows or columns for that at load;
``kv`` = ``"borrowed"``: the mixer has no key and value tensors and writes no
cache: its schedule entry names the entry whose cache its queries read (after
that entry's key norm).  ``cache_window``: how many positions back the cache
must keep keys (at least ``window``; larger where a borrower's window is).

Three more, for designs without a rotation: ``keep_first`` (with a ``window``): the first that many keys of a
sequence stay visible to every later row, at their true places, and their pages are never given back;
``sink`` = ``"zero"`` adds one to the softmax's denominator (a key whose score is 0 and which has no value),
``"learned"`` adds ``exp(sink_h)`` of a tensor ``sink`` [num_heads] (not scaled, counted once a row);
``q_temp`` = {coef, every}: the query of position p is multiplied by
``1 + coef ln(floor((p + 1) / every) + 1)`` (float32, in the fused q/k kernel).  The per-head q/k norm goes with a
``value_dim`` of its own: the norm's mean is then taken over ``head_dim`` columns of the wider cache head.  An odd
``head_dim`` without a position encoding is stored wider in the same way.

Sizes and constants (params): hidden_size, num_heads, num_kv_heads, head_dim,
value_dim, scale, qk_norm_eps (None: no q/k norm), qk_norm ("per_head" |
"projection"), window (None: all keys), cache_window, block (None), values
("projection" | "keys"), kv ("own" | "borrowed"), gate (None | "sigmoid" |
"head_sigmoid"), softmax_weights ("operand" | "float32"), position (a
``position`` PartSpec), bias, keep_first, sink (None | "zero" | "learned"), q_temp.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from ..cache.spec import PagedKVSpec
from ..config.schema import ConfigError, PartSpec
from ..ops import kernels as K
from ..ops.linear import linear
from .base import Part, WeightSpec, make_part, register_part


# Geometry of the attention kernels' work lists (built on the host for every step that has prompt portions).
ROW_TILE = 64              # rows of one segment that the mma.sync prefill kernel takes at a time
BIG_TILE = 128             # rows of the tcgen05 prefill kernel's tiles
SHORT_SEG = 4              # segments of at most this many rows count as decoded tokens: split-KV kernel


def attention_tiles(segs, split_ok: bool = True):
    """Work lists of the tiled prefill kernels for one step (``engine.batch.StepSegments`` in,
    ``engine.batch.PartTables`` out; None for a step of short segments only, which the split-KV kernel takes).

    ``tile_seg`` / ``tile_row0``: segment and first row of every stretch of ROW_TILE consecutive rows of a
    segment.  ``big_tile_seg`` / ``big_tile_row0``: the same in stretches of BIG_TILE rows, those that read the
    most keys first (a kernel that gives a CTA the i-th and the i-th last of them gives every CTA about the same
    work).  A step that mixes decoded tokens with prompt portions: the leading segments of at most SHORT_SEG
    rows (the scheduler puts decodes first) go to the split-KV kernel, made for single rows with long caches,
    and the rest to a tiled one; ``n_short_rows`` / ``n_short_tiles`` are the rows and ROW_TILE tiles of that
    lead (0 if the step is not mixed in this way), and the big tiles then list the other segments only."""
    from ..engine.batch import PartTables

    if split_ok and segs.max_seg_len <= SHORT_SEG:
        return None
    cu, n_seg = segs.cu_rows, segs.n_seg
    tile_seg, tile_row0 = [], []
    for i in range(n_seg):
        for r0 in range(int(cu[i]), int(cu[i + 1]), ROW_TILE):
            tile_seg.append(i)
            tile_row0.append(r0)
    n_short_seg = 0
    while n_short_seg < n_seg and segs.seg_len[n_short_seg] <= SHORT_SEG:
        n_short_seg += 1
    if n_short_seg == n_seg or all(n > SHORT_SEG for n in segs.seg_len):
        n_short_seg = 0                                   # all short or none: one kernel takes the whole step
    big = []
    for i in range(n_short_seg, n_seg):
        for r0 in range(int(cu[i]), int(cu[i + 1]), BIG_TILE):
            last_pos = int(segs.seg_pos[i]) + min(r0 + BIG_TILE, int(cu[i + 1])) - int(cu[i]) - 1
            big.append((-last_pos, i, r0))                # the further on, the more keys
    big.sort()
    i32 = lambda v: np.asarray(v, dtype=np.int32)
    return PartTables(
        arrays={"tile_seg": i32(tile_seg), "tile_row0": i32(tile_row0),
                "big_tile_seg": i32([b[1] for b in big]), "big_tile_row0": i32([b[2] for b in big])},
        scalars={"n_tiles": len(tile_seg), "n_big_tiles": len(big), "n_short_rows": int(cu[n_short_seg]),
                 "n_short_tiles": n_short_seg})


class PagedAttentionKernels:
    """The choice among the attention kernels over the paged cache, shared by the mixers that keep keys and values
    there.  The mixer has ``H``, ``G``, ``hd``, ``scale``, ``window``, ``block``, ``exact_weights``, ``split_ok``
    and ``step_tables_key``; ``keep_first`` and ``sink_w`` (float32 [H] or None) if it has kept first keys or a sink."""

    keep_first = 0
    sink_w = None

    def _read_sink(self, what: str):
        """The parameters ``sink`` and ``keep_first`` (shared by the mixers over the paged cache)."""
        self.sink = self._p("sink", None)
        if self.sink not in (None, "zero", "learned"):
            raise ConfigError(f"{what}: sink='{self.sink}' (expected 'zero', 'learned' or none)")
        self.keep_first = int(self._p("keep_first", 0) or 0)
        if self.keep_first < 0:
            raise ConfigError(f"{what}: keep_first={self.keep_first} must not be negative")
        if self.keep_first and self.window is None:
            self.keep_first = 0                              # without a window every key is read anyway
        if self.keep_first and self.block is not None:
            raise ConfigError(f"{what}: keep_first does not go with blocks of positions")

    def _bind_sink(self, w, device):
        if self.sink == "learned":
            self.sink_w = w["sink"].to(torch.float32).reshape(-1).contiguous()
        elif self.sink == "zero":
            self.sink_w = torch.zeros(self.H, dtype=torch.float32, device=device)
        else:
            self.sink_w = None


    def _tile_setup(self):
        # (the split-key kernel reads keys 16 bytes at a time and shares a kv head among at most 8 query heads;
        # other shapes take the general kernel for every row)
        self.split_ok = self.H // self.G <= K.SPLIT_MAX_RATIO and self.hd % 16 == 0
        self.step_tables_key = ("attention_tiles", self.split_ok)

    def step_tables(self, segs):
        return attention_tiles(segs, self.split_ok)

    def _attend(self, q, ctx, view, cache):
        """Causal attention of the rows ``q`` [n, H hd] over the cache (this step's keys and values already in
        it); returns the heads side by side."""
        H, G, hd = self.H, self.G, self.hd
        o = torch.empty_like(q)
        extra = dict(keep_first=self.keep_first, sink=self.sink_w)
        tiles = ctx.tables.get(self.step_tables_key)
        if self.split_ok and (tiles is None or q.dtype == torch.float32):
            # rows that each read a long cache (decode): split the keys over many CTAs.  The 32-bit path
            # takes this kernel for every row, whatever the length of its segment: its chunks lie at absolute
            # multiples of 256 keys and are summed in order, so a row's bits do not depend on how the step was cut.
            self._split(q, o, ctx, view, cache, ctx.n_rows)
        elif tiles is not None and K.attention_prefill_ok(q, hd):
            lead = tiles.n_short_rows
            if lead and self.split_ok:
                # decoded tokens beside prompt portions: the decoded rows lead the batch and go to the split
                # kernel (in a row tile each would walk its whole cache alone), the portions to the tiled one
                self._split(q, o, ctx, view, cache, lead)
                t0 = tiles.n_short_tiles
                K.attention_prefill(q, cache.tensor, view.block_table, ctx.cu_rows, ctx.seg_pos, tiles.tile_seg[t0:],
                                    tiles.tile_row0[t0:], o, self.scale, self.window, view.page_size, H, G, hd,
                                    tiles.big_tile_seg, tiles.big_tile_row0, block=self.block, exact_weights=self.exact_weights,
                                    **extra)
            else:
                # (with a lead that the split kernel cannot take, the big tiles leave it out: small tiles only)
                big = (None, None) if lead else (tiles.big_tile_seg, tiles.big_tile_row0)
                K.attention_prefill(q, cache.tensor, view.block_table, ctx.cu_rows, ctx.seg_pos, tiles.tile_seg,
                                    tiles.tile_row0, o, self.scale, self.window, view.page_size, H, G, hd, *big,
                                    block=self.block, exact_weights=self.exact_weights, **extra)
        else:
            lead = tiles.n_short_rows if tiles is not None else 0
            if lead and self.split_ok:
                self._split(q, o, ctx, view, cache, lead)
            else:
                lead = 0
            K.attention_rows(q[lead:], cache.tensor, view.block_table, ctx.row_seg[lead:], ctx.positions[lead:], o[lead:],
                             self.scale, self.window, view.page_size, H, G, hd, self.block, **extra)
        return o

    def _split(self, q, o, ctx, view, cache, n_rows):
        """Split-key attention for the first ``n_rows`` rows of the step."""
        H, G, hd = self.H, self.G, self.hd
        n_chunks = -(-ctx.max_context // K.SPLIT_CHUNK)
        need = K.attention_split_scratch(n_rows, H, hd, n_chunks, self.keep_first)
        ws = self.env.shared.get("attn_scratch")
        if ws is None or ws.numel() < need:
            # A captured decode step keeps the address of the scratch it was captured with, so a buffer that
            # has been outgrown is retired, never freed: a replay of an older graph then still writes memory
            # that nobody else owns.  Growth doubles, so the retired buffers together are smaller than the live one.
            if ws is not None:
                self.env.shared.setdefault("attn_scratch_retired", []).append(ws)
            ws = torch.zeros(max(need, 2 * (ws.numel() if ws is not None else 0), 1 << 16), dtype=torch.float32,
                             device=q.device)
            self.env.shared["attn_scratch"] = ws
        K.attention_split(q[:n_rows], cache.tensor, view.block_table, ctx.row_seg[:n_rows], ctx.positions[:n_rows],
                          o[:n_rows], ws, n_chunks, self.scale, self.window, view.page_size, H, G, hd, self.block,
                          self.exact_weights, keep_first=self.keep_first, sink=self.sink_w)


class Attention(PagedAttentionKernels, Part):
    category = "mixer"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.d = int(self._p("hidden_size"))
        self.H = int(self._p("num_heads"))
        self.G = int(self._p("num_kv_heads"))
        self.hd = int(self._p("head_dim"))
        self.scale = float(self._p("scale"))
        eps = self._p("qk_norm_eps", None)
        self.qk_norm_eps: Optional[float] = None if eps is None else float(eps)
        self.window: Optional[int] = self._p("window", None)
        self.bias = bool(self._p("bias", False))
        self.block: Optional[int] = self._p("block", None)
        if self.block is not None and int(self.block) < 1:
            raise ConfigError(f"attention: block={self.block} must be a positive number of positions")
        values = self._p("values", "projection")
        if values not in ("projection", "keys"):
            raise ConfigError(f"attention: values='{values}' (expected 'projection' or 'keys')")
        self.values_are_keys = values == "keys"
        gate = self._p("gate", None)
        if gate not in (None, "sigmoid", "head_sigmoid"):
            raise ConfigError(f"attention: gate='{gate}' (expected 'sigmoid', 'head_sigmoid' or none)")
        self.gated = gate is not None
        self.head_gate = gate == "head_sigmoid"
        sw = self._p("softmax_weights", "operand")
        if sw not in ("operand", "float32"):
            raise ConfigError(f"attention: softmax_weights='{sw}' (expected 'operand' or 'float32')")
        self.exact_weights = sw == "float32"
        self.qk_norm = self._p("qk_norm", "per_head")
        if self.qk_norm not in ("per_head", "projection"):
            raise ConfigError(f"attention: qk_norm='{self.qk_norm}' (expected 'per_head' or 'projection')")
        kv = self._p("kv", "own")
        if kv not in ("own", "borrowed"):
            raise ConfigError(f"attention: kv='{kv}' (expected 'own' or 'borrowed')")
        self.borrows = kv == "borrowed"
        cw = self._p("cache_window", self.window)
        self.cache_window: Optional[int] = None if cw is None else int(cw)
        if self.window is not None and self.cache_window is not None and self.cache_window < int(self.window):
            raise ConfigError(f"attention: cache_window={self.cache_window} is smaller than window={self.window}")
        if self.bias and (self.values_are_keys or self.gated):
            raise ConfigError("attention: biases are not combined with values='keys' or a gate")
        if self.H < 1 or self.G < 1 or self.H % self.G:
            raise ConfigError(f"attention: num_heads={self.H} must be a multiple of num_kv_heads={self.G}")
        # dim, vdim: the heads as the model has them; hd: as the cache and the kernels see them
        self.dim = self.hd
        self.vdim = int(self._p("value_dim", self.dim))
        pos_given = self._p("position", None) is not None
        if self.qk_norm == "projection" or self.vdim != self.dim or (self.dim % 2 and not pos_given):
            # (an odd head size without a rotation is stored wider too: the kernels take even sizes)
            if self.values_are_keys or self.bias:
                raise ConfigError("attention: values='keys' and biases want value_dim = head_dim and the per-head norm")
            if min(self.dim, self.vdim) < 1:
                raise ConfigError("attention: head sizes must be positive")
            self.hd = -(-max(self.dim, self.vdim) // 16) * 16
        if self.borrows and (self.values_are_keys or self.bias or self.qk_norm != "projection"):
            raise ConfigError("attention: kv='borrowed' goes with qk_norm='projection', a value matrix elsewhere and no biases")
        if self.qk_norm == "projection" and self.qk_norm_eps is None:
            raise ConfigError("attention: qk_norm='projection' needs qk_norm_eps")
        if self.hd % 2 or not (2 <= self.hd <= 256):
            raise ConfigError(f"attention: head_dim={self.dim} is not supported by the kernels "
                              "(an even number from 2 to 256)")
        pos = self._p("position", None)
        if pos is None:
            pos = PartSpec("none")
        elif isinstance(pos, dict):
            pos = PartSpec(**pos)
        self.position = make_part("position", pos, env)
        self.graph_safe = bool(self.position.graph_safe)     # a position part that reads host values keeps it eager
        self._read_sink("attention")
        qt = self._p("q_temp", None)
        self.q_temp = None
        if qt is not None:
            coef, every = (qt["coef"], qt["every"]) if isinstance(qt, dict) else qt
            self.q_temp = (float(coef), float(every))
            if not self.q_temp[1] > 0:
                raise ConfigError(f"attention: q_temp.every={every} must be positive")
            if not hasattr(self.position, "fused_rotary") or self.qk_norm == "projection":
                raise ConfigError("attention: q_temp runs in the fused q/k kernel (no position part of its own, per-head norm or none)")
        if self.vdim != self.dim and self.qk_norm != "projection" and self.qk_norm_eps is not None:
            if not hasattr(self.position, "fused_rotary") or self.position.fused_rotary()[2]:
                raise ConfigError("attention: a per-head q/k norm with value_dim != head_dim runs without a rotation")
        if self.values_are_keys and not hasattr(self.position, "fused_rotary"):
            raise ConfigError("attention: values='keys' needs a position encoding that runs in the fused q/k kernel")
        if self.qk_norm == "projection" and (not hasattr(self.position, "fused_rotary") or self.position.fused_rotary()[2]):
            raise ConfigError("attention: qk_norm='projection' runs without a rotation")
        self._tile_setup()

    def weight_specs(self) -> Dict[str, WeightSpec]:
        d, H, G = self.d, self.H, self.G
        s = {"q_proj.weight": WeightSpec((H * self.dim, d)), "out_proj.weight": WeightSpec((d, H * self.vdim))}
        if not self.borrows:
            s["k_proj.weight"] = WeightSpec((G * self.dim, d))
            if not self.values_are_keys:
                s["v_proj.weight"] = WeightSpec((G * self.vdim, d))
        if self.gated:
            s["gate_proj.weight"] = WeightSpec((H if self.head_gate else H * self.vdim, d))
        if self.qk_norm == "projection":
            s["q_norm.weight"] = WeightSpec((H * self.dim,), "norm")
            if not self.borrows:
                s["k_norm.weight"] = WeightSpec((G * self.dim,), "norm")
        elif self.qk_norm_eps is not None:
            s["q_norm.weight"] = WeightSpec((self.dim,), "norm")
            s["k_norm.weight"] = WeightSpec((self.dim,), "norm")
        if self.sink == "learned":
            s["sink"] = WeightSpec((H,), "bias")
        if self.bias:
            hd = self.hd                      # (biases go with value_dim = head_dim)
            for n, sz in (("q_proj", H * hd), ("k_proj", G * hd), ("v_proj", G * hd), ("out_proj", d)):
                s[n + ".bias"] = WeightSpec((sz,), "bias")
        return s

    def _pad_heads(self, w, heads, width):
        """[heads width, ...] -> [heads hd, ...]: every head's rows, then zero rows up to the cache head's width."""
        if width == self.hd:
            return w.contiguous()
        out = torch.zeros((heads, self.hd) + tuple(w.shape[1:]), dtype=w.dtype, device=w.device)
        out[:, :width] = w.reshape((heads, width) + tuple(w.shape[1:]))
        return out.reshape((heads * self.hd,) + tuple(w.shape[1:]))

    def bind(self, w):
        # one product for everything that reads the layer's input: rows [q | k | v (if it has a matrix) | gate]
        H, G, hd = self.H, self.G, self.hd
        rows = [self._pad_heads(w["q_proj.weight"], H, self.dim)]
        if not self.borrows:
            rows.append(self._pad_heads(w["k_proj.weight"], G, self.dim))
            if not self.values_are_keys:
                rows.append(self._pad_heads(w["v_proj.weight"], G, self.vdim))
        self.gate_col = sum(r.shape[0] for r in rows)
        if self.gated:
            rows.append(w["gate_proj.weight"] if self.head_gate else self._pad_heads(w["gate_proj.weight"], H, self.vdim))
        n_rows = sum(r.shape[0] for r in rows)
        if n_rows % 8:
            # zero rows behind the last, so that a row of the product's output starts on a 16-byte boundary
            rows.append(torch.zeros((8 - n_rows % 8, self.d), dtype=rows[0].dtype, device=rows[0].device))
        self.w_qkv = torch.cat(rows, 0).contiguous()
        self.k_col = H * hd
        self.v_col = H * hd if self.values_are_keys else (H + G) * hd
        self.w_o = self._pad_heads(w["out_proj.weight"].t().contiguous(), H, self.vdim).t().contiguous()
        self.b_qkv = self.b_o = None
        if self.bias:
            self.b_qkv = torch.cat([w[n + ".bias"].float() for n in ("q_proj", "k_proj", "v_proj")]).contiguous()
            self.b_o = w["out_proj.bias"].float().contiguous()
        self.q_w = self.k_w = None
        if self.qk_norm == "projection":
            self.q_w = self._pad_heads(w["q_norm.weight"].float(), H, self.dim)
            if not self.borrows:
                self.k_w = self._pad_heads(w["k_norm.weight"].float(), G, self.dim)
        elif self.qk_norm_eps is not None:
            # (a head stored wider than it is: zeros behind the weight's own columns, as behind the head's)
            self.q_w = self._pad_heads(w["q_norm.weight"].float(), 1, self.dim)
            self.k_w = self._pad_heads(w["k_norm.weight"].float(), 1, self.dim)
        self._bind_sink(w, self.w_qkv.device)

    def cache_spec(self):
        # (a borrower names what it reads, so that the engine can see that lender and borrower agree)
        return PagedKVSpec(self.G, self.hd, self.cache_window, None if self.block is None else int(self.block),
                           self.keep_first if self.cache_window is not None else 0)

    def forward(self, h, residual, ctx, cache):
        """``cache``: a :class:`~kappai_b200.cache.storage.KVLayerView`."""
        H, G, hd = self.H, self.G, self.hd
        view = ctx.paged[cache.group]
        qkv = linear(h, self.w_qkv, self.b_qkv)
        q = torch.empty((ctx.n_rows, H * hd), dtype=qkv.dtype, device=qkv.device)
        kv_out = cache.tensor if cache.writes else None
        if self.borrows and cache.writes:
            raise ValueError("attention: a mixer with kv='borrowed' was given a cache of its own")
        if self.qk_norm == "projection":
            K.qk_rownorm_kv(qkv, self.k_col, self.v_col, self.q_w, self.k_w, self.qk_norm_eps, H * self.dim, G * self.dim,
                            view.slot_map, q, kv_out, view.page_size, H, G, hd)
        elif hasattr(self.position, "fused_rotary"):
            cos, sin, rot, inter = self.position.fused_rotary()
            K.qk_norm_rope_kv(qkv, self.q_w, self.k_w, self.qk_norm_eps or 0.0, cos, sin, rot, inter,
                              ctx.positions, view.slot_map, q, kv_out, view.page_size, H, G, hd, self.v_col,
                              norm_dim=self.dim, q_temp=self.q_temp)
        else:
            # a position encoding of its own: norm in place, let it change q and k, then scatter
            if self.q_w is not None:
                K.qk_norm_rope_kv(qkv, self.q_w, self.k_w, self.qk_norm_eps, None, None, 0, False, ctx.positions,
                                  None, None, None, view.page_size, H, G, hd)
            self.position.apply(qkv[:, :H * hd], qkv[:, H * hd:(H + G) * hd], ctx)
            K.qk_norm_rope_kv(qkv, None, None, 0.0, None, None, 0, False, ctx.positions, view.slot_map, q, kv_out,
                              view.page_size, H, G, hd)
        o = self._attend(q, ctx, view, cache)
        if self.head_gate:
            K.head_gate(o, qkv[:, self.gate_col:self.gate_col + H], H, hd)
        elif self.gated:
            K.sigmoid_gate(o, qkv[:, self.gate_col:self.gate_col + H * hd])
        linear(o, self.w_o, self.b_o, out=residual, accumulate=True)


class LatentAttention(PagedAttentionKernels, Part):
    """Attention whose queries, keys and values are expanded from low-rank latents, without positions.

    ``c_q = norm(h Wdq^T) * w_q``, ``q = c_q Wuq^T``; ``c = norm(h Wdkv^T) * w_kv``, ``k = c Wuk^T``,
    ``v = c Wuv^T`` (every head has keys and values of its own, ``head_dim`` and ``value_dim`` wide); causal
    softmax attention with ``scale``; the concatenated heads times ``sigmoid(h Wg^T)`` (``gate`` = ``"sigmoid"``),
    then the output matrix.  The two down-projections and the gate read the same input and run as one product;
    the two latents are normed by one launch; the expanded keys and values go to the paged cache, one kv head a
    query head, and the attention kernels of :class:`Attention` run over it unchanged.  A cache head is as wide
    as the wider of ``head_dim`` and ``value_dim``, rounded up to a multiple of 16 (the expanding matrices, the
    gate's and the output matrix get zero rows or columns for that at load, so that nothing pads at run time).

    ``gate`` = ``"head_sigmoid"``: one gate a head, ``sigmoid(h Wg^T)`` with Wg [num_heads, hidden].  ``window``,
    ``keep_first`` and ``sink`` as in :class:`Attention` (a learned sink is the tensor ``sink`` [num_heads]).

    Params: hidden_size, num_heads, head_dim, value_dim, q_rank, kv_rank, scale, norm_eps, gate (None |
    "sigmoid" | "head_sigmoid"), softmax_weights ("operand" | "float32"), window, block, keep_first, sink.
    """

    category = "mixer"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.d = int(self._p("hidden_size"))
        self.H = int(self._p("num_heads"))
        self.dim = int(self._p("head_dim"))
        self.vdim = int(self._p("value_dim", self.dim))
        self.q_rank = int(self._p("q_rank"))
        self.kv_rank = int(self._p("kv_rank"))
        self.scale = float(self._p("scale"))
        self.eps = float(self._p("norm_eps"))
        self.window: Optional[int] = self._p("window", None)
        self.block: Optional[int] = self._p("block", None)
        gate = self._p("gate", None)
        if gate not in (None, "sigmoid", "head_sigmoid"):
            raise ConfigError(f"latent_attention: gate='{gate}' (expected 'sigmoid', 'head_sigmoid' or none)")
        self.gated = gate is not None
        self.head_gate = gate == "head_sigmoid"
        self._read_sink("latent_attention")
        sw = self._p("softmax_weights", "operand")
        if sw not in ("operand", "float32"):
            raise ConfigError(f"latent_attention: softmax_weights='{sw}' (expected 'operand' or 'float32')")
        self.exact_weights = sw == "float32"
        if min(self.H, self.dim, self.vdim, self.q_rank, self.kv_rank) < 1:
            raise ConfigError("latent_attention: heads, head sizes and ranks must be positive")
        self.G = self.H                                          # the expanded keys and values are per head
        self.hd = -(-max(self.dim, self.vdim) // 16) * 16        # width of a head in the cache
        if self.hd > 256:
            raise ConfigError(f"latent_attention: heads of {max(self.dim, self.vdim)} are not supported by the kernels (at most 256)")
        self._tile_setup()

    def weight_specs(self) -> Dict[str, WeightSpec]:
        d, H = self.d, self.H
        s = {"q_down.weight": WeightSpec((self.q_rank, d)), "q_norm.weight": WeightSpec((self.q_rank,), "norm"),
             "q_up.weight": WeightSpec((H * self.dim, self.q_rank)),
             "kv_down.weight": WeightSpec((self.kv_rank, d)), "kv_norm.weight": WeightSpec((self.kv_rank,), "norm"),
             "k_up.weight": WeightSpec((H * self.dim, self.kv_rank)), "v_up.weight": WeightSpec((H * self.vdim, self.kv_rank)),
             "out_proj.weight": WeightSpec((d, H * self.vdim))}
        if self.gated:
            s["gate_proj.weight"] = WeightSpec((H if self.head_gate else H * self.vdim, d))
        if self.sink == "learned":
            s["sink"] = WeightSpec((H,), "bias")
        return s

    def _pad_rows(self, w, width):
        """[H width, k] -> [H hd, k]: every head's rows, then zero rows up to the cache head's width."""
        if width == self.hd:
            return w.contiguous()
        out = torch.zeros((self.H, self.hd, w.shape[1]), dtype=w.dtype, device=w.device)
        out[:, :width] = w.reshape(self.H, width, w.shape[1])
        return out.reshape(self.H * self.hd, w.shape[1])

    def bind(self, w):
        rows = [w["q_down.weight"], w["kv_down.weight"]]
        if self.gated:
            rows.append(w["gate_proj.weight"] if self.head_gate else self._pad_rows(w["gate_proj.weight"], self.vdim))
        n_rows = sum(r.shape[0] for r in rows)
        if n_rows % 8:
            # zero rows behind the last, so that a row of the product's output starts on a 16-byte boundary
            rows.append(torch.zeros((8 - n_rows % 8, self.d), dtype=rows[0].dtype, device=rows[0].device))
        self.w_down = torch.cat(rows, 0).contiguous()
        self.gate_col = self.q_rank + self.kv_rank
        self.q_norm_w = w["q_norm.weight"].float().contiguous()
        self.kv_norm_w = w["kv_norm.weight"].float().contiguous()
        self.w_uq = self._pad_rows(w["q_up.weight"], self.dim)
        self.w_ukv = torch.cat([self._pad_rows(w["k_up.weight"], self.dim), self._pad_rows(w["v_up.weight"], self.vdim)], 0).contiguous()
        self.w_o = self._pad_rows(w["out_proj.weight"].t().contiguous(), self.vdim).t().contiguous()
        self._bind_sink(w, self.w_down.device)

    def cache_spec(self):
        return PagedKVSpec(self.H, self.hd, self.window, None if self.block is None else int(self.block),
                           self.keep_first if self.window is not None else 0)

    def forward(self, h, residual, ctx, cache):
        H, hd, n = self.H, self.hd, ctx.n_rows
        view = ctx.paged[cache.group]
        p = linear(h, self.w_down)                               # [c_q before its norm | c before its norm | gate]
        cq = torch.empty((n, self.q_rank), dtype=p.dtype, device=p.device)
        c = torch.empty((n, self.kv_rank), dtype=p.dtype, device=p.device)
        K.rmsnorm_cols(p, [(0, self.q_norm_w, cq), (self.q_rank, self.kv_norm_w, c)], self.eps)
        qkv = torch.empty((n, 3 * H * hd), dtype=p.dtype, device=p.device)
        linear(cq, self.w_uq, out=qkv[:, :H * hd])
        linear(c, self.w_ukv, out=qkv[:, H * hd:])
        q = torch.empty((n, H * hd), dtype=p.dtype, device=p.device)
        K.qk_norm_rope_kv(qkv, None, None, 0.0, None, None, 0, False, ctx.positions, view.slot_map, q,
                          cache.tensor if cache.writes else None, view.page_size, H, H, hd)
        o = self._attend(q, ctx, view, cache)
        if self.head_gate:
            K.head_gate(o, p[:, self.gate_col:self.gate_col + H], H, hd)
        elif self.gated:
            K.sigmoid_gate(o, p[:, self.gate_col:self.gate_col + H * hd])
        linear(o, self.w_o, out=residual, accumulate=True)


register_part("mixer", "attention", Attention)
register_part("mixer", "latent_attention", LatentAttention)
