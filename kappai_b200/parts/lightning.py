"""Linear attention with a per-head decay ("lightning attention").

``q, k, v = act(h Wq^T), act(h Wk^T), act(h Wv^T)`` (act = silu; heads side by
side, ``head_dim`` wide for q and k, ``value_dim`` for v); for every head a
state ``S`` [head_dim, value_dim] follows the recurrence

    S_t = a_h S_(t-1) + k_t v_t^T ,   o_t = S_t^T q_t

with one constant decay ``a_h`` a head and no other scale.  The heads of ``o``
side by side are RMS-normed as one row with a weight, multiplied by
``sigmoid(h Wg^T)`` and projected by the output matrix into the residual.  The
state is the request's only memory of this mixer: float32, one slot a request,
zero at position 0.  The four matrices that read the layer's input run as one
product; the recurrence, the norm and the gate are float32 (csrc/lightning.cu,
``norm_gate_rows``).  Decoded tokens and short portions run the scan kernel
(row after row, the same bits however a sequence is cut; the 32-bit mode runs
it always); in 16-bit mode a step with a portion of ``CHUNKED_FROM`` rows or
more runs the chunked kernels (the rows of a chunk as small float32 matrix
products, the chunks of all segments side by side; the list of chunks is a
step table built on the host).

Variants, each a parameter ("retention" is this mixer with all four): ``position``
(a ``position`` PartSpec of kind ``rope``, "rotate half" pairing) rotates q and
k by position as the kernels read them, in float32; ``k_scale`` multiplies k
behind the rotation; ``norm`` = ``"per_head"`` divides every head's ``o`` by
its own root mean square and has no weight (the default ``"all_heads"`` is the
norm above); ``gate`` = ``"silu"`` multiplies by ``silu(h Wg^T)`` instead.

Params: hidden_size, num_heads, head_dim, value_dim, decay (a list, one a
head), norm_eps, activation ("silu" | None), gate ("sigmoid" | "silu"), norm
("all_heads" | "per_head"), position (None | a rope PartSpec), k_scale.
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch

from ..cache.spec import StateSpec
from ..config.schema import ConfigError, PartSpec
from ..ops import kernels as K
from ..ops.linear import linear
from .base import Part, WeightSpec, make_part, register_part


CHUNKED_FROM = 16      # rows of a step's longest segment from which the chunked kernels run (16-bit mode)


def lightning_chunks(segs, chunk_rows: int):
    """The chunks of a step's segments for the chunked kernels (``engine.batch.StepSegments`` in,
    ``engine.batch.PartTables`` out; None for a step of short segments only, which the scan takes): every segment cut
    into stretches of at most ``chunk_rows`` rows, counted from its first row in this step.  The short segments that
    lead the step (decoded tokens, as the scheduler orders them) are left to the scan, which walks a one-row segment
    in a fraction of a chunk's time: ``n_lead`` counts them, and the lists number the other segments from 0."""
    from ..engine.batch import PartTables

    if segs.max_seg_len < CHUNKED_FROM:
        return None
    cu = segs.cu_rows
    n_lead = 0
    while segs.seg_len[n_lead] < CHUNKED_FROM:
        n_lead += 1
    chunk_seg, chunk_row0, seg_chunk0 = [], [], [0]
    for i in range(n_lead, segs.n_seg):
        for r0 in range(int(cu[i]), int(cu[i + 1]), chunk_rows):
            chunk_seg.append(i - n_lead)
            chunk_row0.append(r0)
        seg_chunk0.append(len(chunk_seg))
    i32 = lambda v: np.asarray(v, dtype=np.int32)
    return PartTables(arrays={"chunk_seg": i32(chunk_seg), "chunk_row0": i32(chunk_row0), "seg_chunk0": i32(seg_chunk0)},
                      scalars={"n_chunks": len(chunk_seg), "n_lead": n_lead})


class LightningAttention(Part):
    category = "mixer"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.d = int(self._p("hidden_size"))
        self.H = int(self._p("num_heads"))
        self.dim = int(self._p("head_dim"))
        self.vdim = int(self._p("value_dim", self.dim))
        self.eps = float(self._p("norm_eps"))
        self.activation = self._p("activation", "silu")
        decay = self._p("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != self.H:
            raise ConfigError(f"lightning: decay must list one number for each of the {self.H} heads")
        self.decay = [float(a) for a in decay]
        if any(not (0.0 <= a <= 1.0) for a in self.decay):
            raise ConfigError("lightning: a decay lies between 0 and 1")
        if self.activation not in ("silu", None):
            raise ConfigError(f"lightning: activation='{self.activation}' (expected 'silu' or none)")
        self.gate = self._p("gate", "sigmoid")
        if self.gate not in ("sigmoid", "silu"):
            raise ConfigError(f"lightning: gate='{self.gate}' (expected 'sigmoid' or 'silu')")
        self.norm = self._p("norm", "all_heads")
        if self.norm not in ("all_heads", "per_head"):
            raise ConfigError(f"lightning: norm='{self.norm}' (expected 'all_heads' or 'per_head')")
        self.k_scale = float(self._p("k_scale", 1.0))
        pos = self._p("position", None)
        self.rotary = None
        if pos is not None:
            pos = PartSpec(**pos) if isinstance(pos, dict) else pos
            enc = make_part("position", pos, env)
            if not hasattr(enc, "fused_rotary"):
                raise ConfigError("lightning: the position encoding must be one that the kernels apply themselves")
            cos, sin, rot, interleaved = enc.fused_rotary()
            if rot:
                if interleaved:
                    raise ConfigError("lightning: the kernels rotate pairs (i, i + half) only")
                if rot > self.dim:
                    raise ConfigError(f"lightning: rotary_dim={rot} exceeds head_dim={self.dim}")
                self.rotary = (cos, sin, rot)
        if min(self.H, self.dim, self.vdim) < 1 or self.dim > K.LIGHTNING_MAX_DIM:
            raise ConfigError(f"lightning: head_dim={self.dim} is not supported by the kernels (1 to {K.LIGHTNING_MAX_DIM})")
        self.chunked = env.dtype != torch.float32 and self.dim <= K.LIGHTNING_CHUNK_MAX_DIM and env.device.type == "cuda"
        if self.chunked:
            self.chunk_rows = K.lightning_chunk_rows()
            self.step_tables_key = ("lightning_chunks", self.chunk_rows)

    def step_tables(self, segs):
        return lightning_chunks(segs, self.chunk_rows)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        d, H = self.d, self.H
        s = {"q_proj.weight": WeightSpec((H * self.dim, d)), "k_proj.weight": WeightSpec((H * self.dim, d)),
             "v_proj.weight": WeightSpec((H * self.vdim, d)), "gate_proj.weight": WeightSpec((H * self.vdim, d)),
             "out_proj.weight": WeightSpec((d, H * self.vdim))}
        if self.norm == "all_heads":
            s["norm.weight"] = WeightSpec((H * self.vdim,), "norm")
        return s

    def bind(self, w):
        self.w_in = torch.cat([w["q_proj.weight"], w["k_proj.weight"], w["v_proj.weight"], w["gate_proj.weight"]], 0).contiguous()
        self.w_o = w["out_proj.weight"].contiguous()
        self.norm_w = w["norm.weight"].float().contiguous() if self.norm == "all_heads" else None
        # a decay as a float32 pair: hi the nearest float32, lo what it leaves of the constant
        a = np.asarray(self.decay, dtype=np.float64)
        hi = a.astype(np.float32)
        lo = (a - hi.astype(np.float64)).astype(np.float32)
        dev = self.w_in.device
        self.decay_hi = torch.from_numpy(hi).to(dev)
        self.decay_lo = torch.from_numpy(lo).to(dev)
        # the chunked kernel's table of powers a^0 .. a^rows, made in double
        self.decay_pow = None
        if self.chunked:
            m = np.arange(self.chunk_rows + 1, dtype=np.float64)
            self.decay_pow = torch.from_numpy(np.power(a[:, None], m[None, :]).astype(np.float32)).contiguous().to(dev)

    def cache_spec(self):
        return StateSpec((self.H, self.dim, self.vdim), "float32")

    def forward(self, h, residual, ctx, cache):
        """``cache``: a :class:`~kappai_b200.cache.storage.StateView` with tensor [n_slots, H, head_dim, value_dim]."""
        H, dim, vdim, n = self.H, self.dim, self.vdim, ctx.n_rows
        p = linear(h, self.w_in)                                 # [q | k | v | gate]
        o = torch.empty((n, H * vdim), dtype=torch.float32, device=p.device)
        chunks = ctx.tables.get(self.step_tables_key) if self.chunked else None
        scan = lambda n_seg: K.lightning_scan(p, 0, H * dim, 2 * H * dim, self.decay_hi, self.decay_lo, cache.tensor, ctx.cu_rows,
                                              ctx.seg_pos, ctx.seg_slot, o, n_seg, H, dim, vdim, self.activation, cache.writes,
                                              self.rotary, self.k_scale)
        if chunks is not None:
            # (measured at 2,048 rows against the scan: 32 heads of 64 x 64 151 us against 430, of 128 x 128 620 against 1291)
            nl = chunks.n_lead
            if nl:
                scan(nl)                                         # decoded tokens beside the portions: the scan takes them
            K.lightning_chunks(p, 0, H * dim, 2 * H * dim, self.decay_pow, cache.tensor, ctx.cu_rows[nl:], ctx.seg_pos[nl:],
                               ctx.seg_slot[nl:], chunks.chunk_seg, chunks.chunk_row0, chunks.seg_chunk0, chunks.n_chunks, o,
                               ctx.n_seg - nl, H, dim, vdim, self.activation, cache.writes, self.rotary, self.k_scale)
        else:
            scan(ctx.n_seg)
        g0 = 2 * H * dim + H * vdim
        og = torch.empty((n, H * vdim), dtype=p.dtype, device=p.device)
        gate = p[:, g0:g0 + H * vdim]
        if self.norm == "all_heads" and self.gate == "sigmoid":
            K.norm_gate_rows(o, self.norm_w, gate, self.eps, og)
        else:
            K.group_norm_gate_rows(o, self.norm_w, gate, self.eps, og, H if self.norm == "per_head" else 1, False, self.gate)
        linear(og, self.w_o, out=residual, accumulate=True)


register_part("mixer", "lightning", LightningAttention)
