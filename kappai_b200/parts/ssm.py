"""A selective state space mixer ("mamba2": the scalar-decay form of a state space layer).

One product gives a row ``[z | x | B | C | dt]``: ``z`` and ``x`` are ``inner = num_heads * head_dim`` wide, ``B``
and ``C`` ``groups * state_size`` each, ``dt`` one number a head.  The channels ``[x | B | C]`` pass a causal
convolution a channel (``conv_kernel`` taps, the last on the current token, with a bias) and silu.  With
``dt_t = softplus(dt_t + dt_bias_h)`` (not clamped) every head h keeps a state ``S`` [state_size, head_dim], reads
the B and C of group ``h // (num_heads / groups)`` and follows

    S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T ,    y_t = S_t^T C_t + D_h x_t .

The heads of ``y`` side by side are gated first, ``y * silu(z)``, and the gated row is then cut into ``norm_groups``
stretches of equal width, every stretch scaled to unit root mean square on its own; a weight and the output matrix
follow, into the residual.

What a request keeps between steps is one float32 row in its state slot: the state of every head, then the last
``conv_kernel - 1`` inputs of the convolution; both count as zero at position 0.  Step sizes, decays, the state
and every sum of the recurrence are float32; the storage type holds the projection and the convolution's output
(csrc/ssm.cu).  Decoded tokens and short portions run the scan kernel (row after row, the same bits however a
sequence is cut; the 32-bit mode runs it always); in 16-bit mode a step with a portion of ``CHUNKED_FROM`` rows or
more runs the chunked kernels, whose list of chunks is the step table that the ``lightning`` mixer builds too.

Params: hidden_size, num_heads, head_dim, state_size, groups, conv_kernel, norm_groups, norm_eps.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.spec import StateSpec
from ..config.schema import ConfigError
from ..ops import kernels as K
from ..ops.linear import linear
from .base import Part, WeightSpec, register_part
from .lightning import lightning_chunks


class Mamba2(Part):
    category = "mixer"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.d = int(self._p("hidden_size"))
        self.H = int(self._p("num_heads"))
        self.P = int(self._p("head_dim"))
        self.N = int(self._p("state_size"))
        self.G = int(self._p("groups", 1))
        self.taps = int(self._p("conv_kernel"))
        self.norm_groups = int(self._p("norm_groups", 1))
        self.eps = float(self._p("norm_eps"))
        if min(self.H, self.P, self.N, self.G, self.norm_groups) < 1:
            raise ConfigError("mamba2: heads, sizes and groups must be positive")
        if self.H % self.G:
            raise ConfigError(f"mamba2: num_heads={self.H} must be a multiple of groups={self.G}")
        self.inner = self.H * self.P
        if self.inner % self.norm_groups:
            raise ConfigError(f"mamba2: norm_groups={self.norm_groups} must divide num_heads * head_dim = {self.inner}")
        if not (1 <= self.taps <= K.SSM_MAX_TAPS):
            raise ConfigError(f"mamba2: conv_kernel={self.taps} outside 1..{K.SSM_MAX_TAPS}")
        if self.N > K.SSM_MAX_STATE:
            raise ConfigError(f"mamba2: state_size={self.N} is not supported by the kernels (at most {K.SSM_MAX_STATE})")
        self.C = self.inner + 2 * self.G * self.N                 # channels of the convolution
        self.n_in = 2 * self.inner + 2 * self.G * self.N + self.H
        self.state_len = self.H * self.N * self.P
        self.chunked = env.dtype != torch.float32 and self.N <= K.SSM_CHUNK_MAX_STATE and env.device.type == "cuda"
        if self.chunked:
            self.chunk_rows = K.ssm_chunk_rows()
            self.step_tables_key = ("lightning_chunks", self.chunk_rows)

    def step_tables(self, segs):
        return lightning_chunks(segs, self.chunk_rows)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        H = self.H
        return {"in_proj.weight": WeightSpec((self.n_in, self.d)), "conv.weight": WeightSpec((self.C, self.taps), "conv"),
                "conv.bias": WeightSpec((self.C,), "bias"), "dt_bias": WeightSpec((H,), "bias"),
                "A_log": WeightSpec((H,), "bias"), "D": WeightSpec((H,), "norm"),
                "norm.weight": WeightSpec((self.inner,), "norm"), "out_proj.weight": WeightSpec((self.d, self.inner))}

    def bind(self, w):
        w_in = w["in_proj.weight"]
        if self.n_in % 8:
            # zero rows behind the last, so that a row of the product's output starts on a 16-byte boundary
            w_in = torch.cat([w_in, torch.zeros((8 - self.n_in % 8, self.d), dtype=w_in.dtype, device=w_in.device)], 0)
        self.w_in = w_in.contiguous()
        self.w_o = w["out_proj.weight"].contiguous()
        f32 = lambda name: w[name].float().contiguous()
        self.conv_w, self.conv_b = f32("conv.weight"), f32("conv.bias")
        self.dt_bias, self.a_log, self.D, self.norm_w = f32("dt_bias"), f32("A_log"), f32("D"), f32("norm.weight")

    def cache_spec(self):
        return StateSpec((self.state_len + (self.taps - 1) * self.C,), "float32")

    def forward(self, h, residual, ctx, cache):
        """``cache``: a :class:`~kappai_b200.cache.storage.StateView` with tensor [n_slots, H N P + (taps - 1) C]."""
        H, G, N, P, n = self.H, self.G, self.N, self.P, ctx.n_rows
        inner, C = self.inner, self.C
        p = linear(h, self.w_in)                                 # [z | x | B | C | dt]
        xbc = torch.empty((n, C), dtype=p.dtype, device=p.device)
        dt = torch.empty((n, H), dtype=torch.float32, device=p.device)
        da = torch.empty((n, H), dtype=torch.float32, device=p.device)
        state, kept = cache.tensor, cache.tensor[:, self.state_len:]
        K.ssm_conv(p, inner, inner + C, self.conv_w, self.conv_b, self.dt_bias, self.a_log, kept, ctx.row_seg, ctx.cu_rows,
                   ctx.seg_pos, ctx.seg_slot, xbc, dt, da, ctx.n_seg, ctx.decode_only, cache.writes)
        y = torch.empty((n, inner), dtype=torch.float32, device=p.device)
        chunks = ctx.tables.get(self.step_tables_key) if self.chunked else None
        scan = lambda n_seg: K.ssm_scan(xbc, dt, da, self.D, state, ctx.cu_rows, ctx.seg_pos, ctx.seg_slot, y, n_seg,
                                        H, G, N, P, cache.writes)
        if chunks is not None:
            nl = chunks.n_lead
            if nl:
                scan(nl)                                         # decoded tokens beside the portions: the scan takes them
            K.ssm_chunks(xbc, dt, da, self.D, state, ctx.cu_rows[nl:], ctx.seg_pos[nl:], ctx.seg_slot[nl:], chunks.chunk_seg,
                         chunks.chunk_row0, chunks.seg_chunk0, chunks.n_chunks, y, ctx.n_seg - nl, H, G, N, P, cache.writes)
        else:
            scan(ctx.n_seg)
        og = torch.empty((n, inner), dtype=p.dtype, device=p.device)
        K.group_norm_gate_rows(y, self.norm_w, p[:, :inner], self.eps, og, self.norm_groups, True, "silu")
        linear(og, self.w_o, out=residual, accumulate=True)


register_part("mixer", "mamba2", Mamba2)
