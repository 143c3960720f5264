"""SwiGLU feed-forward.

``f = (silu(h Wg^T) * (h Wu^T)) Wd^T`` added to the residual; gate and up run
as one product against [Wg; Wu], gate rows first (src/recipe/builders.c:344-388,
src/model.c:1575-1610); ``silu(g) = g / (1 + exp(-g))``
(src/backend/cpu/quants.h:369-371).

Params: hidden_size, intermediate_size, bias, activation (``silu`` by default;
``relu`` and ``gelu_tanh`` make the same unit with another function on the gate:
kind ``glu``).

``glu_clamped``: the same three matrices with another unit between them: the
gate is bounded above and the other branch on both sides,
``g = min(h Wg^T + bg, limit)``, ``u = clamp(h Wu^T + bu, -limit, limit)``,
``f = (g sigmoid(alpha g) (u + shift)) Wd^T + bd``.  Params: hidden_size,
intermediate_size, limit, alpha, shift, bias.

``moe``: a mixture of ``num_experts`` such units without biases, of which every
row uses the ``top`` with the largest router logits ``z = h Wr^T + b`` (float32),
weighted by the softmax over those ``top`` logits alone; see csrc/moe.cu.
Params: hidden_size, expert_size, num_experts, top, activation, router_bias.
More of them, each off by default: ``routing`` = ``"softmax_all"`` takes as
scores the softmax over all router outputs, chooses by score + a learned
``correction`` (a tensor; it takes part in the choice only) and weighs a chosen
expert by its score times ``router_scale``, without renormalising;
``identity_experts``: that many further router outputs stand for experts that
return their input (they have no tensors); ``shared_size``: a unit of that size
which every row uses beside its chosen experts, its output times
``sigmoid(w_sg . h)``, one gate a row (``shared_gate`` = ``"sigmoid"``) or
ungated (None).  ``routing`` = ``"sigmoid"``: the ``top`` largest logits are
chosen and a chosen expert's weight is ``sigmoid(z)`` of its own logit times
``router_scale``, not renormalised.  ``weight_on`` = ``"input"``: the weight
multiplies what the expert reads, ``sum_j expert_j(w_j h)``, instead of what it
returns (``"output"``, the default).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels as K
from ..ops.linear import linear, linear_swiglu
from ..config.schema import ConfigError
from .base import Part, WeightSpec, register_part


class SwiGLU(Part):
    category = "feed_forward"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.d = int(self._p("hidden_size"))
        self.ff = int(self._p("intermediate_size"))
        self.bias = bool(self._p("bias", False))
        self.activation = str(self._p("activation", "silu"))
        K.activation_code(self.activation)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {"gate_proj.weight": WeightSpec((self.ff, self.d)), "up_proj.weight": WeightSpec((self.ff, self.d)),
             "down_proj.weight": WeightSpec((self.d, self.ff))}
        if self.bias:
            s["gate_proj.bias"] = WeightSpec((self.ff,), "bias")
            s["up_proj.bias"] = WeightSpec((self.ff,), "bias")
            s["down_proj.bias"] = WeightSpec((self.d,), "bias")
        return s

    def bind(self, w):
        self.w_gu = torch.cat([w["gate_proj.weight"], w["up_proj.weight"]], 0).contiguous()
        self.w_down = w["down_proj.weight"].contiguous()
        self.b_gu = self.b_down = None
        if self.bias:
            self.b_gu = torch.cat([w["gate_proj.bias"].float(), w["up_proj.bias"].float()]).contiguous()
            self.b_down = w["down_proj.bias"].float().contiguous()

    def forward(self, h, residual, ctx):
        act = linear_swiglu(h, self.w_gu, self.b_gu, self.activation)
        linear(act, self.w_down, self.b_down, out=residual, accumulate=True)


class ClampedGLU(SwiGLU):
    """``glu_clamped``: see the module's text.  Gate and up run as one product whose epilogue computes the unit, in
    float32 from their values rounded to the storage type (where no product kernel fits the shape, and in float32
    mode, the product is followed by the row-wise kernel)."""

    def __init__(self, params, env):
        Part.__init__(self, params, env)
        self.d = int(self._p("hidden_size"))
        self.ff = int(self._p("intermediate_size"))
        self.bias = bool(self._p("bias", False))
        self.limit = float(self._p("limit"))
        self.alpha = float(self._p("alpha"))
        self.shift = float(self._p("shift", 0.0))
        if not self.limit > 0:
            raise ConfigError(f"glu_clamped: limit={self.limit} must be positive")

    def forward(self, h, residual, ctx):
        act = linear_swiglu(h, self.w_gu, self.b_gu, glu=(self.limit, self.alpha, self.shift))
        linear(act, self.w_down, self.b_down, out=residual, accumulate=True)


class MixtureOfExperts(Part):
    category = "feed_forward"
    graph_safe = True          # rows meet their experts on the device; the host sees none of it

    def __init__(self, params, env):
        super().__init__(params, env)
        self.d = int(self._p("hidden_size"))
        self.ff = int(self._p("expert_size"))
        self.E = int(self._p("num_experts"))
        self.top = int(self._p("top"))
        self.activation = str(self._p("activation", "silu"))
        self.routing = str(self._p("routing", "top_logits"))
        if self.routing not in K.MOE_ROUTINGS:
            raise ConfigError(f"moe: routing='{self.routing}' (expected one of {', '.join(K.MOE_ROUTINGS)})")
        self.router_bias = bool(self._p("router_bias", self.routing == "top_logits"))
        self.correction = bool(self._p("correction", self.routing == "softmax_all"))
        self.router_scale = float(self._p("router_scale", 1.0))
        self.n_identity = int(self._p("identity_experts", 0))
        self.weight_on = str(self._p("weight_on", "output"))
        if self.weight_on not in ("output", "input"):
            raise ConfigError(f"moe: weight_on='{self.weight_on}' (expected 'output' or 'input')")
        if self.weight_on == "input" and self.n_identity:
            raise ConfigError("moe: weight_on='input' does not go with identity experts")
        self.E_all = self.E + self.n_identity                       # router outputs
        shared = self._p("shared_size", None)
        self.shared_ff = None if shared is None else int(shared)
        self.shared_gate = self._p("shared_gate", None)
        K.activation_code(self.activation)
        if self.E < 1 or self.n_identity < 0 or not (1 <= self.top <= self.E_all):
            raise ConfigError(f"moe: top={self.top} must lie between 1 and the {self.E_all} router outputs")
        if self.top > K.MOE_MAX_TOP or self.E_all > K.MOE_MAX_EXPERTS:
            raise ConfigError(f"moe: the kernels take top <= {K.MOE_MAX_TOP} and at most {K.MOE_MAX_EXPERTS} router outputs")
        if self.routing == "top_logits" and self.correction:
            raise ConfigError("moe: a correction of the choice belongs to routing='softmax_all'")
        if self.routing == "sigmoid" and (self.router_bias or self.correction):
            raise ConfigError("moe: routing='sigmoid' has neither a bias nor a correction")
        if self.routing == "softmax_all" and self.router_bias:
            raise ConfigError("moe: routing='softmax_all' has a correction of the choice, not a bias of the logits")
        if self.shared_gate not in (None, "sigmoid"):
            raise ConfigError(f"moe: shared_gate='{self.shared_gate}' (expected 'sigmoid' or none)")
        if self.shared_ff is not None and self.shared_ff < 1:
            raise ConfigError("moe: shared_size must be positive")

    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {"router.weight": WeightSpec((self.E_all, self.d))}
        if self.router_bias:
            s["router.bias"] = WeightSpec((self.E_all,), "bias")
        if self.correction:
            s["router.correction"] = WeightSpec((self.E_all,), "bias")
        if self.shared_ff is not None:
            s["shared.gate_proj.weight"] = WeightSpec((self.shared_ff, self.d))
            s["shared.up_proj.weight"] = WeightSpec((self.shared_ff, self.d))
            s["shared.down_proj.weight"] = WeightSpec((self.d, self.shared_ff))
            if self.shared_gate is not None:
                s["shared.gate.weight"] = WeightSpec((1, self.d))
        for e in range(self.E):
            s[f"experts.{e}.gate_proj.weight"] = WeightSpec((self.ff, self.d))
            s[f"experts.{e}.up_proj.weight"] = WeightSpec((self.ff, self.d))
            s[f"experts.{e}.down_proj.weight"] = WeightSpec((self.d, self.ff))
        return s

    def bind(self, w):
        # the router is 32-bit whatever the storage of the rest
        self.w_router = w["router.weight"].to(torch.float32).contiguous()
        self.b_router = w["router.bias"].to(torch.float32).contiguous() if self.router_bias else None
        if self.correction:
            self.b_router = w["router.correction"].to(torch.float32).contiguous()
        self.ws_gu = self.ws_down = self.ws_gate = None
        if self.shared_ff is not None:
            self.ws_gu = torch.cat([w["shared.gate_proj.weight"], w["shared.up_proj.weight"]], 0).contiguous()
            self.ws_down = w["shared.down_proj.weight"].contiguous()
            if self.shared_gate is not None:
                self.ws_gate = w["shared.gate.weight"].to(torch.float32).reshape(-1).contiguous()
        self.w_gu = torch.stack([torch.cat([w[f"experts.{e}.gate_proj.weight"], w[f"experts.{e}.up_proj.weight"]], 0)
                                 for e in range(self.E)]).contiguous()                       # [E, 2 ff, d]
        self.w_down = torch.stack([w[f"experts.{e}.down_proj.weight"] for e in range(self.E)]).contiguous()   # [E, d, ff]

    def forward(self, h, residual, ctx):
        n = h.shape[0]
        idx = torch.empty((n, self.top), dtype=torch.int32, device=h.device)
        weights = torch.empty((n, self.top), dtype=torch.float32, device=h.device)
        layout = torch.empty(K.moe_layout_ints(n, self.E_all, self.top), dtype=torch.int32, device=h.device)
        how = dict(routing=self.routing, scale=self.router_scale, n_identity=self.n_identity)
        if K.moe_router_ok(self.d, self.E_all) and h.stride(1) == 1:
            K.moe_router(h, self.w_router, self.b_router, self.top, idx, weights, layout, **how)
        elif self.routing == "top_logits":
            logits = linear(h, self.w_router, self.b_router, out_dtype=torch.float32)
            K.moe_route(logits, self.top, idx, weights, layout, **how)
        else:
            logits = linear(h, self.w_router, None, out_dtype=torch.float32)
            K.moe_route(logits, self.top, idx, weights, layout, bias=self.b_router, **how)
        K.moe_experts(h, self.w_gu, self.w_down, layout, weights, self.top, residual, self.activation,
                      n_identity=self.n_identity, idx=idx, weight_input=self.weight_on == "input")
        if self.ws_gu is not None:
            act = linear_swiglu(h, self.ws_gu, None, self.activation)
            if self.ws_gate is None:
                linear(act, self.ws_down, None, out=residual, accumulate=True)
            else:
                y = linear(act, self.ws_down, None, out_dtype=torch.float32)
                K.row_gate_add(h, self.ws_gate, y, residual)


register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "glu", SwiGLU)
register_part("feed_forward", "glu_clamped", ClampedGLU)
register_part("feed_forward", "moe", MixtureOfExperts)
