"""Tupalorn: a decoder of parallel layers with three kinds of mixer.

    x = embed[token]
    a layer:   h = LN(x) ;  x <- (x + mixer(h)) + ff(h)        (one weighted layer norm without a shift; both sublayers read h)
    output:    logits = c tanh((embed . LN(x)) / c)            (the embedding table is the head; c = logit_softcap)

The mixers: ``mamba2`` (a selective state space layer: a short convolution over [x | B | C], softplus step sizes, a
float32 state a head, a silu gate in front of a grouped RMS norm; parts/ssm.py), ``retention`` (linear attention
with one constant decay a head: q and k rotated by position in "rotate half" pairs, k times ``dim^-1/2`` behind the
rotation, every head's output divided by its own root mean square, the heads times ``silu(h Wg^T)``; it is the
``lightning`` mixer with those parameters, parts/lightning.py) and ``attention`` (grouped-query softmax attention
without positions over a sliding window, q and k RMS-normed over their whole projections, one sigmoid gate a head;
parts/attention.py).  An attention layer with ``kv_from: j`` has no key and value tensors: its queries read the
keys and values that layer j's cache holds.  The feed-forward is a gated unit with limits,
``a sigmoid(1.702 a) (b + 1)`` with ``a = min(gate, limit)`` and ``b = clamp(up, -limit, limit)``; its three matrices
have biases.

This file is the only place that knows the design's ``config.json`` keys and tensor names.  The layers are listed
in ``layers``, each with its ``type`` (the mixer), the mixer's sizes (``mixer``) and its feed-forward (``mlp``, or
nothing where a layer has none); the tensors of layer i are named ``l<i>.*``.  Every size and constant is read from there; what the
design fixes (activations, the kinds of gates and norms, the constants of the gated unit) is written below.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from ..config.schema import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TypedConfig, cfg
from ..config.registry import register_architecture

ARCHITECTURE = "Tupalorn"
GLU_ALPHA = 1.702                  # the gated unit: a sigmoid(GLU_ALPHA a) (b + GLU_SHIFT)
GLU_SHIFT = 1.0
SOFTMAX_WEIGHTS = "float32"        # scores and weights are 32-bit, also where they meet the values
DEFAULT_MAX_POSITIONS = 131072     # the design itself sets no limit; an optional key ``max_positions`` overrides


def _get(d: Any, key: str, where: str, typ=(int, float)):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: missing required key '{where}.{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, typ):
        raise ConfigError(f"config key '{where}.{key}': unexpected value {v!r}")
    return v


def _int(d, key, where, least: int = 1) -> int:
    v = _get(d, key, where)
    if int(v) != v or int(v) < least:
        raise ConfigError(f"config key '{where}.{key}': expected an integer of at least {least}, got {v!r}")
    return int(v)


@dataclass
class TupalornConfig(TypedConfig):
    vocab: int = cfg()
    width: int = cfg()
    layers: List[dict] = cfg()
    norm: dict = cfg()
    logit_softcap: Optional[float] = cfg(None)
    max_positions: int = cfg(DEFAULT_MAX_POSITIONS)
    eos_token_id: Optional[int] = cfg(None)

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1:
            raise ConfigError("vocab and width must be positive")
        if not self.layers:
            raise ConfigError("layers must list at least one layer")
        if self.max_positions < 1:
            raise ConfigError("max_positions must be positive")
        self.eps = float(_get(self.norm, "eps", "norm"))
        if self.eps <= 0:
            raise ConfigError("norm.eps must be positive")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError("logit_softcap must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"config key '{where}': expected an object")
            kind = _get(layer, "type", where, str)
            m, mw = layer.get("mixer"), where + ".mixer"
            H = _int(m, "heads", mw)
            _int(m, "vdim", mw)
            if kind == "mamba2":
                _int(m, "state", mw), _int(m, "conv", mw)
                G, ng = _int(m, "groups", mw), _int(m, "norm_groups", mw)
                if H % G:
                    raise ConfigError(f"{mw}: heads={H} must be a multiple of groups={G}")
                if (H * int(m["vdim"])) % ng:
                    raise ConfigError(f"{mw}: norm_groups={ng} must divide heads * vdim")
            elif kind == "retention":
                dim = _int(m, "dim", mw)
                decay = _get(m, "decay", mw, list)
                if len(decay) != H or any(isinstance(a, bool) or not isinstance(a, (int, float)) for a in decay):
                    raise ConfigError(f"{mw}.decay must list one number for each of the {H} heads")
                rot = m.get("rot")
                if rot:
                    dims = _int(rot, "dims", mw + ".rot")
                    _get(rot, "base", mw + ".rot")
                    if dims < 2 or dims % 2 or dims > dim:
                        raise ConfigError(f"{mw}.rot.dims={dims} must be even and at most dim={dim}")
            elif kind == "attention":
                _int(m, "dim", mw)
                G = _int(m, "kv_heads", mw)
                _get(m, "scale", mw)
                if H % G:
                    raise ConfigError(f"{mw}: heads={H} must be a multiple of kv_heads={G}")
                if m.get("mask"):
                    _int(m["mask"], "size", mw + ".mask")
                if m.get("kv_from") is not None:
                    j = _int(m, "kv_from", mw, 0)
                    lender = self.layers[j] if j < i and isinstance(self.layers[j], dict) else None
                    lm = lender.get("mixer") if lender else None
                    if lender is None or lender.get("type") != "attention" or not isinstance(lm, dict) or lm.get("kv_from") is not None:
                        raise ConfigError(f"{mw}.kv_from={j} must name an earlier attention layer with keys and values of its own")
                    for k in ("kv_heads", "dim", "vdim"):
                        if lm.get(k) != m.get(k):
                            raise ConfigError(f"{mw}: {k}={m.get(k)} differs from layer {j}'s {lm.get(k)}, whose keys and values it reads")
            else:
                raise ConfigError(f"config key '{where}.type'='{kind}': expected 'mamba2', 'retention' or 'attention'")
            mlp = layer.get("mlp")
            if mlp is not None:
                mk = _get(mlp, "kind", where + ".mlp", str)
                if mk != "dense":
                    raise ConfigError(f"config key '{where}.mlp.kind'='{mk}': this design has 'dense' feed-forwards only")
                _int(mlp, "ff", where + ".mlp")
                if not float(_get(mlp, "limit", where + ".mlp")) > 0:
                    raise ConfigError(f"{where}.mlp.limit must be positive")


def _window(m: Dict[str, Any]) -> Optional[int]:
    return int(m["mask"]["size"]) if m.get("mask") else None


def _cache_window(c: TupalornConfig, i: int) -> Optional[int]:
    """How far back layer i's cache must keep keys: its own window, or a wider one of a layer that reads its cache
    (None: everything)."""
    windows = [_window(c.layers[i]["mixer"])]
    for layer in c.layers[i + 1:]:
        if layer["type"] == "attention" and layer["mixer"].get("kv_from") == i:
            windows.append(_window(layer["mixer"]))
    return None if any(w is None for w in windows) else max(windows)


def _mixer_spec(c: TupalornConfig, i: int, prefix: str) -> PartSpec:
    layer = c.layers[i]
    m, kind = layer["mixer"], layer["type"]
    if kind == "mamba2":
        return PartSpec(
            "mamba2",
            {"hidden_size": c.width, "num_heads": int(m["heads"]), "head_dim": int(m["vdim"]), "state_size": int(m["state"]),
             "groups": int(m["groups"]), "conv_kernel": int(m["conv"]), "norm_groups": int(m["norm_groups"]), "norm_eps": c.eps},
            prefix,
            rename={"in_proj.weight": "in", "conv.weight": "conv", "conv.bias": "conv.b", "norm.weight": "norm",
                    "out_proj.weight": "o"})
    if kind == "retention":
        rot = m.get("rot")
        position = None
        if rot:
            position = PartSpec("rope", {"rotary_dim": int(rot["dims"]), "theta": float(rot["base"]), "pairing": "neox"})
        return PartSpec(
            "lightning",
            {"hidden_size": c.width, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]),
             "decay": [float(a) for a in m["decay"]], "norm_eps": c.eps, "activation": None, "gate": "silu",
             "norm": "per_head", "position": position, "k_scale": float(int(m["dim"])) ** -0.5},
            prefix,
            rename={"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "gate_proj.weight": "g",
                    "out_proj.weight": "o"})
    borrowed = m.get("kv_from") is not None
    return PartSpec(
        "attention",
        {"hidden_size": c.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]), "head_dim": int(m["dim"]),
         "value_dim": int(m["vdim"]), "scale": float(m["scale"]), "qk_norm": "projection", "qk_norm_eps": c.eps,
         "window": _window(m), "cache_window": _cache_window(c, int(m["kv_from"]) if borrowed else i),
         "kv": "borrowed" if borrowed else "own", "gate": "head_sigmoid", "softmax_weights": SOFTMAX_WEIGHTS,
         "position": None, "bias": False},
        prefix,
        rename={"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "q_norm.weight": "q.norm",
                "k_norm.weight": "k.norm", "gate_proj.weight": "g", "out_proj.weight": "o"})


def _ffn_spec(c: TupalornConfig, mlp: Optional[Dict[str, Any]], prefix: str) -> Optional[PartSpec]:
    if mlp is None:
        return None
    return PartSpec("glu_clamped", {"hidden_size": c.width, "intermediate_size": int(mlp["ff"]), "bias": True,
                                    "limit": float(mlp["limit"]), "alpha": GLU_ALPHA, "shift": GLU_SHIFT},
                    prefix, rename={"gate_proj.weight": "gate", "gate_proj.bias": "gate.b", "up_proj.weight": "up",
                                    "up_proj.bias": "up.b", "down_proj.weight": "down", "down_proj.bias": "down.b"})


def build_spec(c: TupalornConfig) -> ModelSpec:
    norm = lambda prefix, name: PartSpec("layernorm", {"size": c.width, "eps": c.eps}, prefix, rename={"weight": name})
    layers, schedule = [], []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        layers.append(LayerSpec(mixer=_mixer_spec(c, i, p + "mix."), ffn=_ffn_spec(c, layer.get("mlp"), p + "mlp."),
                                mixer_norm=norm(p, "norm1"), ffn_norm=None, block="parallel_residual"))
        kv_from = layer["mixer"].get("kv_from") if layer["type"] == "attention" else None
        # (every layer runs once and in order, so a layer's number is its schedule entry's)
        schedule.append(ScheduleEntry(i, cache_of=None if kv_from is None else int(kv_from)))
    spec = ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=c.width,
        vocab_size=c.vocab,
        max_positions=c.max_positions,
        embedding=PartSpec("embedding", {"vocab_size": c.vocab, "hidden_size": c.width, "scale": None}, "",
                           rename={"weight": "embed"}),
        layers=layers,
        schedule=schedule,
        final_norm=norm("", "final.norm"),
        head=PartSpec("lm_head", {"vocab_size": c.vocab, "hidden_size": c.width, "tied": True,
                                  "softcap": c.logit_softcap}, ""),
        eos_token_id=c.eos_token_id,
    )
    spec.validate()
    return spec


register_architecture(ARCHITECTURE, TupalornConfig, build_spec)
