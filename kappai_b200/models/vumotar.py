"""Vumotar: a decoder whose layers norm every sublayer on both sides, with three kinds of attention without a
rotation and mixtures of experts whose weights scale the experts' inputs.

    x = embed[token]
    a layer:   x <- x + norm1b(mixer(norm1(x))) ;  x <- x + norm2b(ff(norm2(x)))          (RMS norms with weights)
    a loop:    layers loop.start .. loop.stop - 1 run loop.times times in a row with the same weights, every pass
               with caches of its own; nothing else happens between the passes
    output:    logits = embed . norm(x)                                                    (the table is the head)

The mixers (parts/attention.py): ``attention`` (grouped-query heads, q and k RMS-normed a head with one shared
weight, a sliding window that also keeps the first ``mask.keep_first`` keys of the sequence visible, a softmax with
one more in its denominator), ``attention_2`` (grouped-query heads, causal, plain softmax, the query of position p
times ``1 + q_temp.coef ln(floor((p + 1) / q_temp.every) + 1)``) and ``latent_attention`` (queries, keys and values
expanded from RMS-normed low-rank latents, a sliding window, a softmax whose denominator also holds ``exp(sink_h)``
of a learned number a head, one sigmoid gate a head in front of the output matrix).  No mixer has a position
encoding; every one has its own ``scale`` on the scores.  The feed-forward (parts/ffn.py) is a mixture of silu
units: scores ``sigmoid(W_router h)`` in float32, the ``top`` largest chosen, the chosen scores themselves as
weights (not renormalised), each weight multiplying its unit's *input*, and a shared unit of the same form that
every token runs.

This file is the only place that knows the design's ``config.json`` keys and tensor names.  ``layers`` lists the
layers, each with its ``type`` (the mixer), the mixer's sizes (``mixer``) and its feed-forward (``mlp``, or null
for none); layer i's tensors start with ``l<i>.``.  Every size and constant is read from there; what the design
fixes (the activation, the kinds of sink and gate, the place of the norms, the tied head) is written below.
``loop``, ``mask.keep_first`` and an ``mlp``'s ``shared`` may be left out; a mixer without ``mask`` reads every
earlier key, one without ``q_temp`` has no temperature.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from ..config.schema import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TypedConfig, cfg
from ..config.registry import register_architecture

ARCHITECTURE = "Vumotar"
EXPERT_ACTIVATION = "silu"
SOFTMAX_WEIGHTS = "float32"        # scores and weights are 32-bit, also where they meet the values
DEFAULT_MAX_POSITIONS = 131072     # the design itself sets no limit; an optional key ``max_positions`` overrides
MIXERS = ("attention", "attention_2", "latent_attention")


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
class VumotarConfig(TypedConfig):
    vocab: int = cfg()
    width: int = cfg()
    layers: List[dict] = cfg()
    norm: dict = cfg()
    loop: Optional[dict] = cfg(None)
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
        n = len(self.layers)
        if self.loop is not None:
            a, b = _int(self.loop, "start", "loop", 0), _int(self.loop, "stop", "loop", 0)
            _int(self.loop, "times", "loop")
            if not (0 <= a < b <= n):
                raise ConfigError(f"loop: start={a}, stop={b} must name a stretch of the {n} layers")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"config key '{where}': expected an object")
            kind = _get(layer, "type", where, str)
            if kind not in MIXERS:
                raise ConfigError(f"config key '{where}.type'='{kind}': expected one of {', '.join(MIXERS)}")
            m, mw = layer.get("mixer"), where + ".mixer"
            H = _int(m, "heads", mw)
            _int(m, "dim", mw), _int(m, "vdim", mw)
            _get(m, "scale", mw)
            if m.get("mask") is not None:
                _int(m["mask"], "size", mw + ".mask")
                if m["mask"].get("keep_first") is not None:
                    _int(m["mask"], "keep_first", mw + ".mask", 0)
            if kind == "latent_attention":
                _int(m, "q_rank", mw), _int(m, "kv_rank", mw)
            else:
                G = _int(m, "kv_heads", mw)
                if H % G:
                    raise ConfigError(f"{mw}: heads={H} must be a multiple of kv_heads={G}")
            if m.get("q_temp") is not None:
                qt, qw = m["q_temp"], mw + ".q_temp"
                _get(qt, "coef", qw)
                if not float(_get(qt, "every", qw)) > 0:
                    raise ConfigError(f"{qw}.every must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                mk = _get(mlp, "kind", where + ".mlp", str)
                if mk != "moe":
                    raise ConfigError(f"config key '{where}.mlp.kind'='{mk}': this design has 'moe' feed-forwards only")
                _int(mlp.get("expert"), "ff", where + ".mlp.expert")
                r, rw = mlp.get("router"), where + ".mlp.router"
                E, top = _int(r, "experts", rw), _int(r, "top", rw)
                if top > E:
                    raise ConfigError(f"{rw}: top={top} exceeds the {E} experts")
                if mlp.get("shared"):
                    _int(mlp["shared"], "ff", where + ".mlp.shared")


def _mask(m: Dict[str, Any]):
    """(window, kept first keys) of a mixer; (None, 0) where it has no mask: every earlier key is read."""
    mask = m.get("mask")
    return (None, 0) if mask is None else (int(mask["size"]), int(mask.get("keep_first") or 0))


def _mixer_spec(c: VumotarConfig, layer: Dict[str, Any], prefix: str) -> PartSpec:
    m, kind = layer["mixer"], layer["type"]
    window, keep = _mask(m)
    common = {"hidden_size": c.width, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]),
              "scale": float(m["scale"]), "softmax_weights": SOFTMAX_WEIGHTS}
    if kind == "latent_attention":
        return PartSpec(
            "latent_attention",
            dict(common, q_rank=int(m["q_rank"]), kv_rank=int(m["kv_rank"]), norm_eps=c.eps, gate="head_sigmoid",
                 window=window, keep_first=keep, sink="learned"),
            prefix,
            rename={"q_down.weight": "dq", "q_norm.weight": "dq.norm", "q_up.weight": "uq", "kv_down.weight": "dkv",
                    "kv_norm.weight": "dkv.norm", "k_up.weight": "uk", "v_up.weight": "uv", "gate_proj.weight": "g",
                    "out_proj.weight": "o", "sink": "sink"})
    rename = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "out_proj.weight": "o"}
    common.update(num_kv_heads=int(m["kv_heads"]), position=None, bias=False)
    if kind == "attention":
        rename.update({"q_norm.weight": "q.norm", "k_norm.weight": "k.norm"})
        return PartSpec(
            "attention",
            dict(common, qk_norm="per_head", qk_norm_eps=c.eps, window=window, keep_first=keep, sink="zero"),
            prefix, rename=rename)
    qt = m.get("q_temp")
    return PartSpec("attention", dict(common, qk_norm_eps=None, window=window, keep_first=keep,
                                      q_temp=None if qt is None else {"coef": float(qt["coef"]), "every": float(qt["every"])}),
                    prefix, rename=rename)


def _ffn_spec(c: VumotarConfig, mlp: Optional[Dict[str, Any]], prefix: str) -> Optional[PartSpec]:
    if mlp is None:
        return None
    r = mlp["router"]
    E = int(r["experts"])
    rename = {"router.weight": "router"}
    for e in range(E):
        for local, name in (("gate_proj", "gate"), ("up_proj", "up"), ("down_proj", "down")):
            rename[f"experts.{e}.{local}.weight"] = f"e{e}.{name}"
    params = {"hidden_size": c.width, "expert_size": int(mlp["expert"]["ff"]), "num_experts": E, "top": int(r["top"]),
              "activation": EXPERT_ACTIVATION, "routing": "sigmoid", "weight_on": "input"}
    if mlp.get("shared"):
        params.update(shared_size=int(mlp["shared"]["ff"]), shared_gate=None)
        rename.update({"shared.gate_proj.weight": "shared.gate", "shared.up_proj.weight": "shared.up",
                       "shared.down_proj.weight": "shared.down"})
    return PartSpec("moe", params, prefix, rename=rename)


def layer_schedule(c: VumotarConfig) -> List[ScheduleEntry]:
    """The order in which the layers run: the looped stretch ``times`` times (the same weights, a cache a run)."""
    n = len(c.layers)
    if c.loop is None:
        return [ScheduleEntry(i) for i in range(n)]
    a, b, times = int(c.loop["start"]), int(c.loop["stop"]), int(c.loop["times"])
    return [ScheduleEntry(i) for i in list(range(a)) + list(range(a, b)) * times + list(range(b, n))]


def build_spec(c: VumotarConfig) -> ModelSpec:
    norm = lambda prefix, name: PartSpec("rmsnorm", {"size": c.width, "eps": c.eps}, prefix, rename={"weight": name})
    layers, ignored = [], []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        ffn = _ffn_spec(c, layer.get("mlp"), p + "mlp.")
        if ffn is None:
            ignored += [p + "norm2", p + "norm2b"]       # norms of a feed-forward that the layer does not have
        layers.append(LayerSpec(mixer=_mixer_spec(c, layer, p + "mix."), ffn=ffn, mixer_norm=norm(p, "norm1"),
                                ffn_norm=norm(p, "norm2") if ffn is not None else None,
                                mixer_post_norm=norm(p, "norm1b"),
                                ffn_post_norm=norm(p, "norm2b") if ffn is not None else None,
                                block="sandwich_residual"))
    spec = ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=c.width,
        vocab_size=c.vocab,
        max_positions=c.max_positions,
        embedding=PartSpec("embedding", {"vocab_size": c.vocab, "hidden_size": c.width, "scale": None}, "",
                           rename={"weight": "embed"}),
        layers=layers,
        schedule=layer_schedule(c),
        final_norm=norm("", "final.norm"),
        head=PartSpec("lm_head", {"vocab_size": c.vocab, "hidden_size": c.width, "tied": True}, ""),
        eos_token_id=c.eos_token_id,
        ignored_tensors=ignored,
    )
    spec.validate()
    return spec


register_architecture(ARCHITECTURE, VumotarConfig, build_spec)
