"""Small Vumotar configurations that differ in every size, constant and option, and a writer of model folders whose
weights are large enough that every sublayer moves the residual (with weights of 0.02 a wrong key, a sink left out or
a window one token off would hide below the tolerances)."""
import json
import math
import os
import tempfile

import numpy as np


def _attention(heads, kv_heads, dim, vdim, window, keep_first=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if window is not None:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    return {"type": "attention", "mixer": m}


def _attention_2(heads, kv_heads, dim, vdim, coef, every, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if coef is not None:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention_2", "mixer": m}


def _latent(heads, dim, vdim, q_rank, kv_rank, window, scale=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def _layer(mixer, experts=None, top=None, ff=None, shared=None):
    if experts is None:
        return dict(mixer, mlp=None)
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    return dict(mixer, mlp=mlp)


def _model(vocab, width, layers, eps=1e-5, loop=None, max_positions=None):
    c = {"architecture": "Vumotar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if max_positions is not None:
        c["max_positions"] = max_positions
    return c


# A: every mixer; the middle layers a loop of two passes; values wider than keys in the windowed layer and narrower in
# the latent one; three kept first keys behind a window of 20; two experts of six a token; a layer without a
# feed-forward; a shared unit of another size than the experts
VUM_A = _model(211, 64, [
    _layer(_attention_2(4, 2, 16, 16, 0.7, 8), 6, 2, 40, 24),
    _layer(_attention(4, 2, 16, 24, 20, 3, 0.35), 4, 1, 48, 48),
    _layer(_latent(2, 24, 16, 20, 40, 25, 0.3), None),
    _layer(_attention(2, 1, 32, 16, 9, 1, 0.2), 6, 3, 32),
], loop=(1, 3, 2))
# B: the loop comes first and runs three times; no kept keys (the key is left out); keys wider than values; three heads
# everywhere, every query head with a key head of its own; one expert of three and no shared unit; a temperature whose
# period is no whole number
VUM_B = _model(97, 48, [
    _layer(_attention(3, 3, 24, 8, 33, None), 3, 1, 56),
    _layer(_latent(3, 8, 24, 16, 12, 7), 3, 1, 40, 16),
    _layer(_attention_2(3, 3, 24, 8, 1.5, 6.5, 0.15), 5, 2, 24),
], eps=1e-6, loop=(0, 2, 3), max_positions=400)
# C: sizes the fast kernels refuse (an odd width, odd head sizes, a vocabulary smaller than a warp, five query heads on one key head, odd
# ranks); a window of two with five kept keys (more than the window); a latent window of one; every expert chosen; a
# temperature that changes at every position
VUM_C = _model(19, 37, [
    _layer(_attention(5, 1, 8, 12, 2, 5, 0.5), 3, 3, 20, 12),
    _layer(_latent(1, 37, 12, 9, 7, 1), 2, 1, 28),
    _layer(_attention_2(5, 1, 7, 7, 0.25, 1), 4, 2, 44, 20),
], eps=1e-3)
# D: widths at which the decode products stream their weights and the prompt products run on tcgen05; head sizes 64 and
# 128 (tensor-core attention kernels) with 70 kept keys (more than a key tile) behind a window of two pages; prompts
# whose steps reach the grouped tcgen05 expert tiles; no loop
VUM_D = _model(400, 512, [
    _layer(_attention(8, 2, 64, 64, 128, 70), 8, 2, 256, 256),
    _layer(_attention_2(4, 2, 128, 128, 0.5, 64), 8, 2, 256),
    _layer(_latent(4, 64, 64, 96, 128, 100), 4, 1, 512, 128),
    _layer(_attention(4, 4, 128, 128, 40, 2, 0.05), None),
], max_positions=1024)
# E: sixteen query heads on one key head (more than the split-key kernel shares); the loop reaches the last layer and
# runs once; kept keys that fill more than a page; latent heads of 128 x 64; three experts of five
VUM_E = _model(300, 256, [
    _layer(_latent(2, 128, 64, 64, 48, 50), 5, 3, 64, 64),
    _layer(_attention(16, 1, 32, 32, 30, 20), 5, 1, 128),
    _layer(_attention_2(16, 1, 32, 48, 0.3, 32), 2, 2, 96, 32),
], loop=(1, 3, 1), max_positions=640)

# F: what may be left out is left out: mixers without masks (every earlier key is read, the sinks stay), no temperature,
# no loop, no shared unit; one layer, run twice by a loop over itself, in the middle
VUM_F = _model(64, 32, [
    _layer(_attention(2, 1, 16, 16, None), 4, 2, 16),
    _layer(_latent(2, 16, 8, 12, 20, None), 3, 1, 24),
    _layer(_attention_2(4, 4, 8, 8, None, None), None),
], loop=(1, 2, 2))

CONFIGS = {"A": (VUM_A, 3), "B": (VUM_B, 4), "C": (VUM_C, 5), "D": (VUM_D, 6), "E": (VUM_E, 7), "F": (VUM_F, 8)}


def tensor_shapes(cfg):
    d, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, d), "final.norm": (d,)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H, dim, vdim = m["heads"], m["dim"], m["vdim"]
        out.update({p + "norm1": (d,), p + "norm1b": (d,)})
        if layer["type"] == "latent_attention":
            out.update({p + "mix.dq": (m["q_rank"], d), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (H * dim, m["q_rank"]),
                        p + "mix.dkv": (m["kv_rank"], d), p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (H * dim, m["kv_rank"]),
                        p + "mix.uv": (H * vdim, m["kv_rank"]), p + "mix.sink": (H,), p + "mix.g": (H, d), p + "mix.o": (d, H * vdim)})
        else:
            G = m["kv_heads"]
            out.update({p + "mix.q": (H * dim, d), p + "mix.k": (G * dim, d), p + "mix.v": (G * vdim, d), p + "mix.o": (d, H * vdim)})
            if layer["type"] == "attention":
                out.update({p + "mix.q.norm": (dim,), p + "mix.k.norm": (dim,)})
        mlp = layer["mlp"]
        if mlp is not None:
            out.update({p + "norm2": (d,), p + "norm2b": (d,), p + "mlp.router": (mlp["router"]["experts"], d)})
            units = [(f"e{e}", mlp["expert"]["ff"]) for e in range(mlp["router"]["experts"])]
            if mlp.get("shared"):
                units.append(("shared", mlp["shared"]["ff"]))
            for name, ff in units:
                out.update({p + f"mlp.{name}.gate": (ff, d), p + f"mlp.{name}.up": (ff, d), p + f"mlp.{name}.down": (d, ff)})
    return out


def make_weights(cfg, seed):
    """name -> bfloat16 tensor.  Matrices have unit gain (std 1/sqrt(inputs)), output matrices a gain of 2, the router
    a gain of 3 (scores spread over (0, 1)), norm weights 1 +- 0.2, sinks in [-1, 2], the embedding table std 1."""
    import torch
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(".sink"):
            a = rng.uniform(-1.0, 2.0, shape)
        elif len(shape) == 1:
            a = 1.0 + rng.normal(0.0, 0.2, shape)
        elif name == "embed":
            a = rng.normal(0.0, 1.0, shape)
        else:
            gain = 2.0 if name.endswith((".o", ".down")) else (3.0 if name.endswith(".router") else 1.0)
            a = rng.normal(0.0, gain / math.sqrt(shape[1]), shape)
        out[name] = torch.from_numpy(a.astype(np.float32)).to(torch.bfloat16)
    return out


def write_model_dir(cfg, weights, d):
    from kappai_b200.weights.safetensors_io import save_safetensors

    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_safetensors(os.path.join(d, "model.safetensors"), weights)
    return d


def make_model_dir(name, root=None):
    cfg, seed = CONFIGS[name]
    return write_model_dir(cfg, make_weights(cfg, seed), tempfile.mkdtemp(prefix=f"vum_{name}_", dir=root))
