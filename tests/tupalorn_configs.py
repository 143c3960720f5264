"""Small Tupalorn configurations that differ in every size, constant and option, and a writer of model folders whose
weights are large enough that every sublayer moves the residual (with weights of 0.02 a wrong key, a lost state or a
window one token off would hide below the tolerances)."""
import json
import math
import os
import tempfile

import numpy as np


def _mamba2(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def _retention(heads, dim, vdim, decay, rot=None):
    assert len(decay) == heads
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "retention", "mixer": m}


def _attention(heads, kv_heads, dim, vdim, window, scale=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def _layer(mixer, ff, limit=1.0):
    return dict(mixer, mlp=None if ff is None else {"kind": "dense", "ff": ff, "limit": limit})


def _model(vocab, width, layers, eps=1e-5, softcap=None, max_positions=None):
    c = {"architecture": "Tupalorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if softcap is not None:
        c["logit_softcap"] = softcap
    if max_positions is not None:
        c["max_positions"] = max_positions
    return c


# A: every mixer; a rotation of a part of the head; values twice as wide as keys in the retention layer; two attention
# layers that read the cache of a third, one of them with a wider window than the lender's own; a layer without a
# feed-forward; the state space layer comes last
TUP_A = _model(211, 64, [
    _layer(_retention(2, 16, 32, [0.9, 0.995], rot=(8, 10000.0)), 96, 0.5),
    _layer(_attention(4, 2, 16, 16, 20, 0.3), 80, 0.5),
    _layer(_mamba2(4, 16, 16, 2, 3, 4), None),
    _layer(_attention(4, 2, 16, 16, 33, 0.2, kv_from=1), 96, 2.0),
    _layer(_attention(4, 2, 16, 16, 5, 0.4, kv_from=1), 64, 0.7),
    _layer(_mamba2(2, 32, 24, 1, 2, 1), 72, 1.5),
], softcap=12.0)
# B: keys wider than values (a cache head is padded); attention without a window, and a borrower of it with one;
# three heads everywhere; a full rotation; no soft cap on the logits; one group and one norm group
TUP_B = _model(97, 48, [
    _layer(_mamba2(3, 8, 24, 1, 2, 1), 72, 2.0),
    _layer(_attention(3, 3, 24, 8, None), 64, 1.0),
    _layer(_retention(3, 40, 24, [0.8, 0.97, 0.999], rot=(40, 500.0)), None),
    _layer(_attention(3, 3, 24, 8, 7, kv_from=1), 48, 0.25),
], eps=1e-6, max_positions=400)
# C: sizes the fast kernels refuse (width 36, a vocabulary smaller than a warp, a state of 5, a convolution of one
# tap, five query heads on one key head, values wider than keys); a window of two; no rotation in the retention
# layer; as many norm groups as heads
TUP_C = _model(19, 36, [
    _layer(_attention(5, 1, 8, 12, 2, 0.5), 44, 3.0),
    _layer(_mamba2(5, 4, 5, 5, 1, 5), 20, 1.0),
    _layer(_retention(1, 36, 12, [0.95]), 28, 0.8),
], eps=1e-3, softcap=5.0)
# D: widths at which the decode products stream their weights and the prompt products run on tcgen05; head size 64
# (tensor-core attention kernels) and a window of two pages; a state of 128; prompts of several chunks
TUP_D = _model(400, 512, [
    _layer(_mamba2(8, 64, 128, 1, 4, 1), 1024, 1.0),
    _layer(_retention(4, 64, 64, [0.6, 0.9, 0.99, 0.9999], rot=(32, 5.0e5)), 512, 1.0),
    _layer(_attention(8, 2, 64, 64, 128), 1024, 4.0),
    _layer(_mamba2(16, 32, 64, 4, 4, 2), 512, 1.0),
    _layer(_attention(8, 2, 64, 64, 40, 0.1, kv_from=2), 512, 1.0),
], softcap=25.0, max_positions=1024)
# E: sixteen query heads on one key head (more than the split-key kernel shares); retention heads of 128 x 64; a
# state of 200 rows (the scan keeps it, the chunked kernels do not); a convolution of eight taps
TUP_E = _model(300, 256, [
    _layer(_retention(2, 128, 64, [0.97, 1.0], rot=(64, 100.0)), 256, 1.0),
    _layer(_attention(16, 1, 32, 32, 50), 256, 1.0),
    _layer(_mamba2(4, 32, 200, 2, 8, 2), 128, 1.0),
], softcap=20.0, max_positions=640)

CONFIGS = {"A": (TUP_A, 3), "B": (TUP_B, 4), "C": (TUP_C, 5), "D": (TUP_D, 6), "E": (TUP_E, 7)}


def tensor_shapes(cfg):
    d, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, d), "final.norm": (d,)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H, vdim = m["heads"], m["vdim"]
        out[p + "norm1"] = (d,)
        if layer["type"] == "mamba2":
            inner, gn = H * vdim, m["groups"] * m["state"]
            out.update({p + "mix.in": (2 * inner + 2 * gn + H, d), p + "mix.conv": (inner + 2 * gn, m["conv"]),
                        p + "mix.conv.b": (inner + 2 * gn,), p + "mix.dt_bias": (H,), p + "mix.A_log": (H,), p + "mix.D": (H,),
                        p + "mix.norm": (inner,), p + "mix.o": (d, inner)})
        elif layer["type"] == "retention":
            dim = m["dim"]
            out.update({p + "mix.q": (H * dim, d), p + "mix.k": (H * dim, d), p + "mix.v": (H * vdim, d),
                        p + "mix.g": (H * vdim, d), p + "mix.o": (d, H * vdim)})
        else:
            dim, G = m["dim"], m["kv_heads"]
            out.update({p + "mix.q": (H * dim, d), p + "mix.q.norm": (H * dim,), p + "mix.g": (H, d), p + "mix.o": (d, H * vdim)})
            if m.get("kv_from") is None:
                out.update({p + "mix.k": (G * dim, d), p + "mix.v": (G * vdim, d), p + "mix.k.norm": (G * dim,)})
        mlp = layer["mlp"]
        if mlp is not None:
            ff = mlp["ff"]
            out.update({p + "mlp.gate": (ff, d), p + "mlp.gate.b": (ff,), p + "mlp.up": (ff, d), p + "mlp.up.b": (ff,),
                        p + "mlp.down": (d, ff), p + "mlp.down.b": (d,)})
    return out


def make_weights(cfg, seed):
    """name -> bfloat16 tensor.  Matrices have unit gain (std 1/sqrt(inputs)), output matrices a gain of 2, norm weights
    and the skip weights D 1 +- 0.2, biases std 0.3, the embedding table std 1.  The state space layers get step sizes
    and decay rates that spread the per-token decay from about 0.5 to 0.998: dt_bias in [-3, 0], A_log in [-3, 0]."""
    import torch
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("dt_bias") or name.endswith("A_log"):
            a = rng.uniform(-3.0, 0.0, shape)
        elif name.endswith(".b"):
            a = rng.normal(0.0, 0.3, shape)
        elif name.endswith("mix.conv"):
            a = rng.normal(0.0, 1.0 / math.sqrt(shape[1]), shape)
        elif len(shape) == 1:
            a = 1.0 + rng.normal(0.0, 0.2, shape)
        elif name == "embed":
            a = rng.normal(0.0, 1.0, shape)
        else:
            gain = 2.0 if name.endswith((".o", ".down")) else 1.0
            a = rng.normal(0.0, gain / math.sqrt(shape[1]), shape)
        out[name] = torch.from_numpy(a.astype(np.float32)).to(torch.bfloat16)
    return out


def make_model_dir(name, root=None):
    from kappai_b200.weights.safetensors_io import save_safetensors

    cfg, seed = CONFIGS[name]
    d = tempfile.mkdtemp(prefix=f"tup_{name}_", dir=root)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_safetensors(os.path.join(d, "model.safetensors"), make_weights(cfg, seed))
    return d
