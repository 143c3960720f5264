"""A plain, slow Tupalorn: whole sequences, no cache, one function for each mechanism.

Tupalorn is a decoder-only model of *parallel* layers: with ``h = LN(x)`` (a weighted layer norm
without a shift) both sublayers read the same ``h`` and ``x <- x + (mixer(h) + ff(h))``.  Three mixers:

* ``mamba2``: a selective state space layer.  One projection gives ``[z | x | B | C | dt]``; x, B and C pass a
  causal convolution a channel (with a bias) and silu; ``dt = softplus(dt + dt_bias)``; a head keeps a state
  ``S`` [state, vdim] with ``S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T`` and gives
  ``y_t = S_t^T C_t + D x_t``; y times silu(z) is RMS-normed in ``norm_groups`` equal parts, weighted, projected.
* ``retention``: linear attention with one constant decay a head.  q and k are rotated by position (rotate-half
  pairing over the first ``rot.dims`` dimensions), k is scaled by ``dim^-1/2``; ``S_t = a S_(t-1) + k_t v_t^T``,
  ``o_t = S_t^T q_t``; every head's o is divided by its root mean square, the heads side by side are multiplied
  by ``silu(W_g h)`` and projected.
* ``attention``: grouped-query softmax attention without positions over a sliding window, q and k RMS-normed over
  their *whole* projections (all heads at once) with a weight, scores times ``scale``, every head's output times
  one sigmoid gate a head; a layer with ``kv_from: j`` has no key/value tensors and reads layer j's keys and values.

The feed-forward: ``g = min(W_g h + b, L)``, ``u = clamp(W_u h + b, -L, L)``, ``y = g sigmoid(1.702 g) (u + 1)``,
``W_d y + b``.  Output: layer norm, the embedding table as head, ``cap * tanh(logits / cap)``.

This file shares no code with the package: it reads config.json and the safetensors file itself, with numpy
only, and runs in float64.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


def read_safetensors(path):
    """name -> numpy array (bfloat16 widened exactly; integer tables as they are)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, en = e["data_offsets"]
        raw = data[b:en]
        if e["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
        elif e["dtype"] == "F32":
            a = np.frombuffer(raw, dtype=np.float32)
        elif e["dtype"] == "I32":
            a = np.frombuffer(raw, dtype=np.int32)
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        out[name] = a.reshape(e["shape"]).copy()
    return out


# ------------------------------------------------------------------- mechanisms

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis; var is the mean of the squared deviations."""
    mu = np.mean(x, axis=-1, keepdims=True)
    d = x - mu
    return d / np.sqrt(np.mean(d * d, axis=-1, keepdims=True) + eps) * w


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def causal_conv(u, taps, bias, before=None):
    """y[t, c] = bias[c] + sum_j taps[c, j] u[t - (K - 1) + j, c]: the last tap meets the current token; rows
    before the sequence count as zero, or are ``before`` ([K - 1, channels]: the inputs that came last)."""
    T, C = u.shape
    K = taps.shape[1]
    pad = np.zeros((K - 1, C)) if before is None else np.asarray(before, dtype=np.float64)
    up = np.concatenate([pad, u], 0)
    y = np.tile(np.asarray(bias, dtype=np.float64)[None, :], (T, 1))
    for j in range(K):
        y += up[j:j + T] * taps[:, j][None, :]
    return y


def selective_scan(x, B, C, dt, A_log, D, heads, groups, state=None):
    """x [T, heads, vdim], B and C [T, groups, N], dt [T, heads] (already positive).  Returns y [T, heads, vdim]
    and the last state [heads, N, vdim].  Head h reads group h // (heads / groups)."""
    T, H, P = x.shape
    N = B.shape[2]
    S = np.zeros((H, N, P)) if state is None else np.array(state, dtype=np.float64)
    y = np.zeros((T, H, P))
    per = H // groups
    for t in range(T):
        for h in range(H):
            g = h // per
            a = math.exp(-math.exp(A_log[h]) * dt[t, h])
            S[h] = a * S[h] + dt[t, h] * np.outer(B[t, g], x[t, h])
            y[t, h] = S[h].T @ C[t, g] + D[h] * x[t, h]
    return y, S


def grouped_rms_norm(y, w, parts, eps):
    """y [T, n] cut into ``parts`` equal stretches, each divided by its own root mean square, then times w."""
    T, n = y.shape
    return (unit_rms(y.reshape(T, parts, n // parts), eps)).reshape(T, n) * w


def mamba2(h, w, m, eps):
    """The mamba2 mixer on a whole sequence h [T, width].  ``w``: the mixer's tensors by local name; ``m``: its sizes."""
    H, P, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = H * P
    T = h.shape[0]
    p = h @ w["in"].T
    z, xBC, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xBC = silu(causal_conv(xBC, w["conv"], w["conv.b"]))
    x = xBC[:, :inner].reshape(T, H, P)
    B = xBC[:, inner:inner + G * N].reshape(T, G, N)
    C = xBC[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w["dt_bias"][None, :])
    y, _ = selective_scan(x, B, C, dt, w["A_log"], w["D"], H, G)
    y = y.reshape(T, inner) * silu(z)
    return grouped_rms_norm(y, w["norm"], int(m["norm_groups"]), eps) @ w["o"].T


def rotate_half(x, first_pos, dims, base):
    """x [T, heads, dim]: dimension i < dims/2 of a head is paired with i + dims/2; the pair (u, v) at position p
    becomes (u cos a - v sin a, v cos a + u sin a), a = p base^(-2i/dims).  The other dimensions pass."""
    T = x.shape[0]
    half = dims // 2
    f = np.power(float(base), -2.0 * np.arange(half) / dims)
    a = (first_pos + np.arange(T))[:, None] * f[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def decayed_outer_scan(q, k, v, decay, state=None):
    """S_t = a_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; q, k [T, H, dim], v [T, H, vdim]; returns o and the last state."""
    T, H, dim = q.shape
    P = v.shape[2]
    S = np.zeros((H, dim, P)) if state is None else np.array(state, dtype=np.float64)
    o = np.zeros((T, H, P))
    for t in range(T):
        for h in range(H):
            S[h] = float(decay[h]) * S[h] + np.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o, S


def retention(h, w, m, eps):
    H, dim, P = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = (h @ w["q"].T).reshape(T, H, dim)
    k = (h @ w["k"].T).reshape(T, H, dim)
    v = (h @ w["v"].T).reshape(T, H, P)
    rot = m.get("rot")
    if rot:
        q = rotate_half(q, 0, int(rot["dims"]), float(rot["base"]))
        k = rotate_half(k, 0, int(rot["dims"]), float(rot["base"]))
    k = k * dim ** -0.5
    o, _ = decayed_outer_scan(q, k, v, m["decay"])
    o = unit_rms(o, eps).reshape(T, H * P)
    return (o * silu(h @ w["g"].T)) @ w["o"].T


def attention_keys_values(h, w, m, eps):
    """The keys (after their norm over the whole projection) and values of an attention layer, [T, G, dim], [T, G, vdim]."""
    G, dim, P = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    k = unit_rms(h @ w["k"].T, eps) * w["k.norm"]
    return k.reshape(T, G, dim), (h @ w["v"].T).reshape(T, G, P)


def windowed_attention(q, k, v, scale, window):
    """q [T, H, dim], k [T, G, dim], v [T, G, vdim]: row i sees j with 0 <= i - j < window (all j <= i if None)."""
    T, H, _ = q.shape
    G = k.shape[1]
    per = H // G
    o = np.zeros((T, H, v.shape[2]))
    for i in range(T):
        lo = 0 if window is None else max(0, i - int(window) + 1)
        for hh in range(H):
            g = hh // per
            s = (k[lo:i + 1, g] @ q[i, hh]) * scale
            p = np.exp(s - s.max())
            o[i, hh] = (p / p.sum()) @ v[lo:i + 1, g]
    return o


def attention(h, w, m, eps, k, v):
    """The attention mixer with given keys and values (its own, or those of the layer it borrows from)."""
    H, dim = int(m["heads"]), int(m["dim"])
    T = h.shape[0]
    q = (unit_rms(h @ w["q"].T, eps) * w["q.norm"]).reshape(T, H, dim)
    mask = m.get("mask")
    o = windowed_attention(q, k, v, float(m["scale"]), int(mask["size"]) if mask else None)
    o = o * sigmoid(h @ w["g"].T)[:, :, None]
    return o.reshape(T, -1) @ w["o"].T


def clamped_gated_unit(h, w, limit):
    g = np.minimum(h @ w["gate"].T + w["gate.b"], limit)
    u = np.clip(h @ w["up"].T + w["up.b"], -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T + w["down.b"]


def softcap(z, cap):
    return cap * np.tanh(z / cap)


class PlainTupalorn:
    def __init__(self, model_dir=None, config=None, tensors=None):
        if model_dir is not None:
            with open(os.path.join(model_dir, "config.json")) as f:
                config = json.load(f)
            tensors = read_safetensors(os.path.join(model_dir, "model.safetensors"))
        self.cfg = config
        self.w = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
        self.eps = float(config["norm"]["eps"])

    def _local(self, prefix):
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def forward(self, tokens, layers_out=None):
        """Logits [T, vocab] of a whole sequence; ``layers_out`` (a list) gets the residual after every layer."""
        cfg, w, eps = self.cfg, self.w, self.eps
        x = w["embed"][np.asarray(tokens)]
        kv = {}
        for i, L in enumerate(cfg["layers"]):
            m = L["mixer"]
            h = layer_norm(x, w[f"l{i}.norm1"], eps)
            mw = self._local(f"l{i}.mix.")
            if L["type"] == "mamba2":
                y = mamba2(h, mw, m, eps)
            elif L["type"] == "retention":
                y = retention(h, mw, m, eps)
            elif L["type"] == "attention":
                if m.get("kv_from") is not None:
                    k, v = kv[int(m["kv_from"])]
                else:
                    k, v = kv[i] = attention_keys_values(h, mw, m, eps)
                y = attention(h, mw, m, eps, k, v)
            else:
                raise ValueError(L["type"])
            if L.get("mlp") is not None:
                y = y + clamped_gated_unit(h, self._local(f"l{i}.mlp."), float(L["mlp"]["limit"]))
            x = x + y
            if layers_out is not None:
                layers_out.append(x.copy())
        z = layer_norm(x, w["final.norm"], eps) @ w["embed"].T
        cap = cfg.get("logit_softcap")
        return softcap(z, float(cap)) if cap else z
