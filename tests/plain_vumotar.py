"""A plain, slow Vumotar: whole sequences, no cache, one function for each mechanism.

Vumotar is a decoder-only model whose layers norm each sublayer on both sides,

    x <- x + N1b(mixer(N1(x))) ;  x <- x + N2b(ff(N2(x)))

with N an RMS norm with a weight.  A stretch of the layers (``loop.start .. loop.stop - 1``) runs
``loop.times`` times in a row with the same weights.  Three mixers, none with a rotation:

* *attention*: grouped-query attention, q and k RMS-normed a head, keys inside a sliding window or among the
  first ``keep_first`` positions of the sequence, a softmax whose denominator holds an extra 1;
* *attention_2*: grouped-query causal attention with plain softmax, the query of position p times
  ``1 + coef ln(floor((p + 1) / every) + 1)``;
* *latent_attention*: queries, keys and values expanded from normed low-rank latents, a sliding window, a
  softmax whose denominator holds ``exp(sink_h)`` of a learned number a head, one sigmoid gate a head.

The feed-forward is a mixture of silu units chosen by the largest ``sigmoid(router logits)``; the chosen score
multiplies the unit's *input*; a shared unit runs for every token.  The head is the embedding table.

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

def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def visible(n, window=None, keep_first=0):
    """[n, n] booleans: row i sees column j if j <= i and (no window, or i - j < window, or j < keep_first)."""
    i = np.arange(n)[:, None]
    j = np.arange(n)[None, :]
    ok = j <= i
    if window is not None:
        ok &= (i - j < window) | (j < keep_first)
    return ok


def softmax_with_sink(s, mask, sink=None):
    """Rows of ``exp(s_j) / (sum over visible j of exp(s_j) + exp(sink))``; ``sink`` None: a plain softmax.
    The sink has no value: the rows then sum to less than one."""
    s = np.where(mask, s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    if sink is not None:
        m = np.maximum(m, sink)
    e = np.where(mask, np.exp(s - m), 0.0)
    den = e.sum(axis=-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink - m)
    return e / den


def query_temperature(n, coef, every, first_pos=0):
    """1 + coef ln(floor((p + 1) / every) + 1) for the positions first_pos .. first_pos + n - 1."""
    p = first_pos + np.arange(n)
    return 1.0 + coef * np.log(np.floor((p + 1) / every) + 1.0)


def grouped_attention(q, k, v, scale, mask, sink=None):
    """q [n, H, dim], k [n, G, dim], v [n, G, vdim]; query head h reads kv head h // (H / G).
    ``sink``: None, or one number a head [H].  Returns [n, H * vdim]."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((n, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        p = softmax_with_sink(s, mask, None if sink is None else sink[h])
        out[:, h] = p @ v[:, g]
    return out.reshape(n, -1)


def mixer_mask(n, m):
    """The keys a mixer's rows see: its ``mask`` (a window, with kept first keys), or every earlier key."""
    mask = m.get("mask")
    return visible(n) if not mask else visible(n, mask["size"], mask.get("keep_first") or 0)


def windowed_sink_attention(h, w, m, eps):
    """The mixer 'attention': per-head q/k norm, window with kept first positions, one more in the denominator."""
    n = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ w["q"].T).reshape(n, H, dim), w["q.norm"], eps)
    k = rms_norm((h @ w["k"].T).reshape(n, G, dim), w["k.norm"], eps)
    v = (h @ w["v"].T).reshape(n, G, vdim)
    o = grouped_attention(q, k, v, m["scale"], mixer_mask(n, m), sink=np.zeros(H))
    return o @ w["o"].T


def tempered_attention(h, w, m):
    """The mixer 'attention_2': causal, plain softmax, queries scaled by position."""
    n = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(n, H, dim)
    if m.get("q_temp"):
        q = q * query_temperature(n, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    k = (h @ w["k"].T).reshape(n, G, dim)
    v = (h @ w["v"].T).reshape(n, G, vdim)
    o = grouped_attention(q, k, v, m["scale"], mixer_mask(n, m))
    return o @ w["o"].T


def latent_attention(h, w, m, eps):
    """The mixer 'latent_attention': latents, window, a learned sink a head, a gate a head."""
    n = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(n, H, dim)
    c = rms_norm(h @ w["dkv"].T, w["dkv.norm"], eps)
    k = (c @ w["uk"].T).reshape(n, H, dim)
    v = (c @ w["uv"].T).reshape(n, H, vdim)
    o = grouped_attention(q, k, v, m["scale"], mixer_mask(n, m), sink=w["sink"])
    gate = sigmoid(h @ w["g"].T)                                   # [n, H]
    o = (o.reshape(n, H, vdim) * gate[:, :, None]).reshape(n, -1)
    return o @ w["o"].T


def gated_unit(h, w):
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def route(h, router, top):
    """Scores sigmoid(router h); the ``top`` largest a token (the lower index wins a tie).  Returns (indices
    [n, top], weights [n, top]): the weights are the chosen scores as they are."""
    s = sigmoid(h @ router.T)
    idx = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return idx, np.take_along_axis(s, idx, axis=-1)


def choice_margin(h, router, top):
    """The gap, row by row, between the last chosen router logit and the first one left out (inf if all are chosen)."""
    z = np.sort(h @ router.T, axis=-1)[:, ::-1]
    return z[:, top - 1] - z[:, top] if top < z.shape[1] else np.full(len(h), np.inf)


def mixture(h, w, mlp, margins=None):
    """sum over the chosen experts of expert(weight * h), plus the shared unit.  ``margins`` (a list) gets the rows'
    choice margins."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    idx, wt = route(h, w["router"], top)
    if margins is not None:
        margins.append(choice_margin(h, w["router"], top))
    out = np.zeros_like(h)
    for e in range(E):
        rows, col = np.nonzero(idx == e)
        if len(rows):
            out[rows] += gated_unit(wt[rows, col][:, None] * h[rows], {k: w[f"e{e}.{k}"] for k in ("gate", "up", "down")})
    if mlp.get("shared"):
        out += gated_unit(h, {k: w[f"shared.{k}"] for k in ("gate", "up", "down")})
    return out


# ------------------------------------------------------------------- the model

def sub(weights, prefix):
    return {k[len(prefix):]: v.astype(np.float64) for k, v in weights.items() if k.startswith(prefix)}


def layer_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, t = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * t + list(range(b, n))


def forward(cfg, weights, tokens, return_layers=False, margins=None):
    """Logits [n, vocab] of a whole sequence (float64); with ``return_layers`` also the residual after every
    layer run [runs, n, width]; ``margins`` (a list) gets every mixture run's choice margins [n]."""
    eps = cfg["norm"]["eps"]
    E = weights["embed"].astype(np.float64)
    x = E[np.asarray(tokens)]
    after = []
    for i in layer_order(cfg):
        L = cfg["layers"][i]
        p = f"l{i}."
        g = lambda name: weights[p + name].astype(np.float64)
        h = rms_norm(x, g("norm1"), eps)
        mw = sub(weights, p + "mix.")
        if L["type"] == "attention":
            y = windowed_sink_attention(h, mw, L["mixer"], eps)
        elif L["type"] == "attention_2":
            y = tempered_attention(h, mw, L["mixer"])
        elif L["type"] == "latent_attention":
            y = latent_attention(h, mw, L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + rms_norm(y, g("norm1b"), eps)
        if L.get("mlp") is not None:
            h = rms_norm(x, g("norm2"), eps)
            x = x + rms_norm(mixture(h, sub(weights, p + "mlp."), L["mlp"], margins), g("norm2b"), eps)
        after.append(x.copy())
    logits = rms_norm(x, weights["final.norm"].astype(np.float64), eps) @ E.T
    return (logits, np.stack(after)) if return_layers else logits


def load(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


class PlainVumotar:
    """A model folder (or a configuration and tensors) with the whole-sequence forward pass above."""

    def __init__(self, model_dir=None, config=None, tensors=None):
        if model_dir is not None:
            self.cfg, self.w = load(model_dir)
        else:
            self.cfg, self.w = config, tensors

    def forward(self, tokens, layers_out=None, margins=None):
        """Logits [n, vocab]; the residual after every layer run is appended to ``layers_out`` if it is a list, every
        mixture run's choice margins [n] to ``margins`` if it is one."""
        logits, after = forward(self.cfg, self.w, tokens, True, margins)
        if layers_out is not None:
            layers_out.extend(after)
        return logits

    def logits(self, tokens):
        return self.forward(tokens)
