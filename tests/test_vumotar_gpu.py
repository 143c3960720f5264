"""Vumotar on the GPU: every new mechanism's kernel against the plain functions, the mixers, the mixture and the
layer arrangement as parts in batches cut in two, then whole models through the step function, the trace runner and
the engine in every way of cutting the work."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_vumotar as P
import replay_util as R
from test_kernels_gpu import i32, paged_setup, rt
from tolerances import tol_for
from vumotar_configs import CONFIGS, make_model_dir, make_weights, write_model_dir

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=torch.float32).to(DEV).to(dtype).contiguous()


def host(t):
    return t.detach().double().cpu().numpy()


def close(got, want, dtype, tol16=0.02, tol32=3e-5):
    tol = tol32 if dtype == torch.float32 else tol16
    err = np.abs(got - want).max() / max(1.0, np.abs(want).max())
    assert err <= tol, err


@pytest.fixture(scope="module")
def vum_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("vumotar")
    return {n: make_model_dir(n, str(root)) for n in CONFIGS}


@pytest.fixture(scope="module")
def vum_plain(vum_dirs):
    return {n: P.PlainVumotar(d) for n, d in vum_dirs.items()}


# ------------------------------------------------------------------------------------- the attention kernels

def _plain_rows(qs, ks, vs, scale, window, keep, sink):
    """Whole-sequence attention of one request: q [L, H, hd], k and v [L, G, hd] -> [L, H, hd]."""
    L, H, hd = qs.shape
    return P.grouped_attention(qs, ks, vs, scale, P.visible(L, window, keep), sink).reshape(L, H, hd)


def _release_the_hole(bt, seq_lens, page, window, keep):
    """The block tables as the cache manager leaves them when every request stands at its last position: pages behind
    the window are gone, those of the kept first keys are not."""
    bt = bt.copy()
    for i, L in enumerate(seq_lens):
        first_needed = L - 1 - window + 1
        for b in range(-(-keep // page), max(0, first_needed) // page):
            bt[i, b] = -1
    return bt


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,hd,page,window,keep,sink", [
    (4, 2, 16, 16, 20, 3, "zero"), (5, 1, 48, 32, 2, 5, "learned"), (6, 3, 112, 8, 50, 7, "zero"), (8, 2, 64, 64, 128, 70, "zero"),
    (4, 4, 128, 16, 40, 2, "learned"), (2, 2, 64, 8, 300, 9, None), (3, 3, 32, 16, 7, 0, "learned"), (8, 1, 64, 32, 33, 300, "zero"),
    (16, 1, 32, 16, 30, 20, "zero"), (4, 2, 64, 16, None, 0, "learned")])
def test_decoded_rows_with_kept_first_keys_and_sinks(dtype, H, G, hd, page, window, keep, sink):
    """The last row of requests whose lengths put the window's edge and the kept keys on both sides of page, tile and
    chunk borders, through the split-key kernel (where it takes the shape) and the general kernel, over block tables
    whose pages between the kept keys and the window are released."""
    from kappai_b200.ops import kernels as Kn
    rng = np.random.default_rng(H + hd + (window or 0))
    seq_lens = [1, 4, keep + 1 if keep else 2, (window or 50) + keep, (window or 50) + keep + 1, 255, 256, 257, 700, 513]
    cache, bt, ks, vs = paged_setup(rng, seq_lens, page, G, hd, dtype)
    if window:
        bt = _release_the_hole(bt, seq_lens, page, window, keep)
    scale = 1.0 / math.sqrt(hd)
    sk = None if sink is None else (np.zeros(H) if sink == "zero" else rt(rng.uniform(-1, 3, H), torch.float32))
    qs = [rt(rng.standard_normal((L, H, hd)), dtype) for L in seq_lens]
    pos = [L - 1 for L in seq_lens]
    row_seg = list(range(len(seq_lens)))
    q_rows = np.stack([qs[s][p] for s, p in zip(row_seg, pos)]).reshape(len(pos), H * hd)
    want = np.stack([_plain_rows(qs[s], ks[s], vs[s], scale, window, keep, sk)[-1] for s in row_seg])
    sink_t = None if sk is None else dev(sk)
    args = (dev(q_rows, dtype), dev(cache, dtype), i32(bt), i32(row_seg), i32(pos))
    gen = torch.empty((len(pos), H * hd), dtype=dtype, device=DEV)
    Kn.attention_rows(*args, gen, scale, window, page, H, G, hd, keep_first=keep, sink=sink_t)
    close(host(gen).reshape(want.shape), want, dtype)
    if H // G <= Kn.SPLIT_MAX_RATIO and hd % 16 == 0:
        for n_chunks in (-(-max(seq_lens) // Kn.SPLIT_CHUNK), 7):
            ws = torch.full((Kn.attention_split_scratch(len(pos), H, hd, n_chunks, keep),), float("nan"), device=DEV)
            out = torch.empty_like(gen)
            Kn.attention_split(*args, out, ws, n_chunks, scale, window, page, H, G, hd, exact_weights=True, keep_first=keep, sink=sink_t)
            close(host(out).reshape(want.shape), want, dtype)


@pytest.mark.parametrize("H,G,hd,page,window,keep,sink", [
    (8, 2, 64, 64, 128, 70, "zero"), (4, 4, 128, 16, 40, 2, "learned"), (2, 2, 64, 8, 300, 9, None), (8, 1, 64, 32, 33, 300, "zero"),
    (4, 2, 64, 16, None, 0, "learned"), (6, 3, 128, 32, 100, 64, "zero"), (4, 1, 64, 16, 64, 65, "learned")])
def test_prompt_portions_with_kept_first_keys_and_sinks(H, G, hd, page, window, keep, sink):
    """The tensor-core prompt kernel over whole prompts and late portions (their first rows in the middle of a tile, their
    windows' edges inside key tiles, kept keys that fill more than a key tile), against whole-sequence attention and
    against the general kernel."""
    from kappai_b200.ops import kernels as Kn
    DT = torch.bfloat16
    rng = np.random.default_rng(hd + (window or 1) + keep)
    seq_lens, q_from = [130, 700, 257, 64, 420], [0, 391, 255, 1, 70]
    cache, bt, ks, vs = paged_setup(rng, seq_lens, page, G, hd, DT)
    scale = 1.0 / math.sqrt(hd)
    sk = None if sink is None else (np.zeros(H) if sink == "zero" else rt(rng.uniform(-1, 3, H), torch.float32))
    qs = [rt(rng.standard_normal((L, H, hd)), DT) for L in seq_lens]
    rows, cu, seg_pos, tile_seg, tile_row0, row_seg, positions = [], [0], [], [], [], [], []
    for i, (L, a) in enumerate(zip(seq_lens, q_from)):
        rows.append(qs[i][a:])
        for r0 in range(cu[-1], cu[-1] + L - a, Kn.PREFILL_TILE):
            tile_seg.append(i)
            tile_row0.append(r0)
        cu.append(cu[-1] + L - a)
        seg_pos.append(a)
        row_seg += [i] * (L - a)
        positions += list(range(a, L))
    q_rows = np.concatenate(rows, 0).reshape(cu[-1], H * hd)
    want = np.concatenate([_plain_rows(qs[i], ks[i], vs[i], scale, window, keep, sk)[a:] for i, a in enumerate(q_from)], 0)
    sink_t = None if sk is None else dev(sk)
    out = torch.empty((cu[-1], H * hd), dtype=DT, device=DEV)
    Kn.attention_prefill(dev(q_rows, DT), dev(cache, DT), i32(bt), i32(cu), i32(seg_pos), i32(tile_seg), i32(tile_row0), out, scale,
                         window, page, H, G, hd, exact_weights=True, keep_first=keep, sink=sink_t)
    close(host(out).reshape(want.shape), want, DT)
    assert Kn.attention_mma_status() == 0
    gen = torch.empty_like(out)
    Kn.attention_rows(dev(q_rows, DT), dev(cache, DT), i32(bt), i32(row_seg), i32(positions), gen, scale, window, page, H, G, hd,
                      keep_first=keep, sink=sink_t)
    assert (gen.float() - out.float()).abs().max().item() <= 2.5e-2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["kept", "just_outside", "sink"])
def test_one_score_stands_out(which, dtype):
    """Among 600 keys one has a score 12 above the rest: a kept first key far behind the window (the output is its
    value), the key just outside the window (it must not count), or the sink (the output is almost nothing).  Decoded
    row and prompt portion."""
    from kappai_b200.ops import kernels as Kn
    H, G, hd, page, window, keep, L = 4, 2, 64, 16, 100, 4, 600
    rng = np.random.default_rng(5)
    cache, bt, ks, vs = paged_setup(rng, [L], page, G, hd, dtype)
    q = rt(rng.standard_normal((L, H, hd)) * 0.1, dtype)
    sk = np.zeros(H)
    target = {"kept": 2, "just_outside": L - 1 - window, "sink": None}[which]
    if target is not None:
        # the last row's query points at the target key
        q[-1] = rt(np.repeat(ks[0][target], H // G, axis=0) * (12.0 / (ks[0][target] ** 2).sum(-1)).repeat(H // G)[:, None], dtype)
    else:
        sk = np.full(H, 12.0)
    want = _plain_rows(q, ks[0], vs[0], 1.0, window, keep, sk)[-1]
    if which == "kept":
        assert np.abs(want - np.repeat(vs[0][target], H // G, axis=0)).max() < 0.15       # the far key carries the row
    if which == "sink":
        assert np.abs(want).max() < 0.01
    qr = dev(q.reshape(L, H * hd), dtype)
    gen = torch.empty((1, H * hd), dtype=dtype, device=DEV)
    Kn.attention_rows(qr[-1:], dev(cache, dtype), i32(bt), i32([0]), i32([L - 1]), gen, 1.0, window, page, H, G, hd, keep_first=keep, sink=dev(sk))
    close(host(gen).reshape(H, hd), want, dtype)
    ws = torch.zeros(Kn.attention_split_scratch(1, H, hd, 3, keep), device=DEV)
    out = torch.empty_like(gen)
    Kn.attention_split(qr[-1:], dev(cache, dtype), i32(bt), i32([0]), i32([L - 1]), out, ws, 3, 1.0, window, page, H, G, hd,
                       exact_weights=True, keep_first=keep, sink=dev(sk))
    close(host(out).reshape(H, hd), want, dtype)
    if dtype == torch.bfloat16:
        a = L - 70
        tiles = list(range(0, 70, Kn.PREFILL_TILE))
        pre = torch.empty((70, H * hd), dtype=dtype, device=DEV)
        Kn.attention_prefill(qr[a:].contiguous(), dev(cache, dtype), i32(bt), i32([0, 70]), i32([a]), i32([0] * len(tiles)), i32(tiles), pre,
                             1.0, window, page, H, G, hd, exact_weights=True, keep_first=keep, sink=dev(sk))
        close(host(pre)[-1].reshape(H, hd), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dim,hd,page,norm,temp", [
    (4, 2, 16, 32, 16, True, None), (5, 1, 8, 16, 8, True, None), (8, 2, 64, 64, 64, True, None), (4, 2, 48, 64, 16, True, None),
    (6, 3, 48, 48, 16, False, (0.4, 50.0)), (4, 2, 64, 64, 64, False, (0.7, 8.0)), (3, 3, 24, 32, 8, False, (1.5, 6.5)),
    (2, 1, 128, 128, 32, True, (0.25, 1.0))])
def test_per_head_norm_of_padded_heads_and_query_temperature(H, G, dim, hd, page, norm, temp, dtype):
    from kappai_b200.ops import kernels as Kn
    rng = np.random.default_rng(H * hd)
    n, eps = 37, 1e-5
    pos = rng.integers(0, 400, n)
    qkv = np.zeros((n, (H + 2 * G) * hd))
    heads = qkv.reshape(n, H + 2 * G, hd)
    heads[:, :H + G, :dim] = rng.standard_normal((n, H + G, dim))            # q and k: their own columns, zeros behind
    heads[:, H + G:] = rng.standard_normal((n, G, hd))
    qkv = rt(qkv, dtype)
    heads = qkv.reshape(n, H + 2 * G, hd)
    qw, kw = rt(1 + 0.2 * rng.standard_normal(dim), torch.float32), rt(1 + 0.2 * rng.standard_normal(dim), torch.float32)
    pad = lambda w: np.concatenate([w, np.zeros(hd - dim)])
    n_pages = -(-n // page) + 1
    slots = rng.permutation(n_pages * page)[:n]
    cache = torch.zeros((n_pages, 2, G, page, hd), dtype=dtype, device=DEV)
    q_out = torch.empty((n, H * hd), dtype=dtype, device=DEV)
    Kn.qk_norm_rope_kv(dev(qkv, dtype), dev(pad(qw)) if norm else None, dev(pad(kw)) if norm else None, eps, None, None, 0, False,
                       i32(pos), i32(slots), q_out, cache, page, H, G, hd, norm_dim=dim, q_temp=temp)
    q_want = heads[:, :H, :dim].copy()
    k_want = heads[:, H:H + G, :dim].copy()
    if norm:
        q_want, k_want = P.rms_norm(q_want, qw, eps), P.rms_norm(k_want, kw, eps)
    if temp:
        q_want = q_want * (1.0 + temp[0] * np.log(np.floor((pos + 1) / temp[1]) + 1.0))[:, None, None]
    got_q = host(q_out).reshape(n, H, hd)
    close(got_q[:, :, :dim], q_want, dtype)
    assert np.all(got_q[:, :, dim:] == 0)
    c = host(cache)
    got_k = np.stack([c[s // page, 0, :, s % page] for s in slots])
    got_v = np.stack([c[s // page, 1, :, s % page] for s in slots])
    close(got_k[:, :, :dim], k_want, dtype)
    assert np.array_equal(got_v, heads[:, H + G:])


# ------------------------------------------------------------------------------------- router, experts, norms

@pytest.mark.parametrize("n,E,top,d", [(7, 6, 2, 64), (130, 8, 3, 128), (3, 3, 3, 36), (40, 4, 1, 48), (9, 40, 6, 50), (5, 12, 1, 160)])
def test_router_with_sigmoid_scores(n, E, top, d):
    """Both forms of the router (fused, and logits from a product) against the plain choice: the experts, largest score
    first, and the scores themselves as weights."""
    from kappai_b200.ops import kernels as K
    rng = np.random.default_rng(n + E)
    h = rt(rng.normal(0, 1, (n, d)), torch.bfloat16)
    wr = rt(rng.normal(0, 3 / math.sqrt(d), (E, d)), torch.bfloat16)
    idx_w, wts_w = P.route(h, wr, top)
    assert top == 1 or (wts_w.sum(1) > 1.0 + 1e-3).any()                      # not renormalised: the weights do not sum to one
    for form in ("fused", "product"):
        idx = torch.empty((n, top), dtype=torch.int32, device=DEV)
        wts = torch.empty((n, top), device=DEV)
        layout = torch.empty(K.moe_layout_ints(n, E, top), dtype=torch.int32, device=DEV)
        if form == "fused":
            if not K.moe_router_ok(d, E):
                continue
            K.moe_router(dev(h, torch.bfloat16), dev(wr), None, top, idx, wts, layout, routing="sigmoid")
        else:
            K.moe_route(dev(h @ wr.T), top, idx, wts, layout, routing="sigmoid")
        assert np.array_equal(idx.cpu().numpy(), idx_w), form
        assert np.abs(wts.cpu().numpy() - wts_w).max() <= 2e-6, form
        assert np.array_equal(np.diff(layout.cpu().numpy()[:E + 1]), np.bincount(idx_w.reshape(-1), minlength=E))


def _moe_part(d, ff, E, top, shared, dtype, rng):
    from kappai_b200.config import PartSpec
    from kappai_b200.parts import make_part
    from test_parts_gpu import bind_random, env_for
    params = {"hidden_size": d, "expert_size": ff, "num_experts": E, "top": top, "activation": "silu", "routing": "sigmoid",
              "weight_on": "input"}
    if shared:
        params.update(shared_size=shared, shared_gate=None)
    part = make_part("feed_forward", PartSpec("moe", params), env_for(dtype))
    w = bind_random(part, rng, dtype)
    part.w_router.mul_(3.0)
    plain = {"router": w["router.weight"] * 3.0}
    for e in range(E):
        for a, b in (("gate_proj", "gate"), ("up_proj", "up"), ("down_proj", "down")):
            plain[f"e{e}.{b}"] = w[f"experts.{e}.{a}.weight"]
    if shared:
        for a, b in (("gate_proj", "gate"), ("up_proj", "up"), ("down_proj", "down")):
            plain[f"shared.{b}"] = w[f"shared.{a}.weight"]
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": ff}, "shared": {"ff": shared} if shared else None}
    return part, plain, mlp


def _clear_choice(h, router, top, margin):
    z = np.sort(h @ router.T, axis=1)[:, ::-1]
    return np.full(len(h), True) if top >= z.shape[1] else (z[:, top - 1] - z[:, top] > margin)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,E,top,d,ff,shared", [(6, 6, 2, 64, 24, 40), (300, 8, 3, 128, 64, 128), (5, 3, 3, 36, 20, 28), (33, 4, 1, 48, 32, None),
                                                 (700, 4, 2, 256, 128, 64), (64, 12, 1, 160, 88, 72)])
def test_mixture_part_with_weights_on_the_inputs(n, E, top, d, ff, shared, dtype):
    """The three forms of the grouped products (CUDA cores; mma.sync tiles; tcgen05 tiles from 512 pairs on) read rows
    that were multiplied by their weights, and the outputs join unweighted."""
    rng = np.random.default_rng(n)
    part, plain, mlp = _moe_part(d, ff, E, top, shared, dtype, rng)
    h = rt(rng.normal(0, 1, (n, d)), dtype)
    ok = _clear_choice(h, plain["router"], top, 1e-5 if dtype == torch.float32 else 2e-2)
    want = P.mixture(h, plain, mlp)
    on_output = want.copy()
    idx, wt = P.route(h, plain["router"], top)
    res = torch.zeros((n, d), device=DEV)
    part.forward(dev(h, dtype), res, None)
    got = host(res)
    assert ok.sum() >= n // 2
    tol = 2e-5 if dtype == torch.float32 else 0.03
    assert np.abs(got[ok] - want[ok]).max() <= tol * max(1.0, np.abs(want).max())
    # the other reading (weights on the outputs) is far from it
    other = np.zeros_like(h)
    for e in range(E):
        r, c = np.nonzero(idx == e)
        if len(r):
            other[r] += wt[r, c][:, None] * P.gated_unit(h[r], {k: plain[f"e{e}.{k}"] for k in ("gate", "up", "down")})
    if shared:
        other += P.gated_unit(h, {k: plain[f"shared.{k}"] for k in ("gate", "up", "down")})
    if top >= 2:                                  # (the largest of many scores is all but one: it weighs little either way)
        assert np.abs(other - on_output).mean() > 5 * np.abs(got[ok] - want[ok]).mean()
    from kappai_b200.ops import kernels as K
    assert K.moe_tc_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,d", [(5, 36), (40, 64), (3, 512), (70, 4100), (9, 160)])
def test_norm_behind_a_sublayer_and_in_front_of_the_next_in_one_launch(n, d, dtype):
    from kappai_b200.ops import kernels as K
    rng = np.random.default_rng(n + d)
    y, x = rng.normal(0, 3, (n, d)), rng.normal(0, 1, (n, d))
    wb, wn = 1 + 0.2 * rng.standard_normal(d), 1 + 0.2 * rng.standard_normal(d)
    y, x, wb, wn = (rt(a, torch.float32) for a in (y, x, wb, wn))
    x_want = x + P.rms_norm(y, wb, 1e-5)
    h_want = P.rms_norm(x_want, wn, 1e-3)
    for with_next in (True, False):
        yt, xt = dev(y), dev(x)
        h = torch.empty((n, d), dtype=dtype, device=DEV) if with_next else None
        K.rmsnorm_add_norm_rows(yt, dev(wb), 1e-5, xt, dev(wn) if with_next else None, 1e-3, h)
        assert np.abs(host(xt) - x_want).max() <= 1e-5 * max(1.0, np.abs(x_want).max())
        assert torch.count_nonzero(yt).item() == 0                               # cleared for whoever adds into it next
        if with_next:
            close(host(h), h_want, dtype, tol16=0.01)


# ------------------------------------------------------------------------------------- the mixers as parts

def _bind(part, rng, dtype, sink_range=(-1.0, 3.0)):
    """As test_parts_gpu.bind_random, with sinks over a range in which they matter."""
    ws, vals = {}, {}
    for name, spec in part.weight_specs().items():
        if name == "sink":
            a = rng.uniform(*sink_range, spec.shape)
        elif spec.role == "norm":
            a = 1 + 0.2 * rng.standard_normal(spec.shape)
        else:
            a = rng.standard_normal(spec.shape) / math.sqrt(spec.shape[-1])
        store = dtype if spec.role in ("matrix", "embedding") else torch.float32
        t = torch.as_tensor(a.astype(np.float32)).to(store)
        ws[name] = t.cuda()
        vals[name] = t.double().numpy()
    part.bind(ws)
    return vals


def _run_part(kind, params, names, plain_fn, dtype, d, page=16, lens=(300, 70, 33), cuts=(1, 64, 31), tol16=0.05):
    """Three requests, each in two steps (all in one batch), one of them a single token then the rest."""
    from kappai_b200.config import PartSpec
    from kappai_b200.parts import make_part
    from test_parts_gpu import env_for, run_mixer_two_steps
    rng = np.random.default_rng(len(kind) + d + page)
    part = make_part("mixer", PartSpec(kind, params), env_for(dtype, 1024))
    w = _bind(part, rng, dtype)
    local = {v: w[k] for k, v in names.items() if k in w}
    hs = [rt(rng.normal(0, 1, (L, d)), dtype) for L in lens]
    outs = run_mixer_two_steps(part, hs, list(lens), list(cuts), page, dtype)
    for h, got in zip(hs, outs):
        close(got, plain_fn(h, local), dtype, tol16=tol16)
    return part


ATT_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "out_proj.weight": "o", "q_norm.weight": "q.norm",
             "k_norm.weight": "k.norm"}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dim,vdim,d,window,keep,page,scale", [
    (4, 2, 16, 24, 64, 20, 3, 16, 0.35), (3, 3, 24, 8, 48, 33, 0, 8, 0.2), (5, 1, 8, 12, 36, 2, 5, 32, 0.5), (8, 2, 64, 64, 256, 128, 70, 64, 0.125),
    (16, 1, 32, 32, 128, 30, 20, 16, 0.18), (4, 4, 128, 128, 128, 40, 2, 16, 0.05), (4, 2, 16, 16, 64, 33, 2, 16, 0.9), (2, 1, 48, 112, 64, 50, 7, 64, 0.5),
    (2, 1, 16, 16, 32, 1, 1, 16, 0.25)])
def test_windowed_attention_part_with_kept_keys_and_one_more_in_the_denominator(H, G, dim, vdim, d, window, keep, page, scale, dtype):
    """The normed queries and keys have unit mean square, so ``scale * dim`` is the size of the largest scores: the cases
    with a large scale put a row's softmax on one or two keys, often a kept one, the one at the window's far edge or
    the one just outside it; with a small scale the one in the denominator takes a large share."""
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window, "keep_first": keep}}
    params = {"hidden_size": d, "num_heads": H, "num_kv_heads": G, "head_dim": dim, "value_dim": vdim, "scale": scale,
              "qk_norm": "per_head", "qk_norm_eps": 1e-5, "window": window, "keep_first": keep, "sink": "zero",
              "softmax_weights": "float32", "position": None, "bias": False}
    part = _run_part("attention", params, ATT_NAMES, lambda h, w: P.windowed_sink_attention(h, w, m, 1e-5), dtype, d, page=page,
                     tol16=0.05 if scale * dim < 8 else 0.3)
    assert part.cache_spec().keep_first == keep and part.hd % 16 == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dim,vdim,d,coef,every,page,scale", [
    (4, 2, 16, 16, 64, 0.7, 8, 16, 0.25), (3, 3, 24, 8, 48, 1.5, 6.5, 8, 0.15), (5, 1, 8, 12, 36, 0.25, 1, 32, 0.35), (4, 2, 128, 128, 256, 0.5, 64, 64, 0.09),
    (16, 1, 32, 48, 128, 0.3, 32, 16, 0.18), (6, 3, 48, 48, 144, 0.4, 50, 64, 0.14), (4, 2, 64, 64, 128, 2.0, 100, 16, 0.125)])
def test_causal_attention_part_with_a_query_temperature(H, G, dim, vdim, d, coef, every, page, scale, dtype):
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "scale": scale, "q_temp": {"coef": coef, "every": every}}
    params = {"hidden_size": d, "num_heads": H, "num_kv_heads": G, "head_dim": dim, "value_dim": vdim, "scale": scale,
              "qk_norm_eps": None, "window": None, "q_temp": {"coef": coef, "every": every}, "softmax_weights": "float32",
              "position": None, "bias": False}
    _run_part("attention", params, ATT_NAMES, lambda h, w: P.tempered_attention(h, w, m), dtype, d, page=page)
    # without the temperature the plain outputs differ: the test would notice a factor left out
    rng = np.random.default_rng(1)
    h = rng.normal(0, 1, (int(3 * every) + 8, d))
    w = {k: rng.normal(0, 1 / math.sqrt(d), s) for k, s in (("q", (H * dim, d)), ("k", (G * dim, d)), ("v", (G * vdim, d)), ("o", (d, H * vdim)))}
    flat = dict(m, q_temp={"coef": 0.0, "every": every})
    assert np.abs(P.tempered_attention(h, w, m) - P.tempered_attention(h, w, flat)).max() > 1e-3


LATENT_NAMES = {"q_down.weight": "dq", "q_norm.weight": "dq.norm", "q_up.weight": "uq", "kv_down.weight": "dkv", "kv_norm.weight": "dkv.norm",
                "k_up.weight": "uk", "v_up.weight": "uv", "gate_proj.weight": "g", "out_proj.weight": "o", "sink": "sink"}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dim,vdim,qr,kvr,d,window,page,scale", [
    (2, 24, 16, 20, 40, 64, 25, 16, 0.3), (3, 8, 24, 16, 12, 48, 7, 8, 0.35), (1, 36, 12, 9, 7, 36, 1, 32, 0.2), (4, 64, 64, 96, 128, 256, 100, 64, 0.125),
    (2, 128, 64, 64, 48, 128, 50, 16, 0.09), (4, 48, 112, 72, 104, 160, 90, 64, 0.14), (5, 8, 8, 20, 12, 40, 40, 16, 3.0)])
def test_latent_attention_part_with_a_window_learned_sinks_and_head_gates(H, dim, vdim, qr, kvr, d, window, page, scale, dtype):
    m = {"heads": H, "dim": dim, "vdim": vdim, "q_rank": qr, "kv_rank": kvr, "scale": scale, "mask": {"size": window}}
    params = {"hidden_size": d, "num_heads": H, "head_dim": dim, "value_dim": vdim, "q_rank": qr, "kv_rank": kvr, "scale": scale,
              "norm_eps": 1e-5, "gate": "head_sigmoid", "softmax_weights": "float32", "window": window, "sink": "learned"}
    _run_part("latent_attention", params, LATENT_NAMES, lambda h, w: P.latent_attention(h, w, m, 1e-5), dtype, d, page=page,
              tol16=0.05 if scale * dim < 8 else 0.3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_layer_normed_on_both_sides_carries_the_next_layers_input(dtype):
    """Two sandwich layers in a row (the first hands the second its mixer's input), rows of a batch cut in two, against
    the plain layer."""
    from kappai_b200.config import PartSpec
    from kappai_b200.parts import make_part
    from test_parts_gpu import Batch, env_for
    rng = np.random.default_rng(3)
    d, H, G, dim, page, lens, cuts = 64, 4, 2, 16, 16, [90, 41], [1, 30]
    env = env_for(dtype, 256)
    mlp = {"router": {"experts": 4, "top": 2}, "expert": {"ff": 24}, "shared": {"ff": 16}}
    blocks, plain_w = [], []
    for li in range(2):
        att = make_part("mixer", PartSpec("attention", {"hidden_size": d, "num_heads": H, "num_kv_heads": G, "head_dim": dim, "scale": 0.25,
                                                         "qk_norm_eps": None, "q_temp": {"coef": 0.5, "every": 4}, "softmax_weights": "float32"}), env)
        wa = _bind(att, rng, dtype)
        norms, nw = [], []
        for _ in range(4):
            nrm = make_part("norm", PartSpec("rmsnorm", {"size": d, "eps": 1e-5}), env)
            nw.append(_bind(nrm, rng, dtype)["weight"])
            norms.append(nrm)
        ffn = None
        w = {"mix." + v: wa[k] for k, v in ATT_NAMES.items() if k in wa}
        if li == 0:
            ffn, pw, _ = _moe_part(d, 24, 4, 2, 16, dtype, rng)
            w.update({"mlp." + k: v for k, v in pw.items()})
        w.update({"norm1": nw[0], "norm2": nw[1], "norm1b": nw[2], "norm2b": nw[3]})
        plain_w.append(w)
        block = make_part("block", PartSpec("sandwich_residual", {}), env)
        blocks.append(block.assemble(att, ffn, norms[0], norms[1] if ffn else None, None, post_norms=(norms[2], norms[3] if ffn else None)))
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": dim, "scale": 0.25, "q_temp": {"coef": 0.5, "every": 4}}

    def plain(x):
        for li, w in enumerate(plain_w):
            y = P.tempered_attention(P.rms_norm(x, w["norm1"], 1e-5), P.sub(w, "mix."), m)
            x = x + P.rms_norm(y, w["norm1b"], 1e-5)
            if li == 0:
                x = x + P.rms_norm(P.mixture(P.rms_norm(x, w["norm2"], 1e-5), P.sub(w, "mlp."), mlp), w["norm2b"], 1e-5)
        return x

    xs = [rt(rng.normal(0, 1, (L, d)), torch.float32) for L in lens]
    b = Batch([blk.mixer.cache_spec() for blk in blocks], lens, cuts, page, dtype)
    outs = [np.zeros((L, d)) for L in lens]
    for step in (0, 1):
        ctx, rows = b.context(step)
        x = dev(np.concatenate([xs[i][a:a + n] for i, a, n in rows], 0))
        for li, blk in enumerate(blocks):
            ctx.next_block = blocks[li + 1] if li + 1 < len(blocks) else None
            blk.forward(x, ctx, b.storage.views[li])
            if li == 0:
                assert ctx.sandwich_carry is not None and ctx.sandwich_carry[0] is x
        r = 0
        for i, a, n in rows:
            outs[i][a:a + n] = host(x)[r:r + n]
            r += n
    for x0, got in zip(xs, outs):
        close(got, plain(x0), dtype, tol16=0.06)


# ------------------------------------------------------------------------------------- whole models

# The smallest gap between a chosen and an unchosen router logit that a request's tokens may have.  In 16 bits a row's
# router inputs differ from the plain ones by about half a per cent and its logits (spread: about 3) by a hundredth or
# two, so a closer call may fall the other way, and the token that took another expert stays in the caches behind it.
# Requests grow four tokens at a time, and four tokens that bring a closer call are drawn again.
MARGIN = 0.05
_PLAIN = {}
_REQS = {}


def _requests(plain, name, lengths, seed):
    """Random requests whose router choices all have a margin (``MARGIN``; see there)."""
    key = (name, tuple(lengths), seed)
    if key in _REQS:
        return _REQS[key]
    rng = np.random.default_rng(seed)
    reqs = {}
    for i, n in enumerate(lengths):
        toks = []
        while len(toks) < n:
            new = rng.integers(0, plain.cfg["vocab"], min(4, n - len(toks))).tolist()
            m = []
            plain.forward(toks + new, margins=m)
            if m and min(float(x[len(toks):].min()) for x in m) < MARGIN:
                continue
            toks += new
        reqs[f"r{i}"] = toks
    _REQS[key] = reqs
    return reqs


def _expect(plain, name, toks):
    """(the plain logits [T, vocab], every position's smallest router margin [T]) of a sequence."""
    key = (name, tuple(toks))
    if key not in _PLAIN:
        m = []
        lg = plain.forward(toks, margins=m)
        _PLAIN[key] = (lg, np.min(m, axis=0) if m else np.full(len(toks), np.inf))
    return _PLAIN[key]


# lengths above the longest window of every model (A: 25, B: 33, C: 2, D: 128, E: 50) plus the decoded tail, a request of
# two or three tokens, and lengths that end on and one behind a page's last token
LENGTHS = {"A": [150, 3, 64, 49], "B": [130, 41, 2, 97], "C": [77, 20, 101], "D": [330, 65, 201], "E": [200, 64, 140], "F": [90, 33, 2]}
PROMPTS = {"A": [30, 1, 60, 48], "B": [50, 40, 1, 80], "C": [40, 19, 60], "D": [150, 3, 128], "E": [150, 63, 30], "F": [40, 32, 1]}
N_LAST = {"A": 110, "B": 60, "C": 40, "D": 170, "E": 70, "F": 30}       # the windows pass over decoded tokens only (D: 128 + 40)
BF16_REL_RMS = 0.04    # a row's 16-bit error (rms over the vocabulary / the row's spread): 95 % of the rows; 99 % twice that
BF16_BETWEEN_CUTS = 0.06


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", [("A", 16), ("B", None), ("C", 32), ("D", None), ("E", 8), ("F", 16)])
def test_every_cut_agrees_with_plain(name, page_size, dtype, vum_dirs, vum_plain, tmp_path):
    """Whole prompts, the last tokens decoded one by one (more of them than the longest window), portions down to two
    tokens, and up to four requests mixed in a pool so small that pages and slots go round."""
    plain = vum_plain[name]
    reqs = _requests(plain, name, LENGTHS[name], 31)
    prompt_len = dict(zip(reqs, PROMPTS[name]))
    expected = {rid: _expect(plain, name, t)[0] for rid, t in reqs.items()}
    page = page_size or 64
    rounded = sorted(-(-len(t) // page) * page for t in reqs.values())
    max_tokens = rounded[-1] + rounded[0] + 2 * page          # the longest request and the shortest fit together, not all
    tr = R.Trace()
    R.whole(tr, reqs)
    R.last_decoded(tr, reqs, n_last=N_LAST[name])
    R.portions(tr, reqs)
    b = len(tr.steps)
    R.mixed(tr, reqs, prompt_len, seed=5, max_live=4, page=page, max_tokens=max_tokens)
    assert max(len(s["entries"]) for s in tr.steps[b:]) >= 2
    out = R.run_trace(vum_dirs[name], dtype, tr, str(tmp_path / "out"), max_tokens, page_size)
    rel = []
    for st, rows in zip(tr.steps, tr.rows):
        for j, (rid, pos) in enumerate(rows):
            e = expected[rid][pos]
            rel.append((float(np.sqrt(np.mean((out[st["step"]][j] - e) ** 2)) / e.std()), st["step"], rid, pos))
    r = np.array([x[0] for x in rel])
    print(f"{name} {dtype}: {len(r)} rows, relative rms error median {np.median(r):.2e}, 95 % {np.quantile(r, 0.95):.2e}, worst {r.max():.2e}")
    if dtype == "bfloat16":
        # rounding alone gives a per cent or two (these weights have unit gain: every sublayer moves the residual); a
        # wrong key, a sink left out, a window one token off or a wrong page gives tens
        assert np.quantile(r, 0.95) <= BF16_REL_RMS and np.quantile(r, 0.99) <= 2 * BF16_REL_RMS, max(rel)
        apart = []
        for place, rows in R.rows_by_place(tr, out).items():
            e = expected[place[0]][place[1]]
            apart.append(max(float(np.sqrt(np.mean((x - rows[0]) ** 2)) / e.std()) for x in rows[1:]))
        assert np.quantile(apart, 0.99) <= BF16_BETWEEN_CUTS, max(apart)
    else:
        assert r.max() <= 1e-4, max(rel)
    stats = R.cache_stats(str(tmp_path / "out"))
    assert stats and all(g["reused"] > 0 and g["handed_out"] > g["pages"] for g in stats.values()), stats
    if dtype == "float32":
        for place, rows in R.rows_by_place(tr, out).items():
            assert len(rows) >= 2, place
            for x in rows[1:]:
                assert np.array_equal(rows[0], x), f"{name}: float32 logits of {place} differ between cuts"


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_residual_after_every_layer_run(name, vum_dirs, vum_plain):
    from kappai_b200 import ModelRunner, StepEntry
    plain = vum_plain[name]
    toks = _requests(plain, name, [57], 8)["r0"]
    want = []
    plain.forward(toks, want)
    r = ModelRunner(vum_dirs[name], dtype="float32", max_tokens=256, max_requests=2, cuda_graphs=False)
    got = []
    r.observer = lambda i, x: got.append(x.detach().cpu().numpy().copy())
    r.step([StepEntry("a", toks, [0])])
    assert len(got) == len(want) + 1 == len(P.layer_order(plain.cfg)) + 1
    for i, w in enumerate(want):
        assert np.abs(got[i + 1] - w).max() < 1e-4 * max(1.0, np.abs(w).max()), (i, np.abs(got[i + 1] - w).max())


def test_a_mask_one_token_off_or_a_sink_left_out_would_show(vum_dirs, vum_plain, tmp_path):
    """Model A with scales so large that a softmax row sits on one or two keys: wherever that key is the window's last,
    the first one outside it, or the last kept one, a mask one token off moves the logits by tens of per cent, and so
    does a sink left out where the scores are small.  The plain model with every window one token longer or shorter,
    one kept key more or fewer, and without its sinks is that far away at many positions; the engine is not, for tokens
    of a prompt, of portions of it and for tokens decoded one by one."""
    from kappai_b200 import ModelRunner, StepEntry
    cfg = copy.deepcopy(CONFIGS["A"][0])
    for layer in cfg["layers"]:
        if layer["type"] != "attention_2":
            layer["mixer"]["scale"] = 2.5
    weights = make_weights(cfg, 17)
    d = write_model_dir(cfg, weights, str(tmp_path / "peaked"))
    plain = P.PlainVumotar(d)
    toks = np.random.default_rng(3).integers(0, cfg["vocab"], 140).tolist()
    want = plain.forward(toks)

    def far_rows(other_cfg, other_w=None):
        wrong = P.PlainVumotar(config=other_cfg, tensors=other_w or plain.w).forward(toks)
        return np.sqrt(((wrong - want) ** 2).mean(1)) / want.std(1)

    for delta in (1, -1):
        off = copy.deepcopy(cfg)
        for layer in off["layers"]:
            if layer["type"] != "attention_2":
                layer["mixer"]["mask"]["size"] += delta
        assert (far_rows(off) > 0.1).sum() >= 20, delta
        off = copy.deepcopy(cfg)
        for layer in off["layers"]:
            if layer["type"] == "attention":
                layer["mixer"]["mask"]["keep_first"] += delta
        assert (far_rows(off) > 0.1).sum() >= 20, delta
    no_sink = {k: (v - 30.0 if k.endswith(".sink") else v) for k, v in plain.w.items()}
    assert (far_rows(cfg, no_sink) > 0.1).sum() >= 20
    r = ModelRunner(d, dtype="float32", max_tokens=256, max_requests=2, page_size=16, cuda_graphs=False)
    got = [r.step([StepEntry("a", toks[:37], list(range(37)))]).cpu().numpy()]
    got.append(r.step([StepEntry("a", toks[37:60], list(range(23)))]).cpu().numpy())
    for t in toks[60:]:
        got.append(r.step([StepEntry("a", [t], [0])]).cpu().numpy())
    got = np.concatenate(got, 0)
    err = np.sqrt(((got - want) ** 2).mean(1)) / want.std(1)
    assert err.max() < 2e-4, (int(err.argmax()), err.max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batched_requests_equal_each_alone_and_captured_steps_equal_eager(dtype, vum_dirs, vum_plain):
    """Unequal requests decode together for many steps (the steps are captured into CUDA graphs on the way); every row
    equals the row of the request run alone without graphs."""
    from kappai_b200 import ModelRunner, StepEntry
    n_dec = 40
    reqs = _requests(vum_plain["A"], "A", [61 + n_dec, 9 + n_dec, 30 + n_dec], 12)

    def run(runner, group):
        out = {rid: [] for rid in group}
        lg = runner.step([StepEntry(rid, reqs[rid][:len(reqs[rid]) - n_dec], [len(reqs[rid]) - n_dec - 1]) for rid in group])
        for j, rid in enumerate(group):
            out[rid].append(lg[j].cpu().numpy().copy())
        for s in range(n_dec):
            lg = runner.step([StepEntry(rid, [reqs[rid][len(reqs[rid]) - n_dec + s]], [0]) for rid in group])
            for j, rid in enumerate(group):
                out[rid].append(lg[j].cpu().numpy().copy())
        for rid in group:
            runner.end(rid)
        return out

    r1 = ModelRunner(vum_dirs["A"], dtype=dtype, max_tokens=512, max_requests=4, page_size=16)
    together = run(r1, list(reqs))
    assert r1.model.graph_safe and r1.graphs is not None and len(r1.graphs.graphs) >= 1
    alone_runner = ModelRunner(vum_dirs["A"], dtype=dtype, max_tokens=512, max_requests=4, page_size=16, cuda_graphs=False)
    for rid in reqs:
        alone = run(alone_runner, [rid])[rid]
        for a, b in zip(alone, together[rid]):
            if dtype == "float32":
                assert np.array_equal(a, b)
            else:
                assert np.abs(a - b).max() <= 2 * tol_for(dtype, a)


@pytest.mark.parametrize("name", ["A", "D", "E"])
def test_a_slot_and_pages_used_again_start_empty(name, vum_dirs):
    """One slot and just enough pages for one request: a second request takes the slot and the pages of the first (also
    the pages that held its kept first keys) and gives what it gives alone."""
    from kappai_b200 import ModelRunner, StepEntry
    rng = np.random.default_rng(2)
    V = CONFIGS[name][0]["vocab"]
    a, b = rng.integers(0, V, 60).tolist(), rng.integers(0, V, 45).tolist()
    mk = lambda: ModelRunner(vum_dirs[name], dtype="float32", max_tokens=64, max_requests=1, page_size=16, cuda_graphs=False)
    r = mk()
    r.step([StepEntry("a", a, [len(a) - 1])])
    r.end("a")
    second = r.step([StepEntry("b", b[:7], [6])]).cpu().numpy().copy()
    second2 = r.step([StepEntry("b", b[7:], [len(b) - 8])]).cpu().numpy().copy()
    r.end("b")
    fresh = mk()
    assert np.array_equal(second, fresh.step([StepEntry("x", b[:7], [6])]).cpu().numpy())
    assert np.array_equal(second2, fresh.step([StepEntry("x", b[7:], [len(b) - 8])]).cpu().numpy())


def test_kept_pages_stay_in_the_runner_while_the_window_moves_on(vum_dirs):
    from kappai_b200 import ModelRunner, StepEntry
    from kappai_b200.cache.manager import RELEASED
    r = ModelRunner(vum_dirs["E"], dtype="float32", max_tokens=256, max_requests=2, page_size=8, cuda_graphs=False)
    toks = np.random.default_rng(4).integers(0, CONFIGS["E"][0]["vocab"], 150).tolist()
    r.step([StepEntry("a", toks, [])])
    kept = [gk for gk in r.cache.pools if ("keep_first", 20) in gk]
    assert len(kept) == 1
    t = r.cache.block_table("a", kept[0])
    assert all(p != RELEASED for p in t[:3]) and all(p == RELEASED for p in t[3:(150 - 30 + 1) // 8])
    plain = [gk for gk in r.cache.pools if gk[3] == 50][0]
    assert r.cache.block_table("a", plain)[0] == RELEASED


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_greedy_generation_through_the_engine(name, dtype, vum_dirs, vum_plain):
    from kappai_b200 import Engine, EngineArgs, SamplingParams
    plain = vum_plain[name]
    prompts = list(_requests(plain, name, [5, 26, 60], 21).values())
    n_new = 50
    eng = Engine(EngineArgs(model=vum_dirs[name], dtype=dtype, max_batch=4, max_step_tokens=16, page_size=16, kv_tokens=1024))
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, n_predict=n_new))
    assert [len(o) for o in outs] == [n_new] * len(prompts)
    for p, o in zip(prompts, outs):
        lg, margin = _expect(plain, name, p + o)
        lg, margin = lg[len(p) - 1:-1], margin[len(p) - 1:-1]
        for j, t in enumerate(o):
            if dtype == "bfloat16" and margin[:j + 1].min() < MARGIN:
                break                      # a router call too close for 16 bits: from here on the sequences may part
            best = int(np.argmax(lg[j]))
            assert t == best or lg[j][best] - lg[j][t] <= 4 * tol_for(dtype, lg[j]), (j, t, best)
    assert eng.runner.cache.slots.n_free == 4 and all(p.n_free == p.n_pages for p in eng.runner.cache.pools.values())


def test_command_line_and_random_weights(vum_dirs, vum_plain, tmp_path):
    """The command line runs the design like any other: greedy tokens equal the plain model's, --time names the design's
    kernels, and --random-weights writes a loadable model folder from a Vumotar config.json."""
    import json
    import os
    import subprocess
    import sys
    plain = vum_plain["A"]
    prompt = _requests(plain, "A", [30], 77)["r0"]
    cmd = [sys.executable, "-m", "kappai_b200.cli", "-m", vum_dirs["A"], "-p", ",".join(map(str, prompt)), "-n", "12", "-t", "0",
           "--fp32", "--time"]
    p = subprocess.run(cmd, cwd=R.ROOT, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    out = [int(t) for t in p.stdout.split()]
    assert len(out) == 12
    lg = plain.forward(prompt + out)[len(prompt) - 1:-1]
    for j, t in enumerate(out):
        best = int(np.argmax(lg[j]))
        assert t == best or lg[j][best] - lg[j][t] <= 1e-4, (j, t, best)
    for name in ("rmsnorm_add_norm_rows", "qk_norm_rope_kv", "attention_split", "moe_router", "moe_experts", "head_gate", "rmsnorm_cols"):
        assert name in p.stderr, (name, p.stderr[-3000:])
    cfgp = tmp_path / "c.json"
    cfgp.write_text(json.dumps(CONFIGS["B"][0]))
    made = tmp_path / "rw"
    cmd = [os.path.join(R.ROOT, "bin", "kappai-cli"), "--random-weights", str(cfgp), "-s", "5", "-m", str(made), "-t", "0", "-n", "5",
           "1 2 3"]
    p = subprocess.run(cmd, cwd=str(tmp_path), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert len(p.stdout.split()) == 5 and os.path.isfile(made / "model.safetensors")
