"""Tupalorn without a GPU: the configuration reader and its errors, the tensor names and shapes of every test
configuration, which layer keeps which cache, and the plain mechanisms on cases worked out by hand."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_tupalorn as P
from tupalorn_configs import CONFIGS, make_model_dir, tensor_shapes


def _spec(cfg):
    from kappai_b200.config.registry import config_from_dict
    arch, c = config_from_dict(cfg)
    assert arch.name == "Tupalorn"
    return arch.build_spec(c)


def _model(cfg):
    from kappai_b200.engine.model import Model
    from kappai_b200.parts.base import BuildEnv
    return Model(_spec(cfg), BuildEnv(torch.device("cpu"), torch.float32, 32))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_and_shapes(name):
    cfg = CONFIGS[name][0]
    table = {n: tuple(ws.shape) for n, ws in _model(cfg).weight_table().items()}
    assert table == tensor_shapes(cfg)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_what_every_layer_keeps(name):
    from kappai_b200.cache.spec import PagedKVSpec, StateSpec
    cfg = CONFIGS[name][0]
    m = _model(cfg)
    assert [e.layer for e in m.schedule] == list(range(len(cfg["layers"])))
    specs, borrowed = m.cache_specs(), m.cache_borrowing()
    for i, (layer, s) in enumerate(zip(cfg["layers"], specs)):
        mix = layer["mixer"]
        if layer["type"] == "mamba2":
            channels = mix["heads"] * mix["vdim"] + 2 * mix["groups"] * mix["state"]
            assert s == StateSpec((mix["heads"] * mix["state"] * mix["vdim"] + (mix["conv"] - 1) * channels,), "float32")
        elif layer["type"] == "retention":
            assert s == StateSpec((mix["heads"], mix["dim"], mix["vdim"]), "float32")
        elif mix.get("kv_from") is not None:
            assert s is None and borrowed[i] == mix["kv_from"]
        else:
            assert isinstance(s, PagedKVSpec) and s.num_kv_heads == mix["kv_heads"] and borrowed[i] is None
            assert s.head_dim >= max(mix["dim"], mix["vdim"])
            readers = [mix] + [l["mixer"] for l in cfg["layers"] if l["mixer"].get("kv_from") == i]
            sizes = [r["mask"]["size"] if r.get("mask") else None for r in readers]
            assert s.window == (None if None in sizes else max(sizes))     # the cache keeps what its widest reader sees


def test_a_lender_keeps_keys_for_a_borrower_with_a_wider_window():
    cfg = CONFIGS["A"][0]
    own = cfg["layers"][1]["mixer"]["mask"]["size"]
    wide = cfg["layers"][3]["mixer"]["mask"]["size"]
    assert wide > own
    m = _model(cfg)
    assert m.cache_specs()[1].window == wide
    assert m.blocks[1].mixer.window == own and m.blocks[3].mixer.window == wide and m.blocks[4].mixer.window < own
    assert m.blocks[3].mixer.borrows and not m.blocks[1].mixer.borrows


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][2]["mixer"].update(groups=3), "groups"),
    (lambda c: c["layers"][2]["mixer"].update(norm_groups=7), "norm_groups"),
    (lambda c: c["layers"][2]["mixer"].pop("state"), "state"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "kv_from"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(dim=32), "dim"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
])
def test_configuration_errors_name_the_key(change, word):
    from kappai_b200.config.schema import ConfigError
    cfg = copy.deepcopy(CONFIGS["A"][0])
    change(cfg)
    with pytest.raises(ConfigError) as e:
        _spec(cfg)
    assert word in str(e.value)


def test_options_left_out():
    cfg = copy.deepcopy(CONFIGS["B"][0])
    assert "logit_softcap" not in cfg
    m = _model(cfg)
    assert m.head.softcap is None and m.head.tied
    assert m.blocks[1].mixer.window is None and m.blocks[3].mixer.window == 7 and m.cache_specs()[1].window is None
    cfg = copy.deepcopy(CONFIGS["C"][0])
    assert _model(cfg).blocks[2].mixer.rotary is None          # a retention layer without a rotation


def test_a_written_model_folder_loads_in_the_plain_reader(tmp_path):
    d = make_model_dir("C", str(tmp_path))
    p = P.PlainTupalorn(d)
    assert set(p.w) == set(tensor_shapes(CONFIGS["C"][0]))
    lg = p.forward([1, 2, 3, 4])
    assert lg.shape == (4, 19) and np.isfinite(lg).all() and np.abs(lg).max() < 5.0     # the soft cap bounds the logits


# ----------------------------------------------------------------------------------- the plain mechanisms by hand

def test_layer_norm_by_hand():
    x = np.array([[1.0, 3.0, 5.0, 7.0]])
    y = P.layer_norm(x, np.array([1.0, 2.0, 1.0, 0.5]), 0.0)
    s = math.sqrt(5.0)                                          # deviations -3 -1 1 3: variance 5
    assert np.allclose(y, [[-3 / s, -2 / s, 1 / s, 1.5 / s]])


def test_causal_conv_by_hand_and_with_kept_inputs():
    u = np.array([[1.0], [2.0], [3.0], [4.0]])
    taps, bias = np.array([[10.0, 100.0, 1.0]]), np.array([0.5])       # the last tap meets the current row
    y = P.causal_conv(u, taps, bias)
    assert np.allclose(y[:, 0], [1.5, 102.5, 213.5, 324.5])
    later = P.causal_conv(u[2:], taps, bias, before=u[:2])
    assert np.allclose(later, y[2:])


def test_selective_scan_by_hand_and_carried_state():
    # one head, a state of one row, one value column: S_t = exp(-A dt) S + dt B x ; y = S C + D x
    x = np.array([1.0, 2.0, -1.0]).reshape(3, 1, 1)
    B = np.array([1.0, 0.5, 2.0]).reshape(3, 1, 1)
    C = np.array([1.0, 1.0, 3.0]).reshape(3, 1, 1)
    dt = np.array([0.5, 1.0, 0.25]).reshape(3, 1)
    A_log, D = np.array([math.log(2.0)]), np.array([0.1])
    y, S = P.selective_scan(x, B, C, dt, A_log, D, 1, 1)
    s0 = 0.5
    s1 = math.exp(-2.0) * s0 + 1.0
    s2 = math.exp(-0.5) * s1 - 0.5
    assert np.allclose(y.ravel(), [s0 + 0.1, s1 + 0.2, 3 * s2 - 0.1]) and np.allclose(S.ravel(), [s2])
    y2, S2 = P.selective_scan(x[1:], B[1:], C[1:], dt[1:], A_log, D, 1, 1, state=np.array([[[s0]]]))
    assert np.allclose(y2, y[1:]) and np.allclose(S2, S)


def test_heads_read_their_group():
    rng = np.random.default_rng(0)
    T, H, G, N, Pd = 5, 4, 2, 3, 2
    x, B, C = rng.normal(size=(T, H, Pd)), rng.normal(size=(T, G, N)), rng.normal(size=(T, G, N))
    dt = rng.uniform(0.1, 1, (T, H))
    y, _ = P.selective_scan(x, B, C, dt, np.zeros(H), np.zeros(H), H, G)
    B2 = B.copy()
    B2[:, 1] += 1.0                                             # the second group's B: heads 2 and 3 only
    y2, _ = P.selective_scan(x, B2, C, dt, np.zeros(H), np.zeros(H), H, G)
    assert np.array_equal(y[:, :2], y2[:, :2]) and not np.allclose(y[:, 2:], y2[:, 2:])


def test_rotation_pairs_and_partial_rotation():
    x = np.zeros((2, 1, 6))
    x[:, 0] = [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]
    y = P.rotate_half(x, 0, 4, 100.0)
    assert np.allclose(y[0], x[0])                              # position 0: no turn
    f = [1.0, 100.0 ** -0.5]
    for i in range(2):
        u, v = x[1, 0, i], x[1, 0, i + 2]
        assert np.isclose(y[1, 0, i], u * math.cos(f[i]) - v * math.sin(f[i]))
        assert np.isclose(y[1, 0, i + 2], v * math.cos(f[i]) + u * math.sin(f[i]))
    assert np.array_equal(y[1, 0, 4:], x[1, 0, 4:])             # dimensions behind the rotated ones pass
    assert np.allclose(P.rotate_half(x[1:], 1, 4, 100.0), y[1:])


def test_a_window_sees_itself_and_the_tokens_before():
    T, w = 6, 3
    q = np.ones((T, 1, 1))
    k = np.zeros((T, 1, 1))
    v = np.arange(1.0, T + 1).reshape(T, 1, 1)
    o = P.windowed_attention(q, k, v, 1.0, w)                   # equal scores: the mean of the visible values
    assert np.allclose(o.ravel(), [1.0, 1.5, 2.0, 3.0, 4.0, 5.0])
    assert np.allclose(P.windowed_attention(q, k, v, 1.0, None).ravel(), [1.0, 1.5, 2.0, 2.5, 3.0, 3.5])
    assert np.allclose(P.windowed_attention(q, k, v, 1.0, 1).ravel(), v.ravel())


def test_decayed_state_by_hand():
    q = np.ones((3, 1, 1))
    k = np.ones((3, 1, 1))
    v = np.array([1.0, 10.0, 100.0]).reshape(3, 1, 1)
    o, S = P.decayed_outer_scan(q, k, v, [0.5])
    assert np.allclose(o.ravel(), [1.0, 10.5, 105.25]) and np.allclose(S.ravel(), [105.25])


def test_gated_unit_limits():
    w = {"gate": np.array([[1.0]]), "gate.b": np.array([0.0]), "up": np.array([[1.0]]), "up.b": np.array([0.0]),
         "down": np.array([[1.0]]), "down.b": np.array([0.25])}
    big = P.clamped_gated_unit(np.array([[50.0]]), w, 2.0)      # gate and up both stop at the limit
    assert np.isclose(big[0, 0], 2.0 * P.sigmoid(1.702 * 2.0) * 3.0 + 0.25)
    low = P.clamped_gated_unit(np.array([[-50.0]]), w, 2.0)     # the gate has no lower limit, up has
    assert np.isclose(low[0, 0], -50.0 * P.sigmoid(-1.702 * 50.0) * (-2.0 + 1.0) + 0.25)


def test_grouped_norm_and_softcap():
    y = np.array([[3.0, 4.0, 0.0, 2.0]])
    n = P.grouped_rms_norm(y, np.ones(4), 2, 0.0)
    assert np.allclose(n, [[3 / math.sqrt(12.5), 4 / math.sqrt(12.5), 0.0, math.sqrt(2.0)]])
    assert np.allclose(P.softcap(np.array([0.0, 1e9, -1e9]), 7.0), [0.0, 7.0, -7.0])


def test_the_bench_configurations_are_valid_models():
    """``bench.py --design tupalorn`` times these layer sizes: every one of them reads as a model with one lender and one
    borrower whose window is shorter than the lender's own."""
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_for_test", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    for name, width, H, G, hd, ff, *_ in bench.DESIGN_SIZES:
        cfg = bench.tupalorn_config(width, H, G, hd, ff)
        m = _spec(cfg)
        assert [l.mixer.kind for l in m.layers] == ["mamba2", "lightning", "attention", "attention"], name
        assert [e.cache_of for e in m.schedule] == [None, None, None, 2]
        assert m.layers[2].mixer.params["cache_window"] == bench.DESIGN_BLOCK and m.layers[3].mixer.params["window"] == bench.TUPALORN_WINDOW
