"""Vumotar without a GPU: the configuration reader and its errors, the tensor names and shapes of every test
configuration, the order of layer runs and what every run keeps, pages of kept first keys in the cache manager and the
memory plan, and the plain mechanisms on cases worked out by hand."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_vumotar as P
from vumotar_configs import CONFIGS, make_weights, tensor_shapes


def _spec(cfg):
    from kappai_b200.config.registry import config_from_dict
    arch, c = config_from_dict(cfg)
    assert arch.name == "Vumotar"
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
def test_order_of_layer_runs_and_what_every_run_keeps(name):
    from kappai_b200.cache.spec import PagedKVSpec
    cfg = CONFIGS[name][0]
    m = _model(cfg)
    order = [e.layer for e in m.schedule]
    assert order == P.layer_order(cfg)
    loop = cfg.get("loop")
    if loop:
        assert len(order) == len(cfg["layers"]) + (loop["stop"] - loop["start"]) * (loop["times"] - 1)
    assert not any(e.enter or e.cache_of is not None for e in m.schedule)     # every pass with caches of its own
    for i, s in zip(order, m.cache_specs()):
        layer, mix = cfg["layers"][i], cfg["layers"][i]["mixer"]
        assert isinstance(s, PagedKVSpec) and s.head_dim >= max(mix["dim"], mix["vdim"])
        assert s.head_dim % 16 == 0 or s.head_dim == mix["dim"] == mix["vdim"]     # a head is widened only where its two sizes differ
        mask = mix.get("mask") or {}
        assert s.num_kv_heads == (mix["heads"] if layer["type"] == "latent_attention" else mix["kv_heads"])
        assert (s.window, s.keep_first) == (mask.get("size"), mask.get("keep_first", 0) if mask else 0)


def test_parts_and_their_constants_come_from_the_configuration():
    cfg = CONFIGS["A"][0]
    m = _model(cfg)
    a2, a, lat = m.blocks[0].mixer, m.blocks[1].mixer, m.blocks[2].mixer
    assert a2.q_temp == (0.7, 8.0) and a2.sink is None and a2.window is None and a2.qk_norm_eps is None
    assert a.sink == "zero" and a.keep_first == 3 and a.window == 20 and a.q_temp is None and a.qk_norm_eps == cfg["norm"]["eps"]
    assert (a.dim, a.vdim, a.hd) == (16, 24, 32) and a.scale == 0.35
    assert lat.sink == "learned" and lat.head_gate and lat.window == 25 and lat.keep_first == 0
    f = m.blocks[0].ffn
    assert (f.routing, f.weight_on, f.top, f.E, f.ff, f.shared_ff, f.shared_gate) == ("sigmoid", "input", 2, 6, 40, 24, None)
    assert m.blocks[2].ffn is None and m.blocks[2].ffn_norm is None and m.blocks[2].ffn_post_norm is None
    assert m.blocks[3].ffn.shared_ff is None
    assert all(type(b).__name__ == "SandwichResidualBlock" and b.mixer_post_norm is not None for b in m.blocks)
    assert m.head.tied and m.graph_safe
    assert _spec(cfg).ignored_tensors == ["l2.norm2", "l2.norm2b"]


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].pop("coef"), "coef"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][2]["mixer"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("ff"), "ff"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
])
def test_configuration_errors_name_the_key(change, word):
    from kappai_b200.config.schema import ConfigError
    cfg = copy.deepcopy(CONFIGS["A"][0])
    change(cfg)
    with pytest.raises(ConfigError) as e:
        _spec(cfg)
    assert word in str(e.value)


def test_a_mixer_without_a_mask_reads_every_key_and_one_without_a_temperature_has_none():
    cfg = copy.deepcopy(CONFIGS["A"][0])
    cfg["layers"][0]["mixer"].pop("q_temp")
    cfg["layers"][1]["mixer"].pop("mask")
    cfg["layers"][2]["mixer"].pop("mask")
    m = _model(cfg)
    assert m.blocks[0].mixer.q_temp is None
    assert m.blocks[1].mixer.window is None and m.blocks[1].mixer.keep_first == 0 and m.blocks[1].mixer.sink == "zero"
    assert m.blocks[2].mixer.window is None and m.cache_specs()[2].window is None


def test_parts_refuse_what_they_cannot_do():
    from kappai_b200.config import PartSpec
    from kappai_b200.config.schema import ConfigError
    from kappai_b200.parts import BuildEnv, make_part
    env = BuildEnv(torch.device("cpu"), torch.float32, 32)
    att = {"hidden_size": 32, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16, "scale": 0.25}
    for extra, word in ((dict(sink="big"), "sink"), (dict(keep_first=-2, window=4), "keep_first"),
                        (dict(keep_first=2, window=4, block=8), "blocks"), (dict(q_temp={"coef": 1.0, "every": 0.0}), "every")):
        with pytest.raises(ConfigError) as e:
            make_part("mixer", PartSpec("attention", dict(att, **extra)), env)
        assert word in str(e.value)
    assert make_part("mixer", PartSpec("attention", dict(att, keep_first=5)), env).keep_first == 0      # no window: all keys anyway
    moe = {"hidden_size": 32, "expert_size": 8, "num_experts": 4, "top": 2}
    for extra, word in ((dict(weight_on="both"), "weight_on"), (dict(weight_on="input", identity_experts=1), "identity"),
                        (dict(routing="sigmoid", router_bias=True), "sigmoid")):
        with pytest.raises(ConfigError) as e:
            make_part("feed_forward", PartSpec("moe", dict(moe, **extra)), env)
        assert word in str(e.value)


def test_missing_and_unexpected_tensors_are_listed_and_unread_norms_are_let_through(tmp_path):
    from kappai_b200.weights.loader import WeightError, load_weights
    from vumotar_configs import write_model_dir
    cfg = CONFIGS["A"][0]
    w = make_weights(cfg, 1)
    w["l2.norm2"] = torch.ones(cfg["width"], dtype=torch.bfloat16)          # a norm of the feed-forward that layer 2 lacks
    d = write_model_dir(cfg, w, str(tmp_path / "ok"))
    load_weights(_model(cfg), d)
    del w["l1.mix.q.norm"], w["l2.mix.sink"]
    w["l0.mix.sink"] = torch.zeros(4, dtype=torch.bfloat16)
    d = write_model_dir(cfg, w, str(tmp_path / "bad"))
    with pytest.raises(WeightError) as e:
        load_weights(_model(cfg), d)
    assert e.value.missing == ["l1.mix.q.norm", "l2.mix.sink"] and e.value.unexpected == ["l0.mix.sink"]


# ------------------------------------------------------------------------------------- cache manager and memory plan

def test_pages_of_kept_first_keys_stay_while_the_window_moves_on():
    from kappai_b200.cache.manager import RELEASED, PagePool
    page, window, keep = 8, 10, 11                         # the kept keys fill one page and a part of the next
    pool = PagePool(12, page, window, None, keep)
    plain = PagePool(12, page, window)
    for p in (pool, plain):
        p.open("a")
        p.extend("a", 70)
        p.release_behind("a", 70)
    first_needed = 70 - window + 1
    assert [b for b, pg in enumerate(plain.table("a")) if pg == RELEASED] == list(range(first_needed // page))
    assert [b for b, pg in enumerate(pool.table("a")) if pg == RELEASED] == list(range(2, first_needed // page))
    pool.check()
    held = pool.n_pages - pool.n_free
    pool.close("a")
    assert pool.n_free == pool.n_pages and held == 2 + (9 - first_needed // page)
    # a second request gets the pages back, also those that held kept keys
    pool.open("b")
    pool.extend("b", 12 * page)
    assert pool.n_reused >= 9 and pool.n_free == 0


def test_the_group_key_tells_kept_keys_apart_and_the_plan_counts_their_pages():
    from kappai_b200.cache.spec import PagedKVSpec
    from kappai_b200.engine.memory import GroupNeed, pages_of_group
    a, b, c = PagedKVSpec(2, 32, 20, None, 3), PagedKVSpec(2, 32, 20, None, 0), PagedKVSpec(2, 32, None, None, 3)
    assert a.group_key != b.group_key and b.group_key == PagedKVSpec(2, 32, 20).group_key
    assert c.group_key == PagedKVSpec(2, 32, None).group_key               # without a window nothing is released anyway
    without = pages_of_group(GroupNeed("g", 64, 100), 1000, 16, 4, 32)
    with_kept = pages_of_group(GroupNeed("g", 64, 100, 40), 1000, 16, 4, 32)
    assert with_kept == without + 4 * 3


# ------------------------------------------------------------------------------------- the plain mechanisms by hand

def test_visible_keys_by_hand():
    v = P.visible(9, 3, 2)
    assert v[8].tolist() == [True, True, False, False, False, False, True, True, True]
    assert v[3].tolist() == [True, True, True, True, False, False, False, False, False]
    assert v[4].tolist() == [True, True, True, True, True, False, False, False, False]
    assert v[5].tolist() == [True, True, False, True, True, True, False, False, False]
    assert P.visible(4, 1).tolist() == np.eye(4, dtype=bool).tolist()
    assert P.visible(4).tolist() == np.tril(np.ones((4, 4), dtype=bool)).tolist()


def test_softmax_with_a_sink_by_hand():
    s = np.log(np.array([[1.0, 2.0, 5.0]]))
    m = np.array([[True, True, False]])
    assert np.allclose(P.softmax_with_sink(s, m), [[1 / 3, 2 / 3, 0]])
    assert np.allclose(P.softmax_with_sink(s, m, 0.0), [[1 / 4, 2 / 4, 0]])               # one more in the denominator
    assert np.allclose(P.softmax_with_sink(s, m, math.log(7.0)), [[1 / 10, 2 / 10, 0]])
    assert np.allclose(P.softmax_with_sink(s + 900.0, m, 0.0), [[1 / 3, 2 / 3, 0]])       # no overflow, the sink vanishes
    assert np.allclose(P.softmax_with_sink(s - 900.0, m, 0.0), 0.0)                       # all weight on the sink


def test_query_temperature_by_hand():
    t = P.query_temperature(10, 0.5, 4)
    assert np.allclose(t[:3], 1.0) and np.allclose(t[3:7], 1 + 0.5 * math.log(2)) and np.allclose(t[7:], 1 + 0.5 * math.log(3))
    assert np.allclose(P.query_temperature(2, 2.0, 4, first_pos=9), 1 + 2.0 * math.log(1 + 2))    # positions 9 and 10: floor(10 / 4) = floor(11 / 4) = 2
    assert np.allclose(P.query_temperature(3, 1.0, 2.5), [1.0, 1.0, 1 + math.log(2)])    # floor(1/2.5), floor(2/2.5), floor(3/2.5)


def test_routing_and_weights_on_the_input_by_hand():
    h = np.array([[1.0, 0.0], [0.0, 2.0]])
    router = np.array([[3.0, 0.0], [1.0, 1.0], [0.0, -1.0]])
    idx, wt = P.route(h, router, 2)
    assert idx.tolist() == [[0, 1], [1, 0]]                                  # z = [3, 1, 0] and [0, 2, -2]
    assert np.allclose(wt, [[P.sigmoid(3), P.sigmoid(1)], [P.sigmoid(2), 0.5]])     # each score on its own, no renormalising
    w = {"router": router}
    for e in range(3):
        w.update({f"e{e}.gate": np.eye(2) * (e + 1), f"e{e}.up": np.eye(2), f"e{e}.down": np.eye(2)})
    mlp = {"router": {"experts": 3, "top": 2}}
    got = P.mixture(h, w, mlp)
    unit = lambda x, e: P.silu((e + 1) * x) * x
    want0 = unit(P.sigmoid(3) * h[0], 0) + unit(P.sigmoid(1) * h[0], 1)
    want1 = unit(P.sigmoid(2) * h[1], 1) + unit(0.5 * h[1], 0)
    assert np.allclose(got, [want0, want1])
    assert not np.allclose(got[1], P.sigmoid(2) * unit(h[1], 1) + 0.5 * unit(h[1], 0))   # a weight on the output is another number


def test_a_layer_norms_its_sublayers_on_both_sides_and_the_head_is_the_table():
    cfg = copy.deepcopy(CONFIGS["C"][0])
    w = {k: v.float().numpy() for k, v in make_weights(cfg, 9).items()}
    toks = [3, 1, 4, 1, 5, 9, 2, 6]
    logits, after = P.forward(cfg, w, toks, True)
    assert after.shape == (len(P.layer_order(cfg)), len(toks), cfg["width"])
    x0 = w["embed"].astype(np.float64)[toks]
    eps = cfg["norm"]["eps"]
    mix = P.windowed_sink_attention(P.rms_norm(x0, w["l0.norm1"], eps), P.sub(w, "l0.mix."), cfg["layers"][0]["mixer"], eps)
    x1 = x0 + P.rms_norm(mix, w["l0.norm1b"], eps)
    ff = P.mixture(P.rms_norm(x1, w["l0.norm2"], eps), P.sub(w, "l0.mlp."), cfg["layers"][0]["mlp"])
    assert np.allclose(after[0], x1 + P.rms_norm(ff, w["l0.norm2b"], eps))
    assert np.allclose(logits, P.rms_norm(after[-1], w["final.norm"], eps) @ w["embed"].astype(np.float64).T)
    la = CONFIGS["A"][0]
    assert P.layer_order(la) == [0, 1, 2, 1, 2, 3]
