"""Tabopel without a GPU: its configuration and description (the runs of a stretch that is repeated, each with a cache
of its own; what a pass adds to the stream; which options each mixer switches on), what every run keeps per request,
and the plain implementation's mechanisms against closed forms written here."""
import json
import math

import numpy as np
import pytest

import tabopel_util as tu
from plain import tabopel_plain as plain


def test_config_round_trip_and_description():
    from air_b200.config import load_config, ConfigError
    from air_b200.parts import registry
    from air_b200.engine.model import Model
    for name in ("A", "B", "C", "D", "random4", "random7", "random11"):
        tu.model_folder(name)
        cfg = tu.CONFIGS[name]
        c = load_config(cfg)
        assert c.architecture == "Tabopel" and c.width == cfg["width"] and len(c.layers) == len(cfg["layers"])
        assert load_config(c.to_dict()) == c
        assert load_config(tu.model_folder(name)) == c
        model = Model(registry.architecture(c.architecture).build_spec(c))
        names = {t.name: tuple(t.shape) for t in model.tensor_specs() if not t.optional}
        assert {n: a.shape for n, a in tu.draw_tensors(cfg, 0).items()} == names
    with pytest.raises(ConfigError):
        load_config(dict(tu.CONFIGS["B"], layers=[dict(type="conv", mixer={})]))
    with pytest.raises(ConfigError):
        load_config({k: v for k, v in tu.CONFIGS["B"].items() if k != "norm"})
    with pytest.raises(ConfigError):
        load_config(dict(tu.CONFIGS["A"], loop=dict(start=3, stop=2, times=2)))
    with pytest.raises(ConfigError):
        load_config(dict(tu.CONFIGS["A"], loop=dict(start=0, stop=9, times=2)))
    bad = json.loads(json.dumps(tu.CONFIGS["A"]))
    bad["layers"][0]["mlp"]["router"]["top"] = 7           # five experts and an identity expert
    with pytest.raises(ConfigError):
        load_config(bad)
    bad = json.loads(json.dumps(tu.CONFIGS["A"]))
    bad["layers"][0]["mixer"]["decay"] = [0.5]             # three heads
    with pytest.raises(ConfigError):
        load_config(bad)
    bad = json.loads(json.dumps(tu.CONFIGS["A"]))
    bad["layers"][1]["mixer"]["rot"]["dims"] = 26          # a head of 24
    with pytest.raises(ConfigError):
        load_config(bad)
    bad = json.loads(json.dumps(tu.CONFIGS["A"]))
    bad["layers"][1]["mlp"]["kind"] = "glu"
    with pytest.raises(ConfigError):
        load_config(bad)


def test_runs_of_a_repeated_stretch_and_what_each_keeps():
    from air_b200.config import load_config
    from air_b200.parts import registry
    from air_b200.engine.model import Model
    from air_b200.parts.base import PagedKV, SlotState
    c = load_config(tu.CONFIGS["A"])
    spec = registry.architecture(c.architecture).build_spec(c)
    assert [r.layer for r in spec.order] == [0, 1, 0, 1, 0, 1, 2, 3, 4]
    assert [r.add_row for r in spec.order] == [("loop.step", 0), None, ("loop.step", 1), None, ("loop.step", 2), None,
                                               None, None, None]
    assert not any(r.add_embedding for r in spec.order) and all(r.cache_from is None for r in spec.order)
    assert plain.run_order(tu.CONFIGS["A"]) == [(0, 0), (1, None), (0, 1), (1, None), (0, 2), (1, None), (2, None),
                                                (3, None), (4, None)]
    needs = Model(spec).cache_needs()
    # every pass has a state or pages of its own; the convolutions' last inputs are a state beside the pages
    assert len(needs) == 10 and needs[0] == needs[2] == needs[4] == (SlotState((3, 20, 12)),)
    assert needs[1] == needs[3] == (PagedKV(4, 24, None, 20, None), SlotState((4 * 24 + 4 * 24 + 4 * 20, 2)))
    assert needs[6] == (PagedKV(2, 16, None, 24, None),) and needs[9] == ()
    assert all(b.kind == "sandwich" for b in spec.layers) and "feed_forward" not in spec.layers[2].parts
    first, second = spec.layers[1].parts["mixer"], spec.layers[2].parts["mixer"]
    assert first.kind == second.kind == "normed_attention"
    assert (first["sink"], first["qk_norm"], first["conv"], first["out_gate"], first["qkv_bias"], first["softcap"]) == \
        ("zero", False, 3, True, False, 0.0)
    assert (second["sink"], second["qk_norm"], second["conv"], second["out_gate"], second["qkv_bias"],
            second["softcap"]) == ("learned", "whole", 0, False, True, 3.0)
    assert first["position"]["rule"] == "banded" and first["position"]["scaling"]["original"] == 64
    f = spec.layers[0].parts["feed_forward"]
    assert (f["experts"], f["identity"], f["top"], f["score"], f["choice_bias"], f["gated"], f["weight_on"]) == \
        (5, 1, 2, "softmax", True, False, "output")
    assert spec.embedding_multiplier == 3.0 and spec.stream_tables == (("loop.step", 3),)
    # no stretch: no table, no run adds anything; a stretch that runs once still adds its row
    b = load_config(tu.CONFIGS["B"])
    spec = registry.architecture(b.architecture).build_spec(b)
    assert spec.stream_tables == () and [r.layer for r in spec.order] == [0, 1, 2, 3]
    assert not any(r.add_row for r in spec.order)
    assert spec.layers[0].parts["mixer"]["position"] is None and spec.layers[2].parts["mixer"]["conv"] == 0
    c3 = load_config(tu.CONFIGS["C"])
    spec = registry.architecture(c3.architecture).build_spec(c3)
    assert [(r.layer, r.add_row) for r in spec.order] == [(0, None), (1, ("loop.step", 0)), (2, None)]


def test_cache_keeps_pages_and_states_per_pass_and_frees_everything():
    from air_b200.cache.manager import CacheManager
    from air_b200.config import load_config
    from air_b200.parts import registry
    from air_b200.engine.model import Model
    c = load_config(tu.CONFIGS["A"])
    model = Model(registry.architecture(c.architecture).build_spec(c))
    cache = CacheManager(model.cache_needs(), 16, 12, 2, allocate=False)
    assert sorted(len(g.runs) for g in cache.groups) == [1, 1, 1, 3]      # the looped attention's three passes share a group
    cache.open("a")
    cache.reserve([("a", 40)])
    cache.commit("a", 40)
    assert cache.used_pages("a") == 3
    cache.open("b")
    cache.reserve([("b", 100)])
    cache.commit("b", 100)
    with pytest.raises(Exception):
        cache.reserve([("a", 60)])            # 3 + 7 pages held, 4 more wanted of 12
    cache.close("b")
    cache.reserve([("a", 60)])
    cache.commit("a", 60)
    cache.check()
    cache.close("a")
    assert cache.free_pages() == 12


def test_frequencies_slowed_down_in_bands():
    import torch
    from air_b200.parts.rope import banded_frequencies
    # the three bands by hand: wavelengths below original / high stay, above original / low are divided, between blend
    r = dict(dims=8, base=100.0, scaling=dict(factor=4.0, low=1.0, high=4.0, original=40.0))
    f = np.array([100.0 ** (-2 * i / 8) for i in range(4)])       # wavelengths 6.28, 19.9, 62.8, 198.7
    s1 = (40.0 / (2 * math.pi / f[1]) - 1.0) / 3.0
    want = np.array([f[0], (1 - s1) * f[1] / 4 + s1 * f[1], f[2] / 4, f[3] / 4])
    assert np.allclose(plain.frequencies(r), want)
    assert 10.0 < 2 * math.pi / f[1] < 40.0 and 2 * math.pi / f[0] < 10.0 and 2 * math.pi / f[2] > 40.0
    got, magnitude = banded_frequencies(8, 100.0, r["scaling"])
    assert magnitude == 1.0 and got.dtype == torch.float64 and np.allclose(got.numpy(), want, rtol=1e-14)
    for mx in (l["mixer"] for cfg in tu.CONFIGS.values() for l in cfg["layers"]):
        if mx.get("rot"):
            got, _ = banded_frequencies(mx["rot"]["dims"], mx["rot"]["base"], mx["rot"].get("scaling"))
            assert np.allclose(got.numpy(), plain.frequencies(mx["rot"]), rtol=1e-14)


def test_plain_mechanisms_against_closed_forms():
    rng = np.random.default_rng(0)
    # rotation: a pair at position p turns by p * f; the part behind `dims` stays; scores depend on the distance only
    r = dict(dims=4, base=10.0)
    x = rng.normal(size=(1, 1, 6))
    y = plain.rotate(np.repeat(x, 3, axis=0), [0, 1, 5], r, np.float64)
    assert np.allclose(y[0], x[0]) and np.allclose(y[:, :, 4:], x[:, :, 4:])
    f = plain.frequencies(r)
    a, b = x[0, 0, 1], x[0, 0, 3]
    assert np.allclose(y[2, 0, 1], a * math.cos(5 * f[1]) - b * math.sin(5 * f[1]))
    assert np.allclose(y[2, 0, 3], b * math.cos(5 * f[1]) + a * math.sin(5 * f[1]))
    q, k = rng.normal(size=(1, 1, 4)), rng.normal(size=(1, 1, 4))
    d1 = plain.rotate(q, [7], r, np.float64)[0, 0] @ plain.rotate(k, [3], r, np.float64)[0, 0]
    d2 = plain.rotate(q, [104], r, np.float64)[0, 0] @ plain.rotate(k, [100], r, np.float64)[0, 0]
    assert np.allclose(d1, d2)
    # the convolution: taps on the inputs before, zeros ahead of the sequence, the last tap on the token itself
    u = rng.normal(size=(5, 2))
    w = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 2.0]])
    y = plain.causal_conv(u, w)
    assert np.allclose(y[0, 0], 100 * u[0, 0]) and np.allclose(y[1, 0], 10 * u[0, 0] + 100 * u[1, 0])
    assert np.allclose(y[4, 0], u[2, 0] + 10 * u[3, 0] + 100 * u[4, 0]) and np.allclose(y[:, 1], 2 * u[:, 1])
    # a sink takes weight: one key of score 0 beside a sink of 0 gets half; a sink far below takes nothing
    one = np.ones((1, 1, 2))
    v = np.array([[[3.0, 5.0]]])
    assert np.allclose(plain.softmax_attention(0 * one, one, v, 1.0, sink=np.zeros(1))[0, 0], [1.5, 2.5])
    assert np.allclose(plain.softmax_attention(0 * one, one, v, 1.0, sink=np.full(1, -80.0))[0, 0], [3.0, 5.0])
    # the cap bounds a score: a huge score and one at the cap weigh alike
    q2 = np.array([[[0.0]], [[1000.0]]])
    k2 = np.array([[[0.0]], [[1.0]]])
    v2 = np.array([[[1.0]], [[0.0]]])
    out = plain.softmax_attention(q2, k2, v2, 1.0, softcap=2.0)
    assert np.allclose(out[1, 0, 0], 1.0 / (1.0 + math.exp(2.0)), rtol=1e-6)
    # retention: the state is a geometric sum of the outer products
    H, d, dv, E, T = 1, 2, 3, 4, 6
    w = {"m.q": rng.normal(size=(d, E)), "m.k": rng.normal(size=(d, E)), "m.v": rng.normal(size=(dv, E)),
         "m.g": np.zeros((dv, E)), "m.o": np.eye(dv)}
    h = rng.normal(size=(T, E))
    m = dict(heads=H, dim=d, vdim=dv, decay=[0.5], rot=dict(dims=0, base=1.0))
    out = plain.mixer_retention(w, "m.", h, m, np.arange(T), 0.0, np.float64)
    q, k, v = h @ w["m.q"].T, h @ w["m.k"].T * d ** -0.5, h @ w["m.v"].T
    S = sum(0.5 ** (T - 1 - t) * np.outer(k[t], v[t]) for t in range(T))
    o = S.T @ q[-1]
    assert np.allclose(out[-1], o / np.sqrt((o * o).mean()) * 0.0)       # silu(0) = 0: the gate closes the read-out
    w["m.g"] = rng.normal(size=(dv, E))
    out = plain.mixer_retention(w, "m.", h, m, np.arange(T), 0.0, np.float64)
    assert np.allclose(out[-1], o / np.sqrt((o * o).mean()) * plain.silu(h[-1] @ w["m.g"].T))
    # the router: chosen by score plus correction, weighted by the score; the last outputs return the input
    f = dict(kind="moe", expert=dict(ff=2), router=dict(experts=2, identity=1, top=2))
    w = {"f.router": np.array([[1.0, 0.0], [0.0, 1.0], [0.0, 0.0]]), "f.correction": np.array([0.0, -1.0, 0.3]),
         "f.e0.up": np.eye(2), "f.e0.down": 2 * np.eye(2), "f.e1.up": np.eye(2), "f.e1.down": np.eye(2)}
    u = np.array([[1.0, 2.0]])
    chosen, weights, margin = plain.route(w, "f.", u, f)
    s = np.exp([1.0, 2.0, 0.0]) / np.exp([1.0, 2.0, 0.0]).sum()
    assert chosen.tolist() == [[2, 0]] and np.allclose(weights, [[s[2], s[0]]])      # expert 1 has the best score, and is left
    assert np.allclose(margin, (s[0] + 0.0) - (s[1] - 1.0))
    assert np.allclose(plain.moe_ff(w, "f.", u, f), s[2] * u + s[0] * 2 * u ** 2)
    assert np.allclose(plain.dense_ff({"f.up": np.array([[1.0, -1.0]]), "f.down": np.array([[3.0], [4.0]])}, "f.",
                                      np.array([[5.0, 2.0], [1.0, 2.0]])), [[27.0, 36.0], [0.0, 0.0]])


def test_oracle_in_32_bit_is_close_to_itself_in_64_and_routers_choose_clearly():
    cfg, tensors = tu.plain_model("A")
    toks = tu.tokens_for("A", 60, 1)
    a = plain.forward(cfg, tensors, toks)
    b = plain.forward(cfg, tensors, toks, dtype=np.float32)
    assert np.abs(a - b).max() < 1e-4 * np.abs(a).max()
    for name in ("A", "B", "C", "D"):
        assert tu.plain_run(name, tu.tokens_for(name, 80, 2))[1] > 0.01, name


def test_every_mechanism_of_the_test_models_matters():
    """Leaving one mechanism out of the oracle moves the logits far beyond what rounding does: a test that passes
    would not pass with the mechanism missing."""
    cfg, tensors = tu.plain_model("A")
    toks = tu.tokens_for("A", 70, 3)
    ref = plain.forward(cfg, tensors, toks)
    scale = np.abs(ref).max()

    def moved(change):
        c, t = json.loads(json.dumps(cfg)), dict(tensors)
        change(c, t)
        return np.abs(plain.forward(c, t, toks) - ref).max() / scale

    assert moved(lambda c, t: t.update({"l2.mix.sink": np.full_like(t["l2.mix.sink"], -60.0)})) > 0.02
    assert moved(lambda c, t: c["layers"][2]["mixer"].update(softcap=0.0)) > 0.005
    assert moved(lambda c, t: c["layers"][1]["mixer"]["rot"].pop("scaling")) > 0.02
    assert moved(lambda c, t: t.update({"l1.mix.q.conv": np.roll(t["l1.mix.q.conv"], 1, axis=1)})) > 0.02
    # (the corrections decide a token's further experts, whose scores are small here: the router's test is the part's)
    assert moved(lambda c, t: t.update({"l0.mlp.router": np.roll(t["l0.mlp.router"], 1, axis=0)})) > 0.02
    assert moved(lambda c, t: c["layers"][0]["mixer"].update(decay=[0.9, 0.9, 0.9])) > 0.02
    assert moved(lambda c, t: t.update({"loop.step": np.roll(t["loop.step"], 1, axis=0)})) > 0.02
    assert moved(lambda c, t: c["embedding"].update(scale=1.0)) > 0.02
