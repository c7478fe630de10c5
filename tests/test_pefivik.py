"""Pefivik without a GPU: its configuration and description (the runs of a stretch that is repeated, each with a
cache of its own; what a pass adds to the stream), the state that the embedding keeps, and the plain implementation's
mechanisms against closed forms written here."""
import json

import numpy as np
import pytest

import pefivik_util as pu
from plain import pefivik_plain as plain


def test_config_round_trip_and_description():
    from air_b200.config import load_config, ConfigError
    from air_b200.parts import registry
    from air_b200.engine.model import Model
    for name in ("A", "B", "C", "random4", "random7"):
        pu.model_folder(name)
        cfg = pu.CONFIGS[name]
        c = load_config(cfg)
        assert c.architecture == "Pefivik" and c.width == cfg["width"] and len(c.layers) == len(cfg["layers"])
        assert load_config(c.to_dict()) == c
        model = Model(registry.architecture(c.architecture).build_spec(c))
        names = {t.name: tuple(t.shape) for t in model.tensor_specs() if not t.optional}
        assert {n: a.shape for n, a in pu.draw_tensors(cfg, 0).items()} == names
    with pytest.raises(ConfigError):
        load_config(dict(pu.CONFIGS["B"], layers=[dict(type="conv", mixer={})]))
    with pytest.raises(ConfigError):
        load_config({k: v for k, v in pu.CONFIGS["B"].items() if k != "residual_mult"})
    with pytest.raises(ConfigError):
        load_config({k: v for k, v in pu.CONFIGS["B"].items() if k != "embedding"})
    with pytest.raises(ConfigError):
        load_config(dict(pu.CONFIGS["A"], loop=dict(start=3, stop=2, times=2)))
    with pytest.raises(ConfigError):
        load_config(dict(pu.CONFIGS["A"], loop=dict(start=0, stop=9, times=2)))
    bad = json.loads(json.dumps(pu.CONFIGS["A"]))
    bad["layers"][0]["mlp"]["router"]["top"] = 5           # two groups of two take part
    with pytest.raises(ConfigError):
        load_config(bad)
    bad = json.loads(json.dumps(pu.CONFIGS["A"]))
    bad["layers"][0]["mlp"]["router"]["groups"]["count"] = 4      # six experts
    with pytest.raises(ConfigError):
        load_config(bad)
    bad = json.loads(json.dumps(pu.CONFIGS["A"]))
    bad["layers"][1]["mlp"]["kind"] = "glu"
    with pytest.raises(ConfigError):
        load_config(bad)


def test_runs_of_a_repeated_stretch_and_what_each_keeps():
    from air_b200.config import load_config
    from air_b200.parts import registry
    from air_b200.engine.model import Model
    from air_b200.parts.base import PagedLatent, SlotState
    c = load_config(pu.CONFIGS["A"])
    spec = registry.architecture(c.architecture).build_spec(c)
    assert [r.layer for r in spec.order] == [0, 1, 0, 1, 0, 1, 2, 3, 4]
    assert [r.add_row for r in spec.order] == [("loop.step", 0), None, ("loop.step", 1), None, ("loop.step", 2), None,
                                               None, None, None]
    assert [r.add_embedding for r in spec.order] == [False, False, True, False, True, False, False, False, False]
    assert all(r.cache_from is None for r in spec.order)
    assert [(l, t) for l, t in plain.run_order(5, pu.CONFIGS["A"]["loop"])] == \
        [(0, 0), (1, None), (0, 1), (1, None), (0, 2), (1, None), (2, None), (3, None), (4, None)]
    needs = Model(spec).cache_needs()
    # every pass has a cache of its own; behind the runs, the token before (the embedding's state)
    assert len(needs) == 10 and needs[0] == needs[2] == needs[4] == (PagedLatent(40, None),)
    assert needs[1] == needs[3] == (SlotState((3, 20, 12)),) and needs[9] == (SlotState((1,), "int32"),)
    assert "feed_forward" not in spec.layers[2].parts and spec.layers[2].params["residual_scale"] == 0.6
    f = spec.layers[0].parts["feed_forward"]
    assert f["groups"] == (3, 2) and f["weight_on"] == "output" and f["route_scale"] == 1.7 and f["renormalize"]
    assert spec.logit_softcap == 12.0 and spec.embedding["buckets"] == 389 and spec.stream_tables == (("loop.step", 3),)
    # no stretch: no table, no run adds anything; a stretch that runs once still adds its row
    b = load_config(pu.CONFIGS["B"])
    spec = registry.architecture(b.architecture).build_spec(b)
    assert spec.stream_tables == () and [r.layer for r in spec.order] == [0, 1, 2, 3]
    assert not any(r.add_embedding or r.add_row for r in spec.order)
    c3 = load_config(pu.CONFIGS["C"])
    spec = registry.architecture(c3.architecture).build_spec(c3)
    assert [(r.layer, r.add_row, r.add_embedding) for r in spec.order] == \
        [(0, None, False), (1, ("loop.step", 0), False), (2, None, False)]


def test_cache_keeps_a_state_per_pass_and_frees_everything():
    from air_b200.cache.manager import CacheManager
    from air_b200.config import load_config
    from air_b200.parts import registry
    from air_b200.engine.model import Model
    c = load_config(pu.CONFIGS["A"])
    model = Model(registry.architecture(c.architecture).build_spec(c))
    cache = CacheManager(model.cache_needs(), 16, 12, 2, allocate=False)
    assert len(cache.groups) == 3            # latents of 40, 56 and 24 numbers
    assert sorted(len(g.runs) for g in cache.groups) == [1, 1, 3]
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


def test_plain_mechanisms_against_closed_forms():
    rng = np.random.default_rng(0)
    # the table of pairs: the hash of (previous, current), the last row for a first token
    table, pairs = rng.normal(size=(50, 4)), rng.normal(size=(8, 4))
    x = plain.embed_tokens([3, 10, 49], table, pairs, 7, 5, 3)
    assert np.allclose(x[0], table[3] + pairs[7]) and np.allclose(x[1], table[10] + pairs[(3 * 5 + 10 * 3) % 7])
    assert np.allclose(x[2], table[49] + pairs[(10 * 5 + 49 * 3) % 7])
    # a forget gate that is constant: the state is a geometric sum of what was written
    H, d, dv, E, T = 1, 2, 3, 4, 6
    w = {"q": np.zeros((H * d, E)), "f": np.zeros((H * d, E)), "f.b": np.zeros(H * d), "lower": np.array([0.5, 0.0]),
         "v": rng.normal(size=(H * dv, E)), "norm": np.ones(dv), "o": np.eye(E)[:, :dv]}
    h = rng.normal(size=(T, E))
    state = np.zeros((H, d, dv))
    plain.hgrn2(h, w, dict(heads=H, dim=d, vdim=dv), 1e-6, state)
    f = np.array([0.75, 0.5])                              # l + (1 - l) sigmoid(0)
    v = h @ w["v"].T
    want = sum((f ** (T - 1 - t))[:, None] * (1 - f)[:, None] * v[t][None, :] for t in range(T))
    assert np.allclose(state[0], want)
    # PolyNorm: every power is divided by its own root mean square
    z = rng.normal(size=(2, 9))
    y = plain.poly_norm(z, np.array([2.0, 3.0, 5.0, 7.0]), 0.0)
    n = lambda u: u / np.sqrt((u * u).mean(-1, keepdims=True))
    assert np.allclose(y, 2 * n(z) + 3 * n(z ** 2) + 5 * n(z ** 3) + 7)
    # the router: groups of consecutive experts, marks from the best two scores, the best groups, then the best experts
    s = np.array([0.9, 0.1, 0.5, 0.45, 0.6, 0.3, 0.2, 0.8])
    assert plain.route(s, 2, 4, 2) == [0, 7]               # marks 1.0, 0.95, 0.9, 1.0: groups 0 and 3
    assert plain.route(s, 3, 4, 3) == [0, 7, 2]            # ... and group 1
    assert plain.route(s, 2, 1, 1) == [0, 7] and plain.route(s, 3, 8, 3) == [0, 7, 4]
    assert plain.route(np.full(6, 0.5), 3, 3, 2) == [0, 1, 2]      # equal marks and scores: the lower index
    # a sink takes weight: one key, score 0, sink 0 -> half of the value
    w = {"q": np.zeros((2, 3)), "dkv": np.eye(3)[:2], "dkv.norm": np.ones(2), "uk": np.zeros((2, 2)), "uv": np.eye(2),
         "sink": np.array([0.0]), "g": np.zeros((1, 3)), "o": np.eye(2)}
    out = plain.latent_attention(np.array([[3.0, 4.0, 0.0]]), w, dict(heads=1, dim=2, vdim=2, scale=1.0), 0.0)
    c = np.array([3.0, 4.0]) / np.sqrt(12.5)
    assert np.allclose(out[0], 0.5 * 0.5 * c)              # half to the sink, and the gate sigmoid(0)


def test_oracle_in_32_bit_is_close_to_itself_in_64():
    cfg, tensors = pu.plain_model("A")
    toks = pu.tokens_for("A", 60, 1)
    a = plain.forward(cfg, tensors, toks)
    b = plain.forward(cfg, tensors, toks, dtype=np.float32)
    assert np.abs(a - b).max() < 1e-4 * np.abs(a).max()
    assert pu.plain_run("A", toks)[1] > 0.01
