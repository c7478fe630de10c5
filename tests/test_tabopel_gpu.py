"""Tabopel on the GPU against the plain implementation (tests/plain/tabopel_plain.py, 64-bit): every mechanism alone
through its part or kernel, then whole models through Engine.step, the scheduler and the trace runner, in float32 and
bfloat16, for configurations that differ in every size and option (tabopel_util.CONFIGS)."""
import tempfile
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import tabopel_util as tu
import util
from plain import tabopel_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.ascontiguousarray(a)).to(device=DEV, dtype=dtype)


def i32(a):
    return torch.tensor(list(a), dtype=torch.int32, device=DEV)


def runtime(dtype, page=16):
    from air_b200.parts.base import Runtime
    return Runtime(torch.device(DEV), DT[dtype], page, status=torch.zeros(1, dtype=torch.int32, device=DEV))


def context_for(cache, entries, part=None):
    from air_b200.engine.batch import Entry, build_context
    entries = [Entry(*e) for e in entries]
    for e in entries:
        if e.request not in cache.sequences:
            cache.open(e.request)
    cache.reserve([(e.request, len(e.tokens)) for e in entries])
    return build_context(entries, cache, DEV, status=torch.zeros(1, dtype=torch.int32, device=DEV),
                         planners=[part] if part is not None and part.plan_key() is not None else ())


def summed(y):
    return (y.sum(0) if y.dim() == 3 else y).float().cpu().numpy()


def rounded(w, dtype):
    return {k: tu.bf16(a).astype(np.float64) for k, a in w.items()} if dtype == "bfloat16" else w


WIDE = ("sink", "q.norm", "k.norm", "q.b", "k.b", "v.b", "q.conv", "k.conv", "v.conv", "correction", "router")


def load(part, w, dtype, page=16, prefix="m."):
    part.load({prefix + k: dev(a, torch.float32 if k in WIDE else DT[dtype]) for k, a in w.items()}, runtime(dtype, page))
    return part


def run_in_steps(part, cache, streams, steps, dtype):
    """streams: request -> inputs [T, E]; steps: lists of (request, tokens).  Returns request -> outputs [T, E]."""
    done = {r: 0 for r in streams}
    outs = {r: [] for r in streams}
    for step in steps:
        entries = [(r, [0] * n, []) for r, n in step]
        ctx = context_for(cache, entries, part)
        x = np.concatenate([streams[r][done[r]:done[r] + n] for r, n in step])
        y = summed(part.forward(dev(x, DT[dtype]), ctx, cache.views(0), True))
        at = 0
        for r, n in step:
            outs[r].append(y[at:at + n])
            cache.commit(r, n)
            done[r] += n
            at += n
    assert all(done[r] == len(streams[r]) for r in streams)
    return {r: np.concatenate(o) for r, o in outs.items()}


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,parts", [(13, 72, 3), (5, 90, 1), (300, 256, 2), (2, 2048, 4), (7, 10, 1)])
def test_norm_behind_a_sub_layer_then_sum_then_norm(T, E, parts, dtype):
    """h += n(d; wb); out = n(h; w) in one kernel, d as a tensor or as partial sums; for chosen rows the stream stays."""
    from air_b200.parts.base import NormedSum, Norm
    from air_b200.parts.norm import RMSNorm
    from air_b200.parts.spec import PartSpec
    rng = np.random.default_rng(T + E)
    eps_b, eps = 1e-5, 1e-6
    h, d = rng.normal(size=(T, E)) * 3, rng.normal(size=(parts, T, E)) * rng.uniform(0.01, 30.0, size=(1, T, 1))
    wb, w = rng.normal(1.0, 0.3, size=E), rng.normal(1.0, 0.3, size=E)
    part = RMSNorm(PartSpec("rms", {"size": E, "eps": eps, "tensor": ""}), "n")
    part.load({"n": dev(w)}, runtime(dtype))
    x = h + plain.rms_norm(d.sum(0), wb, eps_b)
    want = plain.rms_norm(x, w, eps)
    tol = 2e-5 if dtype == "float32" else 2e-2
    for term in ((dev(d),) if parts > 1 else (dev(d), dev(d[0]))):
        hd = dev(h)
        out = part.forward(hd, NormedSum(term, dev(wb), eps_b))
        assert np.abs(hd.cpu().numpy() - x).max() < 2e-5 * np.abs(x).max()
        assert np.abs(out.float().cpu().numpy() - want).max() < tol * np.abs(want).max()
    rows = i32([T - 1, 0, T // 2])
    hd = dev(h)
    out = part.forward(hd, NormedSum(dev(d), dev(wb), eps_b), rows=rows)
    assert np.array_equal(hd.cpu().numpy(), h.astype(np.float32))
    assert np.abs(out.float().cpu().numpy() - want[[T - 1, 0, T // 2]]).max() < tol * np.abs(want).max()
    hd = dev(h)
    Norm.add_delta(hd, NormedSum(dev(d), dev(wb), eps_b))
    assert np.abs(hd.cpu().numpy() - x).max() < 2e-5 * np.abs(x).max()


def attention_weights(rng, E, H, G, d, dv, scale, kind, taps, dtype):
    sharp = (2.5 / (scale * d ** 0.5)) ** 0.5
    w = {"v": rng.normal(size=(G * dv, E)) / E ** 0.5, "o": rng.normal(size=(E, H * dv)) / (H * dv) ** 0.5}
    if kind == "attention":
        w.update(q=rng.normal(size=(H * d, E)) * sharp / E ** 0.5, k=rng.normal(size=(G * d, E)) * sharp / E ** 0.5,
                 g=rng.normal(size=(H * dv, E)) * 2.0 / E ** 0.5)
        for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
            if taps:
                w[n + ".conv"] = rng.normal(size=(rows, taps)) / taps ** 0.5 + np.where(np.arange(taps) == taps - 1, 0.6, 0)
    else:
        w.update(q=rng.normal(size=(H * d, E)) / E ** 0.5, k=rng.normal(size=(G * d, E)) / E ** 0.5,
                 sink=rng.normal(1.0, 2.0, size=H))
        w["q.norm"], w["k.norm"] = sharp * rng.normal(1.0, 0.15, size=H * d), sharp * rng.normal(1.0, 0.15, size=G * d)
        for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
            w[n + ".b"] = rng.normal(0.0, 0.3, size=rows)
    return rounded(w, dtype)


def attention_part(kind, E, H, G, d, dv, scale, taps, cap, r, eps):
    from air_b200.parts.normed_attention import NormedAttention
    from air_b200.parts.spec import PartSpec
    first = kind == "attention"
    position = PartSpec("rope_live", {"rotary_dim": r["dims"] if r else 0, "theta": r["base"] if r else 1.0,
                                      "pairing": "half", "rule": "banded", "scaling": (r or {}).get("scaling")})
    return NormedAttention(PartSpec("normed_attention", {
        "hidden": E, "heads": H, "kv_heads": G, "head_dim": d, "v_dim": dv, "scale": scale, "eps": eps,
        "position": position, "qk_norm": False if first else "whole", "sink": "zero" if first else "learned",
        "qkv_bias": not first, "conv": taps if first else 0, "softcap": 0.0 if first else cap, "out_gate": first}), "m.")


ATTENTION_CASES = [
    # kind, H, G, d, dv, taps, cap, rot, page
    ("attention", 4, 4, 24, 20, 3, 0.0, tu.rot(24, 10000.0, (8.0, 1.0, 4.0, 64)), 16),
    ("attention", 2, 1, 40, 8, 2, 0.0, tu.rot(20, 300.0), 16),
    ("attention", 6, 3, 16, 16, 0, 0.0, None, 32),
    ("attention", 4, 2, 64, 64, 5, 0.0, tu.rot(32, 500000.0, (4.0, 1.0, 4.0, 96)), 64),
    ("attention", 3, 1, 10, 6, 1, 0.0, tu.rot(6, 1000.0), 16),
    ("attention_2", 6, 2, 16, 24, 0, 3.0, tu.rot(8, 500000.0), 16),
    ("attention_2", 1, 1, 32, 40, 0, 0.0, tu.rot(32, 10000.0), 16),
    ("attention_2", 2, 1, 128, 64, 0, 6.0, tu.rot(64, 10000.0), 64),
    ("attention_2", 2, 2, 14, 10, 0, 4.0, tu.rot(2, 10000.0), 16),
    # keys and values of one size that the copy-engine decode kernel takes: cap, learned sink (and above: zero sink, gates)
    ("attention_2", 4, 2, 128, 128, 0, 6.0, tu.rot(64, 10000.0), 64),
    ("attention_2", 2, 2, 64, 64, 0, 4.0, tu.rot(32, 500.0), 16),
    ("attention", 8, 1, 128, 128, 4, 0.0, tu.rot(128, 500000.0, (8.0, 1.0, 4.0, 256)), 32),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind,H,G,d,dv,taps,cap,r,page", ATTENTION_CASES)
def test_attention_mixers_through_portions_and_single_tokens(kind, H, G, d, dv, taps, cap, r, page, dtype):
    """A mixer alone over two requests in steps that hold both: long portions (the road of matrix products over gathered
    keys in bfloat16), short ones down to two tokens and single tokens (the kernel that reads the pages), against the
    plain function on each whole sequence.  Scores are as sharp as a trained model's and the sinks of the scores' order
    (a sink that is left out shows: checked on the plain side); the convolution's last inputs travel from step to step,
    and a slot that another request held starts from zeros."""
    from air_b200.cache.manager import CacheManager
    E, scale, eps = 80, 0.2, 1e-5
    rng = np.random.default_rng(H * d + dv)
    w = attention_weights(rng, E, H, G, d, dv, scale, kind, taps, dtype)
    streams = {"a": rng.normal(size=(330, E)), "b": rng.normal(size=(75, E))}
    if dtype == "bfloat16":
        streams = {r_: tu.bf16(x).astype(np.float64) for r_, x in streams.items()}
    m = dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=scale, conv=taps, softcap=cap, rot=r)
    fn = plain.mixer_attention if kind == "attention" else plain.mixer_attention_2
    wp = {"m." + k: a for k, a in w.items()}
    want = {r_: fn(wp, "m.", x, m, np.arange(len(x)), eps, np.float64) for r_, x in streams.items()}
    if kind == "attention_2":
        gone = fn(dict(wp, **{"m.sink": np.full(H, -50.0)}), "m.", streams["b"], m, np.arange(75), eps, np.float64)
        assert np.abs(gone - want["b"]).max() > 0.05
    part = load(attention_part(kind, E, H, G, d, dv, scale, taps, cap, r, eps), w, dtype, page)
    cache = CacheManager([part.cache_needs()], page, 40, 3, dtype=DT[dtype], device=DEV)
    cache.open("other")                                        # the requests under test do not sit in slot 0
    steps = [[("a", 3)], [("a", 61), ("b", 1)], [("b", 2), ("a", 1)], [("a", 150), ("b", 40)], [("a", 2)], [("a", 1), ("b", 1)],
             [("b", 31), ("a", 1)], [("a", 40)], [("a", 70)], [("a", 1)]]
    got = run_in_steps(part, cache, streams, steps, dtype)
    tol = 2e-4 if dtype == "float32" else 4e-2
    for r_ in streams:
        assert np.abs(got[r_] - want[r_]).max() < tol * max(1.0, np.abs(want[r_]).max()), (r_, float(np.abs(got[r_] - want[r_]).max()))
    cache.close("b")
    again = run_in_steps(part, cache, {"c": streams["b"]}, [[("c", 5)], [("c", 1)], [("c", 69)]], dtype)     # b's slot and pages
    assert np.abs(again["c"] - want["b"]).max() < tol * max(1.0, np.abs(want["b"]).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind,cap,d,E", [("attention", 0.0, 16, 64), ("attention_2", 40.0, 16, 64),
                                          ("attention", 0.0, 64, 256), ("attention_2", 40.0, 128, 512)])
def test_attention_finds_a_key_far_away_and_at_page_borders(kind, cap, d, E, dtype):
    """Keys and queries are made by hand: late queries point at the keys of tokens 0, 15, 16, 17 and 200 (a score that
    stands out among hundreds; the query is the key turned back by the distance between them), and the values show
    which key was found.  As one prompt, as a prompt with decoded tokens and in ragged portions, over pages of 16 that
    are scattered.  Heads of 64 and 128 take the tile kernels in bfloat16 (tcgen05 for portions, the copy engine's for
    single tokens), the others the kernels that read the pages in 32-bit."""
    from air_b200.cache.manager import CacheManager
    H, G, dv, T, scale, eps = 2, 1, d, 420, 0.25 * (16 / d) ** 0.5, 1e-6
    r = tu.rot(d // 2, 10000.0)
    rng = np.random.default_rng(5)
    w = attention_weights(rng, E, H, G, d, dv, scale, kind, 0, dtype)
    if kind == "attention_2":      # queries and keys as they are projected: no bias, the norm's weight the same everywhere
        w["q.b"], w["k.b"] = np.zeros(H * d), np.zeros(G * d)
        w["q.norm"], w["k.norm"] = np.full(H * d, 2.0), np.full(G * d, 2.0)
    x = rng.normal(size=(T, E)) * 0.3
    marked = {0: 401, 15: 402, 16: 403, 200: 404, 17: 419}
    for j, i in marked.items():
        key = plain.rotate((x[j:j + 1] @ w["k"].T).reshape(1, G, d), [j], r, np.float64)       # as the cache holds it
        back = plain.rotate(np.repeat(key, H, axis=1), [-i], r, np.float64).reshape(-1)        # q_i turned to i is the key
        # x[i] is chosen so that Wq x[i] is that query, enlarged, and Wk x[i] = 0 (its own key does not draw it)
        x[i] = np.linalg.lstsq(np.concatenate([w["q"], w["k"]]),
                               np.concatenate([back * 30.0 / np.abs(back).max(), np.zeros(G * d)]), rcond=None)[0]
    if dtype == "bfloat16":
        x = tu.bf16(x).astype(np.float64)
    m = dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=scale, softcap=cap, rot=r)
    fn = plain.mixer_attention if kind == "attention" else plain.mixer_attention_2
    wp = {"m." + k: a for k, a in w.items()}
    want = fn(wp, "m.", x, m, np.arange(T), eps, np.float64)
    part = load(attention_part(kind, E, H, G, d, dv, scale, 0, cap, r, eps), w, dtype)
    for cuts in ([T], [400] + [1] * 20, [7, 9, 1, 383, 2, 2, 16]):
        cache = CacheManager([part.cache_needs()], 16, 40, 2, dtype=DT[dtype], device=DEV)
        for g in cache.groups:              # pages in an order of their own
            rng.shuffle(g.pool._free)
        got = run_in_steps(part, cache, {"r": x}, [[("r", n)] for n in cuts], dtype)["r"]
        tol = 2e-4 if dtype == "float32" else 4e-2
        assert np.abs(got - want).max() < tol * max(1.0, np.abs(want).max()), (cuts[:3], float(np.abs(got - want).max()))
    # and the marked keys do carry the rows that point at them: without token 0 row 401 is another row
    gone = fn(wp, "m.", x[1:], m, np.arange(1, T), eps, np.float64)
    assert np.abs(gone[400] - want[401]).max() > 0.1 * np.abs(want[401]).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,d,dv,r", [(3, 20, 12, tu.rot(8, 10000.0)), (1, 64, 32, None), (2, 64, 128, tu.rot(64, 100000.0)),
                                       (4, 8, 24, tu.rot(8, 1000.0, (4.0, 1.0, 2.0, 16))), (3, 10, 6, tu.rot(10, 10000.0)),
                                       (2, 100, 64, tu.rot(50, 500.0))])
def test_retention_carries_its_state_through_portions_and_slots(H, d, dv, r, dtype):
    """The mixer alone: two requests in steps that hold both, portions of many sizes and single tokens; some heads
    forget so slowly (a decay of 0.999) that the first token, thirty times the others, still shows after 300; a slot
    that another request held starts from zeros."""
    from air_b200.cache.manager import CacheManager
    from air_b200.parts.recurrent import Retention
    from air_b200.parts.spec import PartSpec
    E, eps = 72, 1e-5
    rng = np.random.default_rng(H * d)
    decay = [(0.9990234375, 0.9, 0.99609375, 0.5)[h % 4] for h in range(H)]
    w = rounded({"q": rng.normal(size=(H * d, E)) * 1.5 / E ** 0.5, "k": rng.normal(size=(H * d, E)) * 1.5 / E ** 0.5,
                 "v": rng.normal(size=(H * dv, E)) / E ** 0.5, "g": rng.normal(size=(H * dv, E)) * 2 / E ** 0.5,
                 "o": rng.normal(size=(E, H * dv)) / (H * dv) ** 0.5}, dtype)
    streams = {"a": rng.normal(size=(320, E)), "b": rng.normal(size=(75, E))}
    streams["a"][0] *= 30.0                                        # a first token that the slow heads remember
    if dtype == "bfloat16":
        streams = {r_: tu.bf16(x).astype(np.float64) for r_, x in streams.items()}
    m = dict(heads=H, dim=d, vdim=dv, decay=decay, rot=r)
    wp = {"m." + k: a for k, a in w.items()}
    want = {r_: plain.mixer_retention(wp, "m.", x, m, np.arange(len(x)), eps, np.float64) for r_, x in streams.items()}
    short = plain.mixer_retention(wp, "m.", streams["a"][1:], m, np.arange(1, 320), eps, np.float64)
    assert np.abs(short[-1] - want["a"][-1]).max() > 0.02 * np.abs(want["a"][-1]).max()      # the first token still shows
    position = None if r is None else PartSpec("rope_live", {"rotary_dim": r["dims"], "theta": r["base"], "pairing": "half",
                                                             "rule": "banded", "scaling": r.get("scaling")})
    part = load(Retention(PartSpec("retention", {"hidden": E, "heads": H, "head_dim": d, "v_dim": dv, "decay": decay,
                                                 "eps": eps, "position": position}), "m."), w, dtype)
    cache = CacheManager([part.cache_needs()], 16, 40, 3, dtype=DT[dtype], device=DEV)
    cache.open("other")
    steps = [[("a", 3)], [("a", 61), ("b", 1)], [("b", 2), ("a", 1)], [("a", 150), ("b", 40)], [("a", 2)], [("a", 1), ("b", 1)],
             [("b", 31), ("a", 1)], [("a", 30)], [("a", 70)], [("a", 1)]]
    got = run_in_steps(part, cache, streams, steps, dtype)
    tol = 2e-4 if dtype == "float32" else 4e-2
    for r_ in streams:
        assert np.abs(got[r_] - want[r_]).max() < tol * max(1.0, np.abs(want[r_]).max()), (r_, float(np.abs(got[r_] - want[r_]).max()))
    cache.close("a")
    again = run_in_steps(part, cache, {"c": streams["b"]}, [[("c", 5)], [("c", 1)], [("c", 69)]], dtype)     # a's slot
    assert np.abs(again["c"] - want["b"]).max() < tol * max(1.0, np.abs(want["b"]).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,F,T", [(72, 100, 11), (96, 40, 70), (128, 256, 150), (40, 8, 3), (90, 50, 65)])
def test_dense_feed_forward_with_the_squared_rectifier(E, F, T, dtype):
    from air_b200.parts.mlp import Relu2MLP
    from air_b200.parts.spec import PartSpec
    rng = np.random.default_rng(E + F)
    w = rounded({"up": rng.normal(size=(F, E)) * 1.4 / E ** 0.5, "down": rng.normal(size=(E, F)) / F ** 0.5}, dtype)
    x = rng.normal(size=(T, E))
    if dtype == "bfloat16":
        x = tu.bf16(x).astype(np.float64)
    part = load(Relu2MLP(PartSpec("relu2_mlp", {"hidden": E, "intermediate": F}), "m."), w, dtype)
    got = summed(part.forward(dev(x, DT[dtype]), SimpleNamespace(residual=None)))
    want = plain.dense_ff({"m." + k: a for k, a in w.items()}, "m.", x)
    assert np.abs(got - want).max() < (1e-4 if dtype == "float32" else 4e-2) * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("M,N,K,bn", [(600, 384, 256, 128), (1100, 512, 320, 256), (130, 96, 64, 32), (9, 512, 256, 256),
                                      (64, 384, 128, 128)])
def test_squared_rectifier_in_the_epilogue_of_the_tensor_core_products(M, N, K, bn):
    """Both tcgen05 products (rows as the M side for many rows, weights as the M side for few) write max(x W^T, 0)^2."""
    from air_b200.csrc import ops
    rng = np.random.default_rng(M + N)
    x, w = tu.bf16(rng.normal(size=(M, K))), tu.bf16(rng.normal(size=(N, K)) / K ** 0.5)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(dev(x, torch.bfloat16), dev(w, torch.bfloat16), out, bn, ops.EPI_RELU2)
    want = plain.relu_squared(x.astype(np.float64) @ w.astype(np.float64).T)
    assert np.abs(out.float().cpu().numpy() - want).max() < 1e-2 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("n,identity,top", [(5, 1, 2), (3, 0, 3), (1, 1, 1), (4, 2, 4), (12, 0, 5), (1, 2, 2), (37, 3, 8)])
def test_router_chooses_by_score_plus_correction_and_weighs_by_score(n, identity, top):
    """The routing kernel alone against the plain router: corrections as large as the scores, so the choice by score
    plus correction is not the choice by score; identity experts take part in the softmax and in the choice."""
    from air_b200.csrc import ops
    rng = np.random.default_rng(n * 10 + top)
    T, E, total = 300, 24, n + identity
    w = {"f.router": rng.normal(size=(total, E)) * 1.5 / E ** 0.5, "f.correction": rng.normal(0.0, 0.2, size=total)}
    u = rng.normal(size=(T, E))
    f = dict(router=dict(experts=n, identity=identity, top=top))
    chosen, weights, _ = plain.route(w, "f.", u, f)
    by_score = np.argsort(-(u @ w["f.router"].T), axis=-1, kind="stable")[:, :top]
    assert total == top or (np.sort(by_score, -1) != np.sort(chosen, -1)).any()
    z = dev(u @ w["f.router"].T)
    expert = torch.empty((T, top), dtype=torch.int32, device=DEV)
    weight = torch.empty((T, top), dtype=torch.float32, device=DEV)
    ops.moe_route(z, total, top, expert, weight, score="softmax", choice_bias=dev(w["f.correction"]))
    # rows whose oracle margin is clear of 32-bit rounding must agree exactly, in the order of the choice scores
    zz = u @ w["f.router"].T
    s = np.exp(zz - zz.max(-1, keepdims=True))
    s /= s.sum(-1, keepdims=True)
    ranked = np.sort(s + w["f.correction"], axis=-1)[:, ::-1]
    clear = (np.abs(np.diff(ranked, axis=-1)).min(-1) > 1e-5) if total > 1 else np.ones(T, bool)
    assert clear.sum() > T * 0.9
    assert np.array_equal(expert.cpu().numpy()[clear], chosen[clear])
    assert np.abs(weight.cpu().numpy()[clear] - weights[clear]).max() < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,identity,top,E,F,T", [(5, 1, 2, 72, 40, 150), (3, 0, 3, 96, 32, 7), (1, 1, 1, 64, 64, 40),
                                                   (4, 2, 4, 128, 32, 300), (12, 0, 5, 128, 64, 70), (1, 2, 2, 90, 30, 33)])
def test_experts_with_identity_experts_on_both_roads(n, identity, top, E, F, T, dtype, monkeypatch):
    """The feed-forward alone against the plain one: experts without a gate, the squared rectifier, weights on the
    outputs, identity experts that return their input; on the road of the package's grouped product and, in bfloat16, on
    the road of the library's.  Rows whose router margin rounding could tip are left out of the comparison."""
    from air_b200.parts.experts import RoutedExperts
    from air_b200.parts.spec import PartSpec
    rng = np.random.default_rng(n + identity + top)
    total = n + identity
    w = {"router": rng.normal(size=(total, E)) * 1.5 / E ** 0.5, "correction": rng.normal(0.0, 0.2, size=total)}
    for x_ in range(n):
        w[f"e{x_}.up"], w[f"e{x_}.down"] = rng.normal(size=(F, E)) * 1.4 / E ** 0.5, rng.normal(size=(E, F)) / F ** 0.5
    w = rounded(w, dtype)
    x = rng.normal(size=(T, E))
    if dtype == "bfloat16":
        x = tu.bf16(x).astype(np.float64)
    f = dict(kind="moe", expert=dict(ff=F), router=dict(experts=n, identity=identity, top=top))
    wp = {"f." + k: a for k, a in w.items()}
    want = plain.moe_ff(wp, "f.", x, f)
    zz = x @ w["router"].T
    s = np.exp(zz - zz.max(-1, keepdims=True))
    s /= s.sum(-1, keepdims=True)
    ranked = np.sort(s + w["correction"], axis=-1)[:, ::-1]
    clear = (ranked[:, top - 1] - ranked[:, top] > (1e-5 if dtype == "float32" else 2e-2)) if total > top else np.ones(T, bool)
    assert clear.sum() > T // 2
    if identity:
        assert (plain.route(wp, "f.", x, f)[0][clear] >= n).any(), "an identity expert is chosen somewhere"
    spec = PartSpec("routed_experts", {"hidden": E, "experts": n, "top": top, "intermediate": F, "score": "softmax",
                                       "renormalize": False, "weight_on": "output", "gated": False, "activation": "relu2",
                                       "choice_bias": True, "identity": identity})
    for rows in ([RoutedExperts.LIBRARY_ROWS] if dtype == "float32" else [RoutedExperts.LIBRARY_ROWS, 0]):
        monkeypatch.setattr(RoutedExperts, "LIBRARY_ROWS", rows)
        part = load(RoutedExperts(spec, "f."), w, dtype, prefix="f.")
        got = summed(part.forward(dev(x, DT[dtype]), SimpleNamespace(residual=None)))
        tol = 1e-4 if dtype == "float32" else 4e-2
        assert np.abs(got - want)[clear].max() < tol * max(1.0, np.abs(want).max()), rows


# ----------------------------------------------------------------------------- whole models
LENGTHS = {"A": (1, 7, 33, 97, 150), "B": (5, 40, 131, 64), "C": (2, 65, 150, 300), "D": (3, 70, 1, 129),
           "E": (130, 2, 310)}


def streams_for(name, seed=0, lengths=None):
    return {f"{name}{i}": tu.tokens_for(name, n, seed + i) for i, n in enumerate(lengths or LENGTHS[name])}


def replay(name, dtype, steps, page_tokens=16, max_requests=4, peak_page=64):
    return util.replay(tu.model_folder(name), dtype, steps, max_tokens=util.peak_tokens(steps, page=peak_page),
                       page_tokens=page_tokens, max_requests=max_requests)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_stream_after_every_run(name, dtype):
    """Layer by layer: the stream behind every run of the order list (a layer that runs three times counts three
    times) against the plain implementation's, for a prompt in one step."""
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig
    cfg, tensors = tu.plain_model(name)
    toks = tu.tokens_for(name, 90, 3)
    want = []
    plain.forward(cfg, tensors, toks, taps=want)
    engine = Engine.from_folder(tu.model_folder(name), EngineConfig(dtype=dtype, page_tokens=16, max_tokens=256,
                                                                    max_requests=2))
    engine.model.tap = []
    engine.step([Entry("r", toks, [])])
    engine.check_status()
    assert len(engine.model.tap) == len(want) == len(engine.model.spec.order)
    for i, (a, b) in enumerate(zip(engine.model.tap, want)):
        tol = 1e-4 if dtype == "float32" else 0.05
        assert np.abs(a.cpu().numpy() - b).max() < tol * np.abs(b).max(), (i, float(np.abs(a.cpu().numpy() - b).max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole_prompts(name, dtype):
    streams = streams_for(name)
    got, _ = replay(name, dtype, util.trace_whole(streams))
    tu.check(got, name, streams, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "E"])
def test_prompt_then_token_by_token(name, dtype):
    streams = streams_for(name, 10)
    got, _ = replay(name, dtype, util.trace_bulk_tail(streams, tail=75))
    tu.check(got, name, streams, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_down_to_two_tokens(name, dtype):
    streams = streams_for(name, 20)
    got, _ = replay(name, dtype, util.trace_portions(streams))
    tu.check(got, name, streams, dtype)
    got, _ = replay(name, dtype, util.trace_portions(streams, sizes=(2, 2, 1, 3, 16, 15, 17, 64, 63, 65, 2)), page_tokens=64)
    tu.check(got, name, streams, dtype)


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_unequal_requests_together_with_pages_and_slots_used_again(name, dtype, page):
    """Ten requests through three slots and a pool that holds the peak only: every request must come out as it does
    alone (the oracle runs each alone), whatever shared its batches and whoever had its slot (retention's states, the
    convolutions' last inputs) and its pages before."""
    lengths = LENGTHS[name] + ((120, 2, 77, 101, 64, 129) if name != "E" else (77, 1, 64))
    streams = streams_for(name, 50, lengths)
    steps = util.trace_mixed(streams, seed=3, live=3)
    got, engine = replay(name, dtype, steps, page_tokens=page, max_requests=3)
    tu.check(got, name, streams, dtype)
    for group in engine.cache.groups:
        assert group.pool.takes > group.pool.num_pages, "pages were used again"


@pytest.mark.parametrize("name", ["A", "C"])
def test_experts_through_the_librarys_grouped_product(name, monkeypatch):
    from air_b200.parts.experts import RoutedExperts
    monkeypatch.setattr(RoutedExperts, "LIBRARY_ROWS", 0)
    streams = streams_for(name, 70, (3, 150, 41))
    got, _ = replay(name, "bfloat16", util.trace_whole(streams), page_tokens=64)
    tu.check(got, name, streams, "bfloat16")
    got, _ = replay(name, "bfloat16", util.trace_mixed(streams, seed=4, live=3), page_tokens=64, max_requests=3)
    tu.check(got, name, streams, "bfloat16")


@pytest.mark.parametrize("name", ["random1", "random2", "random3", "random5", "random8", "random13", "random21", "random34"])
def test_configurations_drawn_at_random(name):
    """Layer orders, repeated stretches, sizes and constants that nobody chose (tabopel_util.random_config): whole
    prompts and a mixed schedule through three slots, in float32 within its tolerance; bfloat16 must be finite and agree
    with the oracle in the median (how far single rows lie depends on how a drawn model amplifies rounding)."""
    tu.model_folder(name)
    streams = {f"{name}_{i}": tu.tokens_for(name, n, 80 + i) for i, n in enumerate((150, 3, 70, 1, 97))}
    margin = min(tu.plain_run(name, toks)[1] for toks in streams.values())
    whole = util.trace_whole(streams)
    mixed = util.trace_mixed(streams, seed=5, live=3, tail=20)
    got, _ = replay(name, "float32", whole, page_tokens=64)
    tu.check(got, name, streams, "float32")
    got, _ = replay(name, "float32", mixed, page_tokens=16, max_requests=3)
    tu.check(got, name, streams, "float32")
    for steps, page in ((whole, 16), (mixed, 64)):
        got, _ = replay(name, "bfloat16", steps, page_tokens=page, max_requests=3)
        means = []
        for (rid, p), row in got.items():
            ref = tu.plain_logits(name, streams[rid])[p]
            assert np.isfinite(row).all()
            means.append(np.abs(row - ref).mean() / max(1.0, np.abs(tu.plain_logits(name, streams[rid])).max()))
        if margin > 0.01:
            assert np.median(means) <= 2 * tu.BF16_MEDIAN_TOL, (name, float(np.median(means)))


@pytest.mark.parametrize("name", ["A", "C"])
def test_float32_does_not_depend_on_the_cut_or_the_batch(name):
    streams = streams_for(name, 30, (97, 40, 131))
    whole, _ = replay(name, "float32", util.trace_whole(streams))
    cut, _ = replay(name, "float32", util.trace_portions(streams, sizes=(2, 31, 1, 16, 5)))
    mixed, _ = replay(name, "float32", util.trace_mixed(streams, seed=1, live=3), max_requests=3)
    for key, row in whole.items():
        assert np.abs(cut[key] - row).max() < 3e-5
        assert np.abs(mixed[key] - row).max() < 3e-5


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_bfloat16_agrees_with_itself_across_schedules(name):
    streams = streams_for(name, 30, (97, 40, 131))
    whole, _ = replay(name, "bfloat16", util.trace_whole(streams), page_tokens=64)
    cut, _ = replay(name, "bfloat16", util.trace_portions(streams, sizes=(2, 31, 1, 16, 5)), page_tokens=64)
    mixed, _ = replay(name, "bfloat16", util.trace_mixed(streams, seed=1, live=3), page_tokens=64, max_requests=3)
    for other in (cut, mixed):
        means = []
        for key, row in whole.items():
            scale = max(1.0, np.abs(row).max())
            diff = np.abs(other[key] - row)
            assert diff.max() <= 2 * tu.BF16_MAX_TOL * scale and diff.mean() <= 2 * tu.BF16_MEAN_TOL * scale, key
            means.append(diff.mean() / scale)
        assert np.median(means) <= tu.BF16_MEDIAN_TOL


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_page_borders_and_first_tokens(name, dtype):
    """Prompts that end just before, on and just behind a page's last place, then decoded across the border; and
    requests decoded from their very first token (the convolutions see zeros ahead of it, retention an empty state)."""
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig
    engine = Engine.from_folder(tu.model_folder(name), EngineConfig(dtype=dtype, page_tokens=16, max_tokens=1024,
                                                                    max_requests=4))
    for n in (15, 16, 17, 31, 33):
        toks = tu.tokens_for(name, n + 4, n)
        got = [engine.step([Entry("r", toks[:n], range(n))]).cpu().numpy()]
        got += [engine.step([Entry("r", [t], [0])]).cpu().numpy() for t in toks[n:]]
        engine.finish("r")
        tu.check({("r", p): row for p, row in enumerate(np.concatenate(got))}, name, {"r": toks}, dtype)
    toks = tu.tokens_for(name, 6, 99)
    got = np.concatenate([engine.step([Entry("s", [t], [0])]).cpu().numpy() for t in toks])
    tu.check({("s", p): row for p, row in enumerate(got)}, name, {"s": toks}, dtype)
    got = [engine.step([Entry("t", toks[:2], [0, 1])]).cpu().numpy()]
    got += [engine.step([Entry("t", [t], [0])]).cpu().numpy() for t in toks[2:]]
    tu.check({("t", p): row for p, row in enumerate(np.concatenate(got))}, name, {"t": toks}, dtype)
    engine.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding(name, dtype):
    """320 tokens one by one after a prompt of five, across twenty pages (the decode steps replay a CUDA graph)."""
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig
    toks = tu.tokens_for(name, 325, 7)
    engine = Engine.from_folder(tu.model_folder(name), EngineConfig(dtype=dtype, page_tokens=16, max_tokens=384,
                                                                    max_requests=2))
    got = [engine.step([Entry("r", toks[:5], range(5))]).cpu().numpy()]
    got += [engine.step([Entry("r", [t], [0])]).cpu().numpy() for t in toks[5:]]
    tu.check({("r", p): row for p, row in enumerate(np.concatenate(got))}, name, {"r": toks}, dtype)
    assert engine.graphs, "decode steps ran as a graph"
    engine.check_status()


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_service(name):
    """The scheduler cuts prompts into portions of five, decodes one step ahead and feeds the device's own choice back."""
    from air_b200 import GenerationConfig
    from air_b200.engine.engine import Engine, EngineConfig
    from air_b200.engine.service import InferenceService, SchedulerConfig
    engine = Engine.from_folder(tu.model_folder(name), EngineConfig(dtype="float32", page_tokens=16, max_tokens=1024,
                                                                    max_requests=4))
    svc = InferenceService(engine, SchedulerConfig(max_active_requests=4, prefill_quantum_tokens=5,
                                                   token_budget_per_cycle=12))
    prompts = [tu.tokens_for(name, n, 40 + n) for n in (1, 7, 33, 20, 3)]
    want = [tu.plain_greedy(name, p, 12) for p in prompts]
    got = svc.generate_cohort([(p, GenerationConfig(max_new_tokens=12, stop_on_eos=False)) for p in prompts])
    assert [r.tokens for r in got] == want
    assert engine.cache.free_pages() == engine.cache.num_pages
    engine.check_status()


def test_trace_runner_program_and_command_line(capsys):
    """bin/trace_run as a program on a Tabopel folder (the class is chosen by config.json), and the command line."""
    name = "B"
    streams = streams_for(name, 60, (40, 9))
    steps = util.trace_mixed(streams, seed=2, live=2)
    with tempfile.TemporaryDirectory() as out:
        util.run_trace_program(tu.model_folder(name), "float32", steps, util.peak_tokens(steps), out)
        got = util.collect(steps, out, tu.CONFIGS[name]["vocab"])
    tu.check(got, name, streams, "float32")
    from air_b200 import cli
    prompt = tu.tokens_for(name, 9, 70)
    assert cli.main(["cuda", tu.model_folder(name), ",".join(map(str, prompt)), "--tokens", "6", "--dtype", "float32",
                     "--no-stop-on-eos"]) == 0
    assert capsys.readouterr().out.strip() == ",".join(map(str, tu.plain_greedy(name, prompt, 6)))
