"""Pefivik on the GPU against the plain implementation (tests/plain/pefivik_plain.py, 64-bit): every mechanism alone
through its part or kernel, then whole models through Engine.step, the scheduler and the trace runner, in float32 and
bfloat16, for configurations that differ in every size and option (pefivik_util.CONFIGS)."""
import tempfile
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import pefivik_util as pu
import util
from plain import pefivik_plain as plain

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


# ----------------------------------------------------------------------------- mechanisms alone
def test_embedding_with_pairs_and_the_token_before_a_portion():
    """Two requests whose tokens come in portions and one by one, in steps that hold both: the row of the table of
    pairs depends on the token before, which may lie in an earlier step; the first token takes the last row; a slot that
    another request held before starts anew.  A multiplier large enough for the product to leave 32 bits."""
    from air_b200.cache.manager import CacheManager
    from air_b200.parts.embedding import BigramHashEmbedding
    from air_b200.parts.spec import PartSpec
    V, E, buckets, mp, mc = 300, 24, 61, 1000003, 7
    rng = np.random.default_rng(0)
    table, pairs = rng.normal(size=(V, E)), rng.normal(size=(buckets + 1, E))
    part = BigramHashEmbedding(PartSpec("bigram_hash", {"vocab": V, "hidden": E, "buckets": buckets, "mul_prev": mp,
                                                        "mul_cur": mc, "pairs": "pairs"}), "table")
    part.load({"table": dev(table), "pairs": dev(pairs)}, runtime("float32"))
    cache = CacheManager([part.cache_needs()], 16, 8, 2, dtype=torch.float32, device=DEV)
    streams = {"a": rng.integers(0, V, size=40).tolist(), "b": rng.integers(0, V, size=23).tolist()}
    want = {r: plain.embed_tokens(t, table, pairs, buckets, mp, mc) for r, t in streams.items()}
    done = {"a": 0, "b": 0}
    for step in ([("a", 5)], [("a", 1), ("b", 7)], [("b", 1), ("a", 2)], [("a", 30), ("b", 1)], [("b", 14), ("a", 2)]):
        entries = [(r, streams[r][done[r]:done[r] + n], []) for r, n in step]
        ctx = context_for(cache, entries)
        ctx.last_token = None
        h, again = part.forward(ctx, cache.views(0), copies=2)
        at = 0
        for r, n in step:
            assert np.abs(h[at:at + n].cpu().numpy() - want[r][done[r]:done[r] + n]).max() < 1e-6, (step, r)
            assert torch.equal(h, again)
            cache.commit(r, n)
            done[r] += n
            at += n
    cache.close("a")
    ctx = context_for(cache, [("c", streams["b"][:3], [])])       # takes a's slot, whose last token must not show
    ctx.last_token = None
    (h,) = part.forward(ctx, cache.views(0))
    assert np.abs(h.cpu().numpy() - want["b"][:3]).max() < 1e-6


def test_what_a_pass_adds_to_the_stream_and_the_scalar_norm_behind_scaled_sums():
    from air_b200.csrc import ops
    from air_b200.parts.base import ScaledSum
    from air_b200.parts.norm import ScalarRMSNorm
    from air_b200.parts.spec import PartSpec
    rng = np.random.default_rng(1)
    T, E, m, g, eps = 13, 72, 0.65, 1.3, 1e-5
    h, x0, row = rng.normal(size=(T, E)), rng.normal(size=(T, E)), rng.normal(size=E)
    for again, r in ((x0, row), (None, row), (x0, None)):
        hd = dev(h)
        ops.stream_add(hd, None if again is None else dev(again), None if r is None else dev(r))
        want = h + (0 if again is None else again) + (0 if r is None else r)
        assert np.abs(hd.cpu().numpy() - want).max() < 1e-6
    a, b = rng.normal(size=(3, T, E)), rng.normal(size=(T, E))
    for dtype in ("float32", "bfloat16"):
        part = ScalarRMSNorm(PartSpec("rms_scalar", {"size": E, "eps": eps, "tensor": ""}), "n")
        part.load({"n": dev(np.array(g), DT[dtype])}, runtime(dtype))
        scale = torch.full((E,), m, device=DEV)
        hd = dev(h)
        out = part.forward(hd, ScaledSum([(dev(a), scale), (dev(b), scale)]))
        x = h + m * (a.sum(0) + b)
        want = plain.over_rms(x, eps) * float(pu.bf16(np.array(g))) if dtype == "bfloat16" else plain.over_rms(x, eps) * g
        assert np.abs(hd.cpu().numpy() - x).max() < 1e-5
        assert np.abs(out.float().cpu().numpy() - want).max() < (1e-5 if dtype == "float32" else 2e-2)
        rows = i32([7, 2])
        hd = dev(h)
        out = part.forward(hd, ScaledSum([(dev(b), scale)]), rows=rows)
        assert np.array_equal(hd.cpu().numpy(), h.astype(np.float32))
        want = plain.over_rms(h + m * b, eps)[[7, 2]] * g
        assert np.abs(out.float().cpu().numpy() - want).max() < (1e-5 if dtype == "float32" else 2e-2)


def latent_weights(rng, E, H, d, dv, R, scale, dtype):
    gain = (2.5 / (scale * d ** 0.5)) ** 0.5
    w = {"q": rng.normal(size=(H * d, E)) * gain / E ** 0.5, "dkv": rng.normal(size=(R, E)) / E ** 0.5,
         "dkv.norm": rng.normal(1.0, 0.2, size=R), "uk": rng.normal(size=(H * d, R)) * gain / R ** 0.5,
         "uv": rng.normal(size=(H * dv, R)) / R ** 0.5, "sink": rng.normal(1.0, 2.0, size=H),
         "g": rng.normal(size=(H, E)) * 2.0 / E ** 0.5, "o": rng.normal(size=(E, H * dv)) / (H * dv) ** 0.5}
    return {k: pu.bf16(a).astype(np.float64) for k, a in w.items()} if dtype == "bfloat16" else w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,d,dv,R,page", [(4, 24, 20, 40, 16), (1, 32, 40, 56, 16), (8, 64, 48, 128, 64), (3, 8, 8, 300, 16),
                                            (5, 16, 12, 20, 32)])
def test_latent_attention_without_positions_with_sink_and_gates(H, d, dv, R, page, dtype):
    """The mixer alone over a request of 330 tokens in portions and single tokens (the long portions take the road of
    matrix products over gathered keys in bfloat16, the others the kernel that reads the pages), against the plain
    function on the whole sequence.  Scores are as sharp as a trained model's (a standard deviation of 2.5) and the
    sinks of the order of the scores: a sink that is left out shows (checked on the plain side)."""
    from air_b200.cache.manager import CacheManager
    from air_b200.parts.latent_attention import LatentAttention
    from air_b200.parts.spec import PartSpec
    E, T, scale, eps = 80, 330, 0.2, 1e-5
    rng = np.random.default_rng(R + H)
    w = latent_weights(rng, E, H, d, dv, R, scale, dtype)
    x = rng.normal(size=(T, E))
    if dtype == "bfloat16":
        x = pu.bf16(x).astype(np.float64)
    spec = PartSpec("latent_attention", {"hidden": E, "heads": H, "head_dim": d, "rot_dim": 0, "v_dim": dv, "kv_rank": R,
                                         "scale": scale, "window": None, "eps": eps, "sink": True, "head_gate": True})
    part = LatentAttention(spec, "m.")
    part.load({"m." + k: dev(a, torch.float32 if k in ("dkv.norm", "sink") else DT[dtype]) for k, a in w.items()},
              runtime(dtype, page))
    want = plain.latent_attention(x, w, dict(heads=H, dim=d, vdim=dv, scale=scale), eps)
    without_sink = plain.latent_attention(x, dict(w, sink=np.full(H, -50.0)), dict(heads=H, dim=d, vdim=dv, scale=scale), eps)
    assert np.abs(want - without_sink).max() > 0.05
    cache = CacheManager([part.cache_needs()], page, 24, 2, dtype=DT[dtype], device=DEV)
    cache.open("other")                                        # the request under test does not sit in slot 0
    outs, at = [], 0
    for n in (3, 61, 1, 150, 2, 1, 1, 40, 70, 1):
        ctx = context_for(cache, [("r", [0] * n, [])], part)
        outs.append(summed(part.forward(dev(x[at:at + n], DT[dtype]), ctx, cache.views(0), True)))
        cache.commit("r", n)
        at += n
    assert at == T
    got = np.concatenate(outs)
    tol = 2e-4 if dtype == "float32" else 4e-2
    assert np.abs(got - want).max() < tol * max(1.0, np.abs(want).max()), float(np.abs(got - want).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_attention_finds_a_key_far_away_and_at_page_borders(dtype):
    """Keys and queries are made by hand: the latent of tokens 0, 15, 16 and 200 each lies along an axis of its own,
    late queries point at one of them each (a score that stands out among hundreds), and the value expansion shows
    which key was found.  As a prompt portion and token by token, over pages of 16 that are scattered."""
    from air_b200.cache.manager import CacheManager
    from air_b200.parts.latent_attention import LatentAttention
    from air_b200.parts.spec import PartSpec
    E, H, d, dv, R, T, scale, eps = 64, 2, 16, 16, 32, 420, 0.25, 1e-6
    rng = np.random.default_rng(5)
    w = latent_weights(rng, E, H, d, dv, R, scale, dtype)
    x = rng.normal(size=(T, E)) * 0.3
    marked = {0: 401, 15: 402, 16: 403, 200: 404, 17: 419}
    for j, i in marked.items():
        c = plain.over_rms(x[j:j + 1] @ w["dkv"].T, eps)[0] * w["dkv.norm"]
        key = (c @ w["uk"].T).reshape(H, d)
        # x[i] is chosen so that Wq x[i] is the key, enlarged: the least-squares solution of Wq x = target
        target = (key * (16.0 / scale / (key ** 2).sum(-1, keepdims=True))).reshape(-1)
        x[i] = np.linalg.lstsq(w["q"], target, rcond=None)[0]
    if dtype == "bfloat16":
        x = pu.bf16(x).astype(np.float64)
    p = dict(heads=H, dim=d, vdim=dv, scale=scale)
    want = plain.latent_attention(x, w, p, eps)
    spec = PartSpec("latent_attention", {"hidden": E, "heads": H, "head_dim": d, "rot_dim": 0, "v_dim": dv, "kv_rank": R,
                                         "scale": scale, "window": None, "eps": eps, "sink": True, "head_gate": True})
    part = LatentAttention(spec, "m.")
    part.load({"m." + k: dev(a, torch.float32 if k in ("dkv.norm", "sink") else DT[dtype]) for k, a in w.items()},
              runtime(dtype))
    for cuts in ([T], [400] + [1] * 20, [7, 9, 1, 383, 2, 2, 16]):
        cache = CacheManager([part.cache_needs()], 16, 40, 2, dtype=DT[dtype], device=DEV)
        for g in cache.groups:              # pages in an order of their own
            rng.shuffle(g.pool._free)
        outs, at = [], 0
        for n in cuts:
            ctx = context_for(cache, [("r", [0] * n, [])], part)
            outs.append(summed(part.forward(dev(x[at:at + n], DT[dtype]), ctx, cache.views(0), True)))
            cache.commit("r", n)
            at += n
        got = np.concatenate(outs)
        tol = 2e-4 if dtype == "float32" else 4e-2
        assert np.abs(got - want).max() < tol * max(1.0, np.abs(want).max()), (cuts[:3], float(np.abs(got - want).max()))
    # and the marked keys do carry the rows that point at them: without key 0 row 401 is another row
    gone = plain.latent_attention(x[1:], w, p, eps)
    assert np.abs(gone[400] - want[401]).max() > 0.1 * np.abs(want[401]).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,d,dv", [(3, 20, 12), (1, 40, 8), (2, 64, 32), (4, 8, 24), (2, 100, 64)])
def test_hgrn2_carries_its_state_through_portions_and_slots(H, d, dv, dtype):
    """The mixer alone: two requests in steps that hold both, portions of many sizes and single tokens; some channels
    forget so slowly (lower bounds of 0.996) that the first token still shows after 300; a slot that another request
    held starts from zeros."""
    from air_b200.cache.manager import CacheManager
    from air_b200.parts.recurrent import HGRN2
    from air_b200.parts.spec import PartSpec
    E, eps = 72, 1e-5
    rng = np.random.default_rng(H * d)
    w = {"q": rng.normal(size=(H * d, E)) * 1.5 / E ** 0.5, "f": rng.normal(size=(H * d, E)) * 2 / E ** 0.5,
         "f.b": rng.normal(size=H * d), "v": rng.normal(size=(H * dv, E)) / E ** 0.5,
         "lower": np.where(rng.random(H * d) < 0.4, 0.99609375, rng.uniform(0, 0.9, size=H * d)),
         "norm": rng.normal(1.0, 0.2, size=dv), "o": rng.normal(size=(E, H * dv)) / (H * dv) ** 0.5}
    if dtype == "bfloat16":
        w = {k: pu.bf16(a).astype(np.float64) for k, a in w.items()}
    streams = {"a": rng.normal(size=(320, E)), "b": rng.normal(size=(75, E))}
    streams["a"][0] *= 30.0                                        # a first token that the slow channels remember
    if dtype == "bfloat16":
        streams = {r: pu.bf16(x).astype(np.float64) for r, x in streams.items()}
    p = dict(heads=H, dim=d, vdim=dv)
    want = {r: plain.hgrn2(x, w, p, eps) for r, x in streams.items()}
    assert np.abs(plain.hgrn2(streams["a"][1:], w, p, eps)[-1] - want["a"][-1]).max() > 0.02
    part = HGRN2(PartSpec("hgrn2", {"hidden": E, "heads": H, "head_dim": d, "v_dim": dv, "eps": eps}), "m.")
    part.load({"m." + k: dev(a, DT[dtype] if a.ndim == 2 else torch.float32) for k, a in w.items()}, runtime(dtype))
    cache = CacheManager([part.cache_needs()], 16, 64, 2, dtype=DT[dtype], device=DEV)
    done = {"a": 0, "b": 0}
    got = {"a": [], "b": []}
    steps = [[("a", 3)], [("a", 1), ("b", 40)], [("b", 1), ("a", 100)], [("a", 2), ("b", 2)], [("a", 150), ("b", 1)],
             [("b", 31), ("a", 1)], [("a", 63)]]
    for step in steps:
        ctx = context_for(cache, [(r, [0] * n, []) for r, n in step])
        x = np.concatenate([streams[r][done[r]:done[r] + n] for r, n in step])
        y = summed(part.forward(dev(x, DT[dtype]), ctx, cache.views(0), True))
        at = 0
        for r, n in step:
            got[r].append(y[at:at + n])
            cache.commit(r, n)
            done[r] += n
            at += n
    tol = 1e-4 if dtype == "float32" else 4e-2
    for r in streams:
        assert done[r] == len(streams[r])
        diff = np.abs(np.concatenate(got[r]) - want[r]).max()
        assert diff < tol * max(1.0, np.abs(want[r]).max()), (r, float(diff))
    cache.close("a")
    ctx = context_for(cache, [("c", [0] * 5, [])])                 # in a's slot: a's state must be gone
    y = summed(part.forward(dev(streams["b"][:5], DT[dtype]), ctx, cache.views(0), True))
    assert np.abs(y - want["b"][:5]).max() < tol * max(1.0, np.abs(want["b"]).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,F,T", [(72, 100, 11), (96, 40, 70), (128, 256, 150), (40, 8, 3)])
def test_dense_feed_forward_with_polynorm_and_biases(E, F, T, dtype):
    from air_b200.parts.mlp import PolyNormMLP
    from air_b200.parts.spec import PartSpec
    rng = np.random.default_rng(F)
    eps = 1e-5
    w = {"up": rng.normal(size=(F, E)) / E ** 0.5, "up.b": rng.normal(0, 0.5, size=F),
         "down": rng.normal(size=(E, F)) / F ** 0.5, "down.b": rng.normal(0, 0.5, size=E),
         "act": np.array([1.1, 0.4, -0.2, 0.3])}
    x = rng.normal(size=(T, E))
    if dtype == "bfloat16":
        w = {k: pu.bf16(a).astype(np.float64) for k, a in w.items()}
        x = pu.bf16(x).astype(np.float64)
    part = PolyNormMLP(PartSpec("polynorm_mlp", {"hidden": E, "intermediate": F, "eps": eps}), "f.")
    part.load({"f." + k: dev(a, DT[dtype] if a.ndim == 2 else torch.float32) for k, a in w.items()}, runtime(dtype))
    got = summed(part.forward(dev(x, DT[dtype]), SimpleNamespace(residual=None)))
    want = plain.dense_ff(x, w, eps)
    # (every term of the activation matters: without the cube the output is another)
    assert np.abs(plain.dense_ff(x, dict(w, act=np.array([1.1, 0.4, 0.0, 0.3])), eps) - want).max() > 0.05
    tol = 1e-5 if dtype == "float32" else 3e-2
    assert np.abs(got - want).max() < tol * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("n,count,keep,top", [(6, 3, 2, 2), (8, 2, 1, 3), (8, 8, 5, 4), (16, 4, 2, 5), (1, 1, 1, 1),
                                              (12, 1, 1, 5), (130, 13, 4, 9)])
def test_router_chooses_among_the_best_groups(n, count, keep, top):
    """Against the plain router: random logits, rows of equal logits (the lower index wins, for groups and experts),
    and the weights: the chosen scores over their sum, times the router's scale."""
    from air_b200.csrc import ops
    rng = np.random.default_rng(n + count)
    T, scale = 200, 1.7
    z = rng.normal(size=(T, n)) * 2
    z[3] = 0.3
    z[4, : n // 2] = 1.0
    expert = torch.empty((T, top), dtype=torch.int32, device=DEV)
    weight = torch.empty((T, top), device=DEV)
    ops.moe_route(dev(z), n, top, expert, weight, None, renormalize=True, groups=count, keep=keep, route_scale=scale,
                  norm_eps=1e-20)
    s = plain.sigmoid(z.astype(np.float32).astype(np.float64))
    got_e, got_w = expert.cpu().numpy(), weight.cpu().numpy()
    for t in range(T):
        margins = []
        chosen = plain.route(s[t], top, count, keep, margins)
        if margins and min(margins) < 1e-6 and t not in (3, 4):
            continue                    # (a draw that 32-bit rounding can tip)
        assert got_e[t].tolist() == chosen, (t, got_e[t], chosen)
        ws = s[t, chosen] / s[t, chosen].sum() * scale
        assert np.abs(got_w[t] - ws).max() < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,count,keep,top,E,F,S,T", [(6, 3, 2, 2, 72, 40, 48, 150), (4, 1, 1, 4, 96, 32, 0, 7),
                                                       (8, 8, 5, 4, 128, 64, 128, 70), (1, 1, 1, 1, 40, 24, 16, 33)])
def test_experts_weighted_on_their_output(n, count, keep, top, E, F, S, T, dtype, monkeypatch):
    """The feed-forward alone against the plain one: the weight multiplies the expert's output (an expert is not
    linear: with the weight on its input the result is another), a shared expert without gate beside them.  Few rows per
    expert (the package's grouped product) and, in bfloat16, the road of many rows as well."""
    from air_b200.parts.experts import RoutedExperts
    from air_b200.parts.spec import PartSpec
    rng = np.random.default_rng(n * 7 + T)
    w = {"router": rng.normal(size=(n, E)) * 3 / E ** 0.5}
    for e in range(n):
        w[f"e{e}.gate"], w[f"e{e}.up"] = rng.normal(size=(F, E)) * 2 / E ** 0.5, rng.normal(size=(F, E)) * 2 / E ** 0.5
        w[f"e{e}.down"] = rng.normal(size=(E, F)) / F ** 0.5
    if S:
        w["shared.gate"], w["shared.up"] = rng.normal(size=(S, E)) / E ** 0.5, rng.normal(size=(S, E)) / E ** 0.5
        w["shared.down"] = rng.normal(size=(E, S)) / S ** 0.5
    x = rng.normal(size=(T, E))
    if dtype == "bfloat16":
        w = {k: pu.bf16(a).astype(np.float64) for k, a in w.items()}
        x = pu.bf16(x).astype(np.float64)
    p = dict(router=dict(experts=n, top=top, scale=1.4, groups=dict(count=count, keep=keep)), shared=dict(ff=S) if S else None)
    margins = []
    want = plain.moe_ff(x, w, p, margins)
    clear = np.ones(T, dtype=bool)
    if margins:         # rows whose choice rounding could tip are left out of the comparison
        per = len(margins) // T
        clear = np.array(margins).reshape(T, per).min(-1) > (1e-5 if dtype == "float32" else 2e-2)
    assert clear.sum() > T // 2
    spec = PartSpec("routed_experts", {"hidden": E, "experts": n, "top": top, "intermediate": F, "shared_intermediate": S,
                                       "shared_gate": False, "score": "sigmoid", "renormalize": True, "norm_eps": 1e-20,
                                       "route_scale": 1.4, "groups": (count, keep) if count > 1 else None,
                                       "weight_on": "output"})
    for rows in ([RoutedExperts.LIBRARY_ROWS] if dtype == "float32" else [RoutedExperts.LIBRARY_ROWS, 0]):
        monkeypatch.setattr(RoutedExperts, "LIBRARY_ROWS", rows)
        part = RoutedExperts(spec, "f.")
        part.load({"f." + k: dev(a, DT[dtype]) for k, a in w.items()}, runtime(dtype))
        y = part.forward(dev(x, DT[dtype]), SimpleNamespace(residual=None))
        got = summed(y) if isinstance(y, torch.Tensor) else summed(y.a) + summed(y.b)
        tol = 1e-4 if dtype == "float32" else 4e-2
        assert np.abs(got - want)[clear].max() < tol * max(1.0, np.abs(want).max()), rows


# ----------------------------------------------------------------------------- whole models
LENGTHS = {"A": (1, 7, 33, 97, 150), "B": (5, 40, 131, 64), "C": (2, 65, 150, 300), "D": (3, 70, 1, 129)}


def streams_for(name, seed=0, lengths=None):
    return {f"{name}{i}": pu.tokens_for(name, n, seed + i) for i, n in enumerate(lengths or LENGTHS[name])}


def replay(name, dtype, steps, page_tokens=16, max_requests=4, peak_page=64):
    return util.replay(pu.model_folder(name), dtype, steps, max_tokens=util.peak_tokens(steps, page=peak_page),
                       page_tokens=page_tokens, max_requests=max_requests)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_stream_after_every_run(name, dtype):
    """Layer by layer: the stream behind every run of the order list (a layer that runs three times counts three
    times) against the plain implementation's, for a prompt in one step."""
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig
    cfg, tensors = pu.plain_model(name)
    toks = pu.tokens_for(name, 90, 3)
    want = []
    plain.forward(cfg, tensors, toks, layers_out=want)
    engine = Engine.from_folder(pu.model_folder(name), EngineConfig(dtype=dtype, page_tokens=16, max_tokens=256,
                                                                    max_requests=2))
    engine.model.tap = []
    engine.step([Entry("r", toks, [])])
    engine.check_status()
    assert len(engine.model.tap) == len(want) == len(engine.model.spec.order)
    for i, (a, b) in enumerate(zip(engine.model.tap, want)):
        tol = 1e-4 if dtype == "float32" else 0.05
        assert np.abs(a.cpu().numpy() - b).max() < tol * np.abs(b).max(), (i, float(np.abs(a.cpu().numpy() - b).max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts(name, dtype):
    streams = streams_for(name)
    got, _ = replay(name, dtype, util.trace_whole(streams))
    pu.check(got, name, streams, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_prompt_then_token_by_token(name, dtype):
    streams = streams_for(name, 10)
    got, _ = replay(name, dtype, util.trace_bulk_tail(streams, tail=75))
    pu.check(got, name, streams, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_down_to_two_tokens(name, dtype):
    streams = streams_for(name, 20)
    got, _ = replay(name, dtype, util.trace_portions(streams))
    pu.check(got, name, streams, dtype)
    got, _ = replay(name, dtype, util.trace_portions(streams, sizes=(2, 2, 1, 3, 16, 15, 17, 64, 63, 65, 2)), page_tokens=64)
    pu.check(got, name, streams, dtype)


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_unequal_requests_together_with_pages_and_slots_used_again(name, dtype, page):
    """Ten requests through three slots and a pool that holds the peak only: every request must come out as it does
    alone (the oracle runs each alone), whatever shared its batches and whoever had its slot (the states of the state
    mixers, the token before) and its pages before."""
    lengths = LENGTHS[name] + (120, 2, 77, 101, 64, 129)
    streams = streams_for(name, 50, lengths)
    steps = util.trace_mixed(streams, seed=3, live=3)
    got, engine = replay(name, dtype, steps, page_tokens=page, max_requests=3)
    pu.check(got, name, streams, dtype)
    for group in engine.cache.groups:
        assert group.pool.takes > group.pool.num_pages, "pages were used again"


@pytest.mark.parametrize("name", ["A", "C"])
def test_experts_through_the_librarys_grouped_product(name, monkeypatch):
    from air_b200.parts.experts import RoutedExperts
    monkeypatch.setattr(RoutedExperts, "LIBRARY_ROWS", 0)
    streams = streams_for(name, 70, (3, 150, 41))
    got, _ = replay(name, "bfloat16", util.trace_whole(streams), page_tokens=64)
    pu.check(got, name, streams, "bfloat16")
    got, _ = replay(name, "bfloat16", util.trace_mixed(streams, seed=4, live=3), page_tokens=64, max_requests=3)
    pu.check(got, name, streams, "bfloat16")


@pytest.mark.parametrize("name", ["random1", "random2", "random3", "random5", "random8", "random13", "random21", "random34"])
def test_configurations_drawn_at_random(name):
    """Layer orders, repeated stretches, sizes and constants that nobody chose (pefivik_util.random_config): whole
    prompts and a mixed schedule through three slots, in float32 within its tolerance; bfloat16 must be finite and agree
    with the oracle in the median (how far single rows lie depends on how a drawn model amplifies rounding)."""
    pu.model_folder(name)
    streams = {f"{name}_{i}": pu.tokens_for(name, n, 80 + i) for i, n in enumerate((150, 3, 70, 1, 97))}
    margin = min(pu.plain_run(name, toks)[1] for toks in streams.values())
    whole = util.trace_whole(streams)
    mixed = util.trace_mixed(streams, seed=5, live=3, tail=20)
    got, _ = replay(name, "float32", whole, page_tokens=64)
    pu.check(got, name, streams, "float32")
    got, _ = replay(name, "float32", mixed, page_tokens=16, max_requests=3)
    pu.check(got, name, streams, "float32")
    for steps, page in ((whole, 16), (mixed, 64)):
        got, _ = replay(name, "bfloat16", steps, page_tokens=page, max_requests=3)
        means = []
        for (rid, p), row in got.items():
            ref = pu.plain_logits(name, streams[rid])[p]
            assert np.isfinite(row).all()
            means.append(np.abs(row - ref).mean() / max(1.0, np.abs(pu.plain_logits(name, streams[rid])).max()))
        if margin > 0.01:
            assert np.median(means) <= 2 * pu.BF16_MEDIAN_TOL, (name, float(np.median(means)))


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
            assert diff.max() <= 2 * pu.BF16_MAX_TOL * scale and diff.mean() <= 2 * pu.BF16_MEAN_TOL * scale, key
            means.append(diff.mean() / scale)
        assert np.median(means) <= pu.BF16_MEDIAN_TOL


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_page_borders_and_first_tokens(name, dtype):
    """Prompts that end just before, on and just behind a page's last place, then decoded across the border; and
    requests decoded from their very first token (the table of pairs' last row, then the token before)."""
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig
    engine = Engine.from_folder(pu.model_folder(name), EngineConfig(dtype=dtype, page_tokens=16, max_tokens=1024,
                                                                    max_requests=4))
    for n in (15, 16, 17, 31, 33):
        toks = pu.tokens_for(name, n + 4, n)
        got = [engine.step([Entry("r", toks[:n], range(n))]).cpu().numpy()]
        got += [engine.step([Entry("r", [t], [0])]).cpu().numpy() for t in toks[n:]]
        engine.finish("r")
        pu.check({("r", p): row for p, row in enumerate(np.concatenate(got))}, name, {"r": toks}, dtype)
    toks = pu.tokens_for(name, 6, 99)
    got = np.concatenate([engine.step([Entry("s", [t], [0])]).cpu().numpy() for t in toks])
    pu.check({("s", p): row for p, row in enumerate(got)}, name, {"s": toks}, dtype)
    got = [engine.step([Entry("t", toks[:2], [0, 1])]).cpu().numpy()]
    got += [engine.step([Entry("t", [t], [0])]).cpu().numpy() for t in toks[2:]]
    pu.check({("t", p): row for p, row in enumerate(np.concatenate(got))}, name, {"t": toks}, dtype)
    engine.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding(name, dtype):
    """320 tokens one by one after a prompt of five, across twenty pages (the decode steps replay a CUDA graph)."""
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig
    toks = pu.tokens_for(name, 325, 7)
    engine = Engine.from_folder(pu.model_folder(name), EngineConfig(dtype=dtype, page_tokens=16, max_tokens=384,
                                                                    max_requests=2))
    got = [engine.step([Entry("r", toks[:5], range(5))]).cpu().numpy()]
    got += [engine.step([Entry("r", [t], [0])]).cpu().numpy() for t in toks[5:]]
    pu.check({("r", p): row for p, row in enumerate(np.concatenate(got))}, name, {"r": toks}, dtype)
    assert engine.graphs, "decode steps ran as a graph"
    engine.check_status()


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_service(name):
    """The scheduler cuts prompts into portions of five, decodes one step ahead and feeds the device's own choice back
    (the token before then comes from the device too)."""
    from air_b200 import GenerationConfig
    from air_b200.engine.engine import Engine, EngineConfig
    from air_b200.engine.service import InferenceService, SchedulerConfig
    engine = Engine.from_folder(pu.model_folder(name), EngineConfig(dtype="float32", page_tokens=16, max_tokens=1024,
                                                                    max_requests=4))
    svc = InferenceService(engine, SchedulerConfig(max_active_requests=4, prefill_quantum_tokens=5,
                                                   token_budget_per_cycle=12))
    prompts = [pu.tokens_for(name, n, 40 + n) for n in (1, 7, 33, 20, 3)]
    want = [pu.plain_greedy(name, p, 12) for p in prompts]
    got = svc.generate_cohort([(p, GenerationConfig(max_new_tokens=12, stop_on_eos=False)) for p in prompts])
    assert [r.tokens for r in got] == want
    assert engine.cache.free_pages() == engine.cache.num_pages
    engine.check_status()


def test_trace_runner_program_and_command_line(capsys):
    """bin/trace_run as a program on a Pefivik folder (the class is chosen by config.json), and the command line."""
    name = "B"
    streams = streams_for(name, 60, (40, 9))
    steps = util.trace_mixed(streams, seed=2, live=2)
    with tempfile.TemporaryDirectory() as out:
        util.run_trace_program(pu.model_folder(name), "float32", steps, util.peak_tokens(steps), out)
        got = util.collect(steps, out, pu.CONFIGS[name]["vocab"])
    pu.check(got, name, streams, "float32")
    from air_b200 import cli
    prompt = pu.tokens_for(name, 9, 70)
    assert cli.main(["cuda", pu.model_folder(name), ",".join(map(str, prompt)), "--tokens", "6", "--dtype", "float32",
                     "--no-stop-on-eos"]) == 0
    assert capsys.readouterr().out.strip() == ",".join(map(str, pu.plain_greedy(name, prompt, 6)))
