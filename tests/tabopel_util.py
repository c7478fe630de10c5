"""Set-up of the Tabopel tests: small configurations that differ in every size and option, model folders with weights
drawn so that a fault shows, and the comparison with the plain implementation."""
import functools
import tempfile

import numpy as np

from bivizen_util import bf16


def rot(dims, base, scaling=None):
    r = dict(dims=dims, base=base)
    if scaling:
        r["scaling"] = dict(factor=scaling[0], low=scaling[1], high=scaling[2], original=scaling[3])
    return r


def conv_attention(heads, kv_heads, dim, vdim, scale, taps, r):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if r:
        m["rot"] = r
    if taps:
        m["conv"] = taps
    return dict(type="attention", mixer=m)


def normed_attention(heads, kv_heads, dim, vdim, scale, cap, r):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if r:
        m["rot"] = r
    if cap:
        m["softcap"] = cap
    return dict(type="attention_2", mixer=m)


def retention(heads, dim, vdim, decay, r):
    m = dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay))
    if r:
        m["rot"] = r
    return dict(type="retention", mixer=m)


def dense(layer, ff):
    return dict(layer, mlp=dict(kind="dense", ff=ff))


def moe(layer, experts, identity, top, ff):
    return dict(layer, mlp=dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, identity=identity, top=top)))


def bare(layer):
    return dict(layer, mlp=None)


def config(vocab, width, eps, scale, loop, layers):
    d = dict(architecture="Tabopel", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=scale),
             layers=layers)
    if loop:
        d["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return d


# A: a stretch of two layers (retention among them) that runs three times and starts at layer 0; as many key/value heads
#    as query heads, and one for all; keys and values of different sizes everywhere; a rotation of a part of the head in
#    every mixer; frequencies slowed down in bands that the test's positions reach; a layer without feed-forward; an
#    identity expert; every expert chosen; sizes that are no multiples of 8.
# B: no repeated stretch at all; one head; one expert beside one identity expert, one choice; retention without a
#    rotation; attention_2 without a soft cap and with the whole head rotated; attention without a convolution; a dense
#    layer whose ff is smaller than the width; an embedding scale of 1.
# C: a stretch that runs once (it still adds its row), at the model's end; heads of 64 and 128 on pages of 64; a
#    convolution of five taps; no identity expert; twelve experts of which five are taken.
# D: no size is a multiple of 4 (width, heads' sizes, ff): the kernels' roads of one element per access; two identity
#    experts of three; a convolution of two taps.
# E: heads of 64 and 128 with keys and values of one size on pages of 64, as large models have them: single tokens
#    attend through the copy-engine decode kernel (zero sink and gates, cap and learned sinks); the first layer routes.
CONFIGS = {
    "A": config(211, 72, 1e-5, 3.0, (0, 2, 3), [
        moe(retention(3, 20, 12, (0.9, 0.99, 0.9990234375), rot(8, 10000.0)), 5, 1, 2, 40),
        dense(conv_attention(4, 4, 24, 20, 0.2, 3, rot(24, 10000.0, (8.0, 1.0, 4.0, 64))), 100),
        bare(normed_attention(6, 2, 16, 24, 0.25, 3.0, rot(8, 500000.0))),
        moe(conv_attention(2, 1, 40, 8, 0.16, 2, rot(20, 300.0)), 3, 0, 3, 24),
        dense(normed_attention(5, 5, 8, 8, 0.35, 5.0, rot(4, 100.0)), 56)]),
    "B": config(333, 96, 1e-6, 1.0, None, [
        dense(retention(1, 64, 32, (0.96875,), None), 40),
        moe(normed_attention(1, 1, 32, 40, 0.18, 0.0, rot(32, 10000.0)), 1, 1, 1, 64),
        moe(conv_attention(6, 3, 16, 8, 0.25, 0, rot(16, 50000.0, (2.0, 2.0, 8.0, 128))), 4, 2, 4, 32),
        bare(retention(4, 8, 24, (0.5, 0.75, 0.984375, 0.998046875), rot(8, 1000.0)))]),
    "C": config(190, 128, 1e-6, 7.5, (1, 3, 1), [
        dense(conv_attention(4, 2, 64, 64, 0.125, 5, rot(32, 500000.0, (4.0, 1.0, 4.0, 96))), 256),
        moe(normed_attention(2, 1, 128, 64, 0.09, 6.0, rot(64, 10000.0)), 12, 0, 5, 64),
        dense(retention(2, 64, 128, (0.9921875, 0.99951171875), rot(64, 100000.0)), 192)]),
    "D": config(150, 90, 1e-5, 0.5, (1, 3, 2), [
        dense(conv_attention(3, 1, 10, 6, 0.3, 2, rot(6, 1000.0)), 50),
        moe(retention(3, 10, 6, (0.8, 0.95, 0.99), rot(10, 10000.0)), 1, 2, 2, 30),
        dense(normed_attention(2, 2, 14, 10, 0.25, 4.0, rot(2, 10000.0)), 34)]),
    "E": config(300, 256, 1e-6, 10.0, (1, 3, 2), [
        moe(conv_attention(8, 2, 64, 64, 0.125, 4, rot(64, 500000.0, (8.0, 1.0, 4.0, 128))), 6, 2, 3, 96),
        dense(normed_attention(4, 4, 128, 128, 0.09, 8.0, rot(64, 10000.0)), 384),
        moe(retention(4, 64, 64, (0.96875, 0.984375, 0.9921875, 0.998046875), rot(64, 1000000.0)), 3, 1, 2, 128),
        dense(conv_attention(4, 1, 128, 128, 0.09, 2, rot(128, 10000.0)), 320)]),
}
SEEDS = {"A": 41, "B": 42, "C": 43, "D": 44, "E": 45}


def random_config(seed):
    """A configuration drawn at random: 2 to 6 layers in any order, a repeated stretch anywhere (or none), every size
    and constant from a list that includes 1, equal and unequal sizes and sizes that are no multiples of 8 or 16."""
    rng = np.random.default_rng(seed)
    width = int(rng.choice([40, 64, 72, 96, 128, 160, 200]))

    def some_rot(dim):
        if rng.random() < 0.15:
            return None
        dims = int(rng.choice([d for d in (2, 4, 8, 16, 32, 64, dim) if d <= dim and d % 2 == 0]))
        scaling = None
        if rng.random() < 0.5:
            scaling = (float(rng.choice([2.0, 4.0, 8.0])), float(rng.choice([1.0, 2.0])), float(rng.choice([4.0, 8.0])),
                       int(rng.choice([32, 128, 1024])))
        return rot(dims, float(rng.choice([100.0, 10000.0, 500000.0])), scaling)

    layers = []
    for i in range(int(rng.integers(2, 7))):
        u = rng.random()
        dim = int(rng.choice([8, 16, 24, 32, 64]))
        vdim = int(rng.choice([8, 16, 24, 40, 64]))
        kv = int(rng.choice([1, 2, 3]))
        heads = kv * int(rng.choice([1, 2, 4]))
        if u < 0.35:
            layer = conv_attention(heads, kv, dim, vdim, float(rng.choice([0.1, 0.2, 0.3])), int(rng.choice([0, 1, 2, 4, 7])),
                                   some_rot(dim))
        elif u < 0.7:
            layer = normed_attention(heads, kv, dim, vdim, float(rng.choice([0.1, 0.2, 0.3])),
                                     float(rng.choice([0.0, 8.0, 50.0])), some_rot(dim))
        else:
            h = int(rng.choice([1, 2, 3, 4]))
            d = int(rng.choice([4, 8, 20, 32, 48, 64, 100]))
            layer = retention(h, d, int(rng.choice([4, 8, 12, 32, 64])),
                              [float(1.0 - 2.0 ** -rng.integers(1, 11)) for _ in range(h)], some_rot(d))
        u = rng.random()
        if u < 0.15:
            layers.append(bare(layer))
        elif u < 0.5:
            layers.append(dense(layer, int(rng.choice([16, 40, 100, 256, 320]))))
        else:
            experts, identity = int(rng.choice([1, 2, 3, 5, 8, 13])), int(rng.choice([0, 0, 1, 2, 3]))
            layers.append(moe(layer, experts, identity, int(rng.integers(1, min(experts + identity, 6) + 1)),
                              int(rng.choice([16, 24, 40, 64, 100]))))
    n = len(layers)
    loop = None
    if rng.random() < 0.8:
        start = int(rng.integers(0, n))
        loop = (start, int(rng.integers(start + 1, n + 1)), int(rng.choice([1, 2, 2, 3])))
    return config(int(rng.integers(50, 700)), width, float(rng.choice([1e-6, 1e-5, 1e-4])),
                  float(rng.choice([0.7, 1.0, 4.0, 16.0])), loop, layers)


ROUTE_MAGNITUDES = (1.0, 0.85, 0.7, 0.6)


def _bits(n):
    return max(0, int(np.ceil(np.log2(n)))) if n > 1 else 0


def route_channels(cfg):
    """Per layer with experts: (first channel, bits, outputs of the router).  Every such layer has channels of the
    stream of its own."""
    out, at = {}, 0
    for i, layer in enumerate(cfg["layers"]):
        f = layer.get("mlp")
        if f and f["kind"] == "moe":
            total = f["router"]["experts"] + f["router"].get("identity", 0)
            out[i] = (at, _bits(total), total)
            at += _bits(total)
    return out, at


def draw_tensors(cfg, seed):
    """name -> float32 array (bfloat16 values).  The scales are chosen so that every mechanism matters: attention
    scores have a standard deviation of about 2.5 (a key that is lost or added moves the logits far beyond bfloat16's
    rounding), learned sinks are of the order of the scores, the taps of a convolution are all of one order, and the
    rows that a pass adds are as large as the stream.

    A router is a discontinuity: with random router weights one token in a hundred has two experts so close that
    bfloat16's rounding picks the other one, and the logits then differ by a whole expert.  So the routers here decide
    by a few channels of the stream that only the token table touches (the norms behind the sub-layers have the weight
    0 there, and the rows that passes add leave them alone).  Every layer with experts has such channels of its own:
    there a token carries the bits of (a hash of the token) mod (the router's outputs) as signs, and an expert's router
    row the bits of its index, so that the token's own expert has a score near 1 and all others scores near 0.  The
    corrections are all different, in steps of 0.04 (far more than what is left for the other scores), so the further
    choices go by the correction, and the choice by score plus correction is not the choice by score.  Which experts a
    token takes is then a matter of the token, clear of rounding; their weights still depend on everything, through
    the norms and the rest of the router row."""
    rng = np.random.default_rng(seed)
    e = cfg["width"]
    t = {}
    routed, nr = route_channels(cfg)
    assert nr < e // 2 and all(bits <= len(ROUTE_MAGNITUDES) for _, bits, _ in routed.values())

    def mat(out, inp, gain=1.0):
        return rng.normal(0.0, gain / np.sqrt(inp), size=(out, inp))

    def behind(size=e):
        w = 0.5 + rng.normal(0.0, 0.1, size=size)
        w[:nr] = 0.0
        return w

    t["embed"] = rng.normal(0.0, 1.0, size=(cfg["vocab"], e)) / cfg["embedding"]["scale"]
    tokens = np.arange(cfg["vocab"])
    for i, (at, bits, total) in routed.items():
        own = (tokens * (2 * i + 3) + i) % total              # the expert that a token takes first in layer i
        for c in range(bits):
            t["embed"][:, at + c] = np.where((own >> c) & 1, 1.0, -1.0) * ROUTE_MAGNITUDES[c] * 5.0 / cfg["embedding"]["scale"]
    if cfg.get("loop"):
        t["loop.step"] = rng.normal(0.0, 0.7, size=(cfg["loop"]["times"], e))
        t["loop.step"][:, :nr] = 0.0
    t["head"] = mat(cfg["vocab"], e, 2.0)
    t["final.norm"] = 1.0 + rng.normal(0.0, 0.1, size=e)
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
        t[p + "norm1"] = 1.0 + rng.normal(0.0, 0.1, size=e)
        t[p + "norm1b"] = behind()
        if layer["type"] == "retention":
            t[p + "mix.q"], t[p + "mix.k"] = mat(H * d, e, 1.5), mat(H * d, e, 1.5)
            t[p + "mix.v"], t[p + "mix.g"] = mat(H * dv, e, 1.5), mat(H * dv, e, 2.0)
        else:
            G = mx["kv_heads"]
            sharp = (2.5 / (mx["scale"] * d ** 0.5)) ** 0.5
            if layer["type"] == "attention":
                t[p + "mix.q"], t[p + "mix.k"] = mat(H * d, e, sharp), mat(G * d, e, sharp)
                t[p + "mix.g"] = mat(H * dv, e, 2.0)
                taps = mx.get("conv", 0)
                for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                    if taps:
                        t[p + f"mix.{n}.conv"] = rng.normal(0.0, 1.0, size=(rows, taps)) / taps ** 0.5 + \
                            np.where(np.arange(taps) == taps - 1, 0.6, 0.0)
            else:
                t[p + "mix.q"], t[p + "mix.k"] = mat(H * d, e), mat(G * d, e)
                for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                    t[p + f"mix.{n}.b"] = rng.normal(0.0, 0.3, size=rows)
                t[p + "mix.q.norm"] = sharp * (1.0 + rng.normal(0.0, 0.15, size=H * d))
                t[p + "mix.k.norm"] = sharp * (1.0 + rng.normal(0.0, 0.15, size=G * d))
                t[p + "mix.sink"] = rng.normal(1.0, 2.0, size=H)
            t[p + "mix.v"] = mat(G * dv, e, 1.5)
        t[p + "mix.o"] = mat(e, H * dv)
        f = layer.get("mlp")
        if not f:
            continue
        t[p + "norm2"] = 1.0 + rng.normal(0.0, 0.1, size=e)
        t[p + "norm2b"] = behind()
        if f["kind"] == "dense":
            t[p + "mlp.up"], t[p + "mlp.down"] = mat(f["ff"], e, 1.4), mat(e, f["ff"])
            continue
        at, bits, total = routed[i]
        n = f["router"]["experts"]
        t[p + "norm2"][:nr] = 1.0
        t[p + "mlp.router"] = mat(total, e, 0.02)
        t[p + "mlp.correction"] = rng.permutation(total).astype(np.float64) * 0.04 - 0.02 * (total - 1)
        for x in range(total):
            t[p + "mlp.router"][x, :nr] = 0.0
            t[p + "mlp.router"][x, at:at + bits] = [(1.0 if (x >> c) & 1 else -1.0) * 3.0 for c in range(bits)]
        for x in range(n):
            t[f"{p}mlp.e{x}.up"], t[f"{p}mlp.e{x}.down"] = mat(f["expert"]["ff"], e, 1.4), mat(e, f["expert"]["ff"])
    return {n: bf16(a) for n, a in t.items()}


_tmp = []


@functools.lru_cache(maxsize=None)
def model_folder(name):
    """config.json and model.safetensors (bfloat16) of a test configuration, in a temporary place."""
    import torch
    from air_b200.weights.loader import write_model_folder
    d = tempfile.TemporaryDirectory(prefix=f"air_b200_tabopel_{name}_")
    _tmp.append(d)
    if name not in CONFIGS:      # "random<seed>": drawn at random
        seed = int(name[len("random"):])
        CONFIGS[name], SEEDS[name] = random_config(seed), seed
    cfg = CONFIGS[name]
    tensors = {n: torch.from_numpy(np.ascontiguousarray(a)).reshape(a.shape).to(torch.bfloat16)
               for n, a in draw_tensors(cfg, SEEDS[name]).items()}
    write_model_folder(d.name, cfg, tensors)
    return d.name


@functools.lru_cache(maxsize=None)
def plain_model(name):
    from plain import pefivik_plain
    return pefivik_plain.read_model(model_folder(name))


_logits = {}


def plain_run(name, tokens):
    """(logits [T, vocab], the smallest margin by which a router chose)."""
    from plain import tabopel_plain as plain
    key = (name, tuple(tokens))
    if key not in _logits:
        cfg, tensors = plain_model(name)
        margins = []
        logits = plain.forward(cfg, tensors, list(tokens), margins=margins).astype(np.float64)
        _logits[key] = (logits, float(np.min(margins)) if margins else np.inf)
    return _logits[key]


def plain_logits(name, tokens):
    return plain_run(name, tokens)[0]


def tokens_for(name, n, seed):
    return np.random.default_rng(7000 + seed).integers(0, CONFIGS[name]["vocab"], size=n).tolist()


def plain_greedy(name, prompt, n):
    out, toks = [], list(prompt)
    for _ in range(n):
        nxt = int(plain_logits(name, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out


# float32: sums in another order than the 64-bit oracle.  bfloat16: activations rounded to 8 bits at the inputs of the
# products and in the cache, through up to ten runs of sharp attention, retention and experts.  A request's rows must
# all be within the row limits, and their median within the tighter one.  The routers choose with clear margins
# (draw_tensors); check() makes sure of it, since a choice that rounding can tip voids the comparison.
FP32_TOL = 1e-4
BF16_MAX_TOL = 0.3
BF16_MEAN_TOL = 7e-2
BF16_MEDIAN_TOL = 2e-2


def check(got, name, streams, dtype):
    """got: {(request, position): logits}; every request of `streams` must have rows, and the rows must agree."""
    for rid, toks in streams.items():
        ref, margin = plain_run(name, toks)
        assert margin > (1e-4 if dtype == "float32" else 0.01), (rid, margin)
        scale = max(1.0, float(np.abs(ref).max()))
        rows = sorted(p for (r, p) in got if r == rid)
        assert rows, f"no logits for request {rid}"
        means = []
        for p in rows:
            out = got[(rid, p)]
            assert np.isfinite(out).all()
            diff = np.abs(out - ref[p])
            if dtype == "float32":
                assert diff.max() <= FP32_TOL * scale, (rid, p, float(diff.max()), scale)
            else:
                assert diff.max() <= BF16_MAX_TOL * scale, (rid, p, float(diff.max()), scale)
                assert diff.mean() <= BF16_MEAN_TOL * scale, (rid, p, float(diff.mean()), scale)
                means.append(diff.mean() / scale)
        if means and len(means) >= 8:
            assert np.median(means) <= BF16_MEDIAN_TOL, (rid, float(np.median(means)))
