"""Set-up of the Pefivik tests: small configurations that differ in every size and option, model folders with weights
drawn so that a fault shows, and the comparison with the plain implementation."""
import functools
import tempfile

import numpy as np

from bivizen_util import bf16


def latent(heads, dim, vdim, rank, scale):
    return dict(type="latent_attention", mixer=dict(heads=heads, dim=dim, vdim=vdim, kv_rank=rank, scale=scale))


def hgrn(heads, dim, vdim):
    return dict(type="hgrn2", mixer=dict(heads=heads, dim=dim, vdim=vdim))


def dense(layer, ff):
    return dict(layer, mlp=dict(kind="dense", ff=ff))


def moe(layer, experts, top, ff, groups=None, scale=1.0, shared=None):
    r = dict(experts=experts, top=top, scale=scale)
    if groups:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    f = dict(kind="moe", expert=dict(ff=ff), router=r)
    if shared:
        f["shared"] = dict(ff=shared)
    return dict(layer, mlp=f)


def bare(layer):
    return dict(layer, mlp=None)


def config(vocab, width, eps, mult, cap, bigram, loop, layers):
    d = dict(architecture="Pefivik", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=mult,
             logit_softcap=cap, embedding=dict(bigram=dict(buckets=bigram[0], mul_prev=bigram[1], mul_cur=bigram[2])),
             layers=layers)
    if loop:
        d["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return d


# A: a stretch of two layers (a state mixer among them) that runs three times and starts at layer 0; experts in
#    three groups of which two take part; a layer without feed-forward; sizes that are no multiples of 8; more buckets
#    than tokens.
# B: no repeated stretch at all; one head; one expert of one (top == experts == 1, one group); a state mixer first and
#    last; a dense layer whose ff is smaller than the width; no soft cap; no shared expert.
# D: no size is a multiple of 4 (width, heads' sizes, the latent, ff): the kernels' roads of one element per access.
# C: a stretch that is run once (it still adds its row), at the model's end; heads of 64 over a latent of 128 on
#    pages of 64; groups of one expert each; every expert of the kept groups chosen.
CONFIGS = {
    "A": config(211, 72, 1e-5, 0.6, 12.0, (389, 31, 5), (0, 2, 3), [
        moe(latent(4, 24, 20, 40, 0.2), 6, 2, 40, groups=(3, 2), scale=1.7, shared=48),
        dense(hgrn(3, 20, 12), 100),
        bare(latent(2, 16, 24, 56, 0.25)),
        moe(hgrn(1, 40, 8), 8, 3, 24, groups=(2, 1), scale=0.8),
        dense(latent(5, 8, 8, 24, 0.3), 56)]),
    "B": config(333, 96, 1e-6, 1.0, 0.0, (97, 1, 1), None, [
        dense(hgrn(2, 16, 16), 40),
        moe(latent(1, 32, 40, 48, 0.18), 1, 1, 64),
        moe(latent(6, 16, 8, 16, 0.22), 4, 4, 32, scale=2.0, shared=16),
        bare(hgrn(4, 8, 24))]),
    "C": config(190, 128, 1e-6, 0.8, 25.0, (190, 1000003, 17), (1, 3, 1), [
        dense(latent(4, 64, 64, 128, 0.11), 256),
        moe(latent(2, 32, 64, 64, 0.15), 8, 4, 64, groups=(8, 5), scale=1.2, shared=128),
        dense(hgrn(2, 64, 32), 192)]),
    "D": config(150, 90, 1e-5, 0.8, 9.0, (77, 3, 5), (1, 3, 2), [
        dense(latent(3, 10, 6, 18, 0.2), 50),
        moe(hgrn(3, 10, 6), 6, 2, 30, groups=(3, 2), scale=1.0, shared=22),
        dense(latent(2, 14, 10, 22, 0.2), 34)]),
}
SEEDS = {"A": 31, "B": 32, "C": 33, "D": 34}


def random_config(seed):
    """A configuration drawn at random: 2 to 6 layers in any order, a repeated stretch anywhere (or none), every size
    and constant from a list that includes 1, equal and unequal sizes and sizes that are no multiples of 8 or 16."""
    rng = np.random.default_rng(seed)
    width = int(rng.choice([40, 64, 72, 96, 128, 160, 200]))
    layers = []
    for i in range(int(rng.integers(2, 7))):
        if rng.random() < 0.6:
            layer = latent(int(rng.choice([1, 2, 3, 4, 6, 8, 16])), int(rng.choice([8, 16, 24, 32, 64])),
                           int(rng.choice([8, 16, 24, 40, 64])), int(rng.choice([8, 24, 40, 56, 96, 112, 128])),
                           float(rng.choice([0.1, 0.2, 0.3])))
        else:
            layer = hgrn(int(rng.choice([1, 2, 3, 4])), int(rng.choice([4, 8, 20, 32, 48, 64, 100])),
                         int(rng.choice([4, 8, 12, 32, 64])))
        u = rng.random()
        if u < 0.15:
            layers.append(bare(layer))
        elif u < 0.5:
            layers.append(dense(layer, int(rng.choice([16, 40, 100, 256, 320]))))
        else:
            count = int(rng.choice([1, 2, 3, 4]))
            size = int(rng.choice([1, 2, 3, 4]))
            keep = int(rng.integers(1, count + 1))
            top = int(rng.integers(1, keep * size + 1))
            layers.append(moe(layer, count * size, top, int(rng.choice([16, 24, 40, 64, 100])),
                              groups=(count, keep) if count > 1 or rng.random() < 0.5 else None,
                              scale=float(rng.choice([0.5, 1.0, 1.25, 2.5])),
                              shared=None if rng.random() < 0.3 else int(rng.choice([16, 40, 64, 96]))))
    n = len(layers)
    loop = None
    if rng.random() < 0.8:
        start = int(rng.integers(0, n))
        loop = (start, int(rng.integers(start + 1, n + 1)), int(rng.choice([1, 2, 2, 3])))
    return config(int(rng.integers(50, 700)), width, float(rng.choice([1e-6, 1e-5, 1e-4])),
                  float(rng.choice([0.4, 0.75, 1.0, 1.3])), float(rng.choice([0.0, 8.0, 20.0])),
                  (int(rng.choice([1, 61, 521, 4099])), int(rng.choice([0, 1, 131, 65537])), int(rng.choice([1, 11, 31]))),
                  loop, layers)


ROUTE_CHANNELS = (1.0, 0.52, 0.27, 0.14, 0.075)


def _bits(n):
    return max(0, int(np.ceil(np.log2(n)))) if n > 1 else 0


def draw_tensors(cfg, seed):
    """name -> float32 array (bfloat16 values).  The scales are chosen so that every mechanism matters: attention
    scores have a standard deviation of about 2.5 (a key that is lost or added moves the logits far beyond bfloat16's
    rounding), sinks are of the order of the scores, rows of the table of pairs are as large as the token rows (a wrong
    previous token shows), some channels of the state mixers forget slowly (lower bounds near 1), and a sub-layer's
    output is of the order of the stream it is added to.

    A router is a discontinuity: with random router weights one token in a hundred has two experts so close that
    bfloat16's rounding picks the other one, and the logits then differ by a whole expert.  So the routers here decide by
    a few channels of the stream that only the token table and the norms touch (the table of pairs, the rows that
    passes add, the output matrices and their biases leave them alone): a token carries a sign pattern with falling
    magnitudes there, and an expert's router row the pattern of its index, the bits of its group on the channels
    with the large magnitudes and the bits of its place in the group behind them.  Every group then holds the same
    places, so the order of the groups' marks is the order of their own bits, and all sums of the magnitudes with
    signs are apart.  Which experts a token takes is then a matter of the token, clear of rounding; their weights still
    depend on everything, through the norms and the rest of the router row."""
    rng = np.random.default_rng(seed)
    e, m = cfg["width"], cfg["residual_mult"]
    t = {}
    nr = 0
    for layer in cfg["layers"]:
        f = layer.get("mlp")
        if f and f["kind"] == "moe":
            g = (f["router"].get("groups") or {"count": 1})["count"]
            nr = max(nr, _bits(g) + _bits(f["router"]["experts"] // g))
    assert nr <= len(ROUTE_CHANNELS)

    def mat(out, inp, gain=1.0):
        return rng.normal(0.0, gain / np.sqrt(inp), size=(out, inp))

    buckets = cfg["embedding"]["bigram"]["buckets"]
    t["embed"] = rng.normal(0.0, 1.0, size=(cfg["vocab"], e))
    tokens = np.arange(cfg["vocab"])
    for c in range(nr):
        t["embed"][:, c] = np.where((tokens >> c) & 1, 1.0, -1.0) * ROUTE_CHANNELS[c] * 1.5
    t["bigram"] = rng.normal(0.0, 0.8, size=(buckets + 1, e))
    t["bigram"][:, :nr] = 0.0
    if cfg.get("loop"):
        t["loop.step"] = rng.normal(0.0, 0.7, size=(cfg["loop"]["times"], e))
        t["loop.step"][:, :nr] = 0.0
    t["head"] = mat(cfg["vocab"], e, 2.0)
    t["final.norm"] = np.array(1.0 + rng.normal(0.0, 0.1))
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
        t[p + "norm1"] = np.array(1.0 + rng.normal(0.0, 0.1))
        if layer["type"] == "latent_attention":
            R = mx["kv_rank"]
            gain = (2.5 / (mx["scale"] * d ** 0.5)) ** 0.5
            t[p + "mix.q"], t[p + "mix.dkv"] = mat(H * d, e, gain), mat(R, e)
            t[p + "mix.dkv.norm"] = 1.0 + rng.normal(0.0, 0.1, size=R)
            t[p + "mix.uk"], t[p + "mix.uv"] = mat(H * d, R, gain), mat(H * dv, R, 1.5 / m)
            t[p + "mix.sink"] = rng.normal(1.0, 2.0, size=H)
            t[p + "mix.g"] = mat(H, e, 2.0)
        else:
            t[p + "mix.q"], t[p + "mix.f"], t[p + "mix.v"] = mat(H * d, e, 1.5), mat(H * d, e, 2.0), mat(H * dv, e, 1.5)
            t[p + "mix.f.b"] = rng.normal(0.0, 1.0, size=H * d)
            t[p + "mix.lower"] = np.where(rng.random(H * d) < 0.3, rng.uniform(0.97, 0.996, size=H * d),
                                          rng.uniform(0.0, 0.9, size=H * d))
            t[p + "mix.norm"] = 1.0 + rng.normal(0.0, 0.1, size=dv)
        t[p + "mix.o"] = mat(e, H * dv, 1.0 / m)
        t[p + "mix.o"][:nr] = 0.0
        f = layer.get("mlp")
        if not f:
            continue
        t[p + "norm2"] = np.array(1.0 + rng.normal(0.0, 0.1))
        if f["kind"] == "dense":
            t[p + "mlp.up"], t[p + "mlp.up.b"] = mat(f["ff"], e), rng.normal(0.0, 0.3, size=f["ff"])
            t[p + "mlp.down"], t[p + "mlp.down.b"] = mat(e, f["ff"], 0.7 / m), rng.normal(0.0, 0.2, size=e)
            t[p + "mlp.down"][:nr] = 0.0
            t[p + "mlp.down.b"][:nr] = 0.0
            t[p + "mlp.act"] = np.array([rng.normal(1.0, 0.2), rng.normal(0.4, 0.1), rng.normal(-0.15, 0.05),
                                         rng.normal(0.0, 0.1)])
            continue
        r = f["router"]
        n = r["experts"]
        g = (r.get("groups") or {"count": 1})["count"]
        size, gb = n // g, _bits(g)
        t[p + "mlp.router"] = mat(n, e, 0.02)
        for x in range(n):
            code = [(x // size >> c) & 1 for c in range(gb)] + [(x % size >> c) & 1 for c in range(_bits(size))]
            t[p + "mlp.router"][x, :nr] = 0.0
            t[p + "mlp.router"][x, :len(code)] = [(1.0 if b else -1.0) * 1.5 for b in code]
            t[f"{p}mlp.e{x}.gate"], t[f"{p}mlp.e{x}.up"] = mat(f["expert"]["ff"], e, 2.0), mat(f["expert"]["ff"], e, 2.0)
            t[f"{p}mlp.e{x}.down"] = mat(e, f["expert"]["ff"], 0.6 / m)
            t[f"{p}mlp.e{x}.down"][:nr] = 0.0
        if f.get("shared"):
            s = f["shared"]["ff"]
            t[p + "mlp.shared.gate"], t[p + "mlp.shared.up"] = mat(s, e, 1.5), mat(s, e, 1.5)
            t[p + "mlp.shared.down"] = mat(e, s, 0.6 / m)
            t[p + "mlp.shared.down"][:nr] = 0.0
    return {n: bf16(a) for n, a in t.items()}


_tmp = []


@functools.lru_cache(maxsize=None)
def model_folder(name):
    """config.json and model.safetensors (bfloat16) of a test configuration, in a temporary place."""
    import torch
    from air_b200.weights.loader import write_model_folder
    d = tempfile.TemporaryDirectory(prefix=f"air_b200_pefivik_{name}_")
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
    from plain import pefivik_plain as plain
    return plain.read_model(model_folder(name))


_logits = {}


def plain_run(name, tokens):
    """(logits [T, vocab], the smallest margin by which a router chose)."""
    from plain import pefivik_plain as plain
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
    return np.random.default_rng(9000 + seed).integers(0, CONFIGS[name]["vocab"], size=n).tolist()


def plain_greedy(name, prompt, n):
    out, toks = [], list(prompt)
    for _ in range(n):
        nxt = int(plain_logits(name, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out


# float32: sums in another order than the 64-bit oracle.  bfloat16: activations rounded to 8 bits at the inputs of the
# products and in the cache, through up to ten runs of sharp attention (a third of the weight on one key in the mean),
# state mixers and experts.  A request's rows must all be within the row limits, and their median within the tighter
# one.  The routers choose with clear margins (draw_tensors); check() makes sure of it, since a choice that rounding
# can tip voids the comparison.
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
