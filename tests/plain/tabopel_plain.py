"""Plain, slow implementation of the Tabopel decoder: the oracle of the tests.

It shares no code with ``air_b200``: whole sequences, no cache, no batch, numpy on the CPU, one function per
mechanism.  `dtype` is the precision of the arithmetic (float64 for the oracle, float32 to see what 32-bit rounding
alone does).

The design, in this file's notation.  x is the stream [T, E]; n(x; w) = x / sqrt(mean(x^2) + eps) * w.

  embedding     x_t = embed[tok_t] * c, c = embedding.scale.
  order         the layers `start` .. `stop - 1` run `times` times over with the same weights, then the layers behind
                them follow; ahead of pass t the row t of the table loop.step joins the stream (every pass, also t = 0).
  layer         x += n(mixer(n(x; w1)); w1b);  x += n(ff(n(x; w2)); w2b): a norm on each side of every sub-layer.
  rotation      the first R numbers of a head: element i pairs with i + R/2, angle = position * f_i,
                f_i = base^(-2i/R); (a, b) -> (a cos - b sin, b cos + a sin).  With `scaling` (factor F, low, high,
                original L): the wavelength l = 2 pi / f; f stays where l < L/high, becomes f/F where l > L/low, and
                between them (1 - s) f/F + s f with s = (L/l - low) / (high - low).
  attention     q, k, v = projections of the input, each channel then a causal convolution over time (taps w[:, j] on
                the inputs t - taps + 1 + j, zeros ahead of the sequence), rotation of q and k, score = scale q.k,
                causal, weights = exp(s_j) / (1 + sum_j exp(s_j)) (a sink of score 0 without a value), all heads times
                sigmoid(Wg input) element by element, Wo.  Query head h reads key/value head h // (H / G).
  attention_2   projections with biases; q (all heads as ONE vector) and k likewise normalised n(.; w) with a weight
                of that whole size; rotation; score = cap tanh(scale q.k / cap); the softmax's denominator has one
                more term exp(sink_h); Wo.
  retention     q, k rotated, k times dim^(-1/2); S_t = g_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with a constant g_h
                per head; each head's o over its root mean square (no weight), all heads times silu(Wg input), Wo.
  dense         Wdown relu(Wup u)^2.
  moe           z = Wr u; s = softmax(z) over all outputs of the router; the `top` largest of s + correction are
                taken (of equal ones the lower index), their weights are s itself; the last `identity` outputs of the
                router stand for experts that return u; y = sum weight_e expert_e(u), expert = Wdown relu(Wup u)^2.
  output        n(x; final.norm), then the output matrix.
"""
from __future__ import annotations

import math

import numpy as np


# ----------------------------------------------------------------------------- small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_norm(x, w, eps):
    """x over its root mean square along the last axis (eps under the root), times w (None: no weight)."""
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if w is None else y * w


def relu_squared(z):
    r = np.maximum(z, 0.0)
    return r * r


# ----------------------------------------------------------------------------- positions
def frequencies(rot):
    """float64 [dims / 2]: the angle per position of every rotated pair."""
    R = int(rot["dims"])
    f = np.array([float(rot["base"]) ** (-2.0 * i / R) for i in range(R // 2)], dtype=np.float64)
    s = rot.get("scaling")
    if not s:
        return f
    F, low, high, L = float(s["factor"]), float(s["low"]), float(s["high"]), float(s["original"])
    out = f.copy()
    for i, fi in enumerate(f):
        wave = 2.0 * math.pi / fi
        if wave < L / high:
            continue
        if wave > L / low:
            out[i] = fi / F
        else:
            t = (L / wave - low) / (high - low)
            out[i] = (1.0 - t) * fi / F + t * fi
    return out


def rotate(x, positions, rot, dtype):
    """x [T, heads, dim]: the first rot.dims numbers of every head turned by position * frequency."""
    R = int(rot["dims"]) if rot else 0
    if R == 0:
        return x
    f = frequencies(rot)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = np.cos(angle).astype(dtype)[:, None, :], np.sin(angle).astype(dtype)[:, None, :]
    a, b = x[..., :R // 2], x[..., R // 2:R]
    out = x.copy()
    out[..., :R // 2] = a * c - b * s
    out[..., R // 2:R] = b * c + a * s
    return out


# ----------------------------------------------------------------------------- mechanisms
def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros ahead of the sequence."""
    T, taps = u.shape[0], w.shape[1]
    y = np.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def softmax_attention(q, k, v, scale, softcap=0.0, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  Causal.  sink [H]: one more score per head that has no
    value (the denominator gets exp(sink_h))."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, h]) * scale
            if softcap:
                s = softcap * np.tanh(s / softcap)
            extra = float(sink[h]) if sink is not None else None
            m = max(s.max(), extra) if extra is not None else s.max()
            e = np.exp(s - m)
            den = e.sum() + (math.exp(extra - m) if extra is not None else 0.0)
            out[t, h] = (e / den) @ v[:t + 1, g]
    return out


def mixer_attention(w, p, x, m, positions, eps, dtype):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = x.shape[0]
    q, k, v = x @ w[p + "q"].T, x @ w[p + "k"].T, x @ w[p + "v"].T
    if m.get("conv"):
        q, k, v = (causal_conv(u, w[p + n + ".conv"]) for u, n in ((q, "q"), (k, "k"), (v, "v")))
    q = rotate(q.reshape(T, H, d), positions, m.get("rot"), dtype)
    k = rotate(k.reshape(T, G, d), positions, m.get("rot"), dtype)
    o = softmax_attention(q, k, v.reshape(T, G, dv), float(m["scale"]), sink=np.zeros(H))
    o = o.reshape(T, H * dv) * sigmoid(x @ w[p + "g"].T)
    return o @ w[p + "o"].T


def mixer_attention_2(w, p, x, m, positions, eps, dtype):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = x.shape[0]
    q = x @ w[p + "q"].T + w[p + "q.b"]
    k = x @ w[p + "k"].T + w[p + "k.b"]
    v = x @ w[p + "v"].T + w[p + "v.b"]
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    q = rotate(q.reshape(T, H, d), positions, m.get("rot"), dtype)
    k = rotate(k.reshape(T, G, d), positions, m.get("rot"), dtype)
    o = softmax_attention(q, k, v.reshape(T, G, dv), float(m["scale"]), softcap=float(m.get("softcap") or 0.0),
                          sink=w[p + "sink"])
    return o.reshape(T, H * dv) @ w[p + "o"].T


def mixer_retention(w, p, x, m, positions, eps, dtype):
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = x.shape[0]
    q = rotate((x @ w[p + "q"].T).reshape(T, H, d), positions, m.get("rot"), dtype)
    k = rotate((x @ w[p + "k"].T).reshape(T, H, d), positions, m.get("rot"), dtype) * dtype(d ** -0.5)
    v = (x @ w[p + "v"].T).reshape(T, H, dv)
    o = np.zeros((T, H, dv), dtype=dtype)
    for h in range(H):
        S = np.zeros((d, dv), dtype=dtype)
        g = dtype(m["decay"][h])
        for t in range(T):
            S = g * S + np.outer(k[t, h], v[t, h])
            o[t, h] = S.T @ q[t, h]
    o = rms_norm(o, None, eps).reshape(T, H * dv) * silu(x @ w[p + "g"].T)
    return o @ w[p + "o"].T


MIXERS = {"attention": mixer_attention, "attention_2": mixer_attention_2, "retention": mixer_retention}


def dense_ff(w, p, u):
    return relu_squared(u @ w[p + "up"].T) @ w[p + "down"].T


def route(w, p, u, f):
    """(chosen [T, top] indices, weights [T, top], the smallest gap between a taken and a left choice score)."""
    top = f["router"]["top"]
    z = u @ w[p + "router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(axis=-1, keepdims=True)
    choice = s + w[p + "correction"]
    order = np.argsort(-choice, axis=-1, kind="stable")
    chosen = order[:, :top]
    weights = np.take_along_axis(s, chosen, axis=-1)
    ranked = np.take_along_axis(choice, order, axis=-1)
    margin = float((ranked[:, top - 1] - ranked[:, top]).min()) if ranked.shape[1] > top else math.inf
    return chosen, weights, margin


def moe_ff(w, p, u, f, margins=None):
    n = f["router"]["experts"]
    chosen, weights, margin = route(w, p, u, f)
    if margins is not None:
        margins.append(margin)
    y = np.zeros_like(u)
    for t in range(u.shape[0]):
        for e, g in zip(chosen[t], weights[t]):
            y[t] += g * (u[t] if e >= n else dense_ff(w, f"{p}e{e}.", u[t][None])[0])
    return y


def feed_forward(w, p, u, f, margins=None):
    return dense_ff(w, p, u) if f["kind"] == "dense" else moe_ff(w, p, u, f, margins)


# ----------------------------------------------------------------------------- the model
def run_order(config):
    """[(layer, row of loop.step that joins the stream ahead of it or None)] in the order in which the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(n)]
    a, b = loop["start"], loop["stop"]
    order = [(i, None) for i in range(a)]
    for t in range(loop["times"]):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def forward(config, weights, tokens, dtype=np.float64, taps=None, margins=None):
    """Logits [T, vocab] of one sequence.  taps: a list that receives the stream after every run of a layer."""
    w = {k: (v.astype(dtype) if v.dtype.kind == "f" else v) for k, v in weights.items()}
    eps = dtype(config["norm"]["eps"])
    tokens = np.asarray(tokens)
    positions = np.arange(len(tokens))
    x = w["embed"][tokens] * dtype(config["embedding"]["scale"])
    for i, row in run_order(config):
        if row is not None:
            x = x + w["loop.step"][row]
        layer = config["layers"][i]
        p = f"l{i}."
        y = MIXERS[layer["type"]](w, p + "mix.", rms_norm(x, w[p + "norm1"], eps), layer["mixer"], positions, eps, dtype)
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            y = feed_forward(w, p + "mlp.", rms_norm(x, w[p + "norm2"], eps), layer["mlp"], margins)
            x = x + rms_norm(y, w[p + "norm2b"], eps)
        if taps is not None:
            taps.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
