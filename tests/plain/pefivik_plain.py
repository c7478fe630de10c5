"""Plain, slow implementation of the Pefivik decoder: the oracle of the tests.

It shares no code with ``air_b200``: whole sequences, no cache, no batch, numpy on the CPU, one function per
mechanism.  `dtype` is the precision of the arithmetic (float64 for the oracle, float32 to see what 32-bit rounding
alone does).

The design, in this file's notation.  x is the stream [T, E]; m is one constant of the model (residual_mult).

  embedding         x_t = embed[tok_t] + bigram[r_t], r_t = (tok_(t-1) A + tok_t B) mod buckets with A = mul_prev and
                    B = mul_cur; the first token of a sequence takes the table's last row (index `buckets`).
  order             the layers `start` .. `stop - 1` are run `times` times over with the same weights and then the
                    layers behind them follow.  Ahead of pass t (t = 0, 1, ...) of the repeated stretch the stream
                    gets x0 (the embedding's output; not ahead of pass 0) and the row t of the table loop.step.
  layer             x += m mixer(n1(x));  x += m ff(n2(x));  n(x) = x / sqrt(mean(x^2) + eps) g with ONE number g.
  latent_attention  q = x Wq^T (H heads of `dim`); c = rms(x Wdkv^T) w_c (`kv_rank` numbers, what a cache would keep);
                    per head k = c Wuk^T, v = c Wuv^T; score = scale q.k, position i sees j <= i, no positions enter;
                    the softmax's denominator also holds exp(sink_h); head h's output times sigmoid(x Wg^T)_h; Wo.
  hgrn2             q = silu(x Wq^T) (H x dim), v = x Wv^T (H x vdim), f = l + (1 - l) sigmoid(x Wf^T + b_f) per head
                    and channel; S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T; o_t = S_t^T q_t; each head's o divided by its
                    root mean square (times w, one vector [vdim] for all heads); Wo.
  dense             z = x Wup^T + b_up;  y_i = a z_i / r1 + b z_i^2 / r2 + c z_i^3 / r3 + e, r_p = sqrt(mean_i z_i^(2p) + eps)
                    over the row's ff columns;  y Wdown^T + b_down.
  moe               s = sigmoid(x Wr^T); consecutive experts make `count` groups of one size, a group's mark is its best
                    s plus its second best, only the `keep` groups with the highest marks take part; of their experts the `top` with the
                    largest s are taken; weights = s / (sum of the taken s + 1e-20) * router_scale; y = sum_e weight_e
                    expert_e(x) + shared(x); expert(u) = (silu(u Wg^T) * (u Wu^T)) Wd^T.
  output            n(x) with final.norm, the output matrix, then cap * tanh(logits / cap).
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np


def read_safetensors(path):
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n].decode("utf-8"))
    data = memoryview(raw)[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        dt = info["dtype"]
        if dt == "BF16":
            a = (np.frombuffer(data[lo:hi], dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif dt == "F32":
            a = np.frombuffer(data[lo:hi], dtype="<f4")
        elif dt == "I32":
            a = np.frombuffer(data[lo:hi], dtype="<i4")
        else:
            raise ValueError(f"dtype {dt} of {name}")
        out[name] = a.reshape(info["shape"]).copy()
    return out


def read_model(folder):
    with open(f"{folder}/config.json") as f:
        config = json.load(f)
    return config, read_safetensors(f"{folder}/model.safetensors")


# ----------------------------------------------------------------------------- small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def over_rms(x, eps):
    """x divided by its root mean square over the last axis, eps under the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


# ----------------------------------------------------------------------------- mechanisms
def embed_tokens(tokens, table, bigram, buckets, mul_prev, mul_cur):
    tokens = [int(t) for t in tokens]
    rows = [buckets] + [(tokens[i - 1] * mul_prev + tokens[i] * mul_cur) % buckets for i in range(1, len(tokens))]
    return table[tokens] + bigram[rows]


def run_order(n_layers, loop):
    """The runs in order: (layer, pass of the repeated stretch if the run opens one, else None)."""
    start, stop, times = (loop["start"], loop["stop"], loop["times"]) if loop else (0, 0, 1)
    runs = [(i, None) for i in range(start)]
    for t in range(times if stop > start else 0):
        runs += [(i, t if i == start else None) for i in range(start, stop)]
    runs += [(i, None) for i in range(stop if stop > start else start, n_layers)]
    return runs


def latent_attention(h, w, p, eps):
    """h [T, E] -> [T, E].  w: the layer's tensors by what follows 'mix.'."""
    T = h.shape[0]
    H, d, dv = p["heads"], p["dim"], p["vdim"]
    q = (h @ w["q"].T).reshape(T, H, d)
    c = over_rms(h @ w["dkv"].T, eps) * w["dkv.norm"]
    k = (c @ w["uk"].T).reshape(T, H, d)
    v = (c @ w["uv"].T).reshape(T, H, dv)
    gate = sigmoid(h @ w["g"].T)                       # [T, H]
    out = np.zeros((T, H, dv), dtype=h.dtype)
    seen = np.tril(np.ones((T, T), dtype=bool))
    for hd in range(H):
        s = (q[:, hd] @ k[:, hd].T) * p["scale"]
        s = np.where(seen, s, -np.inf)
        top = np.maximum(s.max(axis=1, keepdims=True), w["sink"][hd])
        e = np.exp(s - top)
        weights = e / (e.sum(axis=1, keepdims=True) + np.exp(w["sink"][hd] - top))
        out[:, hd] = (weights @ v[:, hd]) * gate[:, hd:hd + 1]
    return out.reshape(T, H * dv) @ w["o"].T


def hgrn2(h, w, p, eps, state=None):
    """h [T, E] -> [T, E]; state [H, dim, vdim] (zeros at a sequence's start) is updated in place if given."""
    T = h.shape[0]
    H, d, dv = p["heads"], p["dim"], p["vdim"]
    q = silu(h @ w["q"].T).reshape(T, H, d)
    v = (h @ w["v"].T).reshape(T, H, dv)
    low = w["lower"]
    f = (low + (1.0 - low) * sigmoid(h @ w["f"].T + w["f.b"])).reshape(T, H, d)
    S = np.zeros((H, d, dv), dtype=h.dtype) if state is None else state
    o = np.zeros((T, H, dv), dtype=h.dtype)
    for t in range(T):
        S *= f[t][:, :, None]
        S += (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = over_rms(o, eps) * w["norm"]
    return o.reshape(T, H * dv) @ w["o"].T


def poly_norm(z, coef, eps):
    a, b, c, e = (coef[i] for i in range(4))
    return a * over_rms(z, eps) + b * over_rms(z * z, eps) + c * over_rms(z * z * z, eps) + e


def dense_ff(h, w, eps):
    z = h @ w["up"].T + w["up.b"]
    return poly_norm(z, w["act"], eps) @ w["down"].T + w["down.b"]


def gated_expert(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(scores, top, count, keep, margins=None):
    """scores [n] -> the indices of the chosen experts, in falling order of score (of equal ones the lower index).
    margins (a list) receives by how much the choice was made: the smallest gap between a group that takes part and
    one that does not, and between a chosen expert and one that could have been chosen."""
    n = scores.shape[0]
    size = n // count
    marks = []
    for g in range(count):
        part = np.sort(scores[g * size:(g + 1) * size])[::-1]
        marks.append(part[:2].sum())
    order = sorted(range(count), key=lambda g: (-marks[g], g))
    allowed = np.zeros(n, dtype=bool)
    for g in order[:keep]:
        allowed[g * size:(g + 1) * size] = True
    cand = sorted((i for i in range(n) if allowed[i]), key=lambda i: (-scores[i], i))
    if margins is not None:
        if keep < count:
            margins.append(float(marks[order[keep - 1]] - marks[order[keep]]))
        if top < len(cand):
            margins.append(float(scores[cand[top - 1]] - scores[cand[top]]))
    return cand[:top]


def moe_ff(h, w, p, margins=None):
    """w: the layer's tensors by what follows 'mlp.'."""
    r = p["router"]
    top = r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    s = sigmoid(h @ w["router"].T)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = route(s[t], top, groups["count"], groups["keep"], margins)
        total = sum(s[t, e] for e in chosen) + 1e-20
        for e in chosen:
            out[t] += s[t, e] / total * r.get("scale", 1.0) * gated_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"],
                                                                            w[f"e{e}.down"])[0]
    if p.get("shared"):
        out += gated_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    return out


# ----------------------------------------------------------------------------- the model
def _sub(tensors, prefix, dtype):
    return {k[len(prefix):]: v.astype(dtype) if v.dtype.kind == "f" else v for k, v in tensors.items()
            if k.startswith(prefix)}


def forward(config, tensors, tokens, dtype=np.float64, layers_out=None, margins=None):
    """Logits [T, vocab] of one sequence; layers_out (a list) receives the stream after every run, margins (a list)
    by how much every router chose."""
    eps = config["norm"]["eps"]
    m = config["residual_mult"]
    bg = config["embedding"]["bigram"]
    x = embed_tokens(tokens, tensors["embed"].astype(dtype), tensors["bigram"].astype(dtype), bg["buckets"],
                     bg["mul_prev"], bg["mul_cur"])
    x0 = x.copy()
    for i, opens in run_order(len(config["layers"]), config.get("loop")):
        layer = config["layers"][i]
        if opens is not None:
            if opens > 0:
                x = x + x0
            x = x + tensors["loop.step"].astype(dtype)[opens]
        h = over_rms(x, eps) * float(tensors[f"l{i}.norm1"])
        w = _sub(tensors, f"l{i}.mix.", dtype)
        if layer["type"] == "latent_attention":
            y = latent_attention(h, w, layer["mixer"], eps)
        elif layer["type"] == "hgrn2":
            y = hgrn2(h, w, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + m * y
        f = layer.get("mlp")
        if f is not None:
            h = over_rms(x, eps) * float(tensors[f"l{i}.norm2"])
            w = _sub(tensors, f"l{i}.mlp.", dtype)
            if f["kind"] == "dense":
                y = dense_ff(h, w, eps)
            elif f["kind"] == "moe":
                y = moe_ff(h, w, f, margins)
            else:
                raise ValueError(f["kind"])
            x = x + m * y
        if layers_out is not None:
            layers_out.append(x.copy())
    y = over_rms(x, eps) * float(tensors["final.norm"])
    logits = y @ tensors["head"].astype(dtype).T
    cap = config.get("logit_softcap") or 0.0
    if cap > 0:
        logits = cap * np.tanh(logits / cap)
    return logits


def greedy_generate(config, tensors, prompt, new_tokens, dtype=np.float64):
    tokens = list(prompt)
    for _ in range(new_tokens):
        tokens.append(int(np.argmax(forward(config, tensors, tokens, dtype)[-1])))
    return tokens[len(prompt):]
