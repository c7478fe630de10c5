"""Mixers that keep a state of fixed size per request instead of keys and values: a matrix per head that every
token updates and reads (linear attention with gates), and the short convolutions in front of it."""
from __future__ import annotations

import torch

from ..config.model_config import ConfigError
from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import Mixer, SlotState
from .linear import Linear
from .registry import register_mixer


class _StateMixer(Mixer):
    """What the two mixers below share: one product for all their projections of the layer's input, a 32-bit state
    [heads, head_dim, v_dim] per request, and the norm with a gate that follows the read-out."""

    graph_safe = True

    def _project(self, tensors, names, rt):
        ws = [tensors[self.prefix + n] for n in names]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"{self.prefix}: the projections are stored in different precisions")
        self.proj = Linear(torch.cat(ws, dim=0).contiguous(), rt.status)
        self.columns, at = {}, 0
        for n, w in zip(names, ws):
            self.columns[n] = (at, at + w.shape[0])
            at += w.shape[0]

    def _band(self, proj, name):
        lo, hi = self.columns[name]
        return proj[:, lo:hi]

    def _finish(self, o, proj, ctx):
        """norm over each head's read-out, times the weight and silu(gate), then the output projection"""
        T = o.shape[0]
        y = torch.empty((T, self.heads * self.v_dim), dtype=self.rt.dtype, device=o.device)
        ops.gated_rmsnorm(o, self._band(proj, "g"), self.norm_weight, self.eps, y, ctx.token_seq)
        return self.o.f32_sums(y)


@register_mixer("gated_delta")
class GatedDeltaRule(_StateMixer):
    """The gated delta rule.  q, k (kv_heads x head_dim) and v (heads x v_dim) are projections of the input followed by
    a short causal convolution over time per channel (`conv` taps, the last one the current token's) and SiLU; q and k
    are scaled to unit length per head (x / sqrt(sum x^2 + 1e-6)), q also by head_dim^-1/2; head h reads q/k head
    h // (heads / kv_heads).  Per head and token, with b = sigmoid(W_b x) and
    g = exp(-exp(A_log) * softplus(W_a x + dt_bias)):

        S = g S;   u = b (v - S^T k);   S = S + k u^T;   o = S^T q

    then o / sqrt(mean(o^2) + eps) * norm * silu(W_g x), and the output projection.  S and the convolutions' last
    conv - 1 inputs are the request's state, 32-bit, zero at its start.

    params: hidden, heads, kv_heads, head_dim, v_dim, conv, eps.  Tensors: <prefix>q, k, v, each with <name>.conv
    [channels, conv]; b, a [heads, hidden]; A_log, dt_bias [heads]; norm [v_dim]; g [heads*v_dim, hidden];
    o [hidden, heads*v_dim]."""

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = p["hidden"], p["heads"], p["kv_heads"]
        self.head_dim, self.v_dim, self.taps, self.eps = p["head_dim"], p["v_dim"], int(p["conv"]), float(p["eps"])
        if self.heads % self.kv_heads:
            raise ConfigError("data_error", "gated_delta: heads must be a multiple of kv_heads")
        if not (1 <= self.taps <= 16):
            raise ConfigError("unsupported", f"gated_delta: a convolution of {self.taps} taps (the kernel takes 1 to 16)")
        if self.head_dim > 1024:
            raise ConfigError("unsupported", f"gated_delta: {self.head_dim} key channels per head (up to 1,024)")
        self.channels = 2 * self.kv_heads * self.head_dim + self.heads * self.v_dim

    def cache_needs(self):
        return (SlotState((self.heads, self.head_dim, self.v_dim)),
                SlotState((self.channels, max(self.taps - 1, 1))))

    def tensor_specs(self):
        p, e, H, G, d, dv = self.prefix, self.hidden, self.heads, self.kv_heads, self.head_dim, self.v_dim
        rows = {"q": G * d, "k": G * d, "v": H * dv}
        specs = []
        for n in "qkv":
            specs += [TensorSpec(p + n, (rows[n], e)), TensorSpec(p + n + ".conv", (rows[n], self.taps), wide=True, std=0.3)]
        specs += [TensorSpec(p + "b", (H, e)), TensorSpec(p + "A_log", (H,), wide=True),
                  TensorSpec(p + "norm", (dv,), init="one_plus_normal", wide=True), TensorSpec(p + "a", (H, e)),
                  TensorSpec(p + "dt_bias", (H,), wide=True), TensorSpec(p + "g", (H * dv, e)),
                  TensorSpec(p + "o", (e, H * dv))]
        return specs

    def load(self, tensors, rt):
        super().load(tensors, rt)
        p = self.prefix
        self._project(tensors, ["q", "k", "v", "b", "a", "g"], rt)
        f32 = lambda n: tensors[p + n].to(torch.float32).contiguous()
        self.conv_weight = torch.cat([f32(n + ".conv") for n in "qkv"], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm_weight = f32("A_log"), f32("dt_bias"), f32("norm")
        self.o = Linear(tensors[p + "o"], rt.status)

    def forward(self, x, ctx, cache, owns_cache=True):
        state, tail = cache
        T, H, G, d, dv = x.shape[0], self.heads, self.kv_heads, self.head_dim, self.v_dim
        proj = self.proj.f32(x)
        y = torch.empty((T, self.channels), dtype=torch.float32, device=x.device)
        if self.taps > 1:
            ops.short_conv_silu(proj[:, :self.channels], self.conv_weight, tail.state, y, ctx.q_start, ctx.slots,
                                ctx.max_q_len)
        else:
            ops.short_conv_silu(proj[:, :self.channels], self.conv_weight, tail.state[:, :, :0].contiguous(), y,
                                ctx.q_start, ctx.slots, ctx.max_q_len)
        o = torch.empty((T, H, dv), dtype=torch.float32, device=x.device)
        ops.linear_scan(ops.SCAN_DELTA, y[:, :G * d], y[:, G * d:2 * G * d], y[:, 2 * G * d:],
                        self._band(proj, "a"), state.state, o, ctx.q_start, ctx.slots, ctx.token_seq, q_scale=d ** -0.5,
                        beta=self._band(proj, "b"), a_log=self.a_log, dt_bias=self.dt_bias, unit=True, unit_eps=1e-6)
        return self._finish(o, proj, ctx)


@register_mixer("gla")
class GatedLinearAttention(_StateMixer):
    """Gated linear attention.  q = W_q x * head_dim^-1/2, k = W_k x (heads x head_dim), v = W_v x (heads x v_dim);
    a decay per key channel, alpha = sigmoid(W_a2 (W_a1 x) + b_a2)^(1/tau) (a product through a narrow middle);
    per head and token

        S = diag(alpha) S + k v^T;   o = S^T q

    then o / sqrt(mean(o^2) + eps) * norm, times silu(W_g x), and the output projection.  S is the request's state,
    32-bit, zero at its start.  The decay's second product, its sigmoid, logarithm and power are 32-bit.

    params: hidden, heads, head_dim, v_dim, tau, rank (the narrow middle), eps.  Tensors: <prefix>q, k
    [heads*head_dim, hidden]; v, g [heads*v_dim, hidden]; a1 [rank, hidden]; a2 [heads*head_dim, rank]; a2.b
    [heads*head_dim]; norm [v_dim]; o [hidden, heads*v_dim]."""

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.heads, self.head_dim, self.v_dim = p["hidden"], p["heads"], p["head_dim"], p["v_dim"]
        self.tau, self.rank, self.eps = float(p["tau"]), int(p["rank"]), float(p["eps"])
        if self.head_dim > 1024:
            raise ConfigError("unsupported", f"gla: {self.head_dim} key channels per head (up to 1,024)")
        if not (self.tau > 0.0):
            raise ConfigError("data_error", "gla: tau must be positive")

    def cache_needs(self):
        return (SlotState((self.heads, self.head_dim, self.v_dim)),)

    def tensor_specs(self):
        p, e, H, d, dv, r = self.prefix, self.hidden, self.heads, self.head_dim, self.v_dim, self.rank
        return [TensorSpec(p + "q", (H * d, e)), TensorSpec(p + "k", (H * d, e)), TensorSpec(p + "v", (H * dv, e)),
                TensorSpec(p + "g", (H * dv, e)), TensorSpec(p + "o", (e, H * dv)),
                TensorSpec(p + "norm", (dv,), init="one_plus_normal", wide=True), TensorSpec(p + "a1", (r, e)),
                TensorSpec(p + "a2", (H * d, r), wide=True, std=0.3), TensorSpec(p + "a2.b", (H * d,), wide=True)]

    def load(self, tensors, rt):
        super().load(tensors, rt)
        p = self.prefix
        self._project(tensors, ["q", "k", "v", "g", "a1"], rt)
        f32 = lambda n: tensors[p + n].to(torch.float32).contiguous()
        self.a2, self.a2_bias, self.norm_weight = f32("a2"), f32("a2.b"), f32("norm")
        self.o = Linear(tensors[p + "o"], rt.status)

    def forward(self, x, ctx, cache, owns_cache=True):
        (state,) = cache
        T, H, d, dv = x.shape[0], self.heads, self.head_dim, self.v_dim
        proj = self.proj.f32(x)
        z = torch.empty((T, H * d), dtype=torch.float32, device=x.device)
        ops.gemm_f32(self._band(proj, "a1").contiguous(), self.a2, self.a2_bias, z)
        o = torch.empty((T, H, dv), dtype=torch.float32, device=x.device)
        ops.linear_scan(ops.SCAN_GLA, self._band(proj, "q"), self._band(proj, "k"), self._band(proj, "v"), z,
                        state.state, o, ctx.q_start, ctx.slots, ctx.token_seq, q_scale=d ** -0.5, tau=self.tau)
        return self._finish(o, proj, ctx)


@register_mixer("hgrn2")
class HGRN2(_StateMixer):
    """HGRN2: gated linear attention without a key projection; what a channel does not keep of its old state (1 - f) is
    the share of the new value that it takes in.  q = silu(W_q x) (heads x
    head_dim), v = W_v x (heads x v_dim); per head and channel f = l + (1 - l) sigmoid(W_f x + b_f) with a learned lower
    bound l; per head and token

        S = diag(f) S + (1 - f) v^T;   o = S^T q

    (k is not a projection and q carries no factor), then o / sqrt(mean(o^2) + eps) * norm over each head's v_dim numbers (one weight for all
    heads, no gate) and the output projection.  S is the request's state, 32-bit, zero at its start.  The gate, its
    sigmoid and 1 - f are 32-bit; the recurrence is gated linear attention's with k = 1 - f.

    params: hidden, heads, head_dim, v_dim, eps.  Tensors: <prefix>q, f [heads*head_dim, hidden]; f.b, lower
    [heads*head_dim]; v [heads*v_dim, hidden]; norm [v_dim]; o [hidden, heads*v_dim]."""

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.heads, self.head_dim, self.v_dim = p["hidden"], p["heads"], p["head_dim"], p["v_dim"]
        self.eps = float(p["eps"])
        if self.head_dim > 1024:
            raise ConfigError("unsupported", f"hgrn2: {self.head_dim} channels per head (up to 1,024)")

    def cache_needs(self):
        return (SlotState((self.heads, self.head_dim, self.v_dim)),)

    def tensor_specs(self):
        p, e, H, d, dv = self.prefix, self.hidden, self.heads, self.head_dim, self.v_dim
        return [TensorSpec(p + "q", (H * d, e)), TensorSpec(p + "f", (H * d, e)), TensorSpec(p + "f.b", (H * d,), wide=True),
                TensorSpec(p + "lower", (H * d,), init="uniform", std=0.9, wide=True), TensorSpec(p + "v", (H * dv, e)),
                TensorSpec(p + "norm", (dv,), init="one_plus_normal", wide=True), TensorSpec(p + "o", (e, H * dv))]

    def load(self, tensors, rt):
        super().load(tensors, rt)
        p = self.prefix
        self._project(tensors, ["q", "f", "v"], rt)
        f32 = lambda n: tensors[p + n].to(torch.float32).contiguous()
        self.gate_bias, self.lower, self.norm_weight = f32("f.b"), f32("lower"), f32("norm")
        self.o = Linear(tensors[p + "o"], rt.status)

    def forward(self, x, ctx, cache, owns_cache=True):
        (state,) = cache
        T, H, dv = x.shape[0], self.heads, self.v_dim
        proj = self.proj.f32(x)
        o = torch.empty((T, H, dv), dtype=torch.float32, device=x.device)
        ops.linear_scan(ops.SCAN_HGRN, self._band(proj, "q"), None, self._band(proj, "v"), self._band(proj, "f"),
                        state.state, o, ctx.q_start, ctx.slots, ctx.token_seq, lower=self.lower,
                        gate_bias=self.gate_bias)
        y = torch.empty((T, H * dv), dtype=self.rt.dtype, device=o.device)
        ops.gated_rmsnorm(o, None, self.norm_weight, self.eps, y, ctx.token_seq)
        return self.o.f32_sums(y)


@register_mixer("retention")
class Retention(_StateMixer):
    """Retention: linear attention with one constant decay per head and neither softmax nor denominator.  q = W_q x,
    k = W_k x (heads x head_dim), v = W_v x (heads x v_dim); q and k are rotated by the token's position (the position
    encoding's frequencies, the first part of a head), k is then multiplied by head_dim^-1/2; per head and token

        S = g_h S + k v^T;   o = S^T q

    with g_h the head's entry of `decay`; then each head's o over its root mean square (o / sqrt(mean(o^2) + eps), no
    weight), times silu(W_g x), and the output projection.  S is the request's state, 32-bit, zero at its start.  The
    rotation, the state and the norm are 32-bit.

    params: hidden, heads, head_dim, v_dim, decay (a number per head), eps, position (a position encoding that gives
    64-bit frequencies, or none).  Tensors: <prefix>q, k [heads*head_dim, hidden]; v, g [heads*v_dim, hidden];
    o [hidden, heads*v_dim]."""

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        from .registry import POSITION_ENCODINGS
        p = spec.params
        self.hidden, self.heads, self.head_dim, self.v_dim = p["hidden"], p["heads"], p["head_dim"], p["v_dim"]
        self.eps = float(p["eps"])
        self.decay = tuple(float(g) for g in p["decay"])
        if len(self.decay) != self.heads:
            raise ConfigError("data_error", f"retention: {len(self.decay)} decays for {self.heads} heads")
        if self.head_dim > 1024:
            raise ConfigError("unsupported", f"retention: {self.head_dim} key channels per head (up to 1,024)")
        pos = p.get("position")
        self.position = POSITION_ENCODINGS.get(pos.kind)(pos) if pos is not None else None

    def cache_needs(self):
        return (SlotState((self.heads, self.head_dim, self.v_dim)),)

    def tensor_specs(self):
        p, e, H, d, dv = self.prefix, self.hidden, self.heads, self.head_dim, self.v_dim
        return [TensorSpec(p + "q", (H * d, e)), TensorSpec(p + "k", (H * d, e)), TensorSpec(p + "v", (H * dv, e)),
                TensorSpec(p + "g", (H * dv, e)), TensorSpec(p + "o", (e, H * dv))]

    def load(self, tensors, rt):
        super().load(tensors, rt)
        self._project(tensors, ["q", "k", "v", "g"], rt)
        self.o = Linear(tensors[self.prefix + "o"], rt.status)
        self.decays = torch.tensor(self.decay, dtype=torch.float32, device=rt.device)
        self.norm_weight = torch.ones(self.v_dim, dtype=torch.float32, device=rt.device)
        self.freq = None
        if self.position is not None:
            self.position.load(tensors, rt)
            if self.position.rotary_dim:
                if not hasattr(self.position, "frequencies64") or getattr(self.position, "pairing", "half") != "half" \
                        or getattr(self.position, "magnitude", 1.0) != 1.0:
                    raise ConfigError("unsupported", "retention takes a half-split rotation with 64-bit frequencies")
                if self.position.rotary_dim > self.head_dim:
                    raise ConfigError("data_error", "retention: the rotated part is larger than a head")
                self.freq = self.position.frequencies64()

    def forward(self, x, ctx, cache, owns_cache=True):
        (state,) = cache
        T, H, d, dv = x.shape[0], self.heads, self.head_dim, self.v_dim
        proj = self.proj.f32(x)
        o = torch.empty((T, H, dv), dtype=torch.float32, device=x.device)
        ops.linear_scan(ops.SCAN_RETENTION, self._band(proj, "q"), self._band(proj, "k"), self._band(proj, "v"),
                        self.decays, state.state, o, ctx.q_start, ctx.slots, ctx.token_seq, positions=ctx.positions,
                        freq=self.freq, k_scale=d ** -0.5)
        return self._finish(o, proj, ctx)
