"""Grouped-query attention with normalised queries and keys, chunks or a window, and a sink in the softmax."""
from __future__ import annotations

import torch

from ..config.model_config import ConfigError
from ..csrc import ops
from ..weights.loader import TensorSpec
from .attention import TiledAttention
from .base import Mixer, PagedKV, SlotState
from .gathered_attention import PortionAttention
from .linear import Linear
from .registry import register_mixer, POSITION_ENCODINGS


@register_mixer("normed_attention")
class NormedAttention(PortionAttention, Mixer):
    """Causal softmax attention over the paged cache in which

      * keys and queries have one size per head (head_dim) and values another (v_dim); query head h reads key/value
        head h // (heads / kv_heads);
      * with qk_norm every head of q and of k is normalised before it is rotated: x / sqrt(mean(x^2) + eps) * w, one
        weight [head_dim] for all heads of q and one for all heads of k;
      * the position encoding (kind rope_live) rotates the first part of a head, in halves or in neighbouring pairs,
        with frequencies that may be stretched, and a magnitude on cos and sin;
      * the score is scale * q.k with `scale` given;
      * a query sees the keys up to its own: all of them, the last `window` of them, or (chunk) those of its own
        chunk, the chunks counted from position 0 of the request whatever the portions a prompt came in;
      * with sink the softmax's denominator has one more term exp(sink_h), a learned number per head that has no key
        and no value; sink "zero" is such a term with the score 0 for every head and no tensor (the denominator is one
        plus the sum);
      * qk_norm "whole" normalises q as ONE vector over all its heads (and k likewise), with weights of that whole
        size, instead of head by head;
      * qkv_bias adds a bias to each of the three projections;
      * conv > 1 puts a causal convolution over time of `conv` taps on every channel of q, k and v, right behind the
        projection (no activation); its last conv - 1 inputs are a state of the request;
      * softcap > 0 turns a score s into softcap * tanh(s / softcap);
      * out_gate multiplies the heads' outputs, element by element, by sigmoid(Wg x) ahead of the output projection.

    params: hidden, heads, kv_heads, head_dim, v_dim, scale, window, chunk (at most one of the two), qk_norm (False,
    True or "head", "whole"), sink (False, True or "learned", "zero"), eps, position, qkv_bias, conv, softcap, out_gate.
    Tensors: <prefix>q [heads*head_dim, hidden], k [kv_heads*head_dim, hidden], v [kv_heads*v_dim, hidden],
    q.norm, k.norm [head_dim] where qk_norm ([heads*head_dim] and [kv_heads*head_dim] where "whole"), sink [heads] where
    the sink is learned, o [hidden, heads*v_dim]; q.b, k.b, v.b where qkv_bias; q.conv, k.conv, v.conv [channels, conv]
    where conv; g [heads*v_dim, hidden] where out_gate.

    q, k and v are one product; one kernel then normalises, rotates and writes keys and values to the pages; pages of a
    chunk that no later query can see go back to the pool.  Prompt portions attend through matrix products over their
    gathered keys, everything else through the 32-bit kernel that reads the pages (PortionAttention).  Where keys and
    values have one size of 64 or 128, the pages fit the tile kernels and there are no chunks, a bfloat16 engine takes
    the dense decoder's roads instead (TiledAttention's plan of a step's tiles): prompt portions the tcgen05 kernel,
    single tokens the copy-engine kernel, both with the cap in their softmax and the sink's term where a row is
    normalised; the output gates multiply where the decode kernel's key splits are merged, or in a kernel of their own."""

    graph_safe = True

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = p["hidden"], p["heads"], p["kv_heads"]
        self.head_dim, self.v_dim = p["head_dim"], p.get("v_dim") or p["head_dim"]
        self.scale, self.eps = float(p["scale"]), float(p.get("eps", 1e-6))
        self.window, self.chunk = p.get("window"), p.get("chunk")
        norm, sink = p.get("qk_norm", False), p.get("sink", False)
        self.qk_norm = bool(norm)
        self.norm_whole = norm == "whole"
        self.sink = bool(sink)
        self.sink_learned = self.sink and sink != "zero"
        if norm not in (False, True, None, "head", "whole") or sink not in (False, True, None, "learned", "zero"):
            raise ConfigError("data_error", f"normed_attention: qk_norm {norm!r}, sink {sink!r}")
        self.qkv_bias, self.out_gate = bool(p.get("qkv_bias", False)), bool(p.get("out_gate", False))
        self.taps, self.softcap = int(p.get("conv") or 0), float(p.get("softcap") or 0.0)
        if self.taps > 16:
            raise ConfigError("unsupported", f"normed_attention: a convolution of {self.taps} taps (up to 16)")
        if self.window and self.chunk:
            raise ConfigError("data_error", "normed_attention: a window or chunks, not both")
        if self.heads % self.kv_heads:
            raise ConfigError("data_error", "attention: heads must be a multiple of kv_heads")
        if self.head_dim % 2 or max(self.head_dim, self.v_dim) > 256:
            raise ConfigError("unsupported", f"attention: head sizes {self.head_dim} / {self.v_dim}: the kernels take "
                                             "even key sizes, and sizes up to 256")
        pos = p["position"]
        self.position = POSITION_ENCODINGS.get(pos.kind)(pos)

    def tiles_fit(self) -> bool:
        """Whether this layer's attention runs on the dense decoder's tile kernels (see the class's text)."""
        return (self.rt.dtype == torch.bfloat16 and self.head_dim == self.v_dim and not self.chunk
                and self.head_dim in ops.TC_ATTENTION_HEAD_DIMS and ops.tile_pages(self.rt.page_tokens))

    def plan_key(self):
        return TiledAttention.plan_key(self) if self.tiles_fit() else PortionAttention.plan_key(self)

    def plan(self, batch):
        return TiledAttention.plan(self, batch) if self.tiles_fit() else PortionAttention.plan(self, batch)

    def attend_tiles(self, q, kv, bt, ctx, out, plan, gate):
        """The step's attention on the tile kernels: the single next tokens at the head of the batch through the
        copy-engine decode kernel, the other entries through the tcgen05 kernel; kv [pages, 2, K, P, d]."""
        T, H, d = q.shape
        n = plan.decode_prefix
        if n:
            ops.decode_attention(q[:n], kv, bt, ctx.token_seq[:n], ctx.positions[:n], out[:n], self.window, self.scale,
                                 softcap=self.softcap, sink=self.sinks, gate=None if gate is None else gate[:n],
                                 status=ctx.status)
        if plan.tiles.shape[0]:
            if plan.slots and getattr(plan, "scratch", None) is None:
                plan.scratch = ops.prefill_attention_scratch(plan.slots, d, q.device)
            ops.prefill_attention_tc(q, kv, bt, plan.tiles, out, self.window, self.scale, status=ctx.status,
                                     segments=plan.segments, items=plan.items, slots=plan.slots,
                                     scratch=getattr(plan, "scratch", None), softcap=self.softcap, sink=self.sinks)
            if gate is not None and T > n:
                ops.sigmoid_gate(out[n:].view(T - n, H * d), gate[n:], ctx.token_seq[n:])
        return out

    @property
    def channels(self):
        return (self.heads + self.kv_heads) * self.head_dim + self.kv_heads * self.v_dim

    def cache_needs(self):
        pages = PagedKV(self.kv_heads, self.head_dim, self.window, self.v_dim, self.chunk)
        return (pages, SlotState((self.channels, self.taps - 1))) if self.taps > 1 else (pages,)

    def tensor_specs(self):
        p, e = self.prefix, self.hidden
        specs = [TensorSpec(p + "q", (self.heads * self.head_dim, e)),
                 TensorSpec(p + "k", (self.kv_heads * self.head_dim, e)),
                 TensorSpec(p + "v", (self.kv_heads * self.v_dim, e))]
        rows = {"q": self.heads * self.head_dim, "k": self.kv_heads * self.head_dim, "v": self.kv_heads * self.v_dim}
        if self.qkv_bias:
            specs += [TensorSpec(p + n + ".b", (rows[n],), wide=True) for n in "qkv"]
        if self.taps:
            specs += [TensorSpec(p + n + ".conv", (rows[n], self.taps), wide=True, std=0.3) for n in "qkv"]
        if self.qk_norm:
            specs += [TensorSpec(p + n + ".norm", (rows[n] if self.norm_whole else self.head_dim,),
                                 init="one_plus_normal", wide=True) for n in "qk"]
        if self.sink_learned:
            specs.append(TensorSpec(p + "sink", (self.heads,), std=1.0, wide=True))
        if self.out_gate:
            specs.append(TensorSpec(p + "g", (self.heads * self.v_dim, e)))
        specs.append(TensorSpec(p + "o", (e, self.heads * self.v_dim)))
        return specs + self.position.tensor_specs()

    def load(self, tensors, rt):
        super().load(tensors, rt)
        p = self.prefix
        ws = [tensors[p + n] for n in ("qkvg" if self.out_gate else "qkv")]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"{p}: the projections are stored in different precisions")
        self.proj = Linear(torch.cat(ws, dim=0).contiguous(), rt.status)
        self.o = Linear(tensors[p + "o"], rt.status)
        self.q_weight = self.k_weight = self.sinks = None
        if self.qk_norm:
            self.q_weight = tensors[p + "q.norm"].to(torch.float32).contiguous()
            self.k_weight = tensors[p + "k.norm"].to(torch.float32).contiguous()
        if self.sink_learned:
            self.sinks = tensors[p + "sink"].to(torch.float32).contiguous()
        elif self.sink:
            self.sinks = torch.zeros(self.heads, dtype=torch.float32, device=rt.device)
        self.bias = self.conv_weight = None
        if self.qkv_bias:
            self.bias = torch.cat([tensors[p + n + ".b"].to(torch.float32) for n in "qkv"]).contiguous()
        if self.taps:
            self.conv_weight = torch.cat([tensors[p + n + ".conv"].to(torch.float32) for n in "qkv"], dim=0).contiguous()
        self.position.load(tensors, rt)
        if not hasattr(self.position, "frequencies64"):
            raise ConfigError("unsupported", "normed_attention takes a position encoding that gives 64-bit frequencies")
        if self.position.rotary_dim > self.head_dim:
            raise ConfigError("data_error", "normed_attention: the rotated part is larger than a head")

    def forward(self, x, ctx, cache, owns_cache=True):
        if not owns_cache:
            raise ops.KernelError("normed_attention: a run that reads another run's keys and values is not offered")
        pages = cache[0]
        T, H, G, dk, dv = x.shape[0], self.heads, self.kv_heads, self.head_dim, self.v_dim
        rt = self.rt
        P = rt.page_tokens
        proj = full = self.proj.f32(x)
        C = self.channels
        if self.taps:
            # the convolution over time of every channel of q, k and v, from the request's last inputs on
            tail = cache[1].state if self.taps > 1 else torch.empty((ctx.slots.shape[0], C, 0), dtype=torch.float32,
                                                                    device=x.device)
            proj = ops.short_conv_silu(full[:, :C], self.conv_weight, tail,
                                       torch.empty((T, C), dtype=torch.float32, device=x.device), ctx.q_start,
                                       ctx.slots, ctx.max_q_len, act=False)
        elif self.out_gate:
            proj = full[:, :C]
        q = torch.empty((T, H, dk), dtype=rt.dtype, device=x.device)
        bt = ctx.block_tables[pages.group]
        kv = pages.kv.view(pages.kv.shape[0], -1)
        pos = self.position
        ops.qk_normed_prepare(proj, self.q_weight, self.k_weight, self.eps, pos.frequencies64(), pos.pairing,
                              pos.magnitude, ctx.positions, ctx.token_seq, bt, q, kv, G, dv, P, status=ctx.status,
                              bias=self.bias, whole=self.norm_whole)
        out = torch.empty((T, H, dv), dtype=rt.dtype, device=x.device)
        gate = full[:, C:] if self.out_gate else None
        plan = ctx.plans.get(TiledAttention.plan_key(self)) if self.tiles_fit() and not ctx.all_decode else None
        if plan is not None:
            self.attend_tiles(q, pages.kv, bt, ctx, out, plan, gate)
        else:
            self.attend(q, kv, bt, ctx, out, kv_heads=G, page_tokens=P, gate=gate,
                        pages=pages.kv if pages.kv.dim() == 5 else None)
        return self.o.f32_sums(out.view(T, H * dv))
