"""Attention over a compressed latent: per token the cache holds one short row instead of keys and values per head."""
from __future__ import annotations

import torch

from ..config.model_config import ConfigError
from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import Mixer, PagedLatent
from .gathered_attention import PortionAttention
from .linear import Linear
from .registry import register_mixer, POSITION_ENCODINGS


@register_mixer("latent_attention")
class LatentAttention(PortionAttention, Mixer):
    """q = Wq x, per head [head_dim plain | rot_dim rotated].  (c | kr) = Wdkv x: c (kv_rank columns) is normalised,
    c = rms(c) * w_c; kr (rot_dim columns) is one rotated key part for all heads.  Head h has the key [Wuk_h c | kr]
    and the value Wuv_h c; score = scale * (q_plain . Wuk_h c + q_rot . kr); causal softmax over the last `window` keys
    (None: all); output matrix on the concatenated heads.  Only the row [c | kr] is kept per token.
    rot_dim may be 0: no position enters, there is no kr, and `position` is not given.  With sink the softmax's
    denominator has one more term exp(sink_h), a learned number per head without key or value.  With head_gate head
    h's output is multiplied by sigmoid(Wg x)_h, one more projection of the layer's input.

    The key and value expansions are never applied to the cache: q_plain is carried through Wuk_h once per query
    (q'_h = Wuk_h^T q_plain_h, so that q_plain . Wuk_h c = q'_h . c), every head then attends over the same rows [c | kr]
    with the query [q'_h | q_rot_h] and sums the rows' first kv_rank elements, and Wuv_h expands that sum.  The two
    small products per head are one grouped product each.

    params: hidden, heads, head_dim, rot_dim, v_dim, kv_rank, scale, window, eps, sink, head_gate, position (rope_live
    with rotary_dim = rot_dim; absent where rot_dim is 0), borrows (the layer has no Wdkv: its run reads the rows that another layer's run keeps), keep (the
    widest window among the layers that read this layer's rows: pages older than that go back to the pool).
    Tensors: <prefix>q [heads*(head_dim+rot_dim), hidden], dkv [kv_rank+rot_dim, hidden], dkv.norm [kv_rank],
    uk [heads*head_dim, kv_rank], uv [heads*v_dim, kv_rank], o [hidden, heads*v_dim]; sink [heads] where sink; g [heads,
    hidden] where head_gate."""

    graph_safe = True

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.heads, self.head_dim = p["hidden"], p["heads"], p["head_dim"]
        self.rot_dim, self.v_dim, self.rank = p["rot_dim"], p["v_dim"], p["kv_rank"]
        self.scale, self.eps = float(p["scale"]), float(p.get("eps", 1e-6))
        self.window, self.borrows, self.chunk, self.sinks = p.get("window"), bool(p.get("borrows", False)), None, None
        self.keep = p.get("keep", self.window) if self.window else None
        self.sink, self.head_gate = bool(p.get("sink", False)), bool(p.get("head_gate", False))
        if self.rank + self.rot_dim > 640:
            raise ConfigError("unsupported", f"latent attention: rows of {self.rank + self.rot_dim} numbers: the "
                                             "attention kernel takes up to 640")
        pos = p.get("position")
        if (pos is None) != (self.rot_dim == 0):
            raise ConfigError("data_error", "latent attention: a rotated part needs a position encoding, and only it")
        self.position = None if pos is None else POSITION_ENCODINGS.get(pos.kind)(pos)

    def cache_needs(self):
        return () if self.borrows else (PagedLatent(self.rank + self.rot_dim, self.keep),)

    def tensor_specs(self):
        p, e, H = self.prefix, self.hidden, self.heads
        specs = [TensorSpec(p + "q", (H * (self.head_dim + self.rot_dim), e))]
        if not self.borrows:
            specs += [TensorSpec(p + "dkv", (self.rank + self.rot_dim, e)),
                      TensorSpec(p + "dkv.norm", (self.rank,), init="one_plus_normal", wide=True)]
        specs += [TensorSpec(p + "uk", (H * self.head_dim, self.rank)), TensorSpec(p + "uv", (H * self.v_dim, self.rank)),
                  TensorSpec(p + "o", (e, H * self.v_dim))]
        if self.sink:
            specs.append(TensorSpec(p + "sink", (H,), std=1.0, wide=True))
        if self.head_gate:
            specs.append(TensorSpec(p + "g", (H, e)))
        return specs + (self.position.tensor_specs() if self.position is not None else [])

    def load(self, tensors, rt):
        super().load(tensors, rt)
        p, H, d, R = self.prefix, self.heads, self.head_dim, self.rank
        # one product for all projections of the layer's input: q, then (where the layer makes its own latent) the
        # latent's rows, then the gates; rows of zeros fill the matrix up to a multiple of 8, which the tensor-core
        # kernels want
        ws = [tensors[p + "q"]]
        self.c_weight = None
        if not self.borrows:
            ws.append(tensors[p + "dkv"])
            self.c_weight = tensors[p + "dkv.norm"].to(torch.float32).contiguous()
        self.gate_column = sum(w.shape[0] for w in ws)
        if self.head_gate:
            ws.append(tensors[p + "g"])
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"{p}: the projections are stored in different precisions")
        rows = sum(w.shape[0] for w in ws)
        if rows % 8:
            ws.append(torch.zeros((8 - rows % 8, self.hidden), dtype=ws[0].dtype, device=ws[0].device))
        self.proj = Linear(torch.cat(ws, dim=0).contiguous() if len(ws) > 1 else ws[0], rt.status)
        self.sinks = tensors[p + "sink"].to(torch.float32).contiguous() if self.sink else None
        # Wuk_h [d, R] is the product's [K, N]: the grouped product wants [N, K] per head
        self.uk_t = tensors[p + "uk"].view(H, d, R).transpose(1, 2).contiguous()
        self.uv = tensors[p + "uv"].view(H, self.v_dim, R).contiguous()
        self.o = Linear(tensors[p + "o"], rt.status)
        if self.position is not None:
            self.position.load(tensors, rt)
            if not hasattr(self.position, "frequencies64") or self.position.pairing != "half":
                raise ConfigError("unsupported", "latent attention takes a rotation in halves with 64-bit frequencies")
            if self.position.rotary_dim != self.rot_dim:
                raise ConfigError("data_error", "latent attention: the rotation covers the rotated part, all of it")

    def forward(self, x, ctx, cache, owns_cache=True):
        if owns_cache == self.borrows:
            raise ops.KernelError("latent attention: the layer and the run list disagree on whose rows the layer reads")
        (latent,) = cache
        T, H, d, rot, R, dv = x.shape[0], self.heads, self.head_dim, self.rot_dim, self.rank, self.v_dim
        rt = self.rt
        dev = x.device
        bt = ctx.block_tables[latent.group]
        proj = self.proj.f32(x)
        q_plain = torch.empty((T, H, d), dtype=rt.dtype, device=dev)
        q_full = torch.empty((T, H, R + rot), dtype=torch.float32, device=dev)
        gate = torch.empty((T, H), dtype=torch.float32, device=dev) if self.head_gate else None
        ops.latent_prepare(proj, self.c_weight, self.eps,
                           self.position.frequencies64() if self.position is not None else None, ctx.positions,
                           ctx.token_seq, bt, q_plain, q_full, latent.rows, owns_cache, status=ctx.status,
                           gate_out=gate, gate_column=self.gate_column)
        ops.grouped_gemm(q_plain, self.uk_t, q_full, R, d, lda=H * d, ldo=H * (R + rot), groups=H, a_group_stride=d,
                         o_group_stride=R + rot, a_local=True, o_local=True, rows_per_group=T)
        summed = torch.empty((T, H, R), dtype=rt.dtype, device=dev)
        self.attend(q_full, latent.rows, bt, ctx, summed, latent=True)
        out = torch.empty((T, H, dv), dtype=rt.dtype, device=dev)
        ops.grouped_gemm(summed, self.uv, out, dv, R, lda=H * R, ldo=H * dv, groups=H, a_group_stride=R,
                         o_group_stride=dv, a_local=True, o_local=True, rows_per_group=T, o_scale=gate, o_scale_ld=H)
        return self.o.f32_sums(out.view(T, H * dv))
