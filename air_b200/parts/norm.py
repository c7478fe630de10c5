"""RMSNorm fused with the residual addition that precedes it."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import GatedSum, Norm, NormedSum, PreNormed, ScaledSum
from .registry import register_norm


@register_norm("rms")
class RMSNorm(Norm):
    """x * rsqrt(mean(x^2) + eps) * w, product order x*scale*w, no bias, no offset on w
    (AIR: src/reference/reference_executor.cpp:17-27; src/cuda/cuda_backend.cu:789-831).
    params: size, eps; tensor: what follows the prefix in the weight's name ("weight" unless given).
    Tensor: <prefix><tensor> [size].  The sum of squares and the residual sum are 32-bit."""

    graph_safe = True

    def tensor_specs(self):
        return [TensorSpec(self.prefix + self.spec.get("tensor", "weight"), (self.spec["size"],),
                           init="one_plus_normal", wide=True)]

    def load(self, tensors, rt):
        super().load(tensors, rt)
        self.weight = tensors[self.prefix + self.spec.get("tensor", "weight")]
        self.eps = float(self.spec["eps"])
        self.weight_f32()

    prenorm = True      # x * scale(row) * w: forward_prenormed writes bfloat16(x * w) and leaves the scale to the consumer

    def weight_f32(self) -> torch.Tensor:
        """The weight in float32 (made once), for the kernels that take it so."""
        src = self.weight
        if getattr(self, "_weight_f32_of", None) is not src:
            self._weight_f32 = src if src.dtype == torch.float32 else src.to(torch.float32)
            self._weight_f32_of = src
        return self._weight_f32

    @staticmethod
    def _as_terms(delta):
        """A sum of two branches without a gate is a sum of two terms without scales (float32 each)."""
        if isinstance(delta, GatedSum) and delta.gate is None and \
                all(t is None or t.dtype == torch.float32 for t in (delta.a, delta.b)):
            return ScaledSum([(t, None) for t in (delta.a, delta.b) if t is not None])
        return delta

    def forward(self, h, delta, rows=None):
        n = h.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, h.shape[1]), dtype=self.rt.dtype, device=h.device)
        delta = self._as_terms(delta)
        if isinstance(delta, GatedSum):
            if rows is not None:
                raise ops.KernelError("rms: a sum with a gate per row for chosen rows is not offered")
            self.add_delta(h, delta)
            delta = None
        if isinstance(delta, NormedSum):
            # a sub-layer's output with a norm of its own behind it: one kernel takes that norm, completes the stream
            # and normalises it
            return ops.normed_add_norm(h, delta.term, delta.weight, delta.eps, self.weight_f32(), self.eps, out,
                                       rows=rows)
        if isinstance(delta, ScaledSum):
            # the outputs of sub-layers that stand side by side, each with its scale per column: one kernel
            # completes the stream with them and normalises
            return ops.scaled_norm(h, delta.terms, self.weight, self.eps, out, rows=rows)
        return ops.add_rmsnorm(h, delta, self.weight, self.eps, out, rows=rows)

    def forward_prenormed(self, h, delta) -> PreNormed:
        """As forward() without rows, for a part that takes its input as PreNormed: the stream is completed and
        the rows are written short of their scale, by many small blocks that do not wait for one another."""
        T, E = h.shape
        if isinstance(delta, (ScaledSum, GatedSum, NormedSum)):
            self.add_delta(h, delta)
            delta = None
        xg = torch.empty((T, E), dtype=torch.bfloat16, device=h.device)
        ss = torch.empty((-(-E // ops.PRENORM_CHUNK), T), dtype=torch.float32, device=h.device)
        ops.add_prenorm(h, delta, self.weight, xg, ss)
        return PreNormed(xg, ss, self.eps)


@register_norm("rms_scalar")
class ScalarRMSNorm(RMSNorm):
    """x * rsqrt(mean(x^2) + eps) * g with ONE learned number g for all columns.  params: size, eps; tensor as for
    "rms".  Tensor: <prefix><tensor> [] (a scalar).  The kernels are RMSNorm's: g is spread over a vector at load."""

    def tensor_specs(self):
        return [TensorSpec(self.prefix + self.spec.get("tensor", "weight"), (), init="one_plus_normal", wide=True)]

    def load(self, tensors, rt):
        Norm.load(self, tensors, rt)
        g = tensors[self.prefix + self.spec.get("tensor", "weight")]
        self.weight = g.reshape(1).expand(self.spec["size"]).contiguous()
        self.eps = float(self.spec["eps"])


@register_norm("rms_after")
class PostRMSNorm(Norm):
    """The norm of a layer that normalises after the sum: the stream itself becomes rms(alpha * h + delta) * w, with
    rms(x) = x / sqrt(mean(x^2) + eps).  params: size, eps, alpha; tensor: what follows the prefix in the weight's name.
    forward() replaces h in place (float32) and returns the same rows in the compute dtype (h itself in a float32
    engine).  delta: None, a tensor, partial sums, or a GatedSum; everything is summed in 32-bit."""

    graph_safe = True

    def tensor_specs(self):
        return [TensorSpec(self.prefix + self.spec.get("tensor", "weight"), (self.spec["size"],),
                           init="one_plus_normal", wide=True)]

    def load(self, tensors, rt):
        super().load(tensors, rt)
        self.weight = tensors[self.prefix + self.spec.get("tensor", "weight")]
        self.eps, self.alpha = float(self.spec["eps"]), float(self.spec["alpha"])

    def forward(self, h, delta, rows=None):
        if rows is not None:
            raise ops.KernelError("rms_after replaces the whole stream: it takes no rows")
        if isinstance(delta, ScaledSum):
            raise ops.KernelError("rms_after: sums with a scale per column are not offered")
        a, b, gate = (delta.a, delta.b, delta.gate) if isinstance(delta, GatedSum) else (delta, None, None)
        if a is not None and a.dtype != torch.float32:
            a = ops.convert(a, torch.empty(a.shape, dtype=torch.float32, device=a.device))
        out = None if self.rt.is_fp32 else torch.empty(h.shape, dtype=self.rt.dtype, device=h.device)
        ops.post_norm(h, self.alpha, a, b, gate, self.weight, self.eps, out)
        return h if out is None else out
