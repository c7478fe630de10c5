"""How the parts of one layer stand around the residual stream."""
from __future__ import annotations

from .registry import register_block, MIXERS, FEED_FORWARDS, NORMS
from .spec import BlockSpec


class Block:
    """What an arrangement offers to the model: its parts, their tensors, what the layer keeps per
    request, and forward(h, pending, ctx, cache, owns_cache) -> (h, pending).  A subclass builds its
    parts from `spec.part(role)` with the registry of the role's kind and `spec.name(role)` as the
    prefix of their tensors."""

    def __init__(self, spec: BlockSpec):
        self.spec = spec

    def parts(self):
        raise NotImplementedError

    def tensor_specs(self):
        return [s for part in self.parts() for s in part.tensor_specs()]

    def load(self, tensors, rt):
        for part in self.parts():
            part.load(tensors, rt)

    def cache_needs(self):
        """What the layer keeps per request (CacheNeed objects); forward() receives their views as `cache`,
        in the same order."""
        return ()

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False) for part in self.parts())

    def forward(self, h, pending, ctx, cache, owns_cache=True):
        raise NotImplementedError


@register_block("pre_norm")
class PreNormBlock(Block):
    """h = h + m mixer(norm1(h)); h = h + m feed_forward(norm2(h)), m = 1 unless the block's parameter
    residual_scale says otherwise (AIR: src/reference/reference_executor.cpp:343-413).
    Roles: mixer_norm, mixer, and feed_forward_norm with feed_forward (a layer may lack these two).

    The residual stream h is float32.  Each addition is fused into the norm that follows
    it: the block receives the previous block's output still pending, and hands its own
    feed-forward output on in the same way; the model's final norm adds the last one.  A part may
    instead add its output into the stream itself (StepContext.residual) and return None: with
    many rows the library's product does that addition in its epilogue, in 32-bit, and the norm
    that follows reads the stream alone.  With m != 1 the parts return their outputs and the block hands them on
    as a ScaledSum whose scale is m in every column, so the same kernel completes the stream and normalises.
    The parameter idle lists (what follows the prefix, shape) of tensors that a model file may hold for the layer
    although the layer does not use them (the second norm of a layer without feed-forward)."""

    def __init__(self, spec: BlockSpec):
        super().__init__(spec)
        self.mixer_norm = NORMS.get(spec.part("mixer_norm").kind)(spec.part("mixer_norm"), spec.name("mixer_norm"))
        self.mixer = MIXERS.get(spec.part("mixer").kind)(spec.part("mixer"), spec.name("mixer"))
        self.ff_norm = self.feed_forward = None
        if "feed_forward" in spec.parts:
            self.ff_norm = NORMS.get(spec.part("feed_forward_norm").kind)(spec.part("feed_forward_norm"),
                                                                          spec.name("feed_forward_norm"))
            self.feed_forward = FEED_FORWARDS.get(spec.part("feed_forward").kind)(spec.part("feed_forward"),
                                                                                  spec.name("feed_forward"))
        self.residual_scale = float(spec.params.get("residual_scale", 1.0))
        self.scale = None

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward) if p is not None)

    def tensor_specs(self):
        from ..weights.loader import TensorSpec
        return super().tensor_specs() + [TensorSpec(self.spec.prefix + name, tuple(shape), optional=True, wide=True)
                                         for name, shape in self.spec.params.get("idle", ())]

    def load(self, tensors, rt):
        super().load(tensors, rt)
        if self.residual_scale != 1.0:
            import torch
            self.scale = torch.full((self.spec.part("mixer_norm")["size"],), self.residual_scale, dtype=torch.float32,
                                    device=rt.device)

    def cache_needs(self):
        return self.mixer.cache_needs()

    @staticmethod
    def _norm(norm, h, delta, part, ctx, owns_cache=True):
        """The norm before `part`: where the part takes rows short of their scale in this step and the norm can
        write them so, the wide kernel whose blocks do not wait for one another."""
        if getattr(norm, "prenorm", False) and part.accepts_prenormed(ctx, owns_cache):
            return norm.forward_prenormed(h, delta)
        return norm.forward(h, delta)

    def _scaled(self, delta):
        """What a part returned, as the sum that the next norm adds: m times it."""
        if self.scale is None or delta is None:
            return delta
        import torch
        from ..csrc import ops
        from .base import GatedSum, ScaledSum

        def f32(t):
            return t if t.dtype == torch.float32 else ops.convert(t, torch.empty(t.shape, dtype=torch.float32,
                                                                                  device=t.device))
        if isinstance(delta, GatedSum):
            if delta.gate is not None:
                raise ops.KernelError("pre_norm with a residual scale: a gate per row is not offered")
            return ScaledSum([(f32(t), self.scale) for t in (delta.a, delta.b) if t is not None])
        if isinstance(delta, ScaledSum):
            raise ops.KernelError("pre_norm with a residual scale: the part's output is scaled already")
        return ScaledSum([(f32(delta), self.scale)])

    def forward(self, h, pending, ctx, cache, owns_cache=True):
        ctx.residual = h if self.scale is None else None     # scaled outputs are returned, not added by the parts
        x = self._norm(self.mixer_norm, h, pending, self.mixer, ctx, owns_cache)
        a = self._scaled(self.mixer.forward(x, ctx, cache, owns_cache))   # None: the mixer has added its output to h
        if self.feed_forward is None:
            return h, a
        x = self._norm(self.ff_norm, h, a, self.feed_forward, ctx)
        return h, self._scaled(self.feed_forward.forward(x, ctx))


@register_block("sandwich")
class SandwichBlock(Block):
    """h = h + norm_b(mixer(norm_a(h))); h = h + norm_d(feed_forward(norm_c(h))): a norm on each side of every
    sub-layer.  Roles: mixer_norm, mixer, mixer_out_norm, and feed_forward_norm, feed_forward, feed_forward_out_norm (a
    layer may lack the last three).  The norms in front are of a registered kind; the norms behind are weights [hidden]
    named by the roles mixer_out_norm and feed_forward_out_norm (x / sqrt(mean(x^2) + eps) * w with the eps of the parts
    of those roles).

    A sub-layer's output is handed on as a NormedSum, so that ONE kernel takes its norm, adds it to the float32 stream
    and takes the norm in front of the next sub-layer (of this block, of the next one, or the model's last one).  The
    parameter idle lists (what follows the prefix, shape) of tensors that a model file may hold for the layer although
    the layer does not use them."""

    def __init__(self, spec: BlockSpec):
        super().__init__(spec)
        self.mixer_norm = NORMS.get(spec.part("mixer_norm").kind)(spec.part("mixer_norm"), spec.name("mixer_norm"))
        self.mixer = MIXERS.get(spec.part("mixer").kind)(spec.part("mixer"), spec.name("mixer"))
        self.mixer_out = NORMS.get(spec.part("mixer_out_norm").kind)(spec.part("mixer_out_norm"),
                                                                     spec.name("mixer_out_norm"))
        self.ff_norm = self.feed_forward = self.ff_out = None
        if "feed_forward" in spec.parts:
            self.ff_norm = NORMS.get(spec.part("feed_forward_norm").kind)(spec.part("feed_forward_norm"),
                                                                          spec.name("feed_forward_norm"))
            self.feed_forward = FEED_FORWARDS.get(spec.part("feed_forward").kind)(spec.part("feed_forward"),
                                                                                  spec.name("feed_forward"))
            self.ff_out = NORMS.get(spec.part("feed_forward_out_norm").kind)(spec.part("feed_forward_out_norm"),
                                                                             spec.name("feed_forward_out_norm"))

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_out, self.ff_norm, self.feed_forward,
                                 self.ff_out) if p is not None)

    def tensor_specs(self):
        from ..weights.loader import TensorSpec
        return super().tensor_specs() + [TensorSpec(self.spec.prefix + name, tuple(shape), optional=True, wide=True)
                                         for name, shape in self.spec.params.get("idle", ())]

    def cache_needs(self):
        return self.mixer.cache_needs()

    @staticmethod
    def _behind(norm, delta):
        """What a sub-layer returned, as the sum that the next norm adds: its norm with the weight of `norm`."""
        import torch
        from ..csrc import ops
        from .base import GatedSum, NormedSum, ScaledSum
        if isinstance(delta, (GatedSum, ScaledSum, NormedSum)) or delta is None:
            raise ops.KernelError("sandwich: the sub-layer must return its output as a tensor or as partial sums")
        if delta.dtype != torch.float32:
            delta = ops.convert(delta, torch.empty(delta.shape, dtype=torch.float32, device=delta.device))
        return NormedSum(delta, norm.weight_f32(), norm.eps)

    def forward(self, h, pending, ctx, cache, owns_cache=True):
        ctx.residual = None          # a sub-layer's output is normalised before it is added: the parts return it
        x = self.mixer_norm.forward(h, pending)
        a = self._behind(self.mixer_out, self.mixer.forward(x, ctx, cache, owns_cache))
        if self.feed_forward is None:
            return h, a
        x = self.ff_norm.forward(h, a)
        return h, self._behind(self.ff_out, self.feed_forward.forward(x, ctx))


@register_block("parallel")
class ParallelBlock(Block):
    """x = norm(h); h = h + s_m * mixer(x) + s_f * feed_forward(x): one norm whose rows both sub-layers read, their
    outputs added to the stream together, each first multiplied by a learned scale per column (layer scale).
    Roles: norm, mixer, feed_forward (may be absent: a layer of a mixer only).  spec.names may also give
    "mixer_scale" and "feed_forward_scale", what follows the layer's prefix in the names of the two scale vectors
    [hidden]; a scale that is not named is 1.

    The block hands its two outputs on as a ScaledSum: the next block's norm (or the model's last one) completes the
    stream with them in 32-bit in the kernel that normalises."""

    def __init__(self, spec: BlockSpec):
        super().__init__(spec)
        self.norm = NORMS.get(spec.part("norm").kind)(spec.part("norm"), spec.name("norm"))
        self.mixer = MIXERS.get(spec.part("mixer").kind)(spec.part("mixer"), spec.name("mixer"))
        self.feed_forward = None
        if "feed_forward" in spec.parts:
            self.feed_forward = FEED_FORWARDS.get(spec.part("feed_forward").kind)(spec.part("feed_forward"),
                                                                                  spec.name("feed_forward"))
        self.scale_names = {role: spec.prefix + spec.names[role + "_scale"] for role in ("mixer", "feed_forward")
                            if role + "_scale" in spec.names and (role == "mixer" or self.feed_forward is not None)}
        # a scale that is named for a feed-forward that the layer does not have: taken if the file has it, not used
        self.idle_names = [spec.prefix + spec.names["feed_forward_scale"]] \
            if "feed_forward_scale" in spec.names and self.feed_forward is None else []
        self.scales = {}

    def parts(self):
        return tuple(p for p in (self.norm, self.mixer, self.feed_forward) if p is not None)

    def tensor_specs(self):
        from ..weights.loader import TensorSpec
        size = self.spec.part("norm")["size"]
        return super().tensor_specs() + [TensorSpec(name, (size,), init="one_plus_normal", wide=True)
                                         for name in self.scale_names.values()] + \
            [TensorSpec(name, (size,), init="one_plus_normal", wide=True, optional=True) for name in self.idle_names]

    def load(self, tensors, rt):
        super().load(tensors, rt)
        import torch
        self.scales = {role: tensors[name].to(torch.float32).contiguous() for role, name in self.scale_names.items()}

    def cache_needs(self):
        return self.mixer.cache_needs()

    def forward(self, h, pending, ctx, cache, owns_cache=True):
        from .base import ScaledSum
        ctx.residual = None          # the sub-layers' outputs are scaled before they are added: they return them
        x = self.norm.forward(h, pending)
        terms = [(self.mixer.forward(x, ctx, cache, owns_cache), self.scales.get("mixer"))]
        if self.feed_forward is not None:
            terms.append((self.feed_forward.forward(x, ctx), self.scales.get("feed_forward")))
        return h, ScaledSum(terms)


@register_block("post_norm")
class PostNormBlock(Block):
    """h = norm1(alpha h + mixer(h)); h = norm2(alpha h + feed_forward(h)): the norm stands behind the sum, so the
    stream itself is normalised and the sub-layers read it as it is.  Roles: mixer, mixer_norm, and optionally
    feed_forward and feed_forward_norm (a layer without feed-forward may still have the second norm); the norms are of
    a kind that replaces the stream (rms_after), and alpha is their parameter.

    The stream h is float32.  The rows that the matrix products read (the same numbers in the compute dtype) are written
    by the norm's kernel and handed from block to block in ctx.shared."""

    ROWS = "post_norm.rows"

    def __init__(self, spec: BlockSpec):
        super().__init__(spec)
        self.mixer = MIXERS.get(spec.part("mixer").kind)(spec.part("mixer"), spec.name("mixer"))
        self.mixer_norm = NORMS.get(spec.part("mixer_norm").kind)(spec.part("mixer_norm"), spec.name("mixer_norm"))
        self.feed_forward = self.ff_norm = None
        if "feed_forward" in spec.parts:
            self.feed_forward = FEED_FORWARDS.get(spec.part("feed_forward").kind)(spec.part("feed_forward"),
                                                                                  spec.name("feed_forward"))
        if "feed_forward_norm" in spec.parts:
            self.ff_norm = NORMS.get(spec.part("feed_forward_norm").kind)(spec.part("feed_forward_norm"),
                                                                          spec.name("feed_forward_norm"))
        if self.feed_forward is not None and self.ff_norm is None:
            raise ValueError(f"block 'post_norm' at '{spec.prefix}': a feed-forward needs the norm behind it")

    def parts(self):
        return tuple(p for p in (self.mixer, self.mixer_norm, self.feed_forward, self.ff_norm) if p is not None)

    def cache_needs(self):
        return self.mixer.cache_needs()

    def forward(self, h, pending, ctx, cache, owns_cache=True):
        import torch
        from ..csrc import ops
        from .base import Norm
        ctx.residual = None
        x = ctx.shared.pop(self.ROWS, None)
        if pending is not None:
            Norm.add_delta(h, pending)
            x = None
        if x is None:
            rt = self.mixer.rt
            x = h if rt.is_fp32 else ops.convert(h, torch.empty(h.shape, dtype=rt.dtype, device=h.device))
        x = self.mixer_norm.forward(h, self.mixer.forward(x, ctx, cache, owns_cache))
        if self.ff_norm is not None:
            x = self.ff_norm.forward(h, self.feed_forward.forward(x, ctx) if self.feed_forward is not None else None)
        ctx.shared[self.ROWS] = x
        return h, None
