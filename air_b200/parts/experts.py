"""A mixture of gated experts with a router on the device, beside an optional shared expert."""
from __future__ import annotations

import torch

from ..config.model_config import ConfigError
from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, GatedSum
from .linear import Linear
from .mlp import SwiGLU
from .registry import register_feed_forward
from .spec import PartSpec


@register_feed_forward("swiglu_plain_names")
class PlainNamesSwiGLU(SwiGLU):
    """SwiGLU whose three matrices are called <prefix>gate, up and down."""
    NAMES = {"gate": "gate", "up": "up", "down": "down"}


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """y = sum over the token's `top` experts e of expert_e(s_e x)  +  g shared(x).

    Router: z = Wr x in 32-bit; scores s = sigmoid(z) (score "sigmoid") or softmax(z); the `top` largest are chosen
    (of equal scores the lower index); the weights are the chosen scores, divided by their sum (+ norm_eps) where
    renormalize, times route_scale.  With groups = (count, keep) experts g * (experts / count) .. (g + 1) * (experts /
    count) - 1 make group g, a group's mark is its best score plus its second best, and only experts of the `keep`
    groups with the highest marks can be chosen.  With weight_on "input" (the default) the weight multiplies the expert's INPUT (the
    scaled row is rounded to the compute dtype like any input of a product), which is not the same as weighting its
    output, since an expert is not linear; with "output" it multiplies the expert's output, in 32-bit.  expert(u) = Wdown (silu(Wgate u) *
    (Wup u)).  The shared expert (shared_intermediate > 0) has the same form and runs for every token; with shared_gate
    its output is multiplied by g = sigmoid(w_sg . x), one number per token, else g = 1.

    With gated False an expert has no gate: expert(u) = Wdown act(Wup u) with act the square of the rectifier
    (activation "relu2").  With choice_bias the experts are chosen by score + bias (a learned number per expert, the
    tensor `correction`) while the weights stay the scores.  With identity = n the router has n more outputs behind the
    experts' own; they stand for experts without matrices whose output is their input (times the weight), and they
    take part in the softmax and in the choice like the others.

    params: hidden, experts, top, intermediate, shared_intermediate, shared_gate, score, renormalize, norm_eps,
    route_scale, groups, weight_on, gated, activation, choice_bias, identity.
    Tensors: <prefix>router [experts + identity, hidden], e<i>.gate, e<i>.up [intermediate, hidden], e<i>.down [hidden,
    intermediate], shared.gate, shared.up, shared.down, shared.sg [1, hidden], correction [experts + identity].

    Everything happens on the device: a kernel picks the experts, one orders the (token, choice) pairs by expert, and
    two grouped products (gate and up with the activation; down) walk the experts' rows.  The outputs of a token's
    choices land in `top` planes that the norm behind the layer adds in order, so the sum does not depend on the
    batch.  From LIBRARY_ROWS rows per expert (in the mean) on, a bfloat16 step hands the two products to the library's
    grouped product (which also takes the experts' bounds from the device): there the experts' outputs are rounded to
    bfloat16 before they are added up in 32-bit."""

    LIBRARY_ROWS = 32

    graph_safe = True

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.experts, self.top = p["hidden"], p["experts"], p["top"]
        self.inter, self.shared_inter = p["intermediate"], int(p.get("shared_intermediate") or 0)
        self.shared_gate = bool(p.get("shared_gate", False)) and self.shared_inter > 0
        self.score, self.renormalize = p.get("score", "sigmoid"), bool(p.get("renormalize", False))
        self.norm_eps, self.route_scale = float(p.get("norm_eps", 0.0)), float(p.get("route_scale", 1.0))
        self.groups, self.keep = tuple(p["groups"]) if p.get("groups") else (0, 0)
        self.weight_on = p.get("weight_on", "input")
        if self.weight_on not in ("input", "output"):
            raise ConfigError("data_error", f"routed experts: weight_on {self.weight_on!r} (input or output)")
        if self.groups > 1 and (self.experts % self.groups or not (0 < self.keep <= self.groups)
                                or self.top > self.keep * (self.experts // self.groups)):
            raise ConfigError("data_error", "routed experts: the groups must be equal, keep between 1 and their number, "
                                            "and the kept groups must hold at least `top` experts")
        self.gated, self.activation = bool(p.get("gated", True)), p.get("activation", "silu")
        self.choice_bias, self.identity = bool(p.get("choice_bias", False)), int(p.get("identity") or 0)
        self.outputs = self.experts + self.identity          # what the router chooses among
        if (self.gated, self.activation) not in ((True, "silu"), (False, "relu2")):
            raise ConfigError("unsupported", "routed experts: gated experts with SiLU, or plain ones with the squared "
                                             "rectifier")
        if self.identity < 0 or (self.identity and (self.weight_on != "output" or self.groups > 1)):
            raise ConfigError("unsupported", "routed experts: identity experts take their weight on the output, and "
                                             "no groups")
        if self.top > self.outputs:
            raise ConfigError("data_error", "routed experts: more choices than experts")
        if self.outputs > 512 or self.top > 32:
            raise ConfigError("unsupported", "routed experts: up to 512 experts and 32 choices per token")
        self.shared = None
        if self.shared_inter:
            self.shared = PlainNamesSwiGLU(PartSpec("swiglu_plain_names", {"hidden": self.hidden,
                                                                           "intermediate": self.shared_inter}),
                                           prefix + "shared.")

    def tensor_specs(self):
        p, e, f = self.prefix, self.hidden, self.inter
        specs = [TensorSpec(p + "router", (self.outputs, e), wide=True)]
        if self.choice_bias:
            specs.append(TensorSpec(p + "correction", (self.outputs,), wide=True, std=0.01))
        for i in range(self.experts):
            specs += ([TensorSpec(f"{p}e{i}.gate", (f, e))] if self.gated else []) + \
                [TensorSpec(f"{p}e{i}.up", (f, e)), TensorSpec(f"{p}e{i}.down", (e, f))]
        if self.shared is not None:
            specs += self.shared.tensor_specs()
        if self.shared_gate:
            specs.append(TensorSpec(p + "shared.sg", (1, e), wide=True))
        return specs

    def load(self, tensors, rt):
        super().load(tensors, rt)
        p, n = self.prefix, self.experts
        rows = [tensors[p + "router"]] + ([tensors[p + "shared.sg"]] if self.shared_gate else [])
        # The router and the shared expert's gate are one product with 32-bit sums.  In a bfloat16 engine its operands
        # are the stored 16-bit weights and the stream's rows as the other products read them: their products are
        # exact in 32 bits, so the tensor cores' 32-bit accumulation is the 32-bit router (rows of zeros fill the matrix
        # up to a multiple of 8, which those kernels want).  A float32 engine runs the CUDA-core product.
        w = torch.cat([r.to(rt.dtype) for r in rows], dim=0)
        if not rt.is_fp32 and w.shape[0] % 8:
            w = torch.cat([w, torch.zeros((8 - w.shape[0] % 8, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0)
        self.router = Linear(w.contiguous(), rt.status)
        # gate and up of an expert are one matrix, in the dense feed-forward's arrangement (blocks of gate rows and of up
        # rows in turn), so that the same memory serves the grouped product and the dense products per expert
        F = self.inter
        block = next((b for b in (128, 64, 32) if F % b == 0), F) if rt.dtype == torch.bfloat16 else F
        self.block = block

        def arranged(g, u):
            if block == F:
                return torch.cat([g, u], dim=0)
            return torch.stack([g.view(F // block, block, -1), u.view(F // block, block, -1)], dim=1).reshape(2 * F, -1)

        if self.gated:
            self.gate_up = torch.stack([arranged(tensors[f"{p}e{i}.gate"], tensors[f"{p}e{i}.up"])
                                        for i in range(n)]).contiguous()             # [n, 2F, E]
        else:
            self.gate_up = torch.stack([tensors[f"{p}e{i}.up"] for i in range(n)]).contiguous()      # [n, F, E]
        self.correction = tensors[p + "correction"].to(torch.float32).contiguous() if self.choice_bias else None
        self.down = torch.stack([tensors[f"{p}e{i}.down"] for i in range(n)]).contiguous()      # [n, E, F]
        if self.gate_up.dtype != rt.dtype:
            raise ValueError(f"{p}: the experts are stored as {self.gate_up.dtype}, the engine computes in {rt.dtype}")
        if self.shared is not None:
            self.shared.load(tensors, rt)

    def forward(self, x, ctx):
        T, E, F, n, top = x.shape[0], self.hidden, self.inter, self.experts, self.top
        dev = x.device
        z = self.router.f32(x)
        expert = torch.empty((T, top), dtype=torch.int32, device=dev)
        weight = torch.empty((T, top), dtype=torch.float32, device=dev)
        gate = torch.empty((T,), dtype=torch.float32, device=dev) if self.shared_gate else None
        ops.moe_route(z, self.outputs, top, expert, weight, gate, has_gate=self.shared_gate, score=self.score,
                      renormalize=self.renormalize, groups=self.groups, keep=self.keep, route_scale=self.route_scale,
                      norm_eps=self.norm_eps, choice_bias=self.correction)
        on_input = self.weight_on == "input"
        pairs = T * top
        ints = torch.empty(n + 1 + pairs + 2 * (pairs // ops.GROUP_TILE + n) + 1, dtype=torch.int32, device=dev)
        start, pair_of_slot = ints[:n + 1], ints[n + 1:n + 1 + pairs]
        tiles, num_tiles = ints[n + 1 + pairs:-1].view(-1, 2), ints[-1:]
        ops.moe_sort(expert, n, start, pair_of_slot, tiles, num_tiles)
        y = torch.empty((top, T, E), dtype=torch.float32, device=dev)
        if self.identity:
            # (pairs of an expert without matrices get no slot in the order by expert: their planes are written here)
            ops.moe_identity(x, expert, weight, n, y)
        if x.dtype == torch.bfloat16 and pairs >= self.LIBRARY_ROWS * n and E % 16 == 0 and F % 16 == 0:
            self._experts_by_the_library(x, start, pair_of_slot, weight, y)
        else:
            act = torch.empty((pairs, F), dtype=x.dtype, device=dev)
            ops.grouped_gemm(x, self.gate_up, act, F, E, lda=E, ldo=F, groups=n, a_index=pair_of_slot, a_div=top,
                             a_scale=weight.view(-1) if on_input else None, start=start, tiles=tiles,
                             num_tiles=num_tiles, silu_mul=self.gated, gate_block=self.block if self.gated else 0,
                             relu2=not self.gated)
            ops.grouped_gemm(act, self.down, y, E, F, lda=F, ldo=E, groups=n, o_index=pair_of_slot, o_div=top,
                             o_part_stride=T * E, start=start, tiles=tiles, num_tiles=num_tiles,
                             o_scale=None if on_input else weight.view(-1))
        if self.shared is None:
            return y
        return GatedSum(y, self.shared.forward(x, ctx), gate)

    def _experts_by_the_library(self, x, start, pair_of_slot, weight, y):
        """The road of steps with many rows per expert: the rows in the experts' order with their weights on them, the
        library's grouped product (it takes the experts' bounds from the device) for gate and up, the package's
        activation kernel, the grouped product for down, the results back to the planes."""
        top, (T, E) = self.top, x.shape
        pairs = T * top
        on_input = self.weight_on == "input"
        rows = ops.rows_by_index(x, pair_of_slot, top, weight.view(-1) if on_input else None,
                                 torch.empty((pairs, E), dtype=x.dtype, device=x.device))
        ends = start[1:].clone()
        act = torch.empty((pairs, self.inter), dtype=x.dtype, device=x.device)
        hidden = torch._grouped_mm(rows, self.gate_up.transpose(1, 2), offs=ends)
        if self.gated:
            ops.silu_mul(hidden, act, block=self.block)
        else:
            ops.relu2(hidden, act)
        ops.planes_by_index(torch._grouped_mm(act, self.down.transpose(1, 2), offs=ends), pair_of_slot, top, y,
                            scale=None if on_input else weight.view(-1))
