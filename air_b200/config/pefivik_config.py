"""Typed configuration of the Pefivik decoder, read from config.json's own keys.

config.json names the design under "architecture" and gives "vocab", "width", "norm" {"eps"}, "residual_mult" (what a
sub-layer's output is multiplied by before it joins the stream), "logit_softcap", "embedding" {"bigram": {"buckets",
"mul_prev", "mul_cur"}} (the second embedding table, indexed by a hash of a token and the one before it), "loop"
{"start", "stop", "times"} (the layers start .. stop - 1 run `times` times over) and "layers": every entry has a "type"
("latent_attention" or "hgrn2"), the mixer's sizes and constants under "mixer" and its feed-forward under "mlp" (null:
none; kind "dense" or "moe").  Every size and constant that may differ between two models of the design is read from
there; nothing has a default in code except keys that a model may leave out (the loop, the soft cap, a shared expert,
groups of experts).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .bivizen_config import _get
from .model_config import ConfigError

MIXER_TYPES = ("latent_attention", "hgrn2")
# No key of config.json bounds a request's length; the block tables need a width, and this is it.
POSITIONS = 1 << 20


@dataclass(frozen=True)
class PefivikFeedForward:
    """kind "dense": one hidden layer of width ff with biases and the PolyNorm activation.  kind "moe": `experts` gated
    experts of width ff, of which a token takes `top` out of the `keep` best of `groups` groups; the weights are the
    scores over their sum, times `scale`; a shared expert of width shared_ff (0: none) beside them."""
    kind: str
    ff: int
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    scale: float = 1.0
    shared_ff: int = 0


@dataclass(frozen=True)
class PefivikLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    kv_rank: int = 0             # latent attention
    scale: float = 0.0           # latent attention
    mlp: Optional[PefivikFeedForward] = None
    second_norm: bool = False    # a layer without feed-forward: whether the model file still has its second norm


@dataclass(frozen=True)
class PefivikConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_softcap: float
    buckets: int
    mul_prev: int
    mul_cur: int
    loop_start: int
    loop_stop: int
    loop_times: int
    has_loop: bool               # config.json has "loop" (and the model file its table), even if the stretch is empty
    layers: Tuple[PefivikLayer, ...]
    max_positions: int = POSITIONS
    eos_token_id: Optional[int] = None
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False)

    reads_shapes = True      # whether a layer without feed-forward has a second norm shows in the model file only

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], shapes=None) -> "PefivikConfig":
        arch = d.get("architecture") or (d.get("architectures") or [None])[0]
        if arch is None:
            raise ConfigError("data_error", "config.json lacks 'architecture'")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("data_error", "config.json lacks 'layers'")
        layers = []
        for i, entry in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _get(entry, "type", str, where)
            if kind not in MIXER_TYPES:
                raise ConfigError("unsupported", f"{where}: mixer type {kind!r} (known: {', '.join(MIXER_TYPES)})")
            m = entry.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError("data_error", f"config.json lacks 'mixer' in {where}")
            wm = where + ".mixer"
            kw = dict(type=kind, heads=_get(m, "heads", int, wm), dim=_get(m, "dim", int, wm),
                      vdim=_get(m, "vdim", int, wm))
            if kind == "latent_attention":
                kw.update(kv_rank=_get(m, "kv_rank", int, wm), scale=_get(m, "scale", float, wm))
            f = entry.get("mlp")
            if f is not None:
                wf = where + ".mlp"
                fkind = _get(f, "kind", str, wf)
                if fkind == "dense":
                    kw["mlp"] = PefivikFeedForward(kind="dense", ff=_get(f, "ff", int, wf))
                elif fkind == "moe":
                    r, shared = f.get("router"), f.get("shared")
                    wr = wf + ".router"
                    g = r.get("groups") if isinstance(r, Mapping) else None
                    kw["mlp"] = PefivikFeedForward(
                        kind="moe", ff=_get(f.get("expert"), "ff", int, wf + ".expert"),
                        experts=_get(r, "experts", int, wr), top=_get(r, "top", int, wr),
                        groups=_get(g, "count", int, wr + ".groups") if g is not None else 1,
                        keep=_get(g, "keep", int, wr + ".groups") if g is not None else 1,
                        scale=_get(r, "scale", float, wr, 1.0, required=False),
                        shared_ff=_get(shared, "ff", int, wf + ".shared") if shared is not None else 0)
                else:
                    raise ConfigError("unsupported", f"{wf}: feed-forward kind {fkind!r} (known: dense, moe)")
            elif shapes is not None:
                kw["second_norm"] = f"l{i}.norm2" in shapes
            else:
                kw["second_norm"] = bool(entry.get("second_norm", False))
            layers.append(PefivikLayer(**kw))
        where = "config.json"
        bg = (d.get("embedding") or {}).get("bigram") if isinstance(d.get("embedding"), Mapping) else None
        if not isinstance(bg, Mapping):
            raise ConfigError("data_error", "config.json lacks 'embedding.bigram'")
        loop = d.get("loop")
        eos = d.get("eos_token_id")
        cfg = cls(architecture=arch, vocab=_get(d, "vocab", int, where), width=_get(d, "width", int, where),
                  eps=_get(d.get("norm"), "eps", float, "norm"),
                  residual_mult=_get(d, "residual_mult", float, where),
                  logit_softcap=_get(d, "logit_softcap", float, where, 0.0, required=False),
                  buckets=_get(bg, "buckets", int, "embedding.bigram"),
                  mul_prev=_get(bg, "mul_prev", int, "embedding.bigram"),
                  mul_cur=_get(bg, "mul_cur", int, "embedding.bigram"),
                  loop_start=_get(loop, "start", int, "loop") if loop is not None else 0,
                  loop_stop=_get(loop, "stop", int, "loop") if loop is not None else 0,
                  loop_times=_get(loop, "times", int, "loop") if loop is not None else 1,
                  has_loop=loop is not None,
                  layers=tuple(layers),
                  max_positions=_get(d, "max_positions", int, where, POSITIONS, required=False),
                  eos_token_id=eos if isinstance(eos, int) else None, raw=dict(d))
        cfg.validate()
        return cfg

    @property
    def loops(self) -> bool:
        return self.loop_stop > self.loop_start

    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            m = {"heads": l.heads, "dim": l.dim, "vdim": l.vdim}
            if l.type == "latent_attention":
                m.update(kv_rank=l.kv_rank, scale=l.scale)
            f = None
            if l.mlp is not None and l.mlp.kind == "dense":
                f = {"kind": "dense", "ff": l.mlp.ff}
            elif l.mlp is not None:
                f = {"kind": "moe", "expert": {"ff": l.mlp.ff},
                     "router": {"experts": l.mlp.experts, "top": l.mlp.top, "scale": l.mlp.scale,
                                "groups": {"count": l.mlp.groups, "keep": l.mlp.keep}}}
                if l.mlp.shared_ff:
                    f["shared"] = {"ff": l.mlp.shared_ff}
            entry = {"type": l.type, "mixer": m, "mlp": f}
            if l.mlp is None and l.second_norm:
                entry["second_norm"] = True
            layers.append(entry)
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "residual_mult": self.residual_mult, "logit_softcap": self.logit_softcap,
             "embedding": {"bigram": {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}},
             "layers": layers}
        if self.has_loop:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.max_positions != POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("data_error", "Pefivik geometry is incomplete: vocab and width must be positive")
        if not (self.eps > 0.0):
            raise ConfigError("data_error", "Pefivik norm eps is missing or invalid")
        if self.buckets <= 0 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ConfigError("data_error", "embedding.bigram: buckets must be positive, the multipliers not negative")
        if self.logit_softcap < 0.0:
            raise ConfigError("data_error", "logit_softcap must not be negative")
        n = len(self.layers)
        if not (0 <= self.loop_start <= self.loop_stop <= n) or self.loop_times < 1:
            raise ConfigError("data_error", f"loop: 0 <= start <= stop <= {n} layers and times >= 1")
        for i, l in enumerate(self.layers):
            if min(l.heads, l.dim, l.vdim) <= 0:
                raise ConfigError("data_error", f"layers[{i}]: heads, dim and vdim must be positive")
            if l.type == "latent_attention" and l.kv_rank <= 0:
                raise ConfigError("data_error", f"layers[{i}]: kv_rank must be positive")
            f = l.mlp
            if f is None:
                continue
            if f.ff <= 0:
                raise ConfigError("data_error", f"layers[{i}].mlp: ff must be positive")
            if f.kind == "moe":
                if f.experts <= 0 or not (0 < f.top <= f.experts) or f.shared_ff < 0:
                    raise ConfigError("data_error", f"layers[{i}].mlp: experts and top (at most experts) must be positive")
                if f.groups < 1 or f.experts % f.groups or not (1 <= f.keep <= f.groups) \
                        or f.top > f.keep * (f.experts // f.groups):
                    raise ConfigError("data_error", f"layers[{i}].mlp.router.groups: equal groups, 1 <= keep <= count, and "
                                                    "the kept groups must hold at least `top` experts")
