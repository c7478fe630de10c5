"""Typed configuration of the Tabopel decoder, read from config.json's own keys.

config.json names the design under "architecture" and gives "vocab", "width", "norm" {"eps"}, "embedding" {"scale"}
(what a token's row is multiplied by), "loop" {"start", "stop", "times"} (the layers start .. stop - 1 run `times`
times over) and "layers": every entry has a "type" ("attention", "attention_2" or "retention"), the mixer's sizes and
constants under "mixer" and its feed-forward under "mlp" (null: none; kind "dense" or "moe").  A mixer gives "heads",
"dim", "vdim" and "rot" {"base", "dims", "scaling" {"factor", "low", "high", "original"}}; the attentions also
"kv_heads" and "scale", "attention" its "conv" (taps), "attention_2" its "softcap", "retention" its "decay" (a number per
head).  Every size and constant that may differ between two models of the design is read from there; nothing has a
default in code except keys that a model may leave out (the loop, a rotation's scaling, the taps, the soft cap,
identity experts).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .bivizen_config import _get
from .model_config import ConfigError

MIXER_TYPES = ("attention", "attention_2", "retention")
# No key of config.json bounds a request's length; the block tables need a width, and this is it.
POSITIONS = 1 << 20


@dataclass(frozen=True)
class TabopelRotation:
    """The first `dims` numbers of a head are rotated, element i with i + dims / 2, by position * base^(-2i/dims);
    with a scaling, slow pairs are slowed down by `factor`, fast ones kept, the band between blended."""
    dims: int
    base: float
    factor: float = 0.0          # 0: no scaling
    low: float = 0.0
    high: float = 0.0
    original: float = 0.0

    def scaling(self) -> Optional[dict]:
        if not self.factor:
            return None
        return {"factor": self.factor, "low": self.low, "high": self.high, "original": self.original}


@dataclass(frozen=True)
class TabopelFeedForward:
    """kind "dense": one hidden layer of width ff, the squared rectifier between the two matrices.  kind "moe":
    `experts` such layers of width ff and `identity` experts that return their input; a token takes the `top` of
    them whose softmax score plus a learned correction is largest, weighted by the scores themselves."""
    kind: str
    ff: int
    experts: int = 0
    top: int = 0
    identity: int = 0


@dataclass(frozen=True)
class TabopelLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    rot: Optional[TabopelRotation] = None
    kv_heads: int = 0            # the attentions
    scale: float = 0.0           # the attentions
    conv: int = 0                # attention: taps of the convolution behind the projections (0: none)
    softcap: float = 0.0         # attention_2
    decay: Tuple[float, ...] = ()    # retention
    mlp: Optional[TabopelFeedForward] = None
    idle: Tuple[str, ...] = ()   # a layer without feed-forward: the norms of one that the model file still has


@dataclass(frozen=True)
class TabopelConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    loop_start: int
    loop_stop: int
    loop_times: int
    has_loop: bool               # config.json has "loop" (and the model file its table), even if the stretch is empty
    layers: Tuple[TabopelLayer, ...]
    max_positions: int = POSITIONS
    eos_token_id: Optional[int] = None
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False)

    reads_shapes = True      # whether a layer without feed-forward has the norms of one shows in the model file only

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], shapes=None) -> "TabopelConfig":
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
            r = m.get("rot")
            if r is not None:
                wr = wm + ".rot"
                s = r.get("scaling") if isinstance(r, Mapping) else None
                ws = wr + ".scaling"
                kw["rot"] = TabopelRotation(
                    dims=_get(r, "dims", int, wr), base=_get(r, "base", float, wr),
                    **({} if s is None else dict(factor=_get(s, "factor", float, ws), low=_get(s, "low", float, ws),
                                                 high=_get(s, "high", float, ws),
                                                 original=_get(s, "original", float, ws))))
            if kind in ("attention", "attention_2"):
                kw.update(kv_heads=_get(m, "kv_heads", int, wm), scale=_get(m, "scale", float, wm))
            if kind == "attention":
                kw["conv"] = _get(m, "conv", int, wm, 0, required=False)
            elif kind == "attention_2":
                kw["softcap"] = _get(m, "softcap", float, wm, 0.0, required=False)
            else:
                decay = m.get("decay")
                if not isinstance(decay, list) or not all(isinstance(g, (int, float)) and not isinstance(g, bool)
                                                          for g in decay):
                    raise ConfigError("data_error", f"config.json lacks 'decay' (a list of numbers) in {wm}")
                kw["decay"] = tuple(float(g) for g in decay)
            f = entry.get("mlp")
            if f is not None:
                wf = where + ".mlp"
                fkind = _get(f, "kind", str, wf)
                if fkind == "dense":
                    kw["mlp"] = TabopelFeedForward(kind="dense", ff=_get(f, "ff", int, wf))
                elif fkind == "moe":
                    ro = f.get("router")
                    wr = wf + ".router"
                    kw["mlp"] = TabopelFeedForward(
                        kind="moe", ff=_get(f.get("expert"), "ff", int, wf + ".expert"),
                        experts=_get(ro, "experts", int, wr), top=_get(ro, "top", int, wr),
                        identity=_get(ro, "identity", int, wr, 0, required=False))
                else:
                    raise ConfigError("unsupported", f"{wf}: feed-forward kind {fkind!r} (known: dense, moe)")
            elif shapes is not None:
                kw["idle"] = tuple(n for n in ("norm2", "norm2b") if f"l{i}.{n}" in shapes)
            else:
                kw["idle"] = tuple(entry.get("idle", ()))
            layers.append(TabopelLayer(**kw))
        where = "config.json"
        loop = d.get("loop")
        eos = d.get("eos_token_id")
        cfg = cls(architecture=arch, vocab=_get(d, "vocab", int, where), width=_get(d, "width", int, where),
                  eps=_get(d.get("norm"), "eps", float, "norm"),
                  embedding_scale=_get(d.get("embedding"), "scale", float, "embedding", 1.0, required=False),
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
            if l.rot is not None:
                m["rot"] = {"base": l.rot.base, "dims": l.rot.dims}
                if l.rot.scaling():
                    m["rot"]["scaling"] = l.rot.scaling()
            if l.type in ("attention", "attention_2"):
                m.update(kv_heads=l.kv_heads, scale=l.scale)
            if l.type == "attention" and l.conv:
                m["conv"] = l.conv
            if l.type == "attention_2" and l.softcap:
                m["softcap"] = l.softcap
            if l.type == "retention":
                m["decay"] = list(l.decay)
            f = None
            if l.mlp is not None and l.mlp.kind == "dense":
                f = {"kind": "dense", "ff": l.mlp.ff}
            elif l.mlp is not None:
                f = {"kind": "moe", "expert": {"ff": l.mlp.ff},
                     "router": {"experts": l.mlp.experts, "top": l.mlp.top, "identity": l.mlp.identity}}
            entry = {"type": l.type, "mixer": m, "mlp": f}
            if l.mlp is None and l.idle:
                entry["idle"] = list(l.idle)
            layers.append(entry)
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "embedding": {"scale": self.embedding_scale}, "layers": layers}
        if self.has_loop:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.max_positions != POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("data_error", "Tabopel geometry is incomplete: vocab and width must be positive")
        if not (self.eps > 0.0):
            raise ConfigError("data_error", "Tabopel norm eps is missing or invalid")
        n = len(self.layers)
        if not (0 <= self.loop_start <= self.loop_stop <= n) or self.loop_times < 1:
            raise ConfigError("data_error", f"loop: 0 <= start <= stop <= {n} layers and times >= 1")
        for i, l in enumerate(self.layers):
            if min(l.heads, l.dim, l.vdim) <= 0:
                raise ConfigError("data_error", f"layers[{i}]: heads, dim and vdim must be positive")
            if l.rot is not None and (l.rot.dims < 0 or l.rot.dims % 2 or l.rot.dims > l.dim or not (l.rot.base > 0.0)):
                raise ConfigError("data_error", f"layers[{i}].mixer.rot: dims must be even and at most dim, base positive")
            if l.rot is not None and l.rot.factor and (l.rot.factor <= 0.0 or l.rot.original <= 0.0
                                                       or min(l.rot.low, l.rot.high) <= 0.0):
                raise ConfigError("data_error", f"layers[{i}].mixer.rot.scaling: factor, low, high and original must be "
                                                "positive")
            if l.type != "retention":
                if l.kv_heads <= 0 or l.heads % l.kv_heads:
                    raise ConfigError("data_error", f"layers[{i}]: heads must be a multiple of kv_heads")
                if l.conv < 0 or l.softcap < 0.0:
                    raise ConfigError("data_error", f"layers[{i}]: conv and softcap must not be negative")
            elif len(l.decay) != l.heads:
                raise ConfigError("data_error", f"layers[{i}]: retention needs one decay per head")
            f = l.mlp
            if f is None:
                continue
            if f.ff <= 0:
                raise ConfigError("data_error", f"layers[{i}].mlp: ff must be positive")
            if f.kind == "moe" and (f.experts <= 0 or f.identity < 0 or not (0 < f.top <= f.experts + f.identity)):
                raise ConfigError("data_error", f"layers[{i}].mlp: experts and top (at most experts + identity) must be positive")
