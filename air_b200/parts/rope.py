"""Rotary position encoding as a table of cos and sin per position."""
from __future__ import annotations

import torch

from .base import PositionEncoding
from .registry import register_position_encoding


@register_position_encoding("rope_half")
class RopeHalf(PositionEncoding):
    """Half-split rotation: pairs (i, i + rot/2), angle p * theta^(-2i/rot)
    (AIR: src/reference/reference_executor.cpp:37-72; src/cuda/cuda_backend.cu:862-906).
    params: rotary_dim, theta, max_positions.  No tensors.

    The angles are evaluated once, in 64-bit like AIR's CPU executor, and kept as float32
    cos|sin [max_positions, rotary_dim]; the mixer's kernel reads a token's row by its
    position.  Another frequency rule (scaled, interpolated) is another table of the same
    shape.  Layers whose encodings have equal parameters share one table (Runtime.shared), so a
    step reads one row per token whatever the number of layers."""

    def load(self, tensors, rt):
        super().load(tensors, rt)
        rot, theta, n = int(self.spec["rotary_dim"]), float(self.spec["theta"]), int(self.spec["max_positions"])
        if rot % 2:
            raise ValueError("rope_half needs an even rotary width")
        self.rotary_dim = rot
        key = ("rope_half", rot, theta, n)
        table = rt.shared.get(key)
        if table is None:
            i = torch.arange(rot // 2, dtype=torch.float64)
            inv_freq = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), (2.0 * i) / rot)
            angle = torch.arange(n, dtype=torch.float64)[:, None] * inv_freq[None, :]
            table = rt.shared[key] = torch.cat([torch.cos(angle), torch.sin(angle)], dim=1).to(torch.float32).to(rt.device)
        self._table = table

    def table(self):
        return self._table


@register_position_encoding("rope_half_live")
class RopeHalfLive(PositionEncoding):
    """The same rotation (pairs (i, i + rot/2), angle p * theta^(-2i/rot)) without a table and so without a
    longest position: the mixer's kernel multiplies the position by the pair's frequency and takes cos and sin
    itself, in 32-bit.  params: rotary_dim (may be smaller than the head: the rest passes unchanged), theta.
    The frequencies are evaluated in 64-bit once and kept as float32 [rotary_dim / 2]."""

    def load(self, tensors, rt):
        super().load(tensors, rt)
        rot, theta = int(self.spec["rotary_dim"]), float(self.spec["theta"])
        if rot % 2 or rot < 0:
            raise ValueError("rope_half_live needs an even rotary width")
        self.rotary_dim = rot
        key = ("rope_half_live", rot, theta)
        f = rt.shared.get(key)
        if f is None:
            i = torch.arange(rot // 2, dtype=torch.float64)
            f = rt.shared[key] = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * i / max(rot, 1)) \
                .to(torch.float32).to(rt.device)
        self._frequencies = f

    def frequencies(self):
        return self._frequencies if self.rotary_dim else None


@register_position_encoding("none")
class NoPosition(PositionEncoding):
    """No position encoding: the mixer's kernel rotates nothing."""


def bent_frequencies(rot: int, theta: float, scaling=None):
    """(float64 frequencies [rot / 2], what cos and sin are multiplied by) of a rotation whose slow pairs are
    stretched for contexts longer than the model was trained on (the YaRN rule).  scaling: None, or a mapping with
    factor, original (the trained length), fast and slow (turns over the trained length above which a pair is left
    alone, and below which it is divided by factor).  With pair(t) = rot ln(original / (2 pi t)) / (2 ln theta),
    lo = max(floor(pair(fast)), 0), hi = min(ceil(pair(slow)), rot - 1), r_i = clamp((i - lo) / max(hi - lo, 0.001),
    0, 1): frequency i = f_i / factor * r_i + f_i (1 - r_i); the magnitude is 0.1 ln(factor) + 1."""
    import math
    i = torch.arange(rot // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / max(rot, 1))
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair(turns):
        return rot * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(theta)))

    lo = max(math.floor(pair(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair(float(scaling["slow"]))), rot - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def banded_frequencies(rot: int, theta: float, scaling=None):
    """float64 frequencies [rot / 2] of a rotation whose slow pairs are slowed down by a constant factor, the fast ones
    left alone and the band between them blended (the rule of Llama 3.1).  scaling: None, or a mapping with factor,
    original (the trained length), low and high.  With the wavelength l_i = 2 pi / f_i: f_i stays where l_i <
    original / high; becomes f_i / factor where l_i > original / low; and between the two, with s = (original / l_i -
    low) / (high - low), (1 - s) f_i / factor + s f_i.  cos and sin keep their magnitude."""
    import math
    i = torch.arange(rot // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / max(rot, 1))
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    low, high = float(scaling["low"]), float(scaling["high"])
    wave = 2.0 * math.pi / f
    s = (original / wave - low) / (high - low) if high != low else torch.ones_like(f)
    blended = (1.0 - s) * f / factor + s * f
    out = torch.where(wave < original / high, f, torch.where(wave > original / low, f / factor, blended))
    return out, 1.0


@register_position_encoding("rope_live")
class RopeLive(PositionEncoding):
    """A rotation of the first rotary_dim elements of a head without a table: the mixer's kernel takes the angle
    position * frequency in 64-bit and its cos and sin once per token.  params: rotary_dim, theta, pairing ("half":
    element i with i + rotary_dim / 2; "neighbours": element 2i with 2i + 1), scaling (None or the mapping that
    bent_frequencies describes; with rule "banded" the mapping that banded_frequencies describes).  frequencies64(): float64 [rotary_dim / 2] on the device; magnitude: what cos and sin
    are multiplied by."""

    def load(self, tensors, rt):
        super().load(tensors, rt)
        rot, theta = int(self.spec["rotary_dim"]), float(self.spec["theta"])
        self.pairing = self.spec.get("pairing", "half")
        scaling = self.spec.get("scaling")
        if rot % 2 or rot < 0:
            raise ValueError("rope_live needs an even rotary width")
        if self.pairing not in ("half", "neighbours"):
            raise ValueError(f"rope_live: pairing {self.pairing!r}")
        self.rotary_dim = rot
        rule = self.spec.get("rule", "bent")
        if rule not in ("bent", "banded"):
            raise ValueError(f"rope_live: rule {rule!r}")
        key = ("rope_live", rot, theta, rule, tuple(sorted(scaling.items())) if scaling else None)
        made = rt.shared.get(key)
        if made is None:
            f, magnitude = (banded_frequencies if rule == "banded" else bent_frequencies)(rot, theta, scaling)
            made = rt.shared[key] = (f.to(rt.device), float(magnitude))
        self._frequencies64, self.magnitude = made

    def frequencies64(self):
        return self._frequencies64 if self.rotary_dim else None

    def frequencies(self):
        return self._frequencies64.to(torch.float32) if self.rotary_dim else None
