"""Rotary position encoding: per-step cos/sin rows in float32."""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch

from .. import ops
from .base import PositionEncoding, register_position_encoding


class RotaryEncoding(PositionEncoding):
    """Rotate-half RoPE over the first ``rot_dim`` elements of a head.

    ``inv_freq_i = 1 / theta^(2i / rot_dim)`` in float32, angle = position * inv_freq_i as a
    float32 product (crates/vapi-backend-candle/src/models/lfm2.rs:163-183).  The reference
    rounds its cos/sin tables to the model dtype; here they stay float32 and are computed for
    the step's positions only, so there is no table of ``max_positions`` rows to hold.
    ``prepare`` returns ``(cos, sin)`` [n, rot_dim/2] which an attention mixer applies.
    """

    def __init__(self, rot_dim: int, theta: float, max_positions: int, name: str = "rope"):
        if rot_dim <= 0 or rot_dim % 2:
            raise ValueError(f"rotary width {rot_dim} must be a positive even number")
        self.rot_dim, self.theta, self.max_positions, self.name = int(rot_dim), float(theta), int(max_positions), name
        self._inv_freq: Dict[Any, torch.Tensor] = {}

    def inv_freq(self, device: torch.device) -> torch.Tensor:
        key = str(device)
        t = self._inv_freq.get(key)
        if t is None:
            theta = torch.tensor(self.theta, dtype=torch.float32)
            expo = torch.arange(0, self.rot_dim, 2, dtype=torch.float32) / float(self.rot_dim)
            t = (1.0 / torch.pow(theta, expo)).to(device).contiguous()
            self._inv_freq[key] = t
        return t

    def prepare(self, ctx: Any) -> Tuple[torch.Tensor, torch.Tensor]:
        return ops.rope_cos_sin(ctx.positions, self.inv_freq(ctx.positions.device))


class ScaledRotaryEncoding(PositionEncoding):
    """Rotary tables whose frequencies an interpolation rule has changed (YaRN).

    ``f_i = base^(-2i / rot_dim)``.  With ``scaling = (factor, original, fast, slow)``: let
    ``c(t) = rot_dim * ln(original / (2 pi t)) / (2 ln base)`` (the pair index that makes ``t`` turns
    over ``original`` positions), ``lo = max(floor(c(fast)), 0)``, ``hi = min(ceil(c(slow)), rot_dim - 1)``
    and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``; pair i then turns at
    ``f_i / factor * ramp_i + f_i * (1 - ramp_i)`` and cos and sin are both multiplied by
    ``0.1 ln(factor) + 1``.  Without ``scaling`` the tables are the plain ones.  The tables hold one
    column per pair and say nothing about which elements of a head form a pair: the mixer that
    applies them decides that (``layout``).  Angles are float32 products of position and frequency.
    """

    def __init__(self, rot_dim: int, base: float, scaling: Optional[Dict[str, float]] = None, name: str = "rope"):
        if rot_dim <= 0 or rot_dim % 2:
            raise ValueError(f"rotary width {rot_dim} must be a positive even number")
        self.rot_dim, self.base, self.name = int(rot_dim), float(base), name
        self.scaling = dict(scaling) if scaling else None
        self.freqs, self.mult = self.frequencies(self.rot_dim, self.base, self.scaling)
        self._freq: Dict[Any, torch.Tensor] = {}

    @staticmethod
    def frequencies(rot_dim: int, base: float, scaling: Optional[Dict[str, float]]):
        f = [base ** (-2.0 * i / rot_dim) for i in range(rot_dim // 2)]
        if not scaling:
            return f, 1.0
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def pair_of(turns: float) -> float:
            return rot_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
        hi = min(math.ceil(pair_of(float(scaling["slow"]))), rot_dim - 1)
        out = []
        for i, fi in enumerate(f):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(fi / factor * ramp + fi * (1.0 - ramp))
        return out, 0.1 * math.log(factor) + 1.0

    def key(self):
        """What makes two encodings the same tables (layers that agree share one)."""
        sc = tuple(sorted(self.scaling.items())) if self.scaling else None
        return (self.rot_dim, self.base, sc)

    def prepare(self, ctx: Any) -> Tuple[torch.Tensor, torch.Tensor]:
        dev = str(ctx.positions.device)
        t = self._freq.get(dev)
        if t is None:
            t = self._freq[dev] = torch.tensor(self.freqs, dtype=torch.float64).to(torch.float32).to(ctx.positions.device)
        return ops.rope_cos_sin_scaled(ctx.positions, t, self.mult)


register_position_encoding("rope", RotaryEncoding)
register_position_encoding("scaled_rope", ScaledRotaryEncoding)
