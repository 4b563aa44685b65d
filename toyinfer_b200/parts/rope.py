"""Rotary position encoding: the tables, and which elements of a head turn together.

inv_freq_i = theta^(-2i/d) for i < d/2; the pair (x_i, x_{i+d/2}) of a head is
rotated by the angle pos * inv_freq_i:
x_i <- x_i cos - x_{i+d/2} sin,  x_{i+d/2} <- x_{i+d/2} cos + x_i sin.
Reference: src/decode.cu:35-41 (frequencies), src/decode.cu:301-324 and
src/prefill.cu:185-208 (rotation).  The reference evaluates cosf/sinf of a 32-bit
product in every kernel; here the angles are formed once, in 64-bit, into 32-bit
cos and sin tables [max_positions, d/2] that every kernel reads, so that a
position has one angle whichever way the tokens are cut into steps.

``pairing`` "half" is the above; "neighbours" pairs (x_2i, x_2i+1) with the same angle pos * inv_freq_i
(the tables are the same; a mixer whose kernel knows both reads the attribute).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .base import BuildContext, PositionEncoding, register_part


def blended_frequencies(dim: int, theta: float, factor: float, original: int, fast: float, slow: float):
    """Frequencies stretched for contexts longer than ``original`` positions ("YaRN": Peng, Quesnelle, Fan,
    Shippole, 2023): pair i keeps theta^(-2i/dim) where its wave turns more than ``fast`` times over
    ``original`` positions, is divided by ``factor`` where it turns fewer than ``slow`` times, and is blended
    linearly in i between the two pair indices where that happens.  Returns (float64 frequencies, the magnitude
    0.1 ln(factor) + 1 that cos and sin are multiplied by)."""
    half = dim // 2
    i = torch.arange(half, dtype=torch.float64)
    base = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -(2.0 * i) / dim)

    def pair_index(turns: float) -> float:
        return dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(pair_index(fast)), 0)
    hi = min(math.ceil(pair_index(slow)), dim - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return base / factor * ramp + base * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def banded_frequencies(dim: int, theta: float, factor: float, original: int, low: float, high: float):
    """Frequencies rescaled by wavelength bands, as Llama 3.1 stretches its context: with wavelength l = 2 pi / f, a pair
    keeps f where l < original / high, gets f / factor where l > original / low, and between the two, with
    s = (original / l - low) / (high - low), (1 - s) f / factor + s f.  Returns float64 frequencies (no magnitude)."""
    half = dim // 2
    i = torch.arange(half, dtype=torch.float64)
    base = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -(2.0 * i) / dim)
    wavelength = 2.0 * math.pi / base
    s = (original / wavelength - low) / (high - low) if high != low else torch.ones_like(base)
    mid = (1.0 - s) * base / factor + s * base
    return torch.where(wavelength < original / high, base, torch.where(wavelength > original / low, base / factor, mid))


def rotary_tables(dim: int, theta: float, max_positions: int, scaling: Optional[dict] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of pos * f_i with f_i = theta^(-2i/dim) (or the blended frequencies and magnitude of ``scaling``:
    factor, original, fast, slow; or, with ``kind`` "bands", the banded frequencies of factor, original, low, high),
    computed in 64-bit, returned as float32."""
    half = dim // 2
    if scaling and scaling.get("kind") == "bands":
        inv_freq, magnitude = banded_frequencies(dim, float(theta), float(scaling["factor"]), int(scaling["original"]),
                                                 float(scaling["low"]), float(scaling["high"])), 1.0
    elif scaling:
        inv_freq, magnitude = blended_frequencies(dim, float(theta), float(scaling["factor"]), int(scaling["original"]),
                                                  float(scaling["fast"]), float(scaling["slow"]))
    else:
        i = torch.arange(half, dtype=torch.float64)
        inv_freq, magnitude = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -(2.0 * i) / dim), 1.0
    pos = torch.arange(max_positions, dtype=torch.float64)
    ang = pos[:, None] * inv_freq[None, :]
    return (torch.cos(ang) * magnitude).to(torch.float32), (torch.sin(ang) * magnitude).to(torch.float32)


class RotaryHalf(PositionEncoding):
    """``scaling``: None, or the stretch for long contexts (see blended_frequencies; with ``kind`` "bands" see
    banded_frequencies).  ``max_positions`` is the
    most the tables may ever hold; with ``lazy`` they are built for as many positions as ``ensure`` is told (the
    engine says how long its sequences get before the first step), not for the model's nominal limit."""

    def __init__(self, ctx: BuildContext, prefix: str, dim: int, theta: float, max_positions: int,
                 scaling: Optional[dict] = None, lazy: bool = False, pairing: str = "half"):
        if pairing not in ("half", "neighbours"):
            raise ValueError(f"rotary pairing must be 'half' or 'neighbours', got {pairing!r}")
        self.pairing = pairing
        if dim % 2:
            raise ValueError(f"rotary dimension must be even, got {dim}")
        self.dim = int(dim)
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self.scaling = dict(scaling) if scaling else None
        if self.scaling:
            bands = self.scaling.get("kind") == "bands"
            keys = ("factor", "original", "low", "high") if bands else ("factor", "original", "fast", "slow")
            for key in keys:
                if key not in self.scaling:
                    raise ValueError(f"rotary scaling needs {key!r}")
            if not all(self.scaling[key] > 0 for key in keys) or (not bands and self.scaling["factor"] < 1.0):
                raise ValueError(f"rotary scaling out of range: {self.scaling}")
        self.device = ctx.device
        self.cos = self.sin = None
        if not lazy:
            self.ensure(self.max_positions)

    def ensure(self, n_positions: int) -> None:
        """Tables for at least ``n_positions`` positions (never more than ``max_positions``).  Called before steps
        are captured: a captured step keeps the tables' addresses."""
        n = min(int(n_positions), self.max_positions)
        if self.cos is not None and self.cos.shape[0] >= n:
            return
        cos, sin = rotary_tables(self.dim, self.theta, n, self.scaling)
        self.cos = cos.to(self.device).contiguous()
        self.sin = sin.to(self.device).contiguous()

    def rotary_tables(self) -> Optional[Tuple[torch.Tensor, torch.Tensor, int]]:
        if self.cos is None:
            self.ensure(min(self.max_positions, 4096))
        return self.cos, self.sin, self.dim


register_part("position", "rotary_half", RotaryHalf)
