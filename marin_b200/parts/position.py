"""Position encodings.

A rotary encoding hands the attention mixer a table of inverse frequencies and says how
pairs are formed; the fused norm + rotation + cache-write kernel takes both as
parameters.  ``NoPosition`` hands over nothing and the mixer skips the rotation.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import Part, Runtime
from .registry import register_position


class PositionEncoding(Part):
    #: float32 ``[rotary_dim // 2]`` on the device, or None when nothing rotates
    inv_freq: Optional[torch.Tensor] = None
    rotary_dim: int = 0
    #: False: element i pairs with i + rotary_dim/2 ("rotate half"); True: (2i, 2i+1)
    interleaved: bool = False
    #: what sines and cosines are multiplied by (1 unless a rescaled encoding says otherwise)
    magnitude: float = 1.0


@register_position("rope")
class Rotary(PositionEncoding):
    """Rotary embedding with half-split pairing.

    ``f_i = theta^(-(2i/d))`` in float32 and ``angle = float(pos) * f_i``; the pair
    ``(a, b) = (x[i], x[i + d/2])`` becomes ``(a cos - b sin, b cos + a sin)``
    (crates/tensor/src/ops.rs:52-95, crates/cuda/src/kernels.cu:147-162).
    """

    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None, interleaved: bool = False):
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim) if rotary_dim is not None else self.head_dim
        self.interleaved = bool(interleaved)
        if self.rotary_dim % 2 != 0 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")

    def load(self, tensors, rt: Runtime) -> None:
        half = self.rotary_dim // 2
        i = torch.arange(half, dtype=torch.float32)
        exponent = -(i * 2.0 / float(self.rotary_dim))
        self.inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float32), exponent).to(rt.device)


@register_position("rope_yarn")
class RescaledRotary(Rotary):
    """Rotary embedding whose frequencies are stretched for contexts longer than the ``original`` one (YaRN: Peng, Quesnelle,
    Fan, Shippole, "YaRN: Efficient Context Window Extension of Large Language Models").  With ``f_i = theta^(-2i/d)``
    and ``dim(t) = d ln(original / (2 pi t)) / (2 ln theta)`` (the pair that makes ``t`` turns over the original context):
    ``lo = max(floor(dim(fast)), 0)``, ``hi = min(ceil(dim(slow)), d - 1)``, ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``;
    pair ``i`` turns at ``f_i / factor * ramp_i + f_i (1 - ramp_i)``: fast pairs keep their frequency, slow ones are divided by
    ``factor``, those between are blended.  Sines and cosines are multiplied by ``0.1 ln(factor) + 1``.  The table is made in
    float64 on the host and rounded once to float32; angles are float32 products of it."""

    def __init__(self, head_dim: int, theta: float, factor: float, original: float, fast: float, slow: float,
                 rotary_dim: Optional[int] = None, interleaved: bool = False):
        super().__init__(head_dim, theta, rotary_dim, interleaved)
        self.factor, self.original, self.fast, self.slow = float(factor), float(original), float(fast), float(slow)
        if self.factor <= 0 or self.original <= 0 or self.fast <= 0 or self.slow <= 0 or self.theta <= 1:
            raise ValueError("rope_yarn: factor, original, fast and slow must be positive and theta above 1")
        self.magnitude = 0.1 * math.log(self.factor) + 1.0

    def frequencies(self):
        """The angle per position of every pair, as Python floats (float64)."""
        d, half = self.rotary_dim, self.rotary_dim // 2

        def dim_of(turns: float) -> float:
            return d * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

        lo = max(math.floor(dim_of(self.fast)), 0)
        hi = min(math.ceil(dim_of(self.slow)), d - 1)
        out = []
        for i in range(half):
            f = self.theta ** (-2.0 * i / d)
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / self.factor * ramp + f * (1.0 - ramp))
        return out

    def load(self, tensors, rt: Runtime) -> None:
        self.inv_freq = torch.tensor(self.frequencies(), dtype=torch.float64).to(torch.float32).to(rt.device)


@register_position("rope_llama3")
class BandScaledRotary(Rotary):
    """Rotary embedding whose slow pairs are slowed further for contexts longer than the ``original`` one, by wavelength
    bands (the frequency scaling of Llama 3.1).  With ``f_i = theta^(-2i/d)`` and wavelength ``l_i = 2 pi / f_i``: pairs with
    ``l_i < original / high`` keep ``f_i``; pairs with ``l_i > original / low`` turn at ``f_i / factor``; between the two, with
    ``s = (original / l_i - low) / (high - low)``, at ``(1 - s) f_i / factor + s f_i``.  Sines and cosines keep their size.
    The table is made in float64 on the host and rounded once to float32; angles are float32 products of it."""

    def __init__(self, head_dim: int, theta: float, factor: float, low: float, high: float, original: float,
                 rotary_dim: Optional[int] = None, interleaved: bool = False):
        super().__init__(head_dim, theta, rotary_dim, interleaved)
        self.factor, self.low, self.high, self.original = float(factor), float(low), float(high), float(original)
        if self.factor <= 0 or self.original <= 0 or self.low <= 0 or self.high <= self.low:
            raise ValueError("rope_llama3: factor, original and low must be positive and high above low")

    def frequencies(self):
        """The angle per position of every pair, as Python floats (float64)."""
        out = []
        for i in range(self.rotary_dim // 2):
            f = self.theta ** (-2.0 * i / self.rotary_dim)
            wavelength = 2.0 * math.pi / f
            if wavelength > self.original / self.low:
                f = f / self.factor
            elif wavelength >= self.original / self.high:
                s = (self.original / wavelength - self.low) / (self.high - self.low)
                f = (1.0 - s) * f / self.factor + s * f
            out.append(f)
        return out

    def load(self, tensors, rt: Runtime) -> None:
        self.inv_freq = torch.tensor(self.frequencies(), dtype=torch.float64).to(torch.float32).to(rt.device)


@register_position("none")
class NoPosition(PositionEncoding):
    def __init__(self, **_ignored):
        self.inv_freq, self.rotary_dim = None, 0
