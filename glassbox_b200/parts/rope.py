"""Rotary position encoding.

The table is built on the host exactly as Glassbox computes its angles
(crates/glassbox-core/src/model.rs:102-115): the inverse frequency 1 / theta^(2i/dim) is formed
in float64 and rounded to float32; the angle is the float32 product position * inv_freq; sine
and cosine are evaluated in float64 and rounded to float32. Doing the angle in float32 makes
long positions round "like transformers" (model.rs:106), so it is kept.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import Position, register_part


def rescaled_frequencies(theta: float, rotary_dim: int, rescale):
    """(float64 frequencies [rotary_dim/2], the factor on sine and cosine) of a rotation whose frequencies are stretched by
    wavelength (``RopeRescaleSpec``): pair i turns f_i = theta^(-2i / rotary_dim) radians per token; with dim(t) = rotary_dim *
    ln(original / (2 pi t)) / (2 ln theta) the pair index that makes t turns within the original context, the pairs below
    lo = max(floor(dim(fast)), 0) keep f_i, those above hi = min(ceil(dim(slow)), rotary_dim - 1) get f_i / factor, the
    ones between a blend along the ramp clamp((i - lo) / max(hi - lo, 0.001), 0, 1)."""
    half = rotary_dim // 2
    i = np.arange(half, dtype=np.float64)
    f = np.power(np.float64(theta), -2.0 * i / np.float64(rotary_dim))
    if rescale is None:
        return f, 1.0

    def pair_of(turns: float) -> float:
        return rotary_dim * math.log(rescale.original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(pair_of(rescale.fast)), 0)
    hi = min(math.ceil(pair_of(rescale.slow)), rotary_dim - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / rescale.factor * ramp + f * (1.0 - ramp), rescale.magnitude_slope * math.log(rescale.factor) + 1.0


def rotary_table(theta: float, rotary_dim: int, max_position: int, rescale=None) -> torch.Tensor:
    """float32 [max_position, rotary_dim/2, 2] holding (cos, sin), times the rescaling's factor if there is one."""
    freq, magnitude = rescaled_frequencies(theta, rotary_dim, rescale)
    inv = freq.astype(np.float32)
    pos = np.arange(max_position, dtype=np.float32)
    angle = (pos[:, None] * inv[None, :]).astype(np.float32)  # float32 multiply
    a64 = angle.astype(np.float64)
    table = np.stack([(np.cos(a64) * magnitude).astype(np.float32), (np.sin(a64) * magnitude).astype(np.float32)], axis=-1)
    return torch.from_numpy(np.ascontiguousarray(table))


def inverse_frequencies(theta: float, rotary_dim: int) -> torch.Tensor:
    """float32 [rotary_dim/2]: theta^(-2i / rotary_dim), formed in float64 and rounded once."""
    i = np.arange(rotary_dim // 2, dtype=np.float64)
    return torch.from_numpy(np.power(np.float64(theta), -2.0 * i / np.float64(rotary_dim)).astype(np.float32))


class Rope(Position):
    """``pairing`` "half": a (cos, sin) table for the kernels that rotate channel i with channel i + rotary_dim/2.
    ``pairing`` "interleaved" (channel 2i with 2i + 1): no table; the mixers that take it ask for ``inv_freq`` and
    form the angle float32(position) * inv_freq[i] and its sine and cosine on the device, so no largest position has to
    be known beforehand."""
    launches_through_kernels_only = True

    def __init__(self, spec, **_):
        super().__init__(spec)
        if spec.pairing not in ("half", "interleaved"):
            raise ValueError(f"rope pairing {spec.pairing!r} is not supported ('half' or 'interleaved')")
        if spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even")
        if getattr(spec, "rescale", None) is not None and spec.pairing != "half":
            raise ValueError("rescaled frequencies are built into the (cos, sin) table, which only the 'half' pairing uses")
        self.rotary_dim = spec.rotary_dim
        self.pairing = spec.pairing
        self._tables = {}

    def inv_freq(self, device):
        key = ("inv_freq", str(device))
        if key not in self._tables:
            self._tables[key] = inverse_frequencies(self.spec.theta, self.spec.rotary_dim).to(device)
        return self._tables[key]

    def fused_table(self, device):
        if self.pairing != "half":
            return None
        key = str(device)
        if key not in self._tables:
            self._tables[key] = rotary_table(self.spec.theta, self.spec.rotary_dim, self.spec.max_position,
                                             getattr(self.spec, "rescale", None)).to(device)
        return self._tables[key]


class NoPosition(Position):
    launches_through_kernels_only = True

    def __init__(self, spec=None, **_):
        super().__init__(spec)


register_part("position", "rope", Rope, replace=True)
register_part("position", "none", NoPosition, replace=True)
