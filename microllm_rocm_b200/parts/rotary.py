"""Rotary position encoding as a table of inverse frequencies.

inv_freq[i] = theta^(-2 i / rotary_dim), evaluated in fp32 exactly as the reference does
per element (src/ops/ops.cpp:861-864: `std::pow(base, -2.0F * float(pair) / float(head_width))`).
The reference recomputes it inside every kernel call; here it is computed once.  Layout
'split_half' pairs element i with i + rotary_dim/2 (the reference's SplitHalf,
src/model/config.h:9), 'interleaved' pairs 2i with 2i+1.  `rotary_dim` smaller than the
head size leaves the remaining elements untouched.  Optional `scale` divides positions'
frequencies (linear scaling); it defaults to 1.

Optional `stretch` {factor, original, fast, slow} stretches the slow frequencies for contexts longer than `original`
positions: with where(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta) (the pair index whose wave makes t turns
over `original` positions), lo = max(floor(where(fast)), 0), hi = min(ceil(where(slow)), rotary_dim - 1) and
ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns with f_i / factor * ramp_i + f_i * (1 - ramp_i), and
every cosine and sine is multiplied by 0.1 * ln(factor) + 1 (`RotaryTable.magnitude`).

Optional `rescale` {factor, low, high, original} slows the long waves down: with wavelength l_i = 2 pi / f_i, pair i keeps
f_i where l_i < original / high, turns with f_i / factor where l_i > original / low, and in between with
(1 - s) f_i / factor + s f_i, s = (original / l_i - low) / (high - low).  No factor on cosines and sines.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import PositionEncoding, RotaryTable, Runtime, register_position_encoding


def inverse_frequencies(theta: float, rotary_dim: int, scale: float = 1.0) -> np.ndarray:
    i = np.arange(rotary_dim // 2, dtype=np.float32)
    exponent = (np.float32(-2.0) * i) / np.float32(rotary_dim)
    inv = np.power(np.float32(theta), exponent, dtype=np.float32)
    if scale != 1.0:
        inv = (inv / np.float32(scale)).astype(np.float32)
    return inv


def stretched_frequencies(theta: float, rotary_dim: int, stretch: dict):
    """(inverse frequencies [rotary_dim/2] fp32, factor on cos and sin) of the stretched table; float64 on the host."""
    factor, original = float(stretch["factor"]), float(stretch["original"])
    if not (factor > 0 and original > 0 and float(stretch["fast"]) > 0 and float(stretch["slow"]) > 0 and theta != 1.0):
        raise ValueError("rotary stretch: factor, original, fast and slow must be positive")
    where = lambda turns: rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
    lo = max(math.floor(where(float(stretch["fast"]))), 0)
    hi = min(math.ceil(where(float(stretch["slow"]))), rotary_dim - 1)
    out = np.zeros(rotary_dim // 2, dtype=np.float64)
    for i in range(rotary_dim // 2):
        f = float(theta) ** (-2.0 * i / rotary_dim)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f / factor * ramp + f * (1.0 - ramp)
    return out.astype(np.float32), 0.1 * math.log(factor) + 1.0


def rescaled_frequencies(theta: float, rotary_dim: int, rescale: dict) -> np.ndarray:
    """Inverse frequencies [rotary_dim/2] fp32 with the long waves slowed down; float64 on the host."""
    factor, low, high, original = (float(rescale[k]) for k in ("factor", "low", "high", "original"))
    if not (factor > 0 and original > 0 and low > 0 and high > low):
        raise ValueError("rotary rescale: factor, original and low must be positive and high above low")
    out = np.zeros(rotary_dim // 2, dtype=np.float64)
    for i in range(rotary_dim // 2):
        f = float(theta) ** (-2.0 * i / rotary_dim)
        wave = 2.0 * math.pi / f
        if wave > original / low:
            f = f / factor
        elif wave >= original / high:
            s = (original / wave - low) / (high - low)
            f = (1.0 - s) * f / factor + s * f
        out[i] = f
    return out.astype(np.float32)


@register_position_encoding("rotary")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, params: dict, rt: Runtime):
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.layout = params.get("layout", "split_half")
        self.scale = float(params.get("scale", 1.0))
        if self.layout not in ("split_half", "interleaved"):
            raise ValueError(f"rotary layout {self.layout!r} is not one of split_half, interleaved")
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        if not self.theta > 0:
            raise ValueError("rotary theta must be positive")
        magnitude = 1.0
        if params.get("stretch") and params.get("rescale"):
            raise ValueError("rotary: either stretch or rescale")
        if params.get("stretch"):
            inv, magnitude = stretched_frequencies(self.theta, self.rotary_dim, params["stretch"])
        elif params.get("rescale"):
            inv = rescaled_frequencies(self.theta, self.rotary_dim, params["rescale"])
        else:
            inv = inverse_frequencies(self.theta, self.rotary_dim, self.scale)
        self._table = RotaryTable(torch.from_numpy(inv).to(rt.device), self.rotary_dim,
                                  self.layout == "interleaved", magnitude)

    def rotary_table(self, head_dim: int):
        if head_dim != self.head_dim:
            raise ValueError(f"rotary table was built for head_dim {self.head_dim}, asked for {head_dim}")
        return self._table


@register_position_encoding("none")
class NoPositionEncoding(PositionEncoding):
    def __init__(self, params: dict, rt: Runtime):
        pass
