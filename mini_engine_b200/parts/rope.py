"""Rotary position encoding, half-split ("neox") layout.

Reference (layers/rotary_embedding.py:5-25): ``inv_freq[i] = theta^(-2i/d)``, angle
``pos * inv_freq[i]``; for i < d/2: ``o[i] = x[i] cos - x[i+d/2] sin``,
``o[i+d/2] = x[i+d/2] cos + x[i] sin``.  The table is built in float32 exactly as the
reference builds it, and stays float32 (the reference rounds it to the working dtype,
layers/rotary_embedding.py:21-22); the rotation itself runs inside the fused
norm+rotate+cache-write kernel of the attention mixer.
"""
from __future__ import annotations

import torch

from .base import PositionEncoding
from .registry import register_position_encoding


class RotaryEmbedding(PositionEncoding):
    capturable = True

    layout = "half_split"

    def __init__(self, rotary_dim: int, max_position: int, theta: float):
        super().__init__()
        if rotary_dim % 2:
            raise ValueError(f"rotary_dim {rotary_dim} must be even")
        self.rotary_dim = rotary_dim                  # the leading elements of a head that are rotated
        self.max_position = max_position
        self.theta = float(theta)
        self.cos_sin: torch.Tensor | None = None      # [max_position, rotary_dim] = cos | sin halves

    def finalize(self, dtype, device):
        d = self.rotary_dim
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
        t = torch.arange(self.max_position, dtype=torch.float32)
        freqs = torch.outer(t, inv_freq)                       # [P, d/2] float32
        self.cos_sin = torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous().to(device)


class InterleavedRotary(PositionEncoding):
    """Rotary positions on pairs of neighbouring elements: (x[2i], x[2i+1]) at position p becomes
    (u cos a - v sin a, v cos a + u sin a) with a = p * theta^(-2i / rotary_dim), on the first ``rotary_dim`` elements.
    It keeps no table over positions: the kernels form each angle from the position and ``inv_freq`` (float64, so that
    the angle is rounded once, to the float32 cosine and sine), which leaves the longest position open."""
    capturable = True

    layout = "interleaved"

    def __init__(self, rotary_dim: int, theta: float):
        super().__init__()
        if rotary_dim % 2 or rotary_dim < 0:
            raise ValueError(f"rotary_dim {rotary_dim} must be even")
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.inv_freq: torch.Tensor | None = None

    def finalize(self, dtype, device):
        d = self.rotary_dim
        i = torch.arange(0, d, 2, dtype=torch.float64)
        self.inv_freq = (self.theta ** (-i / d) if d else i).contiguous().to(device)


class FrequencyRotary(PositionEncoding):
    """Rotary positions in the half-split layout (element i with element i + rotary_dim / 2) on the first ``rotary_dim``
    elements, from a table of frequencies instead of a table over positions: f_i = theta^(-2i / rotary_dim), optionally
    rescaled by wavelength (``scaling`` = {factor, low, high, original}, the rule Llama 3.1 uses for long contexts: with
    l = 2 pi / f, a frequency with l < original / high stays, one with l > original / low is divided by factor, and between
    the two (1 - s) f / factor + s f with s = (original / l - low) / (high - low)).  The kernels form each angle from the
    position and ``freq`` (float64, so that the angle is rounded once), which leaves the longest position open."""
    capturable = True

    layout = "half_split"

    def __init__(self, rotary_dim: int, theta: float, scaling: "dict | None" = None):
        super().__init__()
        if rotary_dim % 2 or rotary_dim < 0:
            raise ValueError(f"rotary_dim {rotary_dim} must be even")
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.scaling = dict(scaling) if scaling else None
        if self.scaling:
            s = self.scaling
            if not (s["factor"] > 0 and s["original"] > 0 and s["high"] > s["low"] > 0):
                raise ValueError(f"rotary scaling needs factor > 0, original > 0 and high > low > 0, got {s}")
        self.freq: torch.Tensor | None = None

    def frequencies(self) -> list[float]:
        import math
        d = self.rotary_dim
        out = []
        for i in range(d // 2):
            f = self.theta ** (-2.0 * i / d)
            if self.scaling:
                s = self.scaling
                wavelength = 2.0 * math.pi / f
                if wavelength > s["original"] / s["low"]:
                    f = f / s["factor"]
                elif not wavelength < s["original"] / s["high"]:
                    t = (s["original"] / wavelength - s["low"]) / (s["high"] - s["low"])
                    f = (1.0 - t) * f / s["factor"] + t * f
            out.append(f)
        return out

    def finalize(self, dtype, device):
        self.freq = torch.tensor(self.frequencies(), dtype=torch.float64).contiguous().to(device)


register_position_encoding("rope", RotaryEmbedding)
register_position_encoding("rope_frequencies", FrequencyRotary)
register_position_encoding("rope_interleaved", InterleavedRotary)
