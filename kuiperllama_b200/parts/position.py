"""Rotary position encoding: the table of inverse frequencies."""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .base import PositionEncoding, Runtime, register_position


def rotary_inverse_frequencies(rotary_dim: int, theta: float, scaling: Optional[dict]) -> List[float]:
    """freq_j = theta^(-2j / rotary_dim) for j < rotary_dim / 2, in float64
    (ExiledOfCode/KuiperLLama builds sin/cos tables from 1 / pow(theta, d / head_size) with
    theta fixed per build, rope_kernel.cu:38-49,124-135; here theta is a parameter).

    ``scaling`` with rope_type "llama3" rescales by wavelength 2 pi / freq: shorter than
    original / high_freq_factor unchanged; longer than original / low_freq_factor divided
    by factor; between them interpolated linearly in original / wavelength.  KuiperLLama has
    no such rule; this follows the published meaning of those config.json keys."""
    freqs = [1.0 / (float(theta) ** ((2.0 * j) / rotary_dim)) for j in range(rotary_dim // 2)]
    if scaling is None:
        return freqs
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return freqs
    if kind != "llama3":
        raise ValueError(f"unknown rope scaling {kind!r}")
    factor = float(scaling["factor"])
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = []
    for f in freqs:
        wavelength = 2.0 * math.pi / f
        if wavelength < orig / high:
            out.append(f)
        elif wavelength > orig / low:
            out.append(f / factor)
        else:
            smooth = (orig / wavelength - low) / (high - low)
            out.append((1.0 - smooth) * f / factor + smooth * f)
    return out


@register_position("rope")
class RotaryPosition(PositionEncoding):
    """Spec: ``head_dim``, ``theta``, ``scaling`` (None or a llama3 dict) and optionally
    ``rotary_dim`` (default: the whole head).  The rotation itself happens in the mixer's
    fused rope-and-cache-write kernel; this part owns the frequencies."""

    def __init__(self, spec, prefix, tensors, runtime: Runtime):
        super().__init__(spec, prefix, tensors, runtime)
        self.head_dim = int(spec["head_dim"])
        self.rotary_dim = int(spec.get("rotary_dim") or self.head_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        freqs = rotary_inverse_frequencies(self.rotary_dim, float(spec["theta"]), spec.get("scaling"))
        self.inv_freq = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(runtime.device)

    def rotary(self):
        return self.inv_freq, self.rotary_dim
