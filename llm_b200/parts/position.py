"""Rotary position encoding as a table of angles."""
from __future__ import annotations

import math

import torch

from ..errors import Unsupported
from .base import PositionEncoding, register_position


def inverse_frequencies(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """theta^(-2p/D) for pair p (D: the rotated part of a head), in float64 (apps/engine/src/ops.rs:128-131 of
    MythEclipse/llm), then config.json's `rope_scaling` of type llama3: pairs
    whose wavelength exceeds original/low_freq_factor are slowed by `factor`,
    those below original/high_freq_factor are kept, and the band between is
    blended linearly in original/wavelength."""
    pairs = torch.arange(head_dim // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * pairs / head_dim)
    if not scaling:
        return freq
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    if kind == "default":
        return freq
    if kind != "llama3":
        raise Unsupported(f"rope scaling of type '{kind}'")
    factor = float(scaling["factor"])
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    original = float(scaling["original_max_position_embeddings"])
    wavelength = 2.0 * math.pi / freq
    smooth = (original / wavelength - low) / (high - low)
    blended = (1.0 - smooth) * freq / factor + smooth * freq
    out = torch.where(wavelength > original / low, freq / factor, blended)
    return torch.where(wavelength < original / high, freq, out)


class Rope(PositionEncoding):
    """Holds a float32 table [positions, n] on the device, n = rotary_dim or head_dim: cos
    of position * inv_freq[p] in columns [0, n/2), sin in [n/2, n). Angles are computed in
    float64 and rounded once. With n < head_dim the elements of a head beyond n are not
    rotated (the rope dimension count of apps/engine/src/model.rs:93-95 of MythEclipse/llm)."""

    def __init__(self, spec):
        if spec.pairing not in ("half", "interleaved"):
            raise Unsupported(f"rope pairing '{spec.pairing}'")
        self.spec = spec
        self.interleaved = spec.pairing == "interleaved"
        self.rotary_dim = spec.head_dim if getattr(spec, "rotary_dim", None) is None else spec.rotary_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= spec.head_dim:
            raise Unsupported(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {spec.head_dim}")
        self.inv_freq = inverse_frequencies(self.rotary_dim, spec.theta, spec.scaling_dict)
        self.table = None

    def prepare(self, max_positions, device):
        n = min(max_positions, self.spec.max_positions)
        if self.table is not None and self.table.shape[0] >= n and self.table.device == torch.device(device):
            return
        angle = torch.arange(n, dtype=torch.float64)[:, None] * self.inv_freq[None, :]
        table = torch.cat([angle.cos(), angle.sin()], dim=1).to(torch.float32)
        self.table = table.to(device).contiguous()


register_position("rope", Rope)
