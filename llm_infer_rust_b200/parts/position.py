"""Position encodings."""
from __future__ import annotations

import math

import torch

from .base import Part
from .registry import register_part


class HalfSplitRope(Part):
    """Rotary tables for the half-split ("rotate_half") layout.

    angle[p, i] = p * theta^(-2i / rot_dim), i in [0, rot_dim / 2); the pair
    (i, i + rot_dim / 2) of a head is rotated by it (reference:
    src/layers/ops.rs:70-127, which builds the table in float32 on the GPU).
    The angles are computed in float64 and the cosines and sines stored as
    float32 [max_positions, rot_dim / 2]; the rotation itself runs in float.
    """
    category = "position_encoding"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.rot_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        self.max_positions = int(spec["max_positions"])
        if self.rot_dim % 2:
            raise ValueError("rotary_dim must be even")
        i = torch.arange(0, self.rot_dim, 2, dtype=torch.float64)
        inv_freq = torch.exp(i * (-(math.log(self.theta) / self.rot_dim)))
        angle = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
        self.cos = torch.cos(angle).to(torch.float32).to(env.device).contiguous()
        self.sin = torch.sin(angle).to(torch.float32).to(env.device).contiguous()


class RotaryFrequencies(Part):
    """Half-split rotary encoding without a table of positions: only the frequencies
    f_i = theta^(-2i / rot_dim) / scaling_factor, i in [0, rot_dim / 2), as float32 (computed in float64).
    A kernel that rotates forms the angle position * f_i in float and takes its cosine and sine itself, so
    no longest position has to be known.  ``scaling_factor`` (linear scaling) divides every frequency.
    ``wavelength_scaling`` {factor, low, high, original} stretches by wavelength l = 2 pi / f instead: f is kept where
    l < original / high, divided by ``factor`` where l > original / low, and in between blended,
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low).
    ``pairing`` says which coordinates frequency i turns: "half_split" (i and i + rot_dim / 2, the default) or
    "interleaved" (2i and 2i + 1); a mixer's kernel reads it, and a mixer that cannot serve a pairing refuses it."""
    category = "position_encoding"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.rot_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        self.scaling_factor = float(spec.get("scaling_factor", 1.0))
        self.pairing = str(spec.get("pairing", "half_split"))
        if self.pairing not in ("half_split", "interleaved"):
            raise ValueError(f"pairing {self.pairing!r} is refused: half_split or interleaved")
        if self.rot_dim % 2 or self.rot_dim <= 0:
            raise ValueError("rotary_dim must be even and positive")
        i = torch.arange(0, self.rot_dim, 2, dtype=torch.float64)
        inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -i / self.rot_dim) / self.scaling_factor
        stretch = spec.get("wavelength_scaling")
        if stretch:
            factor, low, high = float(stretch["factor"]), float(stretch["low"]), float(stretch["high"])
            original = float(stretch["original"])
            if factor <= 0.0 or high <= low or original <= 0.0:
                raise ValueError("wavelength_scaling needs factor > 0, high > low and original > 0")
            wavelength = 2.0 * math.pi / inv_freq
            blend = torch.clamp((original / wavelength - low) / (high - low), 0.0, 1.0)
            blended = (1.0 - blend) * inv_freq / factor + blend * inv_freq
            # outside the band the blend is exactly 0 or 1, so one expression serves all three ranges
            inv_freq = torch.where(wavelength < original / high, inv_freq,
                                   torch.where(wavelength > original / low, inv_freq / factor, blended))
        self.inv_freq = inv_freq.to(torch.float32).to(env.device).contiguous()


register_part("position_encoding", "half_split_rope", HalfSplitRope)
register_part("position_encoding", "rotary_frequencies", RotaryFrequencies)
