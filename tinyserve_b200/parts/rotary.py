"""Rotary position encoding.  Tables as tinyserve builds them (serve.py:1225-1228):
inv_freq and angles in float64, cos and sin stored in float32, one row per absolute
position up to the engine's max_model_len (serve.py:1621).  ``pairing`` "half"
rotates (i, i + rotary_dim/2) as serve.py:811-814 does; "interleaved" rotates
(2i, 2i+1).  ``rotary_dim`` may be smaller than the head size (partial rotary); the
other dimensions pass through.  ``scaling`` = {factor, low, high, original} stretches the long
waves: with wavelength l = 2 pi / f, f stays where l < original / high, becomes f / factor where
l > original / low, and in between is (1 - s) f / factor + s f with
s = (original / l - low) / (high - low)."""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_position_encoding

class Rotary(PositionEncoding):
    capturable = True

    def __init__(self, rotary_dim: int, theta: float, pairing: str = "half", scaling: dict | None = None):
        super().__init__()
        if rotary_dim % 2:
            raise ValueError("rotary_dim must be even")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"unknown rotary pairing {pairing!r}")
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.interleaved = pairing == "interleaved"
        self.scaling = None
        if scaling:
            self.scaling = tuple(float(scaling[k]) for k in ("factor", "low", "high", "original"))
            factor, low, high, original = self.scaling
            if not (factor > 0 and high > low and original > 0 and low > 0):
                raise ValueError(f"rotary scaling {scaling!r}: factor, low and original positive, high above low")
        self.cos = self.sin = None

    @staticmethod
    def scaled(inv_freq, scaling):
        factor, low, high, original = scaling
        wave = 2.0 * math.pi / inv_freq
        s = ((original / wave - low) / (high - low)).clamp(0.0, 1.0)
        mixed = (1.0 - s) * inv_freq / factor + s * inv_freq
        out = torch.where(wave > original / low, inv_freq / factor, mixed)
        return torch.where(wave < original / high, inv_freq, out)

    @staticmethod
    def tables(rotary_dim, theta, num_positions, scaling=None):
        inv_freq = 1.0 / theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float64) / rotary_dim)
        if scaling:
            inv_freq = Rotary.scaled(inv_freq, scaling)
        freqs = torch.outer(torch.arange(num_positions, dtype=torch.float64), inv_freq)
        return freqs.cos().float(), freqs.sin().float()

    def prepare(self, runtime):
        # one table per (sizes, base) and engine: the layers of a model share it
        key = ("rotary", self.rotary_dim, self.theta, self.scaling)
        if key not in runtime.shared:
            cos, sin = self.tables(self.rotary_dim, self.theta, runtime.max_positions, self.scaling)
            runtime.shared[key] = (cos.to(runtime.device).contiguous(), sin.to(runtime.device).contiguous())
        self.cos, self.sin = runtime.shared[key]


register_position_encoding("rotary", Rotary)
