"""Split-half rotary position encoding (student_engine.py:362-363, :537-554).

inv_freq_j = theta^(-2j/R), j < R/2, formed in float32 on the host exactly as the reference
forms it; the angle float32(position) * inv_freq_j and its sine and cosine are float32 in the
kernel. Component j pairs with component j + R/2 (`rotate_half`). R (`rotary_dim`) defaults
to the head size. With `precise` the frequencies are formed in float64 and rounded once to float32 (half a unit in the
last place instead of the few that a float32 power leaves; at position p an error of the frequency turns the pair by p
times as much).

`scaling` (optional: factor, low, high, original) rescales the frequencies by their wavelength l = 2 pi / f, in the manner of
Llama 3.1: f stays where l < original / high, becomes f / factor where l > original / low, and between the two is
(1 - s) f / factor + s f with s = (original / l - low) / (high - low).

`rotary_interleaved` is the same encoding with component 2j paired with 2j + 1 instead of j with j + R/2; a mixer that
applies the rotation itself asks `interleaved`."""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding
from .registry import register_part


class RotaryHalf(PositionEncoding):
    """params: head_dim, theta, rotary_dim (optional), precise (optional), scaling (optional). No tensors in the weight files."""
    interleaved = False

    def __init__(self, spec):
        super().__init__(spec)
        self.head_dim = int(self.params["head_dim"])
        self.rotary_dim = int(self.params.get("rotary_dim") or self.head_dim)
        self.theta = float(self.params["theta"])
        self.precise = bool(self.params.get("precise", False))
        self.scaling = dict(self.params["scaling"]) if self.params.get("scaling") else None
        if self.scaling is not None:
            missing = [k for k in ("factor", "low", "high", "original") if k not in self.scaling]
            if missing or float(self.scaling["high"]) == float(self.scaling["low"]):
                raise ValueError(f"{self.kind or 'rotary'}: scaling needs factor, low, high (different from low) and original")
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_half: rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.inv_freq = None

    def bind(self, tensors, dtype, device):
        index = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64 if self.precise else torch.float32)
        freq = 1.0 / (self.theta ** (index / self.rotary_dim))
        if self.scaling is not None:
            factor, low, high, original = (float(self.scaling[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / freq
            blend = (original / wavelength - low) / (high - low)
            between = (1.0 - blend) * freq / factor + blend * freq
            freq = torch.where(wavelength < original / high, freq, torch.where(wavelength > original / low, freq / factor, between))
        self.inv_freq = freq.to(torch.float32).to(device)

    def fused_rotary(self):
        return self.inv_freq, self.rotary_dim


class RotaryInterleaved(RotaryHalf):
    interleaved = True


register_part("position", "rotary_half", RotaryHalf)
register_part("position", "rotary_interleaved", RotaryInterleaved)
