"""Rotary position encoding with the llama3 frequency rule.

Inverse frequencies are computed once on the host in double precision from ``theta`` and the
scaling constants, exactly as the table builder of the reference does per position
(inference/operation/RoPE.java:14-28 of the reference project), then cast to float32; the angle
position * frequency and its sine and cosine are evaluated in 32-bit inside the kernel that
rotates queries and keys."""
from __future__ import annotations

import math
import struct

import torch

from .base import PositionEncoding, register_position_encoding

PAIRING_CODES = {"interleaved": 0, "half": 1}


def _f32(x: float) -> float:
    """Round a Python float to the nearest float32, as a Java ``float`` variable would hold it."""
    return struct.unpack("<f", struct.pack("<f", x))[0]


def llama3_inverse_frequencies(head_dim: int, theta: float, scaling: dict | None) -> list[float]:
    """freq_i = theta^(-i/head_dim) for even i; with llama3 scaling, wavelengths longer than
    original/low_freq_factor are slowed by ``factor``, shorter than original/high_freq_factor are
    kept, and those between are blended (RoPE.java:14-28).  The power is taken in double and every
    later quantity is held in float32, as the reference's ``float`` variables are."""
    out = []
    for i in range(0, head_dim, 2):
        freq = _f32(1.0 / math.pow(theta, i / float(head_dim)))
        if scaling is not None:
            factor = _f32(float(scaling["factor"]))
            low = _f32(float(scaling["low_freq_factor"]))
            high = _f32(float(scaling["high_freq_factor"]))
            original = _f32(float(scaling["original_max_position_embeddings"]))
            low_wavelen = _f32(original / low)
            high_wavelen = _f32(original / high)
            wavelen = _f32(2.0 * math.pi / freq)
            if wavelen < high_wavelen:
                pass
            elif wavelen > low_wavelen:
                freq = _f32(freq / factor)
            else:
                smooth = _f32(_f32(_f32(original / wavelen) - low) / _f32(high - low))
                freq = _f32(_f32(_f32(_f32(1.0 - smooth) * freq) / factor) + _f32(smooth * freq))
        out.append(freq)
    return out


class RotaryPositionEncoding(PositionEncoding):
    graph_safe = True
    pad_safe = True

    def __init__(self, head_dim: int, theta: float, pairing: str = "half", scaling: dict | None = None,
                 rotary_dim: int | None = None):
        if pairing not in PAIRING_CODES:
            raise ValueError(f"pairing must be one of {sorted(PAIRING_CODES)}, got {pairing!r}")
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim) if rotary_dim is not None else self.head_dim
        if self.rotary_dim % 2 or not (0 <= self.rotary_dim <= self.head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.theta, self.scaling = float(theta), scaling
        self.pairing = PAIRING_CODES[pairing]
        self._inv_freq: dict = {}

    def inverse_frequencies(self, device) -> torch.Tensor:
        key = str(device)
        t = self._inv_freq.get(key)
        if t is None:
            freqs = llama3_inverse_frequencies(self.rotary_dim, self.theta, self.scaling) or [0.0]
            t = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(device)
            self._inv_freq[key] = t
        return t


    def angles(self, ctx) -> torch.Tensor:
        """float32 [rotary_dim / 2, T, 2]: cosine and sine of every token's angle in this pass, made once per pass
        and shared by all layers whose frequencies are these (a product that rotates in its own epilogue reads them)."""
        from ..kernels import ops

        key = ("rotary angles", self.rotary_dim, self.theta, repr(self.scaling))
        table = ctx.extras.get(key)
        if table is None:
            table = ctx.extras[key] = ops.rope_angles(ctx.positions, self.inverse_frequencies(ctx.device), self.rotary_dim // 2)
        return table


class NoPositionEncoding(PositionEncoding):
    graph_safe = True
    pad_safe = True

    """Queries and keys pass unrotated (rotary_dim = 0)."""

    def __init__(self, head_dim: int = 0):
        self.rotary_dim, self.pairing = 0, 0
        self._inv_freq: dict = {}

    def inverse_frequencies(self, device) -> torch.Tensor:
        key = str(device)
        if key not in self._inv_freq:
            self._inv_freq[key] = torch.zeros(1, dtype=torch.float32, device=device)
        return self._inv_freq[key]


register_position_encoding("rope", RotaryPositionEncoding)
register_position_encoding("none", NoPositionEncoding)
