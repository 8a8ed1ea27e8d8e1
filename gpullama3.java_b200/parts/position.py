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


def yarn_inverse_frequencies(dims: int, base: float, factor: float, original: float, fast: float, slow: float,
                             min_ramp_width: float = 0.001) -> list[float]:
    """f_i = base^(-2i/dims), slowed by ``factor`` where a pair turns fewer than ``slow`` times over ``original`` positions,
    kept where it turns more than ``fast`` times, blended linearly in the pair index between the two: with
    pair(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(pair(fast)), 0), hi = min(ceil(pair(slow)), dims - 1)
    and r_i = clamp((i - lo) / max(hi - lo, min_ramp_width), 0, 1), the frequency is f_i / factor * r_i + f_i (1 - r_i).
    Evaluated in double precision."""
    def pair(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo, hi = max(math.floor(pair(fast)), 0), min(math.ceil(pair(slow)), dims - 1)
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        r = min(max((i - lo) / max(hi - lo, min_ramp_width), 0.0), 1.0)
        out.append(f / factor * r + f * (1.0 - r))
    return out


class YarnRotaryPositionEncoding(PositionEncoding):
    """Rotary encoding over interleaved pairs with frequencies stretched for contexts longer than the ``original`` one
    (``yarn_inverse_frequencies``); cosine and sine are multiplied by ``magnitude`` = magnitude_slope ln(factor) + 1.
    Without ``factor`` (or with 1) it is the plain rotary encoding of base ``base``."""
    graph_safe = True
    pad_safe = True

    def __init__(self, rotary_dim: int, base: float, factor: float | None = None, original: float | None = None,
                 fast: float = 32.0, slow: float = 1.0, magnitude_slope: float = 0.1, min_ramp_width: float = 0.001):
        self.rotary_dim, self.pairing, self.base = int(rotary_dim), PAIRING_CODES["interleaved"], float(base)
        if self.rotary_dim % 2 or self.rotary_dim < 2:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and positive")
        self.factor = float(factor) if factor else 1.0
        if self.factor != 1.0 and not original:
            raise ValueError("stretched rotary frequencies need the original context length")
        self.original, self.fast, self.slow = float(original or 0.0), float(fast), float(slow)
        self.min_ramp_width = float(min_ramp_width)
        self.magnitude = float(magnitude_slope) * math.log(self.factor) + 1.0
        self._inv_freq: dict = {}

    def frequencies(self) -> list[float]:
        if self.factor == 1.0:
            return [self.base ** (-2.0 * i / self.rotary_dim) for i in range(self.rotary_dim // 2)]
        return yarn_inverse_frequencies(self.rotary_dim, self.base, self.factor, self.original, self.fast, self.slow,
                                        self.min_ramp_width)

    def inverse_frequencies(self, device) -> torch.Tensor:
        key = str(device)
        t = self._inv_freq.get(key)
        if t is None:
            t = self._inv_freq[key] = torch.tensor(self.frequencies(), dtype=torch.float64).to(torch.float32).to(device)
        return t


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
register_position_encoding("yarn", YarnRotaryPositionEncoding)
