"""Rotary position encoding, rotate-half ("NEOX") pairing, as the reference applies it
inside its attention kernel (src/kernel/cuda/paged_flash_attention.cu:300-384 for K,
:390-481 for Q) from a table of (cos, sin) of ``pos * exp(-(2i/d) * ln(base))``
(src/kernel/cuda/rope_table.cu:33-36).  The whole head is rotated unless
``rotary_dim`` says otherwise.  The table is float32 and is built by a kernel once."""
from __future__ import annotations

import torch

from ..registry import register_part
from .base import PositionEncoding


@register_part("position", "rotary")
class RotaryPosition(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: int = 0, prefix: str = ""):
        super().__init__(prefix)
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim) if rotary_dim else int(head_dim)
        self.theta = float(theta)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and <= head_dim {self.head_dim}")
        self.table = None

    def prepare(self, ops, device, max_position: int) -> None:
        self.table = torch.empty((max_position, self.rotary_dim // 2, 2), dtype=torch.float32, device=device)
        ops.rope_table(self.table, self.theta, self.rotary_dim)

    def rotary(self):
        return self.table, self.rotary_dim


@register_part("position", "none")
class NoPosition(PositionEncoding):
    def __init__(self, prefix: str = ""):
        super().__init__(prefix)


def scaled_frequencies(rot_dim: int, base: float, scaling=None, linear_factor: float = 1.0):
    """(frequencies as a list of rot_dim/2 floats, magnitude of cos and sin).  Plain: f_i = base^(-2i/rot_dim),
    magnitude 1.  With ``scaling`` = (factor, original, fast, slow), the YaRN rule: the dimension at which a
    position of ``original`` makes ``t`` turns is dim(t) = rot_dim ln(original / (2 pi t)) / (2 ln base);
    between lo = max(floor(dim(fast)), 0) and hi = min(ceil(dim(slow)), rot_dim - 1) a ramp r_i =
    clamp((i - lo) / max(hi - lo, 0.001), 0, 1) takes f_i over to f_i / factor (f_i (1 - r_i) + f_i / factor r_i),
    and cos and sin are multiplied by 0.1 ln(factor) + 1.  ``linear_factor``: every frequency is divided by it (linear
    scaling of the positions).  Evaluated in double; the caller rounds once."""
    import math
    half = rot_dim // 2
    f = [base ** (-2.0 * i / rot_dim) / float(linear_factor) for i in range(half)]
    if scaling is None:
        return f, 1.0
    factor, original, fast, slow = (float(v) for v in scaling)

    def dim_of(turns: float) -> float:
        return rot_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(fast)), 0)
    hi = min(math.ceil(dim_of(slow)), rot_dim - 1)
    out = []
    for i, fi in enumerate(f):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * r + fi * (1.0 - r))
    return out, 0.1 * math.log(factor) + 1.0


@register_part("position", "scaled_rotary")
class ScaledRotary(PositionEncoding):
    """A rotation of the first ``rotary_dim`` dimensions of a head whose angles are computed from the position
    where they are applied (no table, so no longest position): pair i at position p turns by float32(p) *
    float32(f_i).  ``pairing``: "interleaved" pairs dimension 2i with 2i+1, "halves" pairs i with i + rotary_dim/2.
    ``scaling`` rescales the frequencies and the magnitude, ``linear_factor`` divides every frequency (scaled_frequencies
    above)."""
    def __init__(self, rotary_dim: int, theta: float, pairing: str = "halves", scaling=None, linear_factor: float = 1.0,
                 prefix: str = ""):
        super().__init__(prefix)
        self.rotary_dim = int(rotary_dim)
        self.theta = float(theta)
        if pairing not in ("interleaved", "halves"):
            raise ValueError(f"pairing must be 'interleaved' or 'halves', got '{pairing}'")
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and positive")
        self.interleaved = pairing == "interleaved"
        self.scaling = tuple(scaling) if scaling is not None else None
        self.linear_factor = float(linear_factor)
        if not self.linear_factor > 0:
            raise ValueError("linear_factor must be positive")
        self.freq = None
        self.magnitude = 1.0

    def prepare(self, ops, device, max_position: int) -> None:
        f, self.magnitude = scaled_frequencies(self.rotary_dim, self.theta, self.scaling, self.linear_factor)
        self.freq = torch.tensor(f, dtype=torch.float64).to(torch.float32).to(device)

    def frequencies(self):
        return self.freq, self.rotary_dim, self.magnitude, self.interleaved
