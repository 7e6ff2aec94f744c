"""Rotary position encoding, half-split pairing.

inv_freq_j = theta^(-2j/d) and the angle p * inv_freq_j are float32; cos and sin
are tabulated in float32 for every position up to ``max_positions``
(tinyvllm/layers.py:167-226).  The rotation itself is part of the mixer's fused
q/k kernel, which reads these tables at the step's positions (the reference
gathers and casts them per step, tinyvllm/layers.py:229-245).
"""

from __future__ import annotations

import math

import torch

from ..ops import kernels
from .base import BuildContext, Part
from .registry import register_part

_TABLES: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


class RopeHalfSplit(Part):
    # How the fused q/k kernels pair the elements of a head: element j of the first half with
    # element j of the second, rotated by position * inv_freq_j read from the float32 tables
    # ``cos`` and ``sin``.  A position part with another pairing must not hand its tables to them.
    pairing = "half_split"

    def __init__(self, ctx: BuildContext, *, head_dim: int, theta: float, max_positions: int) -> None:
        if head_dim % 2:
            raise ValueError("rotary encoding needs an even head size")
        self.head_dim = head_dim
        self.theta = float(theta)
        self.max_positions = max_positions
        self.device = ctx.device
        self.cos = self.sin = None

    def inverse_frequencies(self) -> torch.Tensor:
        """theta^(-2j/d) in float32, the reference's expression (tinyvllm/layers.py:192-205)."""
        exponent = torch.arange(0, self.head_dim, 2, dtype=torch.float32) / self.head_dim
        return 1.0 / (self.theta ** exponent)

    def finalize(self) -> None:
        """Tabulate once per (sizes, device); layers with equal parameters share the tables."""
        key = (self.head_dim, self.theta, self.max_positions, str(self.device))
        if key not in _TABLES:
            inv_freq = self.inverse_frequencies().to(self.device)
            _TABLES[key] = kernels.rope_tables(inv_freq, self.max_positions)
        self.cos, self.sin = _TABLES[key]


class RopeInterleaved(Part):
    """Rotary encoding with neighbouring dimensions paired: (2i, 2i + 1) of the first ``dims``
    dimensions of a head turn by position * base^(-2i / dims); the rest of the head passes.  No
    tables: the kernel that prepares q and k multiplies the position with ``inv_freq`` (float32)
    and takes sine and cosine itself, so there is no limit on positions.

    ``scaling`` (``factor``, ``original``, ``fast``, ``slow``) stretches the slow pairs for contexts
    beyond ``original`` positions: with d(t) = dims * ln(original / (2 pi t)) / (2 ln base), lo =
    max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo,
    0.001), 0, 1), pair i turns at f_i / factor * ramp_i + f_i * (1 - ramp_i), and cosine and sine are
    multiplied by ``magnitude`` = 0.1 ln(factor) + 1 (1 without scaling).

    A ``scaling`` of (``factor``, ``low``, ``high``, ``original``) is another rule, by wavelength: with l_i = 2 pi /
    f_i, a pair whose wave is shorter than original / high keeps f_i, one whose wave is longer than original /
    low turns at f_i / factor, and between the two, with s = (original / l_i - low) / (high - low), at
    (1 - s) f_i / factor + s f_i; cosine and sine keep their size."""

    pairing = "interleaved"

    def __init__(self, ctx: BuildContext, *, dims: int, base: float, scaling: dict | None = None) -> None:
        if dims <= 0 or dims % 2:
            raise ValueError("rotary encoding needs an even, positive number of dimensions")
        self.rot_dims = dims
        self.base = float(base)
        self.scaling = dict(scaling) if scaling else None
        self.magnitude = 1.0
        self.by_wavelength = self.scaling is not None and "low" in self.scaling
        if self.scaling is not None:
            wanted = ("factor", "original", "low", "high") if self.by_wavelength else ("factor", "original", "fast", "slow")
            missing = [key for key in wanted if key not in self.scaling]
            if missing:
                raise ValueError("rotary scaling lacks " + ", ".join(missing))
            if not self.scaling["factor"] > 0:
                raise ValueError("the scaling factor must be positive")
            if self.by_wavelength:
                if not self.scaling["high"] > self.scaling["low"] > 0 or not self.scaling["original"] > 0:
                    raise ValueError("rotary scaling by wavelength wants 0 < low < high and a positive original length")
            else:
                self.magnitude = 0.1 * math.log(float(self.scaling["factor"])) + 1.0
        self.device = ctx.device
        self.inv_freq = None

    def inverse_frequencies(self) -> torch.Tensor:
        """The pairs' frequencies, evaluated in double precision and rounded to float32 once."""
        exponent = torch.arange(0, self.rot_dims, 2, dtype=torch.float64) / self.rot_dims
        freqs = self.base ** -exponent
        if self.by_wavelength:
            factor, original = float(self.scaling["factor"]), float(self.scaling["original"])
            low, high = float(self.scaling["low"]), float(self.scaling["high"])
            wave = 2.0 * math.pi / freqs
            blend = ((original / wave - low) / (high - low)).clamp(0.0, 1.0)
            blended = (1.0 - blend) * freqs / factor + blend * freqs
            freqs = torch.where(wave < original / high, freqs, torch.where(wave > original / low, freqs / factor, blended))
        elif self.scaling is not None:
            factor, original = float(self.scaling["factor"]), float(self.scaling["original"])

            def dimension(turns: float) -> float:
                return self.rot_dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

            lo = max(math.floor(dimension(float(self.scaling["fast"]))), 0)
            hi = min(math.ceil(dimension(float(self.scaling["slow"]))), self.rot_dims - 1)
            index = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            ramp = ((index - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            freqs = freqs / factor * ramp + freqs * (1.0 - ramp)
        return freqs.to(torch.float32)

    def finalize(self) -> None:
        self.inv_freq = self.inverse_frequencies().to(self.device)


class RopeHalfSplitComputed(RopeInterleaved):
    """The same encoding without tables, but with the halves paired: dimension i of the first ``dims``
    dimensions of a head turns together with dimension i + dims / 2, by position * base^(-2i / dims)."""

    pairing = "half_split"


register_part("position", "rope_half_split", RopeHalfSplit)
register_part("position", "rope_interleaved", RopeInterleaved)
register_part("position", "rope_half_split_computed", RopeHalfSplitComputed)
