"""Rotary position encoding as a table of inverse frequencies.

The reference rotates, per head, the pairs (i, i + head_dim/2) ("half-split") by the
angle ``pos * base^(-2i/head_dim)`` (``rope_neox_yarn``,
src/locus/backend/cpu_ops.cpp:1849-1872; angle cpu_ops.cpp:1807-1814), after the bias and
before the key is cached.  Here the per-pair inverse frequency is computed once on the
host in float64, rounded to float32, and handed to the kernel that also writes K and V;
the angle ``float(pos) * inv_freq[i]`` and its sine and cosine are float32 on the device.
``rot_dim`` < head_dim leaves the tail of each head unrotated; ``interleaved`` pairs
(2i, 2i+1) instead.

``scaling`` = {factor, original, fast, slow} stretches the slow pairs for contexts beyond the
``original`` length and leaves the fast ones alone, with a linear ramp between them over the pair
index i: with turns(t) = rot_dim * ln(original / (2 pi t)) / (2 ln theta) (the index of the pair that
makes t turns over the original length), lo = max(floor(turns(fast)), 0), hi = min(ceil(turns(slow)),
rot_dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency of pair i becomes
f_i / factor * ramp_i + f_i * (1 - ramp_i), and cosine and sine are both multiplied by
0.1 * ln(factor) + 1 (the table's ``magnitude``).  The table also carries the frequencies in float64
for kernels that form their angles in float64.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import PositionEncoding, RotaryTable, register_position


class Rotary(PositionEncoding):
    def __init__(self, prefix: str, *, head_dim: int, theta: float, rot_dim: Optional[int] = None,
                 interleaved: bool = False, scaling: Optional[dict] = None) -> None:
        super().__init__(prefix)
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rot_dim = int(rot_dim) if rot_dim is not None else self.head_dim
        self.interleaved = bool(interleaved)
        if self.rot_dim % 2 or not (0 < self.rot_dim <= self.head_dim):
            raise ValueError(f"rotary: rot_dim {self.rot_dim} must be even and within head_dim {self.head_dim}")
        self.scaling = dict(scaling) if scaling else None
        if self.scaling is not None:
            missing = [k for k in ("factor", "original", "fast", "slow") if not float(self.scaling.get(k, 0)) > 0]
            if missing:
                raise ValueError(f"rotary: scaling needs positive {', '.join(missing)}")
        self._table: Optional[RotaryTable] = None

    def frequencies(self) -> torch.Tensor:
        """float64 [rot_dim / 2]: the angle a position advances pair i by."""
        n = self.rot_dim
        i = torch.arange(n // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / n)
        if self.scaling is None:
            return f
        sc = self.scaling

        def turns(t: float) -> float:
            return n * math.log(float(sc["original"]) / (2.0 * math.pi * t)) / (2.0 * math.log(self.theta))

        lo = max(math.floor(turns(float(sc["fast"]))), 0)
        hi = min(math.ceil(turns(float(sc["slow"]))), n - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / float(sc["factor"]) * ramp + f * (1.0 - ramp)

    def magnitude(self) -> float:
        """What cosine and sine are multiplied by (1 without scaling)."""
        return 1.0 if self.scaling is None else 0.1 * math.log(float(self.scaling["factor"])) + 1.0

    def inv_freq_host(self) -> torch.Tensor:
        return self.frequencies().to(torch.float32)

    def bind(self, rt) -> None:
        f = self.frequencies()
        self._table = RotaryTable(f.to(torch.float32).to(rt.device), self.rot_dim, self.interleaved,
                                  magnitude=self.magnitude(), freq64=f.to(rt.device))

    def rotary_table(self) -> Optional[RotaryTable]:
        return self._table


class NoPosition(PositionEncoding):
    """No position encoding at all (q and k are used as projected)."""

    def __init__(self, prefix: str) -> None:
        super().__init__(prefix)

    def rotary_table(self):
        return None

    def apply(self, q, k, positions) -> None:
        return None


register_position("rotary", Rotary)
register_position("none", NoPosition)
