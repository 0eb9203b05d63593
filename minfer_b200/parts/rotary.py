"""Rotary position encoding: pairs of a head's dimensions are rotated by
``pos * frequency_scale / theta^(2i/rotary_dim)``.

The reference (src/graph/cpu_backend.rs:403-434) rotates the whole head, pairs
``(i, i + hd/2)`` for its ``NonInterleaved`` style (Qwen2, src/models/qwen2/loader.rs:144)
or ``(2i, 2i+1)`` for ``Interleaved`` (src/vec_ops.rs:6-14).  The reference forms the angle
``pos * freq`` in float32, which is off by about 1e-4 rad at position 2,000; here the inverse
frequencies are kept in float64, the angle is formed and reduced modulo 2 pi in float64 on the
device, and its sine and cosine are float32.

``scaling`` (YaRN): with ``factor``, ``original`` (the trained context), ``fast`` and ``slow``
(turns over that context), pair i's frequency f_i becomes f_i / factor * ramp_i + f_i * (1 -
ramp_i), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), lo = max(floor(d(fast)), 0),
hi = min(ceil(d(slow)), rotary_dim - 1), d(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta);
cosine and sine are multiplied by 0.1 ln(factor) + 1 (``magnitude``).
"""
from __future__ import annotations

import math
from typing import Any, Mapping, Optional, Tuple

import torch

from .base import PositionEncoding

STYLES = {"neox": 0, "interleaved": 1}


class Rotary(PositionEncoding):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def __init__(self, head_dim: int, rotary_dim: int, theta: float, frequency_scale: float = 1.0,
                 style: str = "neox", scaling: Optional[Mapping[str, Any]] = None):
        if style not in STYLES:
            raise ValueError(f"rotary style must be one of {sorted(STYLES)}, got {style!r}")
        if rotary_dim % 2 != 0 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and in (0, head_dim={head_dim}]")
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim)
        self.theta = float(theta)
        self.frequency_scale = float(frequency_scale)
        self.style = style
        self.scaling = None
        if scaling is not None:
            self.scaling = {k: float(scaling[k]) for k in ("factor", "original", "fast", "slow")}
            if not (self.scaling["factor"] > 0 and self.scaling["original"] > 0
                    and self.scaling["fast"] > 0 and self.scaling["slow"] > 0):
                raise ValueError("rotary scaling wants positive factor, original, fast and slow")
        self._inv_freq: dict = {}

    def inverse_frequencies(self) -> torch.Tensor:
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        freq = self.frequency_scale / torch.pow(
            torch.tensor(self.theta, dtype=torch.float64), 2.0 * i / self.rotary_dim)
        if self.scaling is None:
            return freq
        sc, dims = self.scaling, self.rotary_dim

        def dim_of(turns: float) -> float:
            return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

        lo = max(math.floor(dim_of(sc["fast"])), 0)
        hi = min(math.ceil(dim_of(sc["slow"])), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return freq / sc["factor"] * ramp + freq * (1.0 - ramp)

    def magnitude(self) -> float:
        """The factor on every cosine and sine (1 without scaling)."""
        return 1.0 if self.scaling is None else 0.1 * math.log(self.scaling["factor"]) + 1.0

    def fused_rotary(self, device: torch.device) -> Optional[Tuple[torch.Tensor, int, int]]:
        if self.scaling is not None and self.magnitude() != 1.0:
            raise ValueError("the fused rotary kernel applies no magnitude; this rotation has one")
        return self.tables(device)

    def tables(self, device: torch.device) -> Tuple[torch.Tensor, int, int]:
        """(inverse frequencies float64 on ``device``, rotary_dim, style code)."""
        key = str(device)
        if key not in self._inv_freq:
            self._inv_freq[key] = self.inverse_frequencies().to(device)
        return self._inv_freq[key], self.rotary_dim, STYLES[self.style]


class NoPosition(PositionEncoding):
    """No position encoding at all: queries and keys pass through."""

    def fused_rotary(self, device: torch.device):
        return None, 0, 0
