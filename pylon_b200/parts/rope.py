"""Rotary position encoding.

Tables as raun6k/Pylon builds them (src/pylon/model/layers.py:43-51): float32
``inv_freq[j] = 1 / theta^(2j / d)``, ``angle[p, j] = p * inv_freq[j]`` formed in float32,
cos and sin of it; the rotation pairs element ``j`` with ``j + d/2`` (layers.py:73-78).
The tables stay float32 and the rotation is done in float32 inside the attention mixer's
fused kernel; only the first ``d/2`` columns are stored since both halves share angles.

Options beyond that.  ``rotary_dim``: only the first so many elements of a head are rotated.  ``layout``:
``"halves"`` pairs element j with j + rotary_dim / 2, ``"neighbours"`` element 2 j with 2 j + 1.  ``scaling``
changes the frequencies f_j = theta^(-2j / rotary_dim) for contexts longer than the ``original`` one:

* ``{"kind": "wavelength", "factor", "low", "high", "original"}``: by wavelength l = 2 pi / f.  Waves shorter
  than ``original / high`` keep f, waves longer than ``original / low`` get ``f / factor``, and between the two
  ``(1 - s) f / factor + s f`` with ``s = (original / l - low) / (high - low)``.
* ``{"kind": "yarn", "factor", "original", "fast", "slow"}``: by pair index.  With
  ``index(r) = rotary_dim ln(original / (2 pi r)) / (2 ln theta)``, ``lo = max(floor(index(fast)), 0)``,
  ``hi = min(ceil(index(slow)), rotary_dim - 1)`` and ``ramp_j = clamp((j - lo) / max(hi - lo, 0.001), 0, 1)`` the frequency is
  ``f_j / factor * ramp_j + f_j (1 - ramp_j)``, and cos and sin are both multiplied by ``0.1 ln(factor) + 1``.

Frequencies and angles of scaled tables are formed in float64 and rounded once to float32.
"""
from __future__ import annotations

import math
from typing import Mapping, Optional

import torch

from pylon_b200.parts.base import POSITION_ENCODINGS, PositionEncoding


@POSITION_ENCODINGS.register("rope")
class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, max_positions: int, rotary_dim: Optional[int] = None,
                 scaling: Optional[Mapping[str, float]] = None, layout: str = "halves") -> None:
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary size {self.rotary_dim} must be even and at most the head size {self.head_dim}")
        if layout not in ("halves", "neighbours"):
            raise ValueError(f"rotary layout is 'halves' or 'neighbours', not {layout!r}")
        if scaling is not None and scaling.get("kind") not in ("wavelength", "yarn"):
            raise ValueError(f"rotary scaling kind is 'wavelength' or 'yarn', not {scaling.get('kind')!r}")
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self.scaling = None if scaling is None else dict(scaling)
        self.layout = layout
        self._tables: Optional[tuple[torch.Tensor, torch.Tensor]] = None

    def set_max_positions(self, positions: int) -> None:
        """The engine shortens the tables to the longest request it will hold."""
        if positions != self.max_positions:
            self.max_positions = int(positions)
            self._tables = None

    def frequencies(self) -> tuple[torch.Tensor, float]:
        """float64 ``[rotary_dim / 2]`` frequencies after scaling, and the factor on cos and sin."""
        pairs = self.rotary_dim // 2
        freq = self.theta ** (-2.0 * torch.arange(pairs, dtype=torch.float64) / self.rotary_dim)
        s = self.scaling
        if s is None:
            return freq, 1.0
        factor, original = float(s["factor"]), float(s["original"])
        if s["kind"] == "wavelength":
            low, high = float(s["low"]), float(s["high"])
            wave = 2.0 * math.pi / freq
            blend = (original / wave - low) / (high - low)
            mixed = (1.0 - blend) * freq / factor + blend * freq
            return torch.where(wave < original / high, freq, torch.where(wave > original / low, freq / factor, mixed)), 1.0

        def index(turns: float) -> float:
            return self.rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

        lo = max(math.floor(index(float(s["fast"]))), 0)
        hi = min(math.ceil(index(float(s["slow"]))), self.rotary_dim - 1)
        ramp = torch.clamp((torch.arange(pairs, dtype=torch.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0

    def tables(self, device: torch.device) -> tuple[torch.Tensor, torch.Tensor, int, str]:
        """(cos, sin, rotary_dim, layout): float32 ``[positions, rotary_dim // 2]`` tables, any scaling and factor included."""
        if self._tables is None or self._tables[0].device != device:
            if self.scaling is None:
                exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
                inv_freq = 1.0 / (self.theta ** exponent)
                angles = torch.arange(self.max_positions, dtype=torch.float32).unsqueeze(1) * inv_freq.unsqueeze(0)
                cos, sin = torch.cos(angles), torch.sin(angles)
            else:
                freq, gain = self.frequencies()
                angles = torch.arange(self.max_positions, dtype=torch.float64).unsqueeze(1) * freq.unsqueeze(0)
                cos, sin = (torch.cos(angles) * gain).to(torch.float32), (torch.sin(angles) * gain).to(torch.float32)
            self._tables = (cos.to(device).contiguous(), sin.to(device).contiguous())
        return self._tables[0], self._tables[1], self.rotary_dim, self.layout

    def rotary_table(self, device: torch.device):
        if self.layout != "halves":
            return None   # the kernels that fuse the rotation pair element j with j + rotary_dim / 2
        cos, sin, rotary_dim, _ = self.tables(device)
        return cos, sin, rotary_dim
