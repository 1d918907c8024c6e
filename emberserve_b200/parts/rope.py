"""Rotary position encoding.  Two pairings share one table: rotate-half ("NeoX"), where
dimension i of a head pairs with dimension i + rotary_dim/2, and interleaved, where dimension
2i pairs with 2i + 1 (``RotaryInterleaved``; a mixer reads the pairing from ``part.pairing``).

``inv_freq[i] = 1 / theta^(2i / rotary_dim)`` and ``angle = pos * inv_freq[i]``, both in
float32, as ``emberserve/model/rope.py:68-82`` computes them; the table of (cos, sin) is
built once on the device by ``ems_rope_table`` and applied by the kernel that also writes
keys and values into the cache (``csrc/elementwise.cu``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import PositionEncoding, register_part


@dataclass(frozen=True)
class RotarySpec:
    rotary_dim: int  # how many leading dimensions of a head rotate (head_dim for Qwen2)
    theta: float
    max_positions: int
    kind: str = "rotary_neox"


def inv_frequencies(rotary_dim: int, theta: float) -> torch.Tensor:
    """float32 ``1 / theta^(2i/rotary_dim)``, i in [0, rotary_dim/2)."""
    exponent = torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim
    return 1.0 / (float(theta) ** exponent)


@register_part("position", "rotary_neox")
class RotaryNeox(PositionEncoding):
    pairing = "half"

    def __init__(self, spec: RotarySpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.rotary_dim % 2 or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim must be a positive even number, got {spec.rotary_dim}")
        self._table: torch.Tensor | None = None

    @property
    def max_positions(self) -> int:
        return self.spec.max_positions

    def rotary(self, device: torch.device) -> tuple[torch.Tensor, int]:
        s: RotarySpec = self.spec
        if self._table is None or self._table.device != device:
            inv = inv_frequencies(s.rotary_dim, s.theta).to(device)
            self._table = K.rope_table(inv, s.max_positions)
        return self._table, s.rotary_dim


@dataclass(frozen=True)
class RotaryInterleavedSpec:
    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rotary_interleaved"


@register_part("position", "rotary_interleaved")
class RotaryInterleaved(RotaryNeox):
    """The same angles (``pos * theta^(-2i/rotary_dim)``) and the same table; the pair that angle i
    turns is (2i, 2i + 1)."""

    pairing = "interleaved"


@dataclass(frozen=True)
class RotaryLinearSpec:
    """Rotary angles with every frequency divided by `factor` (linear position scaling: position p turns
    pair i by ``p * theta^(-2i / rotary_dim) / factor``); `factor` 1 is the plain table.  Either pairing."""

    rotary_dim: int
    theta: float
    max_positions: int
    factor: float = 1.0
    pairing: str = "half"  # or "interleaved"
    kind: str = "rotary_linear"


@register_part("position", "rotary_linear")
class RotaryLinear(RotaryNeox):
    def __init__(self, spec: RotaryLinearSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.pairing not in K.ROTARY_PAIRINGS:
            raise ValueError(f"pairing {spec.pairing!r}: one of {sorted(K.ROTARY_PAIRINGS)}")
        if not spec.factor > 0 or not spec.theta > 0:
            raise ValueError("linear scaling needs a positive factor and a positive base")
        self.pairing = spec.pairing

    def rotary(self, device: torch.device) -> tuple[torch.Tensor, int]:
        s: RotaryLinearSpec = self.spec
        if self._table is None or self._table.device != device:
            # (frequencies in 64 bits, rounded once; the angle is the 32-bit product with the position)
            i = torch.arange(s.rotary_dim // 2, dtype=torch.float64)
            inv = (float(s.theta) ** (-2.0 * i / s.rotary_dim) / float(s.factor)).to(torch.float32)
            self._table = K.rope_table(inv.to(device), s.max_positions)
        return self._table, s.rotary_dim


@dataclass(frozen=True)
class RotaryYarnSpec:
    """Rotary angles whose slow pairs are stretched by `factor` (YaRN: Peng et al., "YaRN: Efficient
    Context Window Extension of Large Language Models").  With ``where(t) = rotary_dim * ln(original /
    (2 pi t)) / (2 ln theta)``, pairs below ``lo = max(floor(where(fast)), 0)`` keep their frequency,
    pairs above ``hi = min(ceil(where(slow)), rotary_dim - 1)`` are divided by `factor`, and those
    between are blended linearly; cos and sin are both multiplied by ``0.1 ln(factor) + 1``."""

    rotary_dim: int
    theta: float
    max_positions: int
    factor: float
    original: int
    fast: float
    slow: float
    pairing: str = "interleaved"  # or "half"
    kind: str = "rotary_yarn"


def yarn_inv_frequencies(s: RotaryYarnSpec) -> tuple[torch.Tensor, float]:
    """(float32 frequency of every pair, the factor on cos and sin); computed in 64 bits, rounded once."""
    half = s.rotary_dim // 2
    i = torch.arange(half, dtype=torch.float64)
    f = float(s.theta) ** (-2.0 * i / s.rotary_dim)

    def where(turns: float) -> float:
        return s.rotary_dim * math.log(s.original / (2 * math.pi * turns)) / (2 * math.log(s.theta))

    lo = max(math.floor(where(s.fast)), 0)
    hi = min(math.ceil(where(s.slow)), s.rotary_dim - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return (f / s.factor * ramp + f * (1 - ramp)).to(torch.float32), 0.1 * math.log(s.factor) + 1.0


@register_part("position", "rotary_yarn")
class RotaryYarn(RotaryNeox):
    """The table holds ``mag * cos`` and ``mag * sin`` of ``pos * frequency[i]``, so the kernels that
    rotate by a table need not know about the scaling."""

    def __init__(self, spec: RotaryYarnSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.pairing not in K.ROTARY_PAIRINGS:
            raise ValueError(f"pairing {spec.pairing!r}: one of {sorted(K.ROTARY_PAIRINGS)}")
        if min(spec.factor, spec.original, spec.fast, spec.slow) <= 0 or spec.theta <= 1:
            raise ValueError("YaRN scaling needs positive factor, original, fast and slow and a base above 1")
        self.pairing = spec.pairing

    def rotary(self, device: torch.device) -> tuple[torch.Tensor, int]:
        s: RotaryYarnSpec = self.spec
        if self._table is None or self._table.device != device:
            inv, mag = yarn_inv_frequencies(s)
            self._table = K.rope_table(inv.to(device), s.max_positions)
            if mag != 1.0:
                self._table.mul_(mag)
        return self._table, s.rotary_dim
