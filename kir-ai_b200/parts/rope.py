"""Rotary position embedding, half-split pairing.

For i < rotary_dim/2: f_i = theta^(-2i/rotary_dim), angle = position * f_i (both
32-bit), and the pair (x_i, x_{i + rotary_dim/2}) is rotated by the angle
(crates/llm-backend/src/core/math.rs:515-529 of the reference).  The frequency
table is made once on the host in 32-bit and kept on the device.

Two options.  ``scaling`` stretches the long wavelengths, the way Llama 3.1 does: with wavelength l = 2 pi / f, a
frequency stays where l < original / high, becomes f / factor where l > original / low, and between the two is
(1 - s) f / factor + s f with s = (original / l - low) / (high - low).  ``offset`` rotates columns [offset, offset +
rotary_dim) of a head instead of its first ones.  With either option the table is worked out in 64-bit and rounded
once.

A second kind of ``scaling`` (keys ``factor``, ``original``, ``fast``, ``slow``; the rule known as YaRN) stretches by
the INDEX of a frequency: with dim(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta), the index at which a
wavelength makes t turns over ``original`` positions, lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)),
rotary_dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency becomes
f_i / factor * ramp_i + f_i * (1 - ramp_i), and cosine and sine are multiplied by ``amplitude`` = 0.1 ln(factor) + 1
(the attention preparation kernel takes that factor; ``apply`` alone does not rotate with it).

``pairing="neighbours"`` pairs column 2i with column 2i + 1 (the interleaved layout) where the default, ``"halves"``,
pairs column i with column i + rotary_dim / 2.  A score is a sum over columns, so it does not change when the columns
of queries AND keys are put in another order: ``head_order()`` gives the order of a head's columns in which neighbours
lie half a rotated part apart, a part that projects queries and keys applies it to the rows of its matrices (and
biases) at load, and the kernels go on rotating halves.  Queries and keys of such a layer exist only in that order;
values are left alone.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding, Runtime


class RotaryEmbedding(PositionEncoding):
    capture_safe = True
    kernels_only = True

    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None, *, offset: int = 0,
                 scaling: Optional[dict] = None, precise: bool = False, pairing: str = "halves"):
        if pairing not in ("halves", "neighbours"):
            raise ValueError(f"columns are paired as 'halves' or as 'neighbours', got {pairing!r}")
        self.pairing = pairing
        self.head_dim = head_dim
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim or offset < 0 or offset + self.rotary_dim > head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} (from column {offset}) must be even and lie inside head_dim {head_dim}")
        self.theta = float(theta)
        self.offset = offset
        self.scaling = None
        self.ramp = None
        self.amplitude = 1.0
        if scaling is not None and "fast" in scaling:
            import math

            self.ramp = {key: float(scaling[key]) for key in ("factor", "original", "fast", "slow")}
            if min(self.ramp.values()) <= 0.0 or self.theta <= 1.0:
                raise ValueError(f"frequency scaling by index needs positive constants and a base above one, got {scaling}")
            self.amplitude = 0.1 * math.log(self.ramp["factor"]) + 1.0
        elif scaling is not None:
            self.scaling = {key: float(scaling[key]) for key in ("factor", "low", "high", "original")}
            if self.scaling["high"] == self.scaling["low"] or self.scaling["factor"] <= 0.0:
                raise ValueError(f"frequency scaling needs high != low and a positive factor, got {scaling}")
        self.precise = precise or scaling is not None or offset != 0
        self.inv_freq: Optional[torch.Tensor] = None

    def frequencies(self) -> torch.Tensor:
        if self.precise:
            return self._frequencies_64()
        half = self.rotary_dim // 2
        exponent = -(2.0 * torch.arange(half, dtype=torch.float32)) / float(self.rotary_dim)
        return torch.pow(torch.tensor(self.theta, dtype=torch.float32), exponent)

    def _frequencies_64(self) -> torch.Tensor:
        import math

        half = self.rotary_dim // 2
        index = torch.arange(half, dtype=torch.float64)
        freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * index / float(self.rotary_dim))
        if self.scaling is not None:
            sc = self.scaling
            wavelength = 2.0 * math.pi / freq
            smooth = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
            between = (1.0 - smooth) * freq / sc["factor"] + smooth * freq
            freq = torch.where(wavelength < sc["original"] / sc["high"], freq,
                               torch.where(wavelength > sc["original"] / sc["low"], freq / sc["factor"], between))
        if self.ramp is not None:
            r = self.ramp

            def index_of(turns: float) -> float:
                return self.rotary_dim * math.log(r["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

            lo = max(math.floor(index_of(r["fast"])), 0)
            hi = min(math.ceil(index_of(r["slow"])), self.rotary_dim - 1)
            ramp = torch.clamp((index - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            freq = freq / r["factor"] * ramp + freq * (1.0 - ramp)
        return freq.to(torch.float32)

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.inv_freq = self.frequencies().to(rt.device)

    def head_order(self) -> Optional[torch.Tensor]:
        """For ``pairing="neighbours"``: the stored columns of a head [head_dim] in the order in which the kernels want
        them (the first of every pair, then the second of every pair, then the columns that are not rotated where they
        were); None when the stored order is already the kernels'."""
        if self.pairing == "halves":
            return None
        order = torch.arange(self.head_dim)
        rotated = torch.arange(self.offset, self.offset + self.rotary_dim)
        order[self.offset : self.offset + self.rotary_dim] = torch.cat([rotated[0::2], rotated[1::2]])
        return order

    def row_order(self, heads: int) -> Optional[torch.Tensor]:
        """``head_order`` for the rows of a matrix [heads * head_dim, in] that projects ``heads`` heads."""
        order = self.head_order()
        if order is None:
            return None
        return (torch.arange(heads)[:, None] * self.head_dim + order[None, :]).reshape(-1)

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        if self.pairing != "halves":
            raise ValueError("a rotation of neighbouring columns runs on projections whose rows were put in order at load")
        if self.amplitude != 1.0:
            raise ValueError("a rotation whose cosine and sine carry a factor runs inside the attention preparation only")
        if self.offset:
            raise ValueError("a rotation that does not start at a head's first column runs inside the attention preparation only")
        self.rt.ops.rope_(q, positions, self.inv_freq, self.rotary_dim)
        self.rt.ops.rope_(k, positions, self.inv_freq, self.rotary_dim)

    def fused_table(self) -> Optional[torch.Tensor]:
        """The frequency table when the whole head is rotated (what the fused
        norm + rotation + cache-write kernel takes), else None."""
        return self.inv_freq if self.rotary_dim == self.head_dim and self.offset == 0 else None
