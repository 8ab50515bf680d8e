"""Position encodings."""

from __future__ import annotations

import math
import weakref

import torch

from .base import PositionEncoding, Runtime
from .registry import register


@register("position", "rotary")
class Rotary(PositionEncoding):
    """Rotate-half rotary positions over the first ``dim`` elements of a head.

    inv_freq[i] = 1 / theta^(2i/dim); angle = position * inv_freq; pairs are
    (i, i + dim/2) (acvram/engine/layers.py:727-730, 934-936, 1006-1009).  The table
    holds, for each position, cos of the dim/2 angles and then their sin, in
    float32: the reference rounds its tables to the model's type
    (acvram/engine/layers.py:829-830); here angles, cos and sin stay 32-bit in both
    precisions.  The attention kernel reads the table itself.

    ``scaling`` = (factor s, original length L, fast, slow) stretches the slow pairs (YaRN: Peng et al., "YaRN:
    Efficient Context Window Extension of Large Language Models"): with c(r) = dim ln(L / (2 pi r)) / (2 ln theta),
    lo = max(floor(c(fast)), 0), hi = min(ceil(c(slow)), dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    pair i turns by inv_freq[i] (1 - ramp_i) + inv_freq[i] / s * ramp_i per position, and cos and sin are multiplied by
    0.1 ln s + 1.  A table with ``scaling`` or ``exact`` is computed in float64 and rounded once (the angle of a far
    position then carries no error of its own).

    Layers with the same (dim, theta, positions) on the same device hold one table between them (the table
    of a model with 40 960 positions and heads of 128 is 21 MB; a copy for each of 36 layers would be 755 MB)."""

    _shared: "weakref.WeakValueDictionary" = weakref.WeakValueDictionary()

    def __init__(self, hidden_size: int, dim: int, theta: float, max_positions: int, scaling: tuple | None = None,
                 exact: bool = False) -> None:
        if dim % 2:
            raise ValueError(f"rotary dim {dim} must be even")
        self.dim, self.theta, self.max_positions = int(dim), float(theta), int(max_positions)
        self.scaling = tuple(float(v) for v in scaling) if scaling is not None else None
        if self.scaling is not None and len(self.scaling) != 4:
            raise ValueError("rotary scaling is (factor, original length, fast, slow)")
        self.exact = bool(exact) or self.scaling is not None
        self.table: torch.Tensor | None = None

    def frequencies(self) -> tuple[torch.Tensor, float]:
        """(angle per position of each pair, float64 [dim/2]; the factor on cos and sin)."""
        i = torch.arange(self.dim // 2, dtype=torch.float64)
        inv = self.theta ** (-2.0 * i / self.dim)
        if self.scaling is None:
            return inv, 1.0
        s, length, fast, slow = self.scaling
        c = lambda r: self.dim * math.log(length / (2.0 * math.pi * r)) / (2.0 * math.log(self.theta))
        lo = max(math.floor(c(fast)), 0)
        hi = min(math.ceil(c(slow)), self.dim - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return inv / s * ramp + inv * (1.0 - ramp), 0.1 * math.log(s) + 1.0

    def load(self, tensors, rt: Runtime) -> None:
        key = (self.dim, self.theta, self.max_positions, self.scaling, self.exact, str(rt.device))
        table = Rotary._shared.get(key)
        if table is None:
            if self.exact:
                inv, mag = self.frequencies()
                ang = torch.outer(torch.arange(self.max_positions, dtype=torch.float64), inv)
                table = (torch.cat((ang.cos(), ang.sin()), dim=-1) * mag).to(torch.float32).contiguous().to(rt.device)
            else:
                inv = 1.0 / (self.theta ** (torch.arange(0, self.dim, 2, dtype=torch.float32) / self.dim))
                ang = torch.outer(torch.arange(self.max_positions, dtype=torch.float32), inv)
                table = torch.cat((ang.cos(), ang.sin()), dim=-1).contiguous().to(rt.device)
            Rotary._shared[key] = table
        self.table = table

    def rotary_table(self):
        return self.table


@register("position", "none")
class NoPosition(PositionEncoding):
    """No position signal (the mixer sees order through causality only)."""

    def __init__(self, hidden_size: int) -> None:
        pass

    def apply(self, q, k, ctx) -> None:
        return None
