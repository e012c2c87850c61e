"""Position encodings.  A mixer builds the one its spec names and asks it for per-step tables."""
from __future__ import annotations

from typing import Any, Dict, Tuple

import math

import torch

from ..csrc import kernels as K
from .base import Runtime, StepContext
from .registry import register_position


@register_position("rope_neox")
class RotaryNeoX:
    """Rotary positions with NeoX pairing (i, i + rotary_dim/2): angle = pos * theta^(-2i/rotary_dim)
    (pkg/ops/rope_tables.go:6-20, pkg/ops/rope_heads.go:30-38).  Angles, cos and sin are computed in
    float64 once per step for all layers that share (theta, rotary_dim) and stored as float32."""

    pairing = "halves"

    def __init__(self, params: Dict[str, Any], rt: Runtime):
        self.theta = float(params["theta"])
        self.rotary_dim = int(params["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {self.rotary_dim}")
        half = self.rotary_dim // 2
        i = torch.arange(half, dtype=torch.float64)
        self.inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                                  -2.0 * i / self.rotary_dim).to(rt.device)
        self.magnitude = 1.0                                  # factor on cos and sin
        self.key = ("rope", self.theta, self.rotary_dim)     # the tables do not depend on the pairing

    def tables(self, ctx: StepContext) -> Tuple[torch.Tensor, torch.Tensor]:
        got = ctx.shared.get(self.key)
        if got is None:
            half = self.rotary_dim // 2
            tag = "_".join(str(k) for k in self.key[1:])
            cos = ctx.ws.get(f"rope_cos_{tag}", (ctx.n_tokens, half), torch.float32)
            sin = ctx.ws.get(f"rope_sin_{tag}", (ctx.n_tokens, half), torch.float32)
            K.rope_tables(ctx.positions, self.inv_freq, cos, sin, self.magnitude)
            got = ctx.shared[self.key] = (cos, sin)
        return got


@register_position("rope_yarn")
class RotaryYarn(RotaryNeoX):
    """NeoX pairing with frequencies stretched for contexts beyond the trained length: pairs that turn often
    within `original` positions keep their frequency, pairs that turn seldom are slowed by `factor`, with a linear
    ramp between.  d(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta) is the pair index that makes t turns in
    `original` positions; lo = max(floor d(fast), 0), hi = min(ceil d(slow), rotary_dim - 1),
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), f_i <- f_i / factor * r_i + f_i (1 - r_i); cos and sin are
    both multiplied by `magnitude_slope` ln(factor) + 1 (slope 0.1 unless given), which lengthens the rotated
    pairs.  Parameters: theta, rotary_dim, factor, original, fast, slow."""

    def __init__(self, params: Dict[str, Any], rt: Runtime):
        super().__init__(params, rt)
        factor, original = float(params["factor"]), float(params["original"])
        fast, slow = float(params["fast"]), float(params["slow"])
        if not (factor > 0 and original > 0 and fast > 0 and slow > 0 and self.theta > 1):
            raise ValueError("rope_yarn: factor, original, fast and slow must be positive and theta above one")
        dims = self.rotary_dim

        def pair_of(turns: float) -> float:
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

        lo = max(math.floor(pair_of(fast)), 0)
        hi = min(math.ceil(pair_of(slow)), dims - 1)
        i = torch.arange(dims // 2, dtype=torch.float64)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0).to(self.inv_freq.device)
        self.inv_freq = (self.inv_freq / factor * ramp + self.inv_freq * (1.0 - ramp)).contiguous()
        self.magnitude = float(params.get("magnitude_slope", 0.1)) * math.log(factor) + 1.0
        self.key = ("rope_yarn", self.theta, dims, factor, original, fast, slow, self.magnitude)


@register_position("rope_adjacent")
class RotaryAdjacent(RotaryNeoX):
    """The same angles with the other pairing: element 2i turns with element 2i + 1 (the interleaved layout),
    angle = pos * theta^(-2i/rotary_dim).  The tables are those of `RotaryNeoX` (column i is pair i), so layers
    of both kinds with equal base and size share them; which elements form a pair is the business of the
    kernel that applies them, and a mixer states the pairing it implements in `pairing`."""

    pairing = "adjacent"


@register_position("rope_yarn_adjacent")
class RotaryYarnAdjacent(RotaryYarn):
    """The stretched frequencies and the magnitude of `rope_yarn` with the other pairing: element 2i turns with
    element 2i + 1.  The tables are those of `RotaryYarn` (column i is pair i)."""

    pairing = "adjacent"
