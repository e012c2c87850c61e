"""Operations on the residual stream as a whole, run by an arrangement before and after a block's parts.

`depth_average`: with X_0 the embedded rows and X_(i+1) what block i leaves, the rows that go on to block i + 1
(and after the last block to the output) are sum_(j <= i+1) c_i[j] X_j, c_i a stored vector of i + 2 coefficients.
The X_j of the step live in one float32 workspace buffer [depth + 1, T, hidden]; block 0 also files the embedded
rows there before its parts change them.

Spec parameters: index (the block's place i), depth (how many blocks file their result), tensor (the stored
coefficients, named relative to the part's prefix).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..weights.loader import TensorDecl
from .base import Runtime, StepContext
from .registry import register_stream


@register_stream("depth_average")
class DepthAverage:
    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        return {spec.get("tensor", "weight"): TensorDecl(shape=(int(spec["index"]) + 2,), init="mean")}

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.index, self.depth = int(spec["index"]), int(spec["depth"])
        if not (0 <= self.index < self.depth):
            raise ValueError(f"depth_average: index {self.index} outside 0..{self.depth - 1}")
        self.coeff = rt.vector(weights[spec.get("tensor", "weight")])

    def _history(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return ctx.ws.get("depth_history", (self.depth + 1,) + tuple(x.shape), torch.float32)

    def begin(self, x: torch.Tensor, ctx: StepContext) -> None:
        if self.index == 0:
            K.depth_mix(self._history(x, ctx), x, None, 0, 0)

    def finish(self, x: torch.Tensor, ctx: StepContext) -> None:
        K.depth_mix(self._history(x, ctx), x, self.coeff, self.index + 1, self.index + 2)
