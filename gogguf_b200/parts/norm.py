"""RMSNorm: out = x * (1/sqrt(mean(x^2) + eps)) * weight (pkg/ops/rmsnorm.go:10-25).

Two optional parameters of the spec: ``tensor`` names the stored vector under the part's prefix (default
"weight"), and ``weight_offset`` is added to the stored vector when the model is built, for checkpoints that
keep their norm weights as the distance from one (the factor applied is then 1 + w)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..weights.loader import TensorDecl
from .base import Runtime
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm:
    # out = x / rms(x) * weight: a projection after it can take `weight` into its columns and apply
    # 1 / rms(x) to its own output rows (parts.base.RowStats)
    foldable = True

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        offset = float(spec.get("weight_offset", 0.0))
        return {spec.get("tensor", "weight"): TensorDecl(shape=(spec["size"],),
                                                         init="ones_normal" if offset == 0.0 else "zeros_normal")}

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = rt.vector(weights[spec.get("tensor", "weight")])
        offset = float(spec.get("weight_offset", 0.0))
        if offset != 0.0:
            self.weight = (self.weight + offset).contiguous()      # float32: the sum is exact to a rounding

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        """x: float32 rows of the residual stream; out: compute dtype; rows: optional row gather."""
        K.rmsnorm(x, self.weight, self.eps, out, rows)


@register_norm("group_rmsnorm")
class GroupRMSNorm:
    """RMS norm in groups: the row is cut into `groups` equal consecutive runs, each is divided by its own
    sqrt(mean(run^2) + eps), and the whole is multiplied by the stored weight.  ``scale_tensor`` (optional) names a
    second stored vector of the row's size that multiplies the result element by element (a layer scale); the two
    vectors are multiplied once, in float32, when the model is built.  With one group and no scale this is
    `rmsnorm`; it is not offered to a product as a folded norm."""

    foldable = False

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        t = {spec.get("tensor", "weight"): TensorDecl(shape=(spec["size"],), init="ones_normal")}
        if spec.get("scale_tensor"):
            t[spec["scale_tensor"]] = TensorDecl(shape=(spec["size"],), init="ones_normal")
        return t

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.groups = int(spec.get("groups", 1))
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"group_rmsnorm: {self.size} columns do not form {self.groups} equal runs")
        self.weight = rt.vector(weights[spec.get("tensor", "weight")])
        if spec.get("scale_tensor"):
            self.weight = (self.weight * rt.vector(weights[spec["scale_tensor"]])).contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        K.rmsnorm(x, self.weight, self.eps, out, rows, groups=self.groups)
