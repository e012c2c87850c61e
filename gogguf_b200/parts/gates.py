"""Gates on a part's output: what an arrangement multiplies a part's result by, element by element.

`sigmoid_gate`: sigmoid(W h + b), with h the rows the arrangement hands to the part (the normed residual rows).
The product runs like every projection (tensor cores in the bfloat16 path, CUDA cores in the 32-bit path) and
leaves float32 logits; the bias, the sigmoid and the multiplication happen in float32 inside the kernel that
norms the part's output and adds it to the residual stream.

Spec parameters: in_size, out_size, names (keys weight, bias; the bias is left out with ``bias=False``).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorDecl
from .base import Linear, Runtime, StepContext
from .registry import register_gate


@register_gate("sigmoid_gate")
class SigmoidGate:
    @classmethod
    def _names(cls, spec: PartSpec) -> Dict[str, str]:
        n = dict(weight="weight", bias="bias")
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        n = cls._names(spec)
        t = {n["weight"]: TensorDecl(shape=(spec["out_size"], spec["in_size"]))}
        if spec.get("bias", True):
            t[n["bias"]] = TensorDecl(shape=(spec["out_size"],), init="small_normal")
        return t

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        n = self._names(spec)
        self.size = int(spec["out_size"])
        self.proj = Linear(weights[n["weight"]], rt)
        self.bias = rt.vector(weights[n["bias"]]) if spec.get("bias", True) else None
        self.key = "gate_logits"

    def logits(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        g = ctx.ws.get(self.key, (ctx.n_tokens, self.size), torch.float32)
        self.proj(h, g, ws=ctx.ws)
        return g
