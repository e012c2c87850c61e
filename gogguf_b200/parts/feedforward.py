"""Dense feed-forwards.

`swiglu`: down( silu(gate h) * (up h) ), no bias (pkg/model/qwen3/model.go:273-286, pkg/ops/inplace.go:14-19).
``names`` of the spec renames the stored matrices (keys gate, up, down, row_gate).  ``row_gate`` (optional, True):
a stored vector g of the input's width (names key row_gate, stored [1, hidden] or [hidden]) makes one gate per
token, and the unit's output is multiplied by sigmoid(g . h); the factor goes onto the activation rows in float32,
before the down projection (which is linear).

`gelu_mlp`: down( gelu(up h) ), no bias; ``approximate`` "none" (default: the exact erf form) or "tanh"."""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..weights.loader import TensorDecl
from .base import Linear, Runtime, StepContext
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU:
    @classmethod
    def _names(cls, spec: PartSpec) -> Dict[str, str]:
        n = dict(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight", row_gate="row_gate.weight")
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        h, i = spec["hidden_size"], spec["intermediate_size"]
        n = cls._names(spec)
        t = {n["gate"]: TensorDecl(shape=(i, h)), n["up"]: TensorDecl(shape=(i, h)),
             n["down"]: TensorDecl(shape=(h, i))}
        if spec.get("row_gate"):
            t[n["row_gate"]] = TensorDecl(shape=tuple(spec.get("row_gate_shape") or (1, h)))
        return t

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        n = self._names(spec)
        g, u = rt.matrix(weights[n["gate"]]), rt.matrix(weights[n["up"]])
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.rt = rt
        self.fused = None
        if (rt.fast and rt.dtype == torch.bfloat16 and g.dtype == torch.bfloat16 and self.inter % 64 == 0
                and self.inter >= 128 and self.hidden % 8 == 0):
            # gate and up rows interleaved in blocks of 64: the product's epilogue applies silu(gate) * up
            # and writes the activation directly, so the [T, 2 I] intermediate never exists
            from ..csrc import tcgen05_gemm
            self.fused = Linear(tcgen05_gemm.interleave_gate_up(g, u), rt, swiglu=True)
        if self.fused is None:
            # gate rows first, then up rows: one product for both, then the activation kernel
            self.gate_up = Linear(torch.cat([g, u], dim=0), rt)
        self.down = Linear(weights[n["down"]], rt)
        self.row_gate = rt.vector(weights[n["row_gate"]]).reshape(-1).contiguous() if spec.get("row_gate") else None

    def absorb_norm(self, norm) -> bool:
        """Take the block's pre-norm into the gate/up projection; `forward` then gets RowStats as `h`."""
        first = self.fused if self.fused is not None else self.gate_up
        if not first.can_fold or norm.size != self.hidden or self.row_gate is not None:
            return False
        first.fold_input_norm(norm.weight, norm.eps)
        return True

    def forward(self, h, residual: torch.Tensor, ctx: StepContext) -> None:
        T = ctx.n_tokens
        act = ctx.ws.get("ffn_act", (T, self.inter), self.rt.dtype)
        if self.fused is not None:
            self.fused(h, act, ws=ctx.ws)
        else:
            gu = ctx.ws.get("ffn_gate_up", (T, 2 * self.inter), self.rt.dtype)
            self.gate_up(h, gu, ws=ctx.ws)
            K.swiglu(gu, act, T, self.inter)
        if self.row_gate is not None:
            K.row_gate(act, h, self.row_gate, ctx.seq_of_token, T)
        self.down(act, residual, accumulate=True, ws=ctx.ws, emit=ctx.shared.get("row_stats"))


@register_feed_forward("gelu_mlp")
class GeluMLP:
    @classmethod
    def _names(cls, spec: PartSpec) -> Dict[str, str]:
        n = dict(up="up_proj.weight", down="down_proj.weight")
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        h, i = spec["hidden_size"], spec["intermediate_size"]
        n = cls._names(spec)
        return {n["up"]: TensorDecl(shape=(i, h)), n["down"]: TensorDecl(shape=(h, i))}

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.rt = rt
        self.hidden, self.inter = int(spec["hidden_size"]), int(spec["intermediate_size"])
        form = spec.get("approximate", "none")
        if form not in ("none", "tanh"):
            raise ValueError(f"gelu_mlp: approximate must be 'none' or 'tanh', got {form!r}")
        self.tanh_form = form == "tanh"
        n = self._names(spec)
        self.up = Linear(weights[n["up"]], rt)
        self.down = Linear(weights[n["down"]], rt)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        T = ctx.n_tokens
        z = ctx.ws.get("ffn_act", (T, self.inter), self.rt.dtype)
        self.up(h, z, ws=ctx.ws)
        K.gelu(z, z, self.tanh_form)
        self.down(z, residual, accumulate=True, ws=ctx.ws)
