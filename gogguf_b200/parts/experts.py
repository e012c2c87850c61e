"""Feed-forwards beyond the dense SwiGLU: a two-matrix layer around the xIELU activation, and routed experts.

xIELU (`xielu_mlp`): down(f(up h)) with f(z) = a_p z^2 + z/2 for z > 0 and a_q (exp(z) - 1 - z) + z/2 otherwise,
a_p = softplus(p), a_q = 1/2 + softplus(q); the stored tensor `act` holds (p, q).

Routed experts (`routed_experts`): router logits W_r h in float32, scores by sigmoid (or softmax), the `top_k`
largest chosen, weights the chosen scores (optionally renormalised), the weight applied to the expert's input
or to its output.  `correction` (a stored vector, named in `names`) is added to the scores for the choice only, the
weights stay the scores themselves; `groups` {count, keep}: the experts form `count` equal runs of neighbours, a
group's score is the sum of its two largest choice scores, and only experts of the `keep` best groups can be chosen.  An expert is a gated unit: y = act(Wg x, Wu x), out = Wd y, with
act "clamped_glu": g' = min(g, limit), u' = clamp(u, -limit, limit), g' sigmoid(slope g') (u' + up_offset)
(up_offset 1 unless given); act "silu_glu": silu(g) u, the same unit without a limit, with slope 1 and offset 0.
`shared` (optional: intermediate_size, prefix, names, row_gate) adds one dense gated unit that every token runs
(the `swiglu` feed-forward under the given prefix), summed with the routed experts' output; with `row_gate` its
output is multiplied by one sigmoid gate per token.  `identity` (a count, default 0): the router has that many
outputs beyond `num_experts` with no matrices behind them; choosing one adds the token's own input row times the
weight.  `weight_scale` multiplies the weights after the renormalisation (which divides by the chosen scores' sum
+ 1e-20).
The experts' matrices are reached through the chosen index with nothing read back: on the CUDA cores pair by pair
(the 32-bit path, sizes the tensor-core forms do not take), or in bfloat16 on mma.sync, a CTA per expert and 64
output rows with the expert's pairs as the operand (decode steps, short prompts).  Steps of many tokens in
bfloat16 sort the (token, choice) pairs by expert and run one tcgen05 product per expert on its rows.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..weights.loader import TensorDecl
from .base import Linear, Runtime, StepContext
from .registry import FEED_FORWARDS, lookup, register_feed_forward


SORTED_FORM_MIN_WORK = 1.5e9      # rows per expert x inner width x width from which prompts take the sorted form


def _softplus(v: float) -> float:
    return math.log1p(math.exp(-abs(v))) + max(v, 0.0)


@register_feed_forward("xielu_mlp")
class XieluMLP:
    @classmethod
    def _names(cls, spec: PartSpec) -> Dict[str, str]:
        n = dict(up="up_proj.weight", down="down_proj.weight", act="act")
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        h, i = spec["hidden_size"], spec["intermediate_size"]
        n = cls._names(spec)
        return {n["up"]: TensorDecl(shape=(i, h)), n["down"]: TensorDecl(shape=(h, i)),
                n["act"]: TensorDecl(shape=(2,), init="small_normal")}

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.rt = rt
        self.hidden, self.inter = int(spec["hidden_size"]), int(spec["intermediate_size"])
        n = self._names(spec)
        self.up = Linear(weights[n["up"]], rt)
        self.down = Linear(weights[n["down"]], rt)
        p, q = (float(v) for v in weights[n["act"]].detach().float().cpu().tolist())
        self.ap, self.aq = _softplus(p), 0.5 + _softplus(q)
        self.out_scale = 1.0

    def scale_output(self, mult: float) -> bool:
        """The factor goes onto the activation in float32, before it is rounded for the down projection."""
        self.out_scale = float(mult)
        return True

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        T = ctx.n_tokens
        z = ctx.ws.get("ffn_act", (T, self.inter), self.rt.dtype)
        self.up(h, z, ws=ctx.ws)
        K.xielu(z, z, self.ap, self.aq, self.out_scale)
        self.down(z, residual, accumulate=True, ws=ctx.ws)


@register_feed_forward("routed_experts")
class RoutedExperts:
    @classmethod
    def _names(cls, spec: PartSpec) -> Dict[str, str]:
        n = dict(router="router.weight", expert="experts.{}.", gate="gate_proj.weight", up="up_proj.weight",
                 down="down_proj.weight", correction="router.correction")
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        h, i, E = spec["hidden_size"], spec["intermediate_size"], spec["num_experts"]
        R = E + int(spec.get("identity", 0))          # router outputs
        n = cls._names(spec)
        t = {n["router"]: TensorDecl(shape=(R, h))}
        if spec.get("correction"):
            # (a correction evens out the experts' load: small next to the scores' spread, or the choice is its alone)
            t[n["correction"]] = TensorDecl(shape=(R,), init="zeros_normal")
        for e in range(E):
            p = n["expert"].format(e)
            t[p + n["gate"]] = TensorDecl(shape=(i, h))
            t[p + n["up"]] = TensorDecl(shape=(i, h))
            t[p + n["down"]] = TensorDecl(shape=(h, i))
        sh = cls._shared_spec(spec)
        if sh is not None:
            for local, decl in lookup(FEED_FORWARDS, sh.kind, "feed-forward").tensors(sh).items():
                t[sh.prefix + local] = decl
        return t

    @classmethod
    def _shared_spec(cls, spec: PartSpec):
        """The shared unit as a part spec of its own (prefix relative to this part), or None."""
        sh = spec.get("shared")
        if not sh:
            return None
        params = dict(hidden_size=spec["hidden_size"], intermediate_size=sh["intermediate_size"])
        if sh.get("names"):
            params["names"] = dict(sh["names"])
        if sh.get("row_gate"):
            params["row_gate"] = True
        return PartSpec(kind=sh.get("kind", "swiglu"), prefix=sh.get("prefix", "shared."), params=params)

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.rt = rt
        self.hidden, self.inter = int(spec["hidden_size"]), int(spec["intermediate_size"])
        self.E, self.top = int(spec["num_experts"]), int(spec["top_k"])
        self.identity = int(spec.get("identity", 0))
        self.R = self.E + self.identity              # router outputs
        self.weight_scale = float(spec.get("weight_scale", 1.0))
        if self.identity < 0 or self.top > self.R:
            raise ValueError(f"routed experts: top_k={self.top} of {self.R} router outputs")
        score = spec.get("score", "sigmoid")
        if score not in ("sigmoid", "softmax"):
            raise ValueError(f"routed experts: unknown score {score!r} (sigmoid, softmax)")
        self.softmax = score == "softmax"
        self.renorm = bool(spec.get("renormalize", False))
        where = spec.get("weight_on", "output")
        if where not in ("input", "output"):
            raise ValueError(f"routed experts: weight_on must be 'input' or 'output', got {where!r}")
        self.on_input = where == "input"
        act = dict(spec.get("activation") or {})
        kind = act.get("kind", "clamped_glu")
        if kind == "clamped_glu":
            self.limit = float(act.get("limit", float("inf")))
            self.slope = float(act.get("slope", 1.0))
            self.up_offset = float(act.get("up_offset", 1.0))
        elif kind == "silu_glu":
            self.limit, self.slope, self.up_offset = float("inf"), 1.0, 0.0
        else:
            raise ValueError(f"routed experts: unknown activation {kind!r} (clamped_glu, silu_glu)")
        n = self._names(spec)
        self.router_w = rt.matrix(weights[n["router"]])
        self.correction = rt.vector(weights[n["correction"]]) if spec.get("correction") else None
        gr = dict(spec.get("groups") or {})
        self.groups = int(gr.get("count", 1))
        self.keep = int(gr.get("keep", self.groups))
        if self.groups < 1 or self.R % self.groups or not (1 <= self.keep <= self.groups):
            raise ValueError(f"routed experts: {self.R} experts do not form {self.groups} equal groups of which "
                             f"{self.keep} are kept")
        if self.top > (self.R // self.groups) * self.keep:
            raise ValueError(f"routed experts: top_k={self.top} exceeds the experts of the {self.keep} kept groups")
        gu: List[torch.Tensor] = []
        dn: List[torch.Tensor] = []
        for e in range(self.E):
            p = n["expert"].format(e)
            g, u = rt.matrix(weights.pop(p + n["gate"])), rt.matrix(weights.pop(p + n["up"]))
            if g.dtype != u.dtype:
                g, u = g.float(), u.float()
            gu.append(torch.stack([g, u], dim=0))
            dn.append(rt.matrix(weights.pop(p + n["down"])))
        if len({t.dtype for t in gu} | {t.dtype for t in dn}) != 1:
            gu, dn = [t.float() for t in gu], [t.float() for t in dn]
        self.w_gu = torch.stack(gu, dim=0).contiguous()       # [E, 2, F, W]
        self.w_d = torch.stack(dn, dim=0).contiguous()        # [E, W, F]
        self.out_scale = 1.0
        self.shared = None
        sh = self._shared_spec(spec)
        if sh is not None:
            cls = lookup(FEED_FORWARDS, sh.kind, "feed-forward")
            self.shared = cls(sh, {local: weights.pop(sh.prefix + local) for local in cls.tensors(sh)}, rt)
        self._grouped = None
        # rows on 16-byte boundaries: what the tensor-core forms (mma.sync for few pairs, tcgen05 for many) take
        self._mma = (rt.fast and rt.dtype == torch.bfloat16 and self.w_gu.dtype == torch.bfloat16
                     and self.hidden % 8 == 0 and self.inter % 8 == 0)
        if rt.fast and rt.dtype == torch.bfloat16 and self.w_gu.dtype == torch.bfloat16:
            from . import experts_grouped
            self._grouped = experts_grouped.try_make(self)

    def scale_output(self, mult: float) -> bool:
        """The factor goes onto the experts' activations in float32 (the down projections are linear).  With a
        shared unit the part does not take a factor: the block applies it to the sum."""
        if self.shared is not None:
            return False
        self.out_scale = float(mult)
        return True

    def route(self, h: torch.Tensor, ctx: StepContext):
        T = ctx.n_tokens
        z = ctx.ws.get("moe_logits", (T, self.R), torch.float32)
        K.moe_router_logits(h, self.router_w, z, T)      # CUDA cores, float32 sums: the router is never reduced
        idx = ctx.ws.get("moe_idx", (T, self.top), torch.int32)
        wts = ctx.ws.get("moe_wts", (T, self.top), torch.float32)
        K.moe_route(z, self.top, idx, wts, ctx.seq_of_token, softmax=self.softmax, renormalize=self.renorm, rows=T,
                    correction=self.correction, groups=self.groups, keep=self.keep,
                    n_real=self.E if self.identity else 0, scale=self.weight_scale)
        return idx, wts

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        if self.shared is not None:
            self.shared.forward(h, residual, ctx)
        self._routed(h, residual, ctx)

    def _routed(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        T = ctx.n_tokens
        idx, wts = self.route(h, ctx)
        if self.identity:
            if self.on_input:
                raise ValueError("routed experts: identity experts take their weight on the output")
            K.moe_identity(h, idx, wts, residual, T, self.top, ctx.seq_of_token)
        P = T * self.top
        # the sorted form pays one launch per expert and matrix behind a read-back: worth it where an expert's
        # product is large (measured: 256 rows of 2,048 x 4,096 yes, of 1,024 x 2,048 no)
        prefer_mma = (self._mma and P <= K.MOE_MMA_MAX_PAIRS
                      and (P / self.E) * self.inter * self.hidden < SORTED_FORM_MIN_WORK)
        if self._grouped is not None and self._grouped.takes(ctx) and not prefer_mma:
            self._grouped.run(h, idx, wts, residual, ctx)
            return
        if self._mma and h.dtype == torch.bfloat16 and (P <= K.MOE_MMA_MAX_PAIRS or self._grouped is None):
            # few pairs in bfloat16: the experts' rows stream once through mma.sync, the pairs' rows as the operand
            # (more pairs than one launch takes, where the sorted form does not serve: a launch per slice of pairs)
            xs = ctx.ws.get("moe_rows_in", (P, self.hidden), torch.bfloat16)
            K.moe_gather(h, wts, None, xs, P, self.top, self.on_input)
            yb = ctx.ws.get("moe_act_rows", (P, self.inter), torch.bfloat16)
            rows = ctx.ws.get("moe_rows_out", (P, self.hidden), torch.float32)
            flat_idx, flat_wts = idx.view(-1), wts.view(-1)
            for p0 in range(0, P, K.MOE_MMA_MAX_PAIRS):
                p1 = min(P, p0 + K.MOE_MMA_MAX_PAIRS)
                K.moe_expert_mma(xs[p0:p1], self.w_gu, flat_idx[p0:p1], p1 - p0, yb[p0:p1], True, self.limit, self.slope,
                                 self.out_scale, None if self.on_input else flat_wts[p0:p1], up_offset=self.up_offset)
                K.moe_expert_mma(yb[p0:p1], self.w_d, flat_idx[p0:p1], p1 - p0, rows[p0:p1], False)
            K.moe_combine(rows, None, residual, T, self.top, ctx.seq_of_token, idx=idx if self.identity else None)
            return
        y = ctx.ws.get("moe_act", (T * self.top, self.inter), torch.float32)
        K.moe_gate_up(h, self.w_gu, idx, wts, y, T, self.top, self.on_input, self.limit, self.slope, self.out_scale,
                      up_offset=self.up_offset)
        K.moe_down(y, self.w_d, idx, residual, T, self.top, ctx.seq_of_token)
