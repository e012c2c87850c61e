"""Mixers that keep a matrix state per head and sequence: S_t = diag(g_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.

Two kinds, one scan kernel (`csrc/recurrence.cu`):

`lightning` (a fixed decay per head):
    q = silu(W_q h), k = silu(W_k h) [heads x dim], v = silu(W_v h) [heads x vdim];  g_t = decay_h
    y = W_o ( N(concat_h o_t; w) * sigmoid(W_g h) )          N over all heads' outputs together, weight [heads vdim]

`hgrn2` (a forget gate per channel that also decides what is written):
    q = silu(W_q h) [heads x dim], v = W_v h [heads x vdim]
    f = l + (1 - l) sigmoid(W_f h + b)                        l: a stored lower bound per channel
    g_t = f_t, k_t = 1 - f_t
    y = W_o concat_h N(o_t; w)                                N over each head's vdim outputs, weight [vdim] shared

N(z; w) = z / sqrt(mean(z^2) + eps) * w.  What a layer keeps per sequence is S alone (`StateRequest`
[heads, dim, vdim], float32), read at the start of a step and written back at its end, so prompts may come in
portions and decoding goes on from them.  The projections of h run as one product in the compute dtype; the
activations, the gate, the decays, the state, the outputs' norm and the output gate are float32 in both paths.

Spec parameters: hidden_size, num_heads, head_dim, value_dim, eps, names; `lightning` also decay (one number per
head).  The activations, the norm's extent and the output gate are parameters too (q_act, k_act, v_act: "silu" or
"none"; norm: "whole" or "head"; out_gate: "sigmoid", "silu" or "none"), with the kinds' own values as defaults.
"""
from __future__ import annotations

import os
from typing import Dict, List

import torch

from ..cache.sequence_cache import StateRequest, StateView
from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..weights.loader import TensorDecl
from .base import Linear, Runtime, StepContext
from .registry import register_mixer

CHUNKED_FROM = 64       # new tokens of one sequence from which a step takes the chunked form

_ACT = {"none": 0, "silu": 1}
_GATE = {"none": 0, "sigmoid": 1, "silu": 2}


class _MatrixStateMixer:
    """What the two kinds share: one product for every projection of h, the scan from and into the slot's state,
    norm and output gate, the output product."""

    kind = ""
    defaults: Dict[str, str] = {}
    names_default: Dict[str, str] = {}
    rows: List[str] = []            # the projections of h, in the order of their rows in the fused product

    @classmethod
    def _names(cls, spec: PartSpec) -> Dict[str, str]:
        n = dict(cls.names_default)
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def _opt(cls, spec: PartSpec, key: str) -> str:
        return str(spec.get(key) or cls.defaults[key])

    @classmethod
    def _sizes(cls, spec: PartSpec):
        return int(spec["hidden_size"]), int(spec["num_heads"]), int(spec["head_dim"]), int(spec["value_dim"])

    @classmethod
    def _row_count(cls, spec: PartSpec, key: str) -> int:
        _, H, d, dv = cls._sizes(spec)
        return H * d if key in ("q", "k", "f") else H * dv

    @classmethod
    def cache_request(cls, spec: PartSpec) -> StateRequest:
        _, H, d, dv = cls._sizes(spec)
        return StateRequest(shape=(H, d, dv), dtype=torch.float32)

    def _common(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime) -> Dict[str, str]:
        self.rt = rt
        self.hidden, self.H, self.d, self.dv = self._sizes(spec)
        self.eps = float(spec["eps"])
        self.act_q, self.act_k, self.act_v = (_ACT[self._opt(spec, k)] for k in ("q_act", "k_act", "v_act"))
        norm = self._opt(spec, "norm")
        if norm not in ("whole", "head"):
            raise ValueError(f"{self.kind}: norm must be 'whole' or 'head', got {norm!r}")
        self.whole = norm == "whole"
        self.gate = _GATE[self._opt(spec, "out_gate")]
        n = self._names(spec)
        rows = [k for k in self.rows if k != "g" or self.gate]
        mats = [rt.matrix(weights[n[k]]) for k in rows]
        if len({m.dtype for m in mats}) != 1:
            mats = [m.float() for m in mats]
        self.proj = Linear(torch.cat(mats, dim=0), rt)
        self.off: Dict[str, int] = {}
        at = 0
        for k in rows:
            self.off[k] = at
            at += self._row_count(spec, k)
        self.width = at
        self.norm_weight = rt.vector(weights[n["norm"]])
        self.o = Linear(weights[n["o"]], rt)
        self.out_scale = 1.0
        # prompts: chunks over many CTAs where the head sizes allow and the projections are 16-bit (the running
        # sums of logarithms the chunks work with are rounding next to those, not next to 32-bit projections);
        # GOGGUF_B200_SCAN_CHUNKED=0: token by token everywhere, the form of decode steps
        self._chunked = (os.environ.get("GOGGUF_B200_SCAN_CHUNKED", "1") != "0" and rt.dtype != torch.float32
                         and max(self.d, self.dv) <= K.SCAN_CHUNKS_MAX_HEAD)
        return n

    def scale_output(self, mult: float) -> bool:
        """A factor on this mixer's output: it multiplies the normed heads in float32, before the output product."""
        self.out_scale = float(mult)
        return True

    def _gate_args(self) -> Dict[str, object]:
        raise NotImplementedError

    def _scan(self, x, raw, cache, ctx) -> None:
        T, H, d, dv = ctx.n_tokens, self.H, self.d, self.dv
        if self._chunked and ctx.max_new >= CHUNKED_FROM:
            n = K.gated_scan_chunks_scratch(T, ctx.n_seqs, H, d, dv)
            K.gated_scan_chunks(x, self.off["q"], self.off[self.rows[1]], self.off["v"], raw,
                                ctx.ws.get("recurrence_chunk_states", (n,), torch.float32), cache.state, ctx.cu_seqlens,
                                ctx.slots, ctx.seq_of_token, T, ctx.n_seqs, H, d, dv, **self._gate_args())
            return
        K.gated_scan(x, self.off["q"], self.off[self.rows[1]], self.off["v"], raw, cache.state, ctx.cu_seqlens, ctx.slots,
                     ctx.seq_of_token, T, ctx.n_seqs, H, d, dv, **self._gate_args())

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache: StateView,
                writes_cache: bool = True) -> None:
        if not writes_cache:
            raise ValueError(f"{self.kind}: a layer's state cannot be read by another layer")
        T, H, dv = ctx.n_tokens, self.H, self.dv
        x = ctx.ws.get("recurrence_proj", (T, self.width), self.rt.dtype)
        self.proj(h, x, ws=ctx.ws)
        raw = ctx.ws.get("recurrence_raw", (T, H * dv), torch.float32)
        self._scan(x, raw, cache, ctx)
        y = ctx.ws.get("recurrence_out", (T, H * dv), self.rt.dtype)
        K.scan_finish(raw, x if self.gate else None, self.off.get("g", 0), y, self.norm_weight, ctx.seq_of_token, T, H, dv,
                      self.eps, self.out_scale, whole=self.whole, gate=self.gate)
        self.o(y, residual, accumulate=True, ws=ctx.ws)


@register_mixer("lightning")
class LightningMixer(_MatrixStateMixer):
    kind = "lightning"
    defaults = dict(q_act="silu", k_act="silu", v_act="silu", norm="whole", out_gate="sigmoid")
    names_default = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", g="g_proj.weight", norm="norm.weight",
                         o="o_proj.weight")
    rows = ["q", "k", "v", "g"]

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        W, H, d, dv = cls._sizes(spec)
        n = cls._names(spec)
        t = {n["q"]: TensorDecl(shape=(H * d, W)), n["k"]: TensorDecl(shape=(H * d, W)),
             n["v"]: TensorDecl(shape=(H * dv, W)), n["o"]: TensorDecl(shape=(W, H * dv))}
        t[n["norm"]] = TensorDecl(shape=(H * dv if cls._opt(spec, "norm") == "whole" else dv,), init="ones_normal")
        if cls._opt(spec, "out_gate") != "none":
            t[n["g"]] = TensorDecl(shape=(H * dv, W))
        return t

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self._common(spec, weights, rt)
        decay = [float(a) for a in spec["decay"]]
        if len(decay) != self.H:
            raise ValueError(f"lightning: {len(decay)} decays for {self.H} heads")
        if not all(0.0 <= a <= 1.0 for a in decay):
            raise ValueError("lightning: every decay must lie in [0, 1]")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=rt.device)

    def _gate_args(self) -> Dict[str, object]:
        return dict(decay=self.decay, act_q=self.act_q, act_k=self.act_k, act_v=self.act_v)


@register_mixer("hgrn2")
class Hgrn2Mixer(_MatrixStateMixer):
    kind = "hgrn2"
    defaults = dict(q_act="silu", k_act="none", v_act="none", norm="head", out_gate="none")
    names_default = dict(q="q_proj.weight", f="f_proj.weight", f_bias="f_proj.bias", lower="lower_bound",
                         v="v_proj.weight", g="g_proj.weight", norm="norm.weight", o="o_proj.weight")
    rows = ["q", "f", "v", "g"]

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        W, H, d, dv = cls._sizes(spec)
        n = cls._names(spec)
        t = {n["q"]: TensorDecl(shape=(H * d, W)), n["f"]: TensorDecl(shape=(H * d, W)),
             n["f_bias"]: TensorDecl(shape=(H * d,), init="small_normal"),
             n["lower"]: TensorDecl(shape=(H * d,), init="unit_interval"),
             n["v"]: TensorDecl(shape=(H * dv, W)), n["o"]: TensorDecl(shape=(W, H * dv))}
        t[n["norm"]] = TensorDecl(shape=(H * dv if cls._opt(spec, "norm") == "whole" else dv,), init="ones_normal")
        if cls._opt(spec, "out_gate") != "none":
            t[n["g"]] = TensorDecl(shape=(H * dv, W))
        return t

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        n = self._common(spec, weights, rt)
        self.f_bias = rt.vector(weights[n["f_bias"]])
        self.lower = rt.vector(weights[n["lower"]])

    def _gate_args(self) -> Dict[str, object]:
        return dict(forget_bias=self.f_bias, forget_lower=self.lower, act_q=self.act_q, act_v=self.act_v)
