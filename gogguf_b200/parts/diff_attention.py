"""Differential attention: every query head holds two attention maps over the same values, and their outputs are
subtracted.

    q = W_q h  [heads x 2 x dim],  k = W_k h  [kv_heads x 2 x dim],  v = W_v h  [kv_heads x vdim]     (no biases)
    every (head, map) run of q and k: divided by its root mean square, times a weight [dim] that heads and maps
    share, then its first `rotary_dim` elements turned in adjacent pairs (2i, 2i + 1) by the position's angle
    a_m = softmax over j <= i of cap(scale * q_m . k_m,j) applied to v        cap(s) = softcap tanh(s / softcap)
    lambda = exp(sum(lq1 * lk1)) - exp(sum(lq2 * lk2)) + diff                 (stored vectors of size dim)
    o = unit(a_1 - lambda a_2) * (1 - diff)                                    unit: over the head's vdim values
    y = W_o concat_h o

Query head h reads kv head h / (heads / kv_heads).  The cache holds the keys as they enter the scores (normed,
rotated), both maps of a kv head side by side, and the values.  With `kv_source` {entry, member} the layer has
no key or value tensors: it reads the cache that the named schedule entry writes (its head counts, sizes and
rotation equal this layer's) with queries of its own.

Spec parameters: hidden_size, num_heads, num_kv_heads, head_dim, value_dim, scale, softcap (0 or absent: none),
diff, eps, window (absent: none), position {kind, ...} (absent or rotary_dim 0: none), kv_source, names.
Norms, rotation, scores, softmax, the difference and its norm are float32 in both compute paths.  In the bfloat16
path, head sizes of 32, 64 and 128 run on the tensor cores (`csrc/diff_attention.cu`: the softmax weights enter the
product with the values as two bfloat16 terms, the sums that norm them are float32); GOGGUF_B200_DIFF_ATTN_MMA=0
keeps the plain kernel, its twin.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional

import torch

from ..cache.sequence_cache import KVRequest, KVView, SharedView
from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..weights.loader import TensorDecl
from .base import Linear, Runtime, StepContext
from .registry import POSITIONS, lookup, register_mixer

MAX_VALUE_DIM = 512


@register_mixer("diff_attention")
class DiffAttentionMixer:
    @classmethod
    def _names(cls, spec: PartSpec) -> Dict[str, str]:
        n = dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm", lq1="lq1", lk1="lk1", lq2="lq2", lk2="lk2")
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def _sizes(cls, spec: PartSpec):
        return (int(spec["hidden_size"]), int(spec["num_heads"]), int(spec["num_kv_heads"]), int(spec["head_dim"]),
                int(spec["value_dim"]))

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        W, H, G, d, dv = cls._sizes(spec)
        n = cls._names(spec)
        t = {n["q"]: TensorDecl(shape=(H * 2 * d, W)), n["o"]: TensorDecl(shape=(W, H * dv)),
             n["q_norm"]: TensorDecl(shape=(d,), init="ones_normal")}
        for key in ("lq1", "lk1", "lq2", "lk2"):
            t[n[key]] = TensorDecl(shape=(d,), init="zeros_normal")
        if spec.get("kv_source") is None:
            t[n["k"]] = TensorDecl(shape=(G * 2 * d, W))
            t[n["v"]] = TensorDecl(shape=(G * dv, W))
            t[n["k_norm"]] = TensorDecl(shape=(d,), init="ones_normal")
        return t

    @classmethod
    def cache_request(cls, spec: PartSpec):
        _, _, G, d, dv = cls._sizes(spec)
        own = KVRequest(num_kv_heads=G, head_dim=2 * d, window=spec.get("window"), value_dim=dv)
        src = spec.get("kv_source")
        if src is None:
            return own
        return SharedView(entry=int(src["entry"]), member=src.get("member"), expects=own)

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.rt = rt
        self.hidden, self.H, self.G, self.d, self.dv = self._sizes(spec)
        if self.H % self.G:
            raise ValueError(f"diff_attention: {self.H} query heads are not a multiple of {self.G} kv heads")
        if self.dv > MAX_VALUE_DIM:
            raise ValueError(f"diff_attention: value_dim={self.dv} is not supported (at most {MAX_VALUE_DIM})")
        self.scale = float(spec.get("scale") or 1.0 / math.sqrt(self.d))
        self.cap = float(spec.get("softcap") or 0.0)
        self.diff = float(spec.get("diff", 0.0))
        self.eps = float(spec["eps"])
        self.window = int(spec.get("window") or 0)
        self.own_kv = spec.get("kv_source") is None
        pos = dict(spec.get("position") or {})
        self.rot = int(pos.get("rotary_dim", 0)) if pos else 0
        if self.rot > self.d or self.rot % 2:
            raise ValueError("diff_attention: rotary_dim is even and at most head_dim")
        self.position = None
        if self.rot:
            self.position = lookup(POSITIONS, pos["kind"], "position encoding")(pos, rt)
            if getattr(self.position, "pairing", "halves") != "adjacent":
                raise ValueError("diff_attention: its rotation turns adjacent pairs; the position part must say so")
        n = self._names(spec)
        mats = [rt.matrix(weights[n["q"]])]
        if self.own_kv:
            mats += [rt.matrix(weights[n["k"]]), rt.matrix(weights[n["v"]])]
        if len({m.dtype for m in mats}) != 1:
            mats = [m.float() for m in mats]
        # rows: q heads, then (a layer with keys and values of its own) k heads, then v heads
        self.proj = Linear(torch.cat(mats, dim=0) if len(mats) > 1 else mats[0], rt)
        self.width = self.proj.out_features
        self.o = Linear(weights[n["o"]], rt)
        self.q_norm = rt.vector(weights[n["q_norm"]])
        self.k_norm = rt.vector(weights[n["k_norm"]]) if self.own_kv else None
        lam = [weights[n[key]].detach().double().cpu() for key in ("lq1", "lk1", "lq2", "lk2")]
        self.lam = math.exp(float((lam[0] * lam[1]).sum())) - math.exp(float((lam[2] * lam[3]).sum())) + self.diff
        self.out_scale = 1.0 - self.diff
        self._mma = (rt.fast and rt.dtype == torch.bfloat16 and os.environ.get("GOGGUF_B200_DIFF_ATTN_MMA", "1") != "0")

    def prepare(self, ctx: StepContext) -> None:
        if self.position is not None:
            self.position.tables(ctx)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache: KVView,
                writes_cache: bool = True) -> None:
        if self.own_kv and not writes_cache:
            raise ValueError("diff_attention: a layer with keys of its own writes them; name the source layer with "
                             "kv_source instead of sharing the schedule entry's cache")
        T, H, G, d, dv = ctx.n_tokens, self.H, self.G, self.d, self.dv
        dt = self.rt.dtype
        qkv = ctx.ws.get("diff_attn_proj", (T, self.width), dt)
        self.proj(h, qkv, ws=ctx.ws)
        q = ctx.ws.get("diff_attn_q", (T, H * 2 * d), dt)
        cos, sin = self.position.tables(ctx) if self.position is not None else (None, None)
        table = ctx.page_tables[cache.group]
        K.diff_qk_prep(qkv, q, self.q_norm, self.k_norm, self.eps, cos, sin, ctx.positions, ctx.seq_of_token, table,
                       cache.page_size, cache.k if self.own_kv else None, cache.v if self.own_kv else None, T, H, G, d, dv,
                       self.rot)
        o = ctx.ws.get("diff_attn_out", (T, H * dv), dt)
        if self._mma and K.diff_attention_mma_takes(H, G, d, dv, cache.page_size):
            # steps of few rows over long contexts (decode steps): the key tiles are shared out over several CTAs
            nsplit = K.diff_attention_splits(T, ctx.n_seqs, H, G, int(ctx.max_ctx)) if ctx.max_new <= 4 else 1
            partial = (ctx.ws.get("diff_attn_shares", (K.diff_attention_partial_elems(T, H, dv, nsplit),), torch.float32)
                       if nsplit > 1 else None)
            K.diff_attention_mma(q, cache.k, cache.v, o, ctx.positions, ctx.seq_of_token, ctx.cu_seqlens, table,
                                 cache.page_size, T, ctx.n_seqs, H, G, d, dv, self.scale, self.cap, self.window, self.lam,
                                 self.eps, self.out_scale, nsplit=nsplit, partial=partial, max_new=int(ctx.max_new))
        else:
            K.diff_attention(q, cache.k, cache.v, o, ctx.positions, ctx.seq_of_token, table, cache.page_size, T, H, G, d, dv,
                             self.scale, self.cap, self.window, self.lam, self.eps, self.out_scale)
        self.o(o, residual, accumulate=True, ws=ctx.ws)
