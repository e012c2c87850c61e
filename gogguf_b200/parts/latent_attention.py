"""Latent attention: keys and values of all heads are linear images of one cached vector per position.

    q          = Wq h                         per head [plain (nope_dim) | rot (rope_dim)]
    [l | k_r]  = Wdown h                      latent (latent_dim) and one rotated key part all heads share
    c          = l / rms(l) * w_latent_norm
    key_h      = [Wuk_h c | rotate(k_r)],     value_h = Wuv_h c
    score      = scale * q_h . key_h          softmax over the visible positions (causal, optional window)
    out        = Wo concat_h(sum_j p_j value_h,j)

Only c and the rotated k_r are cached (`LatentRequest`: latent_dim + rope_dim numbers per position and layer,
whatever the number of heads).  Since key and value are linear in c, the step never builds them: the query's
plain part is taken through Wuk_h^T once per token and head (the *absorbed* query, latent_dim wide), attention
runs over the cached rows with all heads sharing every row it reads, and Wuv_h is applied to the weighted sum
of latents afterwards.  That formulation serves prompts, portions of prompts and decoding alike.  A step in which
every sequence starts at position 0 (whole prompts) may instead build the step's keys and values once by a
product and run attention in the ordinary per-head form, which costs a third of the arithmetic; both forms
compute the same sums, so a position's result does not depend on how its sequence was cut into steps beyond
rounding.

The rotation is the adjacent-pair kind (`rope_adjacent`), applied to the first `rotary_dim` elements of the
rot part; `rope_dim` may be 0 (no rotated part, no position encoding: `position` is then left out).

Two options.  `q_latent_dim` (Rq): the queries go through a latent of their own, c_q = N(W_dq h; w_q) (RMS norm with
a plain weight, `latent_norm_eps`), q = W_uq c_q; W_dq and the key/value down projection run as one product.
`sink`: a stored number per head whose exponential joins the softmax's denominator; it has no key and no value, is
not scaled, and counts once.

Spec parameters: hidden_size, num_heads, nope_dim, rope_dim, value_dim, latent_dim, scale, window,
latent_norm_eps, position, q_latent_dim, sink, and optionally `names` (local tensor names of q, down, latent_norm,
up_k, up_v, out; with a query latent q_down, q_latent_norm and q (the up projection); with a sink, sink).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.sequence_cache import LatentRequest, LatentView
from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..weights.loader import TensorDecl
from .base import Linear, Runtime, StepContext
from .registry import POSITIONS, lookup, register_mixer

PROMPT_FORM_MIN_TOKENS = 32      # whole prompts of at least this many tokens take the expanded form

_NAMES = dict(q="q_proj.weight", down="kv_down_proj.weight", latent_norm="kv_norm.weight", up_k="k_up_proj.weight",
              up_v="v_up_proj.weight", out="o_proj.weight", q_down="q_down_proj.weight", q_latent_norm="q_norm.weight",
              sink="sink")


def _names(spec: PartSpec) -> Dict[str, str]:
    n = dict(_NAMES)
    n.update(spec.get("names") or {})
    return n


@register_mixer("latent_attention")
class LatentAttentionMixer:
    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        W, H = spec["hidden_size"], spec["num_heads"]
        d, r, dv, R = spec["nope_dim"], spec["rope_dim"], spec["value_dim"], spec["latent_dim"]
        n = _names(spec)
        Rq = int(spec.get("q_latent_dim") or 0)
        extra = {}
        if Rq:
            extra[n["q_down"]] = TensorDecl(shape=(Rq, W))
            extra[n["q_latent_norm"]] = TensorDecl(shape=(Rq,), init="ones_normal")
        if spec.get("sink"):
            extra[n["sink"]] = TensorDecl(shape=(H,), init="small_normal")
        return {
            **extra,
            n["q"]: TensorDecl(shape=(H * (d + r), Rq or W)),
            n["down"]: TensorDecl(shape=(R + r, W)),
            n["latent_norm"]: TensorDecl(shape=(R,), init="ones_normal"),
            n["up_k"]: TensorDecl(shape=(H * d, R)),
            n["up_v"]: TensorDecl(shape=(H * dv, R)),
            n["out"]: TensorDecl(shape=(W, H * dv)),
        }

    @classmethod
    def cache_request(cls, spec: PartSpec) -> LatentRequest:
        return LatentRequest(width=int(spec["latent_dim"]) + int(spec["rope_dim"]), window=spec.get("window"))

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.rt = rt
        self.hidden, self.H = int(spec["hidden_size"]), int(spec["num_heads"])
        self.d, self.r = int(spec["nope_dim"]), int(spec["rope_dim"])
        self.dv, self.R = int(spec["value_dim"]), int(spec["latent_dim"])
        self.scale = float(spec["scale"])
        self.window = int(spec.get("window") or 0)
        self.eps = float(spec["latent_norm_eps"])
        self.position = None
        self.rot = 0
        if self.r > 0:
            pos = dict(spec["position"])
            self.position = lookup(POSITIONS, pos["kind"], "position encoding")(pos, rt)
            if getattr(self.position, "pairing", None) != "adjacent":
                raise ValueError("latent attention rotates adjacent pairs; its position encoding must be of that kind")
            self.rot = int(pos.get("rotary_dim", self.r))
            if self.rot > self.r or self.rot % 2:
                raise ValueError(f"latent attention: rotary_dim={self.rot} must be even and at most rope_dim={self.r}")
        n = _names(spec)
        H, d, r, dv, R = self.H, self.d, self.r, self.dv, self.R
        self.Rq = int(spec.get("q_latent_dim") or 0)
        # with a query latent the first product makes [query latent | latent | key part] and the queries follow
        # from the normed query latent by a product of their own
        wq = rt.matrix(weights[n["q_down"] if self.Rq else n["q"]])
        wdown = rt.matrix(weights[n["down"]])
        if wq.dtype != wdown.dtype:
            wq, wdown = wq.float(), wdown.float()
        # one product for the queries and the down projection: rows [all q heads | latent | shared key part]
        self.q_down = Linear(torch.cat([wq, wdown], dim=0), rt)
        self.nq = self.Rq or H * (d + r)
        self.q_up = Linear(weights[n["q"]], rt) if self.Rq else None
        self.q_latent_norm = rt.vector(weights[n["q_latent_norm"]]) if self.Rq else None
        self.sink = rt.vector(weights[n["sink"]]) if spec.get("sink") else None
        self.latent_norm = rt.vector(weights[n["latent_norm"]])
        # per head: Wuk_h^T as [latent_dim, nope_dim] (the absorbed query is Wuk_h^T q_plain), Wuv_h as stored
        self.uk_t = rt.matrix(weights[n["up_k"]]).view(H, d, R).transpose(1, 2).contiguous()
        self.uv = rt.matrix(weights[n["up_v"]]).view(H, dv, R).contiguous()
        self.o = Linear(weights[n["out"]], rt)
        self.out_scale = 1.0
        self._fast = None
        self.kv_up = None
        if rt.fast and rt.dtype == torch.bfloat16 and self.uk_t.dtype == torch.bfloat16:
            from ..csrc import fast_latent
            self._fast = fast_latent.try_make(H, d, R, r, H * (d + r) if self.Rq else self.nq + R + r, self.scale,
                                              self.window, self.sink)
            # whole prompts: keys and values of all heads by one product, attention in the expanded form
            if (self._fast is not None and fast_latent.prompt_takes(d, r, dv) and R % 8 == 0 and (H * d) % 8 == 0
                    and (H * dv) % 8 == 0):
                kv_up = Linear(torch.cat([rt.matrix(weights[n["up_k"]]), rt.matrix(weights[n["up_v"]])], dim=0), rt)
                self.kv_up = kv_up if kv_up.tensor_core else None

    def scale_output(self, mult: float) -> bool:
        """Multiply what this part adds to the residual by `mult`: the factor goes onto the heads' outputs in
        float32 before they are rounded for the output projection (which is linear)."""
        self.out_scale = float(mult)
        return True

    def prepare(self, ctx: StepContext) -> None:
        if self.position is not None:
            self.position.tables(ctx)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache: LatentView,
                writes_cache: bool = True) -> None:
        T, H, d, r, dv, R = ctx.n_tokens, self.H, self.d, self.r, self.dv, self.R
        dt = self.rt.dtype
        # the tensor-core kernel takes bfloat16 queries; the plain kernels keep the absorbed query and the
        # latent output in float32 whatever the compute dtype
        mid = torch.bfloat16 if self._fast is not None else torch.float32
        width = self.nq + R + r
        qd = ctx.ws.get("lat_q_down", (T, width), dt)
        self.q_down(h, qd, ws=ctx.ws)
        dkv = qd[:, self.nq:]
        if self.Rq:
            # queries through their own latent: norm of the first Rq columns, then the up projection
            cq = ctx.ws.get("lat_q_latent", (T, self.Rq), dt)
            K.rmsnorm_rows(qd[:, :self.Rq], self.q_latent_norm, self.eps, cq, T)
            qd = ctx.ws.get("lat_q_heads", (T, H * (d + r)), dt)
            self.q_up(cq, qd, ws=ctx.ws)
            width = H * (d + r)
        qh = qd[:, :H * (d + r)]
        qcat = ctx.ws.get("lat_qcat", (T, H, R + r), mid)
        cos, sin = self.position.tables(ctx) if self.position is not None else (None, None)
        table = ctx.page_tables[cache.group]
        av = ctx.ws.get("lat_values", (T, H * dv), dt)
        if self.kv_up is not None and ctx.fresh and ctx.max_new >= PROMPT_FORM_MIN_TOKENS:
            # every sequence starts at position 0: what a token reads is among the step's own tokens
            from ..csrc import fast_latent
            ckr = ctx.ws.get("lat_rows_dense", (T, R + r), dt)
            K.latent_prep(qh, dkv, self.latent_norm, self.eps, cos, sin, self.rot,
                          ctx.positions, ctx.seq_of_token, table, cache.page_size,
                          cache.pool if writes_cache else None, qcat, T, H, d, r, R, dense=ckr)
            kv = ctx.ws.get("lat_keys_values", (T, H * (d + dv)), dt)
            self.kv_up(ckr[:, :R], kv, ws=ctx.ws)
            fast_latent.latent_prompt_mma(qd, qcat, kv, ckr, av, ctx.cu_seqlens, ctx.seq_of_token, ctx.n_seqs, T, H, d, r,
                                          dv, R, self.scale, self.window, self.out_scale, self.sink)
            self.o(av, residual, accumulate=True, ws=ctx.ws)
            return
        K.latent_prep(qh, dkv, self.latent_norm, self.eps, cos, sin, self.rot,
                      ctx.positions, ctx.seq_of_token, table, cache.page_size, cache.pool if writes_cache else None,
                      qcat, T, H, d, r, R)
        if self._fast is not None:
            self._fast.absorb(qd, width, d + r, self.uk_t, qcat, T)
        else:
            K.headwise_gemm(qd, width, d + r, self.uk_t, qcat, H * (R + r), R + r, T)
        olat = ctx.ws.get("lat_out", (T, H, R), mid)
        if self._fast is not None:
            self._fast.attention(qcat, cache.pool, olat, ctx, table, cache.page_size)
        else:
            K.latent_attention_plain(qcat, cache.pool, olat, ctx.positions, ctx.seq_of_token, table,
                                     cache.page_size, T, H, R, r, self.scale, self.window, self.sink)
        if self._fast is not None:
            self._fast.expand(olat, self.uv, av, T, self.out_scale)
        else:
            K.headwise_gemm(olat, H * R, R, self.uv, av, H * dv, dv, T, alpha=self.out_scale)
        self.o(av, residual, accumulate=True, ws=ctx.ws)
