"""Mixers whose state is carried by a gated linear recurrence behind a short convolution of a projection.

`rglru` (the recurrent block with a real-gated linear recurrent unit; state: a vector [width]):
    y = gelu_tanh(W_y h + b_y);   u = conv(W_x h + b_x)                 conv: per channel over time, with a bias
    u in `blocks` equal runs n:   r = sigmoid(A_n u_n + a_n),  i = sigmoid(I_n u_n + i_n)         A_n, I_n square
    log a = -c r softplus(lam)  (c = decay_scale),   S_t = a S_(t-1) + sqrt(1 - a^2) i u,   out = W_o (S_t * y)

`mamba2` (a selective state space with one decay per head and token; state: a matrix [state, vdim] per head):
    W_in h = [z: inner | x: inner | B: groups x state | C: groups x state | dt: heads],  inner = heads x vdim
    (x, B, C) <- silu(conv([x, B, C]));   dt <- softplus(dt + dt_bias)
    S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T,   y_t = S_t^T C_t + D_h x_t      head h reads group h / (heads / groups)
    out = W_o ( groupnorm(y * silu(z); norm_groups runs) * w )                           the gate comes before the norm

conv(v)_t = bias + sum_j c[:, j] v_(t - taps + 1 + j) inside a sequence (the last tap meets the token itself, zeros
before the start).  What a layer keeps per sequence is the convolution's last taps - 1 inputs and S (two
`StateRequest`s: the part's cache request is the pair), so prompts may come in portions and decoding goes on from
them.  The projections of h run as one product on the compute dtype's rows and matrices and leave their float32
sums unrounded; the convolution's sums, the gates, decays, step sizes, the state, the outputs' norm and gate are
float32 in both compute paths.

Spec parameters: hidden_size, taps, names; `rglru`: width, blocks, decay_scale (8 unless given); `mamba2`:
num_heads, value_dim, state_dim, groups, norm_groups, eps.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.sequence_cache import StateRequest
from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..weights.loader import TensorDecl
from .base import Linear, Runtime, StepContext
from .registry import register_mixer


CHUNKED_FROM = 128      # new tokens of one sequence from which a step takes the recurrences' chunked forms
SCAN_CHUNK = 64         # rows per chunk of the matrix-state recurrence's chunked form


def _states(cache, what: str):
    if not isinstance(cache, tuple) or len(cache) != 2:
        raise ValueError(f"{what}: the convolution's state and the recurrence's state are expected")
    return cache


@register_mixer("rglru")
class RGLRUMixer:
    @classmethod
    def _names(cls, spec: PartSpec) -> Dict[str, str]:
        n = dict(y="y", y_bias="y.b", x="x", x_bias="x.b", conv="conv", conv_bias="conv.b", gate_a="ra", gate_a_bias="ra.b",
                 gate_i="ri", gate_i_bias="ri.b", decay="lam", o="o")
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        W, C, nb, taps = int(spec["hidden_size"]), int(spec["width"]), int(spec["blocks"]), int(spec["taps"])
        if nb < 1 or C % nb:
            raise ValueError(f"rglru: a width of {C} does not form {nb} equal runs")
        bw = C // nb
        n = cls._names(spec)
        return {n["y"]: TensorDecl(shape=(C, W)), n["y_bias"]: TensorDecl(shape=(C,), init="zeros_normal"),
                n["x"]: TensorDecl(shape=(C, W)), n["x_bias"]: TensorDecl(shape=(C,), init="zeros_normal"),
                n["conv"]: TensorDecl(shape=(C, taps), init="small_normal"),
                n["conv_bias"]: TensorDecl(shape=(C,), init="zeros_normal"),
                n["gate_a"]: TensorDecl(shape=(nb, bw, bw)), n["gate_a_bias"]: TensorDecl(shape=(nb, bw), init="zeros_normal"),
                n["gate_i"]: TensorDecl(shape=(nb, bw, bw)), n["gate_i_bias"]: TensorDecl(shape=(nb, bw), init="zeros_normal"),
                n["decay"]: TensorDecl(shape=(C,), init="small_normal"), n["o"]: TensorDecl(shape=(W, C))}

    @classmethod
    def cache_request(cls, spec: PartSpec):
        C, taps = int(spec["width"]), int(spec["taps"])
        tail = StateRequest(shape=(taps - 1, C), dtype=torch.float32) if taps > 1 else None
        return (tail, StateRequest(shape=(C,), dtype=torch.float32))

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.rt = rt
        self.hidden, self.C, self.taps = int(spec["hidden_size"]), int(spec["width"]), int(spec["taps"])
        if self.taps < 1:
            raise ValueError("rglru: taps must be at least 1")
        n = self._names(spec)
        y, x = rt.matrix(weights[n["y"]]), rt.matrix(weights[n["x"]])
        if y.dtype != x.dtype:
            y, x = y.float(), x.float()
        self.proj = Linear(torch.cat([y, x], dim=0), rt)           # rows: the y branch, then the x branch
        self.y_bias, self.x_bias = rt.vector(weights[n["y_bias"]]), rt.vector(weights[n["x_bias"]])
        self.conv = rt.vector(weights[n["conv"]]).t().contiguous()  # [taps, C]: a tap's weights side by side
        self.conv_bias = rt.vector(weights[n["conv_bias"]])
        # the gates' square blocks, transposed to [block, in, out]; kept in float32: they make the recurrence's gates
        self.wa = rt.vector(weights[n["gate_a"]]).transpose(1, 2).contiguous()
        self.wi = rt.vector(weights[n["gate_i"]]).transpose(1, 2).contiguous()
        self.ba = rt.vector(weights[n["gate_a_bias"]]).reshape(-1).contiguous()
        self.bi = rt.vector(weights[n["gate_i_bias"]]).reshape(-1).contiguous()
        lam = rt.vector(weights[n["decay"]])
        self.c = (-float(spec.get("decay_scale", 8.0)) * torch.nn.functional.softplus(lam)).contiguous()
        self.o = Linear(weights[n["o"]], rt)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache, writes_cache: bool = True) -> None:
        if not writes_cache:
            raise ValueError("rglru: a layer's state cannot be read by another layer")
        tail, st = _states(cache, "rglru")
        T, C = ctx.n_tokens, self.C
        # (the projection's sums leave the product in float32: what enters the recurrence is not rounded on the way)
        p = ctx.ws.get("rglru_proj", (T, 2 * C), torch.float32)
        self.proj(h, p, ws=ctx.ws)
        u = ctx.ws.get("rglru_u", (T, C), torch.float32)
        K.column_conv(p[:, C:], u, self.conv, self.conv_bias, self.x_bias, tail.state if tail is not None else None,
                      ctx.cu_seqlens, ctx.slots, ctx.seq_of_token, T, ctx.n_seqs, act=0, max_new=int(ctx.max_new))
        a = ctx.ws.get("rglru_a", (T, C), torch.float32)
        b = ctx.ws.get("rglru_b", (T, C), torch.float32)
        K.rglru_gates(u, self.wa, self.wi, self.ba, self.bi, self.c, a, b, ctx.seq_of_token, T)
        out = ctx.ws.get("rglru_out", (T, C), self.rt.dtype)
        if ctx.max_new >= CHUNKED_FROM:
            # prompts: chunks of rows over many threads (the same sums in another bracketing)
            sums = ctx.ws.get("rglru_chunk_sums", (K.diag_scan_chunks_scratch(T, ctx.n_seqs, C),), torch.float32)
            K.diag_scan_chunks(a, b, p[:, :C], self.y_bias, out, sums, st.state, ctx.cu_seqlens, ctx.slots, ctx.seq_of_token,
                               T, ctx.n_seqs)
        else:
            K.diag_scan(a, b, p[:, :C], self.y_bias, out, st.state, ctx.cu_seqlens, ctx.slots, ctx.seq_of_token, T, ctx.n_seqs)
        self.o(out, residual, accumulate=True, ws=ctx.ws)


@register_mixer("mamba2")
class Mamba2Mixer:
    @classmethod
    def _names(cls, spec: PartSpec) -> Dict[str, str]:
        n = dict(in_proj="in", conv="conv", conv_bias="conv.b", dt_bias="dt_bias", a_log="A_log", skip="D", norm="norm", o="o")
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def _sizes(cls, spec: PartSpec):
        W, H, P, N, G = (int(spec[k]) for k in ("hidden_size", "num_heads", "value_dim", "state_dim", "groups"))
        if G < 1 or H % G:
            raise ValueError(f"mamba2: {H} heads do not form {G} equal groups")
        return W, H, P, N, G

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        W, H, P, N, G = cls._sizes(spec)
        inner, conv = H * P, H * P + 2 * G * N
        n = cls._names(spec)
        return {n["in_proj"]: TensorDecl(shape=(2 * inner + 2 * G * N + H, W)),
                n["conv"]: TensorDecl(shape=(conv, int(spec["taps"])), init="small_normal"),
                n["conv_bias"]: TensorDecl(shape=(conv,), init="zeros_normal"),
                n["dt_bias"]: TensorDecl(shape=(H,), init="small_normal"), n["a_log"]: TensorDecl(shape=(H,), init="small_normal"),
                n["skip"]: TensorDecl(shape=(H,), init="ones_normal"), n["norm"]: TensorDecl(shape=(inner,), init="ones_normal"),
                n["o"]: TensorDecl(shape=(W, inner))}

    @classmethod
    def cache_request(cls, spec: PartSpec):
        _, H, P, N, G = cls._sizes(spec)
        taps = int(spec["taps"])
        tail = StateRequest(shape=(taps - 1, H * P + 2 * G * N), dtype=torch.float32) if taps > 1 else None
        return (tail, StateRequest(shape=(H, N, P), dtype=torch.float32))

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.rt = rt
        self.hidden, self.H, self.P, self.N, self.G = self._sizes(spec)
        self.inner = self.H * self.P
        self.conv_ch = self.inner + 2 * self.G * self.N
        self.taps = int(spec["taps"])
        self.norm_groups = int(spec.get("norm_groups", 1))
        if self.norm_groups < 1 or self.inner % self.norm_groups:
            raise ValueError(f"mamba2: {self.inner} outputs do not form {self.norm_groups} equal runs")
        self.eps = float(spec["eps"])
        n = self._names(spec)
        self.proj = Linear(weights[n["in_proj"]], rt)               # rows: z, x, B, C, dt
        self.conv = rt.vector(weights[n["conv"]]).t().contiguous()  # [taps, channels]
        self.conv_bias = rt.vector(weights[n["conv_bias"]])
        self.dt_bias = rt.vector(weights[n["dt_bias"]])
        self.neg_a = (-torch.exp(rt.vector(weights[n["a_log"]]))).contiguous()
        self.skip = rt.vector(weights[n["skip"]])
        self.norm_weight = rt.vector(weights[n["norm"]])
        self.o = Linear(weights[n["o"]], rt)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache, writes_cache: bool = True) -> None:
        if not writes_cache:
            raise ValueError("mamba2: a layer's state cannot be read by another layer")
        tail, st = _states(cache, "mamba2")
        T, H, P, N, G, inner = ctx.n_tokens, self.H, self.P, self.N, self.G, self.inner
        p = ctx.ws.get("mamba2_proj", (T, self.proj.out_features), torch.float32)
        self.proj(h, p, ws=ctx.ws)
        xc = ctx.ws.get("mamba2_conv", (T, self.conv_ch), torch.float32)
        K.column_conv(p[:, inner:inner + self.conv_ch], xc, self.conv, self.conv_bias, None,
                      tail.state if tail is not None else None, ctx.cu_seqlens, ctx.slots, ctx.seq_of_token, T, ctx.n_seqs,
                      act=1, max_new=int(ctx.max_new))
        raw = ctx.ws.get("mamba2_raw", (T, inner), torch.float32)
        chunk, scratch = 0, None
        if ctx.max_new >= CHUNKED_FROM:
            # prompts: chunks of rows over many CTAs (the same sums in another bracketing)
            chunk = SCAN_CHUNK
            scratch = ctx.ws.get("mamba2_chunk_states", (K.stepsize_scan_scratch(T, ctx.n_seqs, H, N, P, chunk),), torch.float32)
        K.stepsize_scan(xc, inner, inner + G * N, p, inner + self.conv_ch, raw, st.state, ctx.cu_seqlens, ctx.slots,
                        ctx.seq_of_token, self.dt_bias, self.neg_a, T, ctx.n_seqs, H, G, N, P, chunk=chunk, scratch=scratch)
        y = ctx.ws.get("mamba2_out", (T, inner), self.rt.dtype)
        K.stepsize_finish(raw, xc, p, 0, self.skip, self.norm_weight, y, ctx.seq_of_token, T, H, P, self.norm_groups, self.eps)
        self.o(y, residual, accumulate=True, ws=ctx.ws)
