"""Python face of the CUDA kernels: one thin function per launcher.

Arguments are torch tensors on the GPU; every function launches on torch's current stream and
allocates nothing (outputs and scratch are passed in).  There is no CPU or library fallback: a
tensor that is not on a CUDA device, or a missing compiler, raises.
"""
from __future__ import annotations

from typing import Optional

import torch

from .build import KernelError, kernel

F32, BF16 = 0, 1


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dt}")


def _p(t: Optional[torch.Tensor]) -> int:
    if t is None:
        return 0
    if not t.is_cuda:
        raise KernelError("kernel argument is not on a CUDA device (there is no CPU path)")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, dt: torch.dtype, what: str) -> None:
    if t.dtype != dt:
        raise KernelError(f"{what} must be {dt}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


# ------------------------------------------------------------------------------- elementwise
def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t, :] (float32) = table[tokens[t], :] * scale; negative ids give zero rows."""
    _need(tokens, torch.int32, "tokens")
    _need(out, torch.float32, "out")
    V, H = table.shape
    kernel("elementwise", "gg_embed_gather")(_p(table), dtype_code(table.dtype), _p(tokens), _p(out),
                                              tokens.numel(), H, V, float(scale), _stream())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, groups: int = 1) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight; x float32, weight float32, out float32/bfloat16.  groups > 1:
    the row is cut into that many equal runs, each divided by its own root mean square."""
    _need(x, torch.float32, "x")
    _need(weight, torch.float32, "norm weight")
    H = x.shape[-1]
    R = rows.numel() if rows is not None else x.numel() // H
    if rows is not None:
        _need(rows, torch.int32, "rows")
    if weight.numel() != H or out.shape[-1] != H or out.numel() < R * H:
        raise KernelError("rmsnorm: shapes disagree")
    if groups > 1:
        if H % groups:
            raise KernelError(f"rmsnorm: {H} columns do not form {groups} equal runs")
        kernel("elementwise", "gg_group_rmsnorm")(_p(x), _p(rows), _p(weight), _p(out), dtype_code(out.dtype), R, H,
                                                   int(groups), float(eps), _stream())
        return
    kernel("elementwise", "gg_rmsnorm")(_p(x), _p(rows), _p(weight), _p(out), dtype_code(out.dtype),
                                         R, H, float(eps), _stream())


def row_stats(x: torch.Tensor, xhat: torch.Tensor, ssq: torch.Tensor) -> None:
    """xhat = bfloat16(x) and ssq[t, p] = sum of x[t, 128 p : 128 p + 128]^2 for float32 rows x [T, H]."""
    _need(x, torch.float32, "x")
    _need(xhat, torch.bfloat16, "xhat")
    _need(ssq, torch.float32, "ssq")
    H = x.shape[-1]
    T = x.numel() // H
    if xhat.numel() != T * H or ssq.numel() != T * ((H + 127) // 128):
        raise KernelError("row_stats: shapes disagree")
    kernel("elementwise", "gg_row_stats")(_p(x), _p(xhat), _p(ssq), T, H, _stream())


def rope_tables(positions: torch.Tensor, inv_freq: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                mag: float = 1.0) -> None:
    """cos, sin [T, half] (float32) = mag * cos / sin of positions[t] * inv_freq[i], angles in float64."""
    _need(positions, torch.int32, "positions")
    _need(inv_freq, torch.float64, "inv_freq")
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    T, half = positions.numel(), inv_freq.numel()
    kernel("elementwise", "gg_rope_tables")(_p(positions), _p(inv_freq), _p(cos), _p(sin), T, half, float(mag), _stream())


def qk_norm_rope_cache(qkv: torch.Tensor, q_out: torch.Tensor, q_weight: Optional[torch.Tensor],
                       k_weight: Optional[torch.Tensor], eps: float, cos: torch.Tensor, sin: torch.Tensor,
                       positions: torch.Tensor, seq_of_token: torch.Tensor, page_table: torch.Tensor,
                       page_size: int, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                       n_tokens: int, nq: int, nkv: int, d: int, rot: int) -> None:
    if q_out.dtype != qkv.dtype or (k_pool is not None and k_pool.dtype != qkv.dtype):
        raise KernelError("qk_norm_rope_cache: qkv, q_out and the cache must share one dtype")
    from .tcgen05_gemm import status_word
    kernel("elementwise", "gg_qk_norm_rope_cache")(
        _p(qkv), dtype_code(qkv.dtype), _p(q_out), _p(q_weight), _p(k_weight), float(eps), _p(cos), _p(sin),
        _p(positions), _p(seq_of_token), _p(page_table), page_table.shape[-1], page_size,
        k_pool.shape[0] if k_pool is not None else 0, _p(k_pool), _p(v_pool),
        n_tokens, nq, nkv, d, rot, _p(status_word(qkv.device)), _stream())


def qkv_prep(qkv: torch.Tensor, q_out: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
             eps: float, norm_mode: int, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor,
             seq_of_token: torch.Tensor, page_table: torch.Tensor, page_size: int, k_pool: Optional[torch.Tensor],
             v_pool: Optional[torch.Tensor], n_tokens: int, nq: int, nkv: int, d: int, dv: int, rot: int) -> None:
    """The general q/k/v preparation: qkv [T, nq*d + nkv*d + nkv*dv]; norm_mode 0 none, 1 per head (weights of
    size d), 2 over the whole q and the whole k projection (weights of size nq*d and nkv*d); rotation of the first
    `rot` elements of each q and k head; q to q_out, k and v into the paged pools (head sizes d and dv)."""
    if q_out.dtype != qkv.dtype or (k_pool is not None and (k_pool.dtype != qkv.dtype or v_pool.dtype != qkv.dtype)):
        raise KernelError("qkv_prep: qkv, q_out and the cache must share one dtype")
    if not qkv.is_contiguous() or qkv.shape[-1] != (nq + nkv) * d + nkv * dv:
        raise KernelError("qkv_prep: qkv must be contiguous [T, nq*d + nkv*d + nkv*dv]")
    if norm_mode:
        want = (d, d) if norm_mode == 1 else (nq * d, nkv * d)
        _need(q_weight, torch.float32, "q norm weight")
        _need(k_weight, torch.float32, "k norm weight")
        if (q_weight.numel(), k_weight.numel()) != want:
            raise KernelError(f"qkv_prep: norm weights of {q_weight.numel()} and {k_weight.numel()} elements, "
                              f"{want[0]} and {want[1]} expected")
    from .tcgen05_gemm import status_word
    kernel("elementwise", "gg_qkv_prep")(
        _p(qkv), dtype_code(qkv.dtype), _p(q_out), _p(q_weight), _p(k_weight), float(eps), int(norm_mode), _p(cos),
        _p(sin), _p(positions), _p(seq_of_token), _p(page_table), page_table.shape[-1], page_size,
        k_pool.shape[0] if k_pool is not None else 0, _p(k_pool), _p(v_pool),
        n_tokens, nq, nkv, d, dv, rot, _p(status_word(qkv.device)), _stream())


def rmsnorm_add(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float,
                xhat: Optional[torch.Tensor] = None, ssq: Optional[torch.Tensor] = None, zero_y: bool = False,
                gate: Optional[torch.Tensor] = None, gate_bias: Optional[torch.Tensor] = None, groups: int = 1) -> None:
    """x[r] += y[r] / sqrt(mean(y[r]^2) + eps) * weight, all float32.  With `gate` (float32 like y) and `gate_bias`
    (float32 [H], optional) y is first multiplied by sigmoid(gate + gate_bias), and the norm is the product's.  With `xhat` (bfloat16 like x) and `ssq`
    (float32 [rows, ceil(H / 128)]) the updated rows' bfloat16 copy and sums of squares per 128 columns are left too
    (what `row_stats` makes).  zero_y: y is left zeroed."""
    _need(x, torch.float32, "x")
    _need(y, torch.float32, "y")
    _need(weight, torch.float32, "norm weight")
    H = x.shape[-1]
    if y.shape != x.shape or weight.numel() != H:
        raise KernelError("rmsnorm_add: shapes disagree")
    if groups > 1:
        # the norm in `groups` equal runs of the row, each over its own root mean square (no gate, no statistics)
        if xhat is not None or gate is not None or H % groups:
            raise KernelError("rmsnorm_add: the grouped form takes no gate and leaves no statistics; the runs are equal")
        kernel("elementwise", "gg_group_rmsnorm_add")(_p(x), _p(y), _p(weight), x.numel() // H, H, int(groups), float(eps),
                                                       int(zero_y), _stream())
        return
    if (xhat is None) != (ssq is None):
        raise KernelError("rmsnorm_add: xhat and ssq come together")
    if xhat is not None:
        _need(xhat, torch.bfloat16, "xhat")
        _need(ssq, torch.float32, "ssq")
        if xhat.numel() != x.numel() or ssq.numel() != (x.numel() // H) * ((H + 127) // 128):
            raise KernelError("rmsnorm_add: shapes of xhat / ssq disagree")
    if gate is not None:
        _need(gate, torch.float32, "gate")
        if gate.shape != y.shape:
            raise KernelError("rmsnorm_add: the gate has the shape of y")
        if gate_bias is not None:
            _need(gate_bias, torch.float32, "gate bias")
            if gate_bias.numel() != H:
                raise KernelError("rmsnorm_add: the gate's bias has one number per column")
    elif gate_bias is not None:
        raise KernelError("rmsnorm_add: a gate bias without a gate")
    kernel("elementwise", "gg_rmsnorm_add")(_p(x), _p(y), _p(weight), x.numel() // H, H, float(eps), _p(xhat), _p(ssq),
                                             int(zero_y), _p(gate), _p(gate_bias), _stream())


def short_conv(h: torch.Tensor, out: torch.Tensor, weight: torch.Tensor, state: Optional[torch.Tensor],
               cu_seqlens: torch.Tensor, slots: torch.Tensor, seq_of_token: torch.Tensor, n_tokens: int, n_seqs: int,
               keep: float = 1.0, max_new: int = 0) -> None:
    """out[t] = keep * h[t] + sum_j weight[j] * h[t - taps + 1 + j] per channel inside each sequence (weight is
    [taps, W]: a tap's weights side by side, the last tap meets the token itself); rows before
    the step come from state [slots, taps - 1, W] (float32), which is then moved on to the step's last rows.
    max_new: the most tokens one sequence brings, where the caller knows it (1: a single launch does both)."""
    taps, W = weight.shape
    if not weight.is_contiguous():
        raise KernelError("short_conv: the taps are a contiguous [taps, W]")
    if h.dtype != out.dtype or not h.is_contiguous() or not out.is_contiguous() or h.shape[-1] != W:
        raise KernelError("short_conv: h and out are contiguous [T, W] of one dtype")
    if h.data_ptr() == out.data_ptr():
        raise KernelError("short_conv: out may not be h")
    _need(weight, torch.float32, "taps")
    if taps > 1:
        _need(state, torch.float32, "state")
        if tuple(state.shape[1:]) != (taps - 1, W):
            raise KernelError("short_conv: the state is [slots, taps - 1, W]")
    kernel("elementwise", "gg_short_conv")(_p(h), _p(out), dtype_code(h.dtype), _p(weight), _p(state), _p(cu_seqlens),
                                            _p(slots), _p(seq_of_token), int(n_tokens), int(n_seqs), W, taps, float(keep),
                                            int(max_new), _stream())


def token_shift(x: torch.Tensor, out: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor,
                slots: torch.Tensor, seq_of_token: torch.Tensor, n_tokens: int, n_seqs: int, max_new: int = 0) -> None:
    """out[t] = x[t] + (x[t - 1] - x[t]) * mu inside each sequence (x float32, out the compute dtype); the row before
    a sequence's first row of the step is state[slot] (float32 [slots, W]), which is then moved on to the step's last
    row.  max_new: the most tokens one sequence brings, where the caller knows it (1: a single launch does both)."""
    _need(x, torch.float32, "x")
    _need(mu, torch.float32, "mu")
    _need(state, torch.float32, "state")
    W = x.shape[-1]
    if mu.numel() != W or state.shape[-1] != W or not out.is_contiguous() or out.shape[-1] != W:
        raise KernelError("token_shift: shapes disagree")
    kernel("elementwise", "gg_token_shift")(_p(x), _p(out), dtype_code(out.dtype), _p(mu), _p(state), _p(cu_seqlens),
                                             _p(slots), _p(seq_of_token), int(n_tokens), int(n_seqs), W, int(max_new),
                                             _stream())


def depth_mix(hist: torch.Tensor, x: torch.Tensor, coeff: Optional[torch.Tensor], store_at: int, n_terms: int) -> None:
    """hist[store_at] = x; then, with n_terms > 0, x = sum_{j < n_terms} coeff[j] * hist[j] (all float32; hist is
    [depth, *x.shape])."""
    _need(hist, torch.float32, "hist")
    _need(x, torch.float32, "x")
    n = x.numel()
    if hist.numel() < (max(store_at, n_terms - 1) + 1) * n:
        raise KernelError("depth_mix: the history is too small")
    if n_terms > 0:
        _need(coeff, torch.float32, "coeff")
        if coeff.numel() < n_terms:
            raise KernelError("depth_mix: a coefficient per term")
    kernel("elementwise", "gg_depth_mix")(_p(hist), _p(x), _p(coeff), int(store_at), int(n_terms), n, _stream())


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x (float32) in the dtype of out."""
    _need(x, torch.float32, "x")
    if out.numel() != x.numel() or not out.is_contiguous():
        raise KernelError("cast_rows: shapes disagree")
    kernel("elementwise", "gg_cast_rows")(_p(x), _p(out), dtype_code(out.dtype), x.numel(), _stream())


def gelu(z: torch.Tensor, out: torch.Tensor, tanh_form: bool = False) -> None:
    """out = gelu(z), the exact (erf) form or the tanh form; float32 arithmetic; out may be z."""
    if z.dtype != out.dtype or z.numel() != out.numel() or not z.is_contiguous() or not out.is_contiguous():
        raise KernelError("gelu: input and output must be contiguous and alike")
    kernel("elementwise", "gg_gelu")(_p(z), _p(out), dtype_code(z.dtype), int(tanh_form), z.numel(), _stream())


def row_gate(act: torch.Tensor, h: torch.Tensor, g: torch.Tensor, seq_of_token: Optional[torch.Tensor], n_tokens: int) -> None:
    """act[t] *= sigmoid(g . h[t]) for every token: one gate per row from the row's input h and a stored vector g."""
    _need(g, torch.float32, "gate vector")
    if act.dtype != h.dtype or not act.is_contiguous() or not h.is_contiguous() or g.numel() != h.shape[-1]:
        raise KernelError("row_gate: shapes disagree")
    kernel("elementwise", "gg_row_gate")(_p(act), act.shape[-1], _p(h), h.shape[-1], dtype_code(act.dtype), _p(g),
                                          _p(seq_of_token), int(n_tokens), _stream())


def column_conv(h: torch.Tensor, out: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                in_bias: Optional[torch.Tensor], state: Optional[torch.Tensor], cu_seqlens: torch.Tensor,
                slots: torch.Tensor, seq_of_token: torch.Tensor, n_tokens: int, n_seqs: int, act: int = 0,
                max_new: int = 0) -> None:
    """out[t] = act(bias + sum_j weight[j] * v[t - taps + 1 + j]) per channel inside each sequence, v = h + in_bias;
    h [T, C] may be a column range of a wider buffer (compute dtype), out [T, C] is float32 (likewise), weight is
    [taps, C] float32; rows before the step come from state [slots, taps - 1, C] (float32), which is then moved on.
    act 0 none, 1 silu."""
    taps, C = weight.shape
    _need(weight, torch.float32, "taps")
    if out.dtype != torch.float32 or h.stride(-1) != 1 or out.stride(-1) != 1 or h.shape[-1] != C or out.shape[-1] != C:
        raise KernelError("column_conv: h [T, C] and out [T, C] (float32) have unit column stride")
    for t in (bias, in_bias):
        if t is not None:
            _need(t, torch.float32, "bias")
            if t.numel() != C:
                raise KernelError("column_conv: a bias per channel")
    if taps > 1:
        _need(state, torch.float32, "state")
        if tuple(state.shape[1:]) != (taps - 1, C):
            raise KernelError("column_conv: the state is [slots, taps - 1, C]")
    kernel("elementwise", "gg_column_conv")(_p(h), h.stride(0), dtype_code(h.dtype), _p(out), out.stride(0), _p(weight),
                                             _p(bias), _p(in_bias), _p(state), _p(cu_seqlens), _p(slots), _p(seq_of_token),
                                             int(n_tokens), int(n_seqs), C, taps, int(act), int(max_new), _stream())


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, rows: int) -> None:
    """out[t] = x[t] / rms(x[t]) * weight for rows that may be column ranges of wider buffers (same dtype)."""
    n = weight.numel()
    if x.dtype != out.dtype or x.stride(-1) != 1 or out.stride(-1) != 1 or x.shape[-1] != n or out.shape[-1] != n:
        raise KernelError("rmsnorm_rows: x and out are [T, n] views of one dtype with unit column stride")
    _need(weight, torch.float32, "norm weight")
    kernel("elementwise", "gg_rmsnorm_rows")(_p(x), x.stride(0), dtype_code(x.dtype), _p(weight), _p(out), out.stride(0),
                                              int(rows), n, float(eps), _stream())


def softcap(z: torch.Tensor, cap: float, n: Optional[int] = None) -> None:
    """z <- cap * tanh(z / cap) in place (float32)."""
    _need(z, torch.float32, "logits")
    kernel("elementwise", "gg_softcap")(_p(z), float(cap), int(z.numel() if n is None else n), _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, n_tokens: int, inter: int) -> None:
    if gate_up.dtype != out.dtype:
        raise KernelError("swiglu: input and output must share one dtype")
    kernel("elementwise", "gg_swiglu")(_p(gate_up), dtype_code(gate_up.dtype), _p(out), n_tokens, inter, _stream())


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    _need(x, torch.float32, "x")
    if delta.numel() != x.numel() or not delta.is_contiguous():
        raise KernelError("residual_add: shapes disagree")
    kernel("elementwise", "gg_residual_add")(_p(x), _p(delta), dtype_code(delta.dtype), x.numel(), _stream())


def residual_axpy(x: torch.Tensor, delta: torch.Tensor, alpha: float) -> None:
    """x (float32) += alpha * delta."""
    _need(x, torch.float32, "x")
    if delta.numel() != x.numel() or not delta.is_contiguous():
        raise KernelError("residual_axpy: shapes disagree")
    kernel("elementwise", "gg_residual_axpy")(_p(x), _p(delta), dtype_code(delta.dtype), float(alpha), x.numel(), _stream())


def xielu(z: torch.Tensor, out: torch.Tensor, ap: float, aq: float, out_scale: float = 1.0) -> None:
    """out = out_scale * (ap z^2 + z/2 where z > 0, aq (exp(z) - 1 - z) + z/2 elsewhere), float32 arithmetic."""
    if z.dtype != out.dtype or z.numel() != out.numel() or not z.is_contiguous() or not out.is_contiguous():
        raise KernelError("xielu: input and output must be contiguous and alike")
    kernel("elementwise", "gg_xielu")(_p(z), dtype_code(z.dtype), _p(out), float(ap), float(aq), float(out_scale),
                                       z.numel(), _stream())


def feed_tokens(tokens: torch.Tensor, src: torch.Tensor, sampled: torch.Tensor, n: int) -> None:
    """tokens[i] = sampled[src[i]] where src[i] >= 0 (all int32, on the device)."""
    _need(tokens, torch.int32, "tokens")
    _need(src, torch.int32, "src")
    _need(sampled, torch.int32, "sampled")
    kernel("elementwise", "gg_feed_tokens")(_p(tokens), _p(src), _p(sampled), n, _stream())


# ------------------------------------------------------------------------------- matrix product
def gemm_plain(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
               m: Optional[int] = None) -> None:
    """out[M, N] (+)= x[M, K] @ w[N, K]^T on the CUDA cores with float32 accumulation."""
    N, K = w.shape
    M = x.shape[0] if m is None else m
    if x.shape[-1] != K or out.shape[-1] != N:
        raise KernelError(f"gemm: x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    if x.stride(-1) != 1 or out.stride(-1) != 1 or not w.is_contiguous():
        raise KernelError("gemm: operands must be row-major")
    kernel("gemm_plain", "gg_gemm_plain")(_p(x), dtype_code(x.dtype), _p(w), dtype_code(w.dtype), _p(out),
                                           dtype_code(out.dtype), int(accumulate), M, N, K,
                                           x.stride(0), out.stride(0), _stream())


# ------------------------------------------------------------------------------- attention
def attention_plain(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                    positions: torch.Tensor, seq_of_token: torch.Tensor, page_table: torch.Tensor,
                    page_size: int, n_tokens: int, nq: int, nkv: int, d: int, scale: float, window: int,
                    dv: Optional[int] = None, sink: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> None:
    """Attention over the paged cache on the CUDA cores; `dv` is the values' head size (default d), `sink` one
    float32 per query head that joins the softmax's denominator, `out_scale` a factor on the result."""
    if not (q.dtype == k_pool.dtype == v_pool.dtype == out.dtype):
        raise KernelError("attention: q, cache and out must share one dtype")
    dv = d if dv is None else int(dv)
    if k_pool.shape[-1] != d or v_pool.shape[-1] != dv:
        raise KernelError("attention: the pools' head sizes disagree with d and dv")
    if sink is not None:
        _need(sink, torch.float32, "sink")
    from .tcgen05_gemm import status_word
    kernel("attention_plain", "gg_attention_plain")(
        _p(q), _p(k_pool), _p(v_pool), _p(out), dtype_code(q.dtype), _p(positions), _p(seq_of_token),
        _p(page_table), page_table.shape[-1], page_size, k_pool.shape[0], n_tokens, nq, nkv, d, dv, float(scale),
        int(window), _p(sink), float(out_scale), _p(status_word(q.device)), _stream())


def diff_qk_prep(qkv: torch.Tensor, q_out: torch.Tensor, q_weight: torch.Tensor, k_weight: Optional[torch.Tensor],
                 eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
                 seq_of_token: torch.Tensor, page_table: torch.Tensor, page_size: int, k_pool: Optional[torch.Tensor],
                 v_pool: Optional[torch.Tensor], n_tokens: int, heads: int, kv_heads: int, d: int, dv: int, rot: int) -> None:
    """Preparation for differential attention: qkv [T, heads*2*d (+ kv_heads*2*d + kv_heads*dv with pools)]; every
    (head, map) run of d is normed with a shared weight [d] and its first `rot` elements turned in adjacent pairs; q
    to q_out [T, heads, 2, d], k into k_pool [page][kv_head][page_size][2 d], v into v_pool [..][dv]."""
    if q_out.dtype != qkv.dtype or (k_pool is not None and (k_pool.dtype != qkv.dtype or v_pool.dtype != qkv.dtype)):
        raise KernelError("diff_qk_prep: qkv, q_out and the cache must share one dtype")
    want = heads * 2 * d + (kv_heads * (2 * d + dv) if k_pool is not None else 0)
    if qkv.stride(-1) != 1 or qkv.shape[-1] != want or not q_out.is_contiguous():
        raise KernelError("diff_qk_prep: the projection row's width does not fit the heads")
    _need(q_weight, torch.float32, "q norm weight")
    if k_pool is not None:
        _need(k_weight, torch.float32, "k norm weight")
        if k_pool.shape[-1] != 2 * d or v_pool.shape[-1] != dv or k_pool.shape[1] != kv_heads:
            raise KernelError("diff_qk_prep: the pools do not fit the heads")
    from .tcgen05_gemm import status_word
    kernel("diff_attention", "gg_diff_qk_prep")(
        _p(qkv), qkv.stride(0), dtype_code(qkv.dtype), _p(q_out), _p(q_weight), _p(k_weight), float(eps), _p(cos), _p(sin),
        _p(positions), _p(seq_of_token), _p(page_table), page_table.shape[-1], int(page_size),
        k_pool.shape[0] if k_pool is not None else 0, _p(k_pool), _p(v_pool), int(n_tokens), int(heads), int(kv_heads),
        int(d), int(dv), int(rot), _p(status_word(qkv.device)), _stream())


def diff_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                   seq_of_token: torch.Tensor, page_table: torch.Tensor, page_size: int, n_tokens: int, heads: int,
                   kv_heads: int, d: int, dv: int, scale: float, cap: float, window: int, lam: float, eps: float,
                   out_scale: float) -> None:
    """out[t, h] = out_scale * unit(a1 - lam * a2): two softmax attentions per head over the paged cache (keys
    [page][kv_head][page_size][2 d], both maps side by side; values [..][dv]), scores bounded by cap tanh(s / cap)
    where cap > 0, the difference divided by its root mean square (eps inside)."""
    if not (q.dtype == k_pool.dtype == v_pool.dtype == out.dtype):
        raise KernelError("diff_attention: q, cache and out must share one dtype")
    if k_pool.shape[-1] != 2 * d or v_pool.shape[-1] != dv or k_pool.shape[1] != kv_heads:
        raise KernelError("diff_attention: the pools do not fit the heads")
    from .tcgen05_gemm import status_word
    kernel("diff_attention", "gg_diff_attention")(
        _p(q), _p(k_pool), _p(v_pool), _p(out), dtype_code(q.dtype), _p(positions), _p(seq_of_token), _p(page_table),
        page_table.shape[-1], int(page_size), k_pool.shape[0], int(n_tokens), int(heads), int(kv_heads), int(d), int(dv),
        float(scale), float(cap), int(window), float(lam), float(eps), float(out_scale), _p(status_word(q.device)),
        _stream())


def diff_attention_mma_takes(heads: int, kv_heads: int, d: int, dv: int, page_size: int) -> bool:
    """Does the tensor-core form of differential attention take these sizes (bfloat16 tensors)?"""
    from .build import module
    return bool(module("diff_attention").lib.gg_diff_attention_mma_takes(int(heads), int(kv_heads), int(d), int(dv),
                                                                          int(page_size)))


def diff_attention_mma(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                       positions: torch.Tensor, seq_of_token: torch.Tensor, cu_seqlens: torch.Tensor,
                       page_table: torch.Tensor, page_size: int, n_tokens: int, n_seqs: int, heads: int, kv_heads: int,
                       d: int, dv: int, scale: float, cap: float, window: int, lam: float, eps: float,
                       out_scale: float, nsplit: int = 1, partial: Optional[torch.Tensor] = None, max_new: int = 0) -> None:
    """`diff_attention` on the tensor cores (mma.sync) for bfloat16 tensors: the query heads of a kv head and up to
    64 / (heads / kv_heads) consecutive tokens of a sequence share a CTA and every page they read.  nsplit > 1: the
    key tiles of every such CTA are shared out over nsplit CTAs and merged by a second kernel (`partial`: float32
    scratch of `diff_attention_partial_elems`).  max_new: the most rows one sequence brings, where the caller knows
    it; with max_new * (heads / kv_heads) <= 16 a CTA holds 16 rows and its four warps share out every page's keys."""
    if nsplit > 1:
        _need(partial, torch.float32, "partial")
        if partial.numel() < diff_attention_partial_elems(n_tokens, heads, dv, nsplit):
            raise KernelError("diff_attention_mma: the scratch for the shares is too small")
    for t, n in ((q, "q"), (k_pool, "k_pool"), (v_pool, "v_pool"), (out, "out")):
        _need(t, torch.bfloat16, n)
    if k_pool.shape[-1] != 2 * d or v_pool.shape[-1] != dv or k_pool.shape[1] != kv_heads:
        raise KernelError("diff_attention_mma: the pools do not fit the heads")
    from .tcgen05_gemm import status_word
    kernel("diff_attention", "gg_diff_attention_mma")(
        _p(q), _p(k_pool), _p(v_pool), _p(out), _p(positions), _p(seq_of_token), _p(cu_seqlens), _p(page_table),
        page_table.shape[-1], int(page_size), k_pool.shape[0], int(n_tokens), int(n_seqs), int(heads), int(kv_heads),
        int(d), int(dv), float(scale), float(cap), int(window), float(lam), float(eps), float(out_scale), int(nsplit),
        _p(partial), int(max_new), _p(status_word(q.device)), _stream())


def diff_attention_partial_elems(n_tokens: int, heads: int, dv: int, nsplit: int) -> int:
    return n_tokens * heads * nsplit * 2 * (2 + dv)


def diff_attention_splits(n_tokens: int, n_seqs: int, heads: int, kv_heads: int, max_ctx: int) -> int:
    """Into how many shares a step's key tiles are cut: none while the step's (tile, kv head) pairs fill the GPU or
    the contexts are short, else towards two CTAs a multiprocessor, at least two tiles a share."""
    tpt = max(1, 64 // (heads // kv_heads))
    ctas = max(n_seqs, -(-n_tokens // tpt)) * kv_heads
    tiles = -(-max_ctx // 64)
    if ctas >= 148 or tiles < 4:
        return 1
    return int(max(1, min(32, 296 // max(ctas, 1), tiles // 2)))


# ------------------------------------------------------------------------------- latent attention
def latent_prep(q: torch.Tensor, dkv: torch.Tensor, norm_weight: torch.Tensor, eps: float, cos: torch.Tensor,
                sin: torch.Tensor, rot_dims: int, positions: torch.Tensor, seq_of_token: torch.Tensor,
                page_table: torch.Tensor, page_size: int, pool: Optional[torch.Tensor], qcat: torch.Tensor,
                n_tokens: int, heads: int, d: int, r: int, R: int, dense: Optional[torch.Tensor] = None) -> None:
    """Norm of the latent, rotation of the shared key part and of the queries' rotated parts, cache write.
    q [T, heads * (d + r)] and dkv [T, R + r] may be column ranges of one buffer (row strides are passed);
    pool [page][page_size][row]; qcat [T, heads, R + r] receives the rotated parts at [..., R:]; dense (optional,
    contiguous [T, R + r] in the cache's dtype) receives the rows the cache gets, token by token."""
    if q.dtype != dkv.dtype or (pool is not None and pool.dtype != q.dtype):
        raise KernelError("latent_prep: q, dkv and the cache must share one dtype")
    if q.stride(-1) != 1 or dkv.stride(-1) != 1 or not qcat.is_contiguous():
        raise KernelError("latent_prep: rows must be contiguous")
    _need(norm_weight, torch.float32, "norm weight")
    if dense is not None and (dense.dtype != q.dtype or not dense.is_contiguous() or dense.shape[-1] != R + r):
        raise KernelError("latent_prep: the dense copy is contiguous [T, R + r] in the dtype of q")
    from .tcgen05_gemm import status_word
    kernel("latent_attention", "gg_latent_prep")(
        _p(q), q.stride(0), _p(dkv), dkv.stride(0), dtype_code(q.dtype), _p(norm_weight), float(eps), _p(cos), _p(sin),
        int(rot_dims), _p(positions), _p(seq_of_token), _p(page_table), page_table.shape[-1], int(page_size),
        pool.shape[0] if pool is not None else 0, _p(pool), pool.shape[-1] if pool is not None else R + r,
        _p(qcat), dtype_code(qcat.dtype), n_tokens, heads, d, r, R, _p(dense), _p(status_word(q.device)), _stream())


def headwise_gemm(x: torch.Tensor, ldx: int, hx: int, w: torch.Tensor, out: torch.Tensor, ldo: int, ho: int,
                  m: int, alpha: float = 1.0) -> None:
    """out[t, h, :] = alpha * w[h] @ x[t, h, :] for w [H, N, K]; x[t, h] starts at t * ldx + h * hx elements
    into x, out[t, h] at t * ldo + h * ho into out."""
    H, N, K = w.shape
    if not w.is_contiguous():
        raise KernelError("headwise_gemm: the weights must be contiguous [H, N, K]")
    kernel("latent_attention", "gg_headwise_gemm")(_p(x), dtype_code(x.dtype), int(ldx), int(hx), _p(w),
                                                    dtype_code(w.dtype), _p(out), dtype_code(out.dtype), int(ldo),
                                                    int(ho), int(m), N, K, H, float(alpha), _stream())


def latent_attention_plain(qcat: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                           seq_of_token: torch.Tensor, page_table: torch.Tensor, page_size: int, n_tokens: int,
                           heads: int, R: int, r: int, scale: float, window: int,
                           sink: Optional[torch.Tensor] = None) -> None:
    """sink (float32 [heads], optional): exp(sink_h) joins the softmax's denominator, without key or value."""
    from .tcgen05_gemm import status_word
    if sink is not None:
        _need(sink, torch.float32, "sink")
    kernel("latent_attention", "gg_latent_attention_plain")(
        _p(qcat), dtype_code(qcat.dtype), _p(pool), dtype_code(pool.dtype), pool.shape[-1], _p(out),
        dtype_code(out.dtype), _p(positions), _p(seq_of_token), _p(page_table), page_table.shape[-1], int(page_size),
        pool.shape[0], n_tokens, heads, R, r, float(scale), int(window), _p(sink), _p(status_word(qcat.device)), _stream())


# ------------------------------------------------------------------------------- retention
def retention_chunk_takes(d: int, dv: int) -> bool:
    """Does the chunked form hold a head of these sizes (state and chunk in one block's shared memory)?"""
    rc, dvs = 32, dv + 1        # RET_RC and the padded row of csrc/retention.cu (the launcher checks again)
    return (2 * rc * d + 2 * rc * dvs + rc * (rc + 1) + d * dvs + rc + 1) * 4 <= 200 * 1024


def retention(qkvg: torch.Tensor, out: torch.Tensor, raw: Optional[torch.Tensor], state: torch.Tensor,
              cos: torch.Tensor, sin: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor,
              seq_of_token: torch.Tensor, decay: torch.Tensor, n_tokens: int, n_seqs: int, heads: int, d: int, dv: int,
              rot: int, key_scale: float, eps: float, out_scale: float, form: int) -> None:
    """Retention over the step's tokens, sequence by sequence, from and into state [slots][heads][d][dv] (float32).
    qkvg [T, 2*heads*d + 2*heads*dv]: q heads, k heads, v heads, gate; out [T, heads*dv] in the same dtype gets
    o / rms(o) * silu(gate) * out_scale.  form 0: token by token; 1: in chunks (see csrc/retention.cu)."""
    if qkvg.dtype != out.dtype or not qkvg.is_contiguous() or not out.is_contiguous():
        raise KernelError("retention: qkvg and out must be contiguous and share one dtype")
    if qkvg.shape[-1] != 2 * heads * (d + dv) or out.shape[-1] != heads * dv:
        raise KernelError("retention: shapes disagree")
    _need(state, torch.float32, "state")
    _need(decay, torch.float32, "decay")
    if tuple(state.shape[1:]) != (heads, d, dv) or decay.numel() != heads:
        raise KernelError("retention: the state must be [slots, heads, d, dv] and decay one number per head")
    if raw is not None:
        _need(raw, torch.float32, "raw")
    kernel("retention", "gg_retention")(
        _p(qkvg), dtype_code(qkvg.dtype), qkvg.shape[-1], _p(out), _p(raw), _p(state), _p(cos), _p(sin),
        _p(cu_seqlens), _p(slots), _p(seq_of_token), _p(decay), int(n_tokens), int(n_seqs), int(heads), int(d), int(dv),
        int(rot), float(key_scale), float(eps), float(out_scale), int(form), _stream())


RETENTION_CHUNK = 64          # tokens per chunk of the many-CTA form (RET_PC in csrc/retention.cu)
RETENTION_CHUNKS_MAX_HEAD = 128


def retention_chunks_scratch(n_tokens: int, n_seqs: int, heads: int, d: int, dv: int) -> int:
    """Floats of scratch `retention_chunks` needs: a state per chunk and head."""
    return (n_tokens // RETENTION_CHUNK + n_seqs) * heads * d * dv


def retention_chunks(qkvg: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, state: torch.Tensor,
                     cos: torch.Tensor, sin: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor,
                     seq_of_token: torch.Tensor, decay: torch.Tensor, n_tokens: int, n_seqs: int, heads: int, d: int,
                     dv: int, rot: int, key_scale: float, eps: float, out_scale: float) -> None:
    """`retention` for prompts, cut so that every chunk of 64 tokens of every head is a CTA of its own: what each
    chunk adds to the state, a walk over the chunks' states, the outputs chunk by chunk (head sizes up to 128)."""
    if qkvg.dtype != out.dtype or not qkvg.is_contiguous() or not out.is_contiguous():
        raise KernelError("retention: qkvg and out must be contiguous and share one dtype")
    if qkvg.shape[-1] != 2 * heads * (d + dv) or out.shape[-1] != heads * dv:
        raise KernelError("retention: shapes disagree")
    _need(state, torch.float32, "state")
    _need(decay, torch.float32, "decay")
    _need(scratch, torch.float32, "scratch")
    if tuple(state.shape[1:]) != (heads, d, dv) or decay.numel() != heads:
        raise KernelError("retention: the state must be [slots, heads, d, dv] and decay one number per head")
    if scratch.numel() < retention_chunks_scratch(n_tokens, n_seqs, heads, d, dv):
        raise KernelError("retention: the scratch is too small")
    kernel("retention", "gg_retention_chunks")(
        _p(qkvg), dtype_code(qkvg.dtype), qkvg.shape[-1], _p(out), _p(scratch), _p(state), _p(cos), _p(sin),
        _p(cu_seqlens), _p(slots), _p(seq_of_token), _p(decay), int(n_tokens), int(n_seqs), int(heads), int(d), int(dv),
        int(rot), float(key_scale), float(eps), float(out_scale), _stream())


# ------------------------------------------------------------------------------- linear recurrences
def gated_scan(x: torch.Tensor, q_off: int, k_off: int, v_off: int, raw: torch.Tensor, state: torch.Tensor,
               cu_seqlens: torch.Tensor, slots: torch.Tensor, seq_of_token: torch.Tensor, n_tokens: int, n_seqs: int,
               heads: int, d: int, dv: int, decay: Optional[torch.Tensor] = None,
               forget_bias: Optional[torch.Tensor] = None, forget_lower: Optional[torch.Tensor] = None,
               act_q: int = 0, act_k: int = 0, act_v: int = 0) -> None:
    """S_t = diag(g_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head over the step's tokens, sequence by sequence,
    from and into state [slots, heads, d, dv] (float32); raw [T, heads * dv] (float32) gets o_t.  x [T, ld] holds
    the projections: q heads at column q_off, v heads at v_off; with `decay` ([heads]) g is that number and the k
    heads are at k_off; with `forget_bias` and `forget_lower` ([heads * d]) the columns at k_off are the forget
    gate's pre-activation z, f = lower + (1 - lower) sigmoid(z + bias), g = f and k = 1 - f.  act_*: 0 as it is,
    1 silu (csrc/recurrence.cu)."""
    if x.stride(-1) != 1:
        raise KernelError("gated_scan: rows of x must be contiguous")
    _need(raw, torch.float32, "raw")
    _need(state, torch.float32, "state")
    if tuple(state.shape[1:]) != (heads, d, dv) or raw.shape[-1] != heads * dv:
        raise KernelError("gated_scan: the state must be [slots, heads, d, dv] and raw [T, heads * dv]")
    gate = 0 if decay is not None else 1
    for t, n in ((decay, heads), (forget_bias, heads * d), (forget_lower, heads * d)):
        if t is not None:
            _need(t, torch.float32, "recurrence constants")
            if t.numel() != n:
                raise KernelError("gated_scan: decay is [heads], the forget gate's bias and lower bound [heads * d]")
    kernel("recurrence", "gg_gated_scan")(
        _p(x), dtype_code(x.dtype), x.stride(0), int(q_off), int(k_off), int(v_off), _p(raw), _p(state), _p(cu_seqlens),
        _p(slots), _p(seq_of_token), _p(decay), _p(forget_bias), _p(forget_lower), gate, int(n_tokens), int(n_seqs),
        int(heads), int(d), int(dv), int(act_q), int(act_k), int(act_v), _stream())


SCAN_CHUNK = 64               # tokens per chunk of the many-CTA form (REC_PC in csrc/recurrence.cu)
SCAN_CHUNKS_MAX_HEAD = 128


def gated_scan_chunks_scratch(n_tokens: int, n_seqs: int, heads: int, d: int, dv: int) -> int:
    """Floats of scratch `gated_scan_chunks` needs: a state and a decay per chunk and head."""
    return (n_tokens // SCAN_CHUNK + n_seqs) * heads * d * (dv + 1)


def gated_scan_chunks(x: torch.Tensor, q_off: int, k_off: int, v_off: int, raw: torch.Tensor, scratch: torch.Tensor,
                      state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, seq_of_token: torch.Tensor,
                      n_tokens: int, n_seqs: int, heads: int, d: int, dv: int, decay: Optional[torch.Tensor] = None,
                      forget_bias: Optional[torch.Tensor] = None, forget_lower: Optional[torch.Tensor] = None,
                      act_q: int = 0, act_k: int = 0, act_v: int = 0) -> None:
    """`gated_scan` for prompts, cut so that every chunk of 64 tokens of every head is a CTA of its own: what each
    chunk adds to the state, a walk over the chunks' states, the outputs chunk by chunk (head sizes up to 128)."""
    if x.stride(-1) != 1:
        raise KernelError("gated_scan: rows of x must be contiguous")
    _need(raw, torch.float32, "raw")
    _need(state, torch.float32, "state")
    _need(scratch, torch.float32, "scratch")
    if tuple(state.shape[1:]) != (heads, d, dv) or raw.shape[-1] != heads * dv:
        raise KernelError("gated_scan: the state must be [slots, heads, d, dv] and raw [T, heads * dv]")
    if scratch.numel() < gated_scan_chunks_scratch(n_tokens, n_seqs, heads, d, dv):
        raise KernelError("gated_scan: the scratch is too small")
    gate = 0 if decay is not None else 1
    for t, n in ((decay, heads), (forget_bias, heads * d), (forget_lower, heads * d)):
        if t is not None:
            _need(t, torch.float32, "recurrence constants")
            if t.numel() != n:
                raise KernelError("gated_scan: decay is [heads], the forget gate's bias and lower bound [heads * d]")
    kernel("recurrence", "gg_gated_scan_chunks")(
        _p(x), dtype_code(x.dtype), x.stride(0), int(q_off), int(k_off), int(v_off), _p(raw), _p(scratch), _p(state),
        _p(cu_seqlens), _p(slots), _p(seq_of_token), _p(decay), _p(forget_bias), _p(forget_lower), gate, int(n_tokens),
        int(n_seqs), int(heads), int(d), int(dv), int(act_q), int(act_k), int(act_v), _stream())


def scan_finish(raw: torch.Tensor, x: Optional[torch.Tensor], g_off: int, out: torch.Tensor,
                weight: Optional[torch.Tensor], seq_of_token: torch.Tensor, n_tokens: int, heads: int, dv: int,
                eps: float, out_scale: float = 1.0, whole: bool = False, gate: int = 0) -> None:
    """out[t] = norm(raw[t]) * gate * out_scale in the dtype of `out`: every head over its dv outputs with weight
    [dv], or (whole) all heads together with weight [heads * dv]; gate 0 none, 1 sigmoid, 2 silu of x[t, g_off:]."""
    _need(raw, torch.float32, "raw")
    if not out.is_contiguous() or out.shape[-1] != heads * dv:
        raise KernelError("scan_finish: out is contiguous [T, heads * dv]")
    if weight is not None:
        _need(weight, torch.float32, "norm weight")
        if weight.numel() != (heads * dv if whole else dv):
            raise KernelError("scan_finish: the weight's size does not fit the norm")
    if gate and (x is None or x.dtype != out.dtype or x.stride(-1) != 1):
        raise KernelError("scan_finish: the gate's rows come in the dtype of out")
    kernel("recurrence", "gg_scan_finish")(
        _p(raw), _p(x), dtype_code(out.dtype), x.stride(0) if x is not None else 0, int(g_off), _p(out), _p(weight),
        _p(seq_of_token), int(n_tokens), int(heads), int(dv), float(eps), float(out_scale), int(whole), int(gate), _stream())


def stepsize_scan_scratch(n_tokens: int, n_seqs: int, heads: int, d: int, dv: int, chunk: int) -> int:
    """Floats of scratch the chunked form of `stepsize_scan` needs: a state and a decay per chunk and head."""
    return (n_tokens // chunk + n_seqs) * heads * (d * dv + 1)


def stepsize_scan(xc: torch.Tensor, b_off: int, c_off: int, xd: torch.Tensor, dt_off: int, raw: torch.Tensor,
                  state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, seq_of_token: torch.Tensor,
                  dt_bias: torch.Tensor, neg_a: torch.Tensor, n_tokens: int, n_seqs: int, heads: int, groups: int, d: int,
                  dv: int, chunk: int = 0, scratch: Optional[torch.Tensor] = None) -> None:
    """S_t = g_t S_(t-1) + (dt B_t) v_t^T, o_t = S_t^T C_t per head with dt = softplus(x_dt + dt_bias), g = exp(neg_a
    dt), from and into state [slots, heads, d, dv] (float32); raw [T, heads * dv] (float32) gets o_t.  xc [T, .]
    float32 holds v heads at column 0, B [groups, d] at b_off, C at c_off; xd [T, .] (compute dtype) x_dt at dt_off."""
    _need(raw, torch.float32, "raw")
    _need(state, torch.float32, "state")
    _need(dt_bias, torch.float32, "dt_bias")
    _need(neg_a, torch.float32, "neg_a")
    if xc.dtype != torch.float32 or xc.stride(-1) != 1 or xd.stride(-1) != 1:
        raise KernelError("stepsize_scan: xc is float32 and rows are contiguous")
    if tuple(state.shape[1:]) != (heads, d, dv) or raw.shape[-1] != heads * dv or dt_bias.numel() != heads or neg_a.numel() != heads:
        raise KernelError("stepsize_scan: the state must be [slots, heads, d, dv], raw [T, heads * dv], constants [heads]")
    if chunk:
        # prompts: what every chunk of `chunk` rows adds to the state, a walk over the chunks, the outputs chunk by chunk
        _need(scratch, torch.float32, "scratch")
        if scratch.numel() < stepsize_scan_scratch(n_tokens, n_seqs, heads, d, dv, chunk):
            raise KernelError("stepsize_scan: the scratch is too small")
    kernel("recurrence", "gg_stepsize_scan")(
        _p(xc), xc.stride(0), int(b_off), int(c_off), _p(xd), dtype_code(xd.dtype), xd.stride(0), int(dt_off), _p(raw),
        _p(state), _p(cu_seqlens), _p(slots), _p(seq_of_token), _p(dt_bias), _p(neg_a), int(n_tokens), int(n_seqs),
        int(heads), int(groups), int(d), int(dv), int(chunk), _p(scratch), _stream())


def stepsize_finish(raw: torch.Tensor, xc: torch.Tensor, xd: torch.Tensor, z_off: int, skip: torch.Tensor,
                    weight: torch.Tensor, out: torch.Tensor, seq_of_token: torch.Tensor, n_tokens: int, heads: int, dv: int,
                    norm_groups: int, eps: float) -> None:
    """out[t] = groupnorm((raw[t] + skip_h * v[t]) * silu(z[t])) * weight in the dtype of out: v the heads' inputs
    (xc columns 0.., float32), z the gate columns of xd at z_off; the norm in `norm_groups` equal runs."""
    _need(raw, torch.float32, "raw")
    _need(skip, torch.float32, "skip")
    _need(weight, torch.float32, "norm weight")
    if not out.is_contiguous() or out.shape[-1] != heads * dv or weight.numel() != heads * dv:
        raise KernelError("stepsize_finish: shapes disagree")
    kernel("recurrence", "gg_stepsize_finish")(
        _p(raw), _p(xc), xc.stride(0), _p(xd), dtype_code(xd.dtype), dtype_code(out.dtype), xd.stride(0), int(z_off), _p(skip), _p(weight), _p(out),
        _p(seq_of_token), int(n_tokens), int(heads), int(dv), int(norm_groups), float(eps), _stream())


# ------------------------------------------------------------------------------- vector-state recurrences
def rglru_gates(u: torch.Tensor, wa_t: torch.Tensor, wi_t: torch.Tensor, ba: torch.Tensor, bi: torch.Tensor,
                c: torch.Tensor, a: torch.Tensor, b: torch.Tensor, seq_of_token: torch.Tensor, n_tokens: int) -> None:
    """a = exp(c * sigmoid(Wa u + ba)), b = sqrt(1 - a^2) * sigmoid(Wi u + bi) * u with block-diagonal Wa, Wi given
    transposed as [blocks, in, out]; everything float32, u, a, b [T, C]."""
    for t, n in ((u, "u"), (wa_t, "wa"), (wi_t, "wi"), (ba, "ba"), (bi, "bi"), (c, "c"), (a, "a"), (b, "b")):
        _need(t, torch.float32, n)
    blocks, bw, _ = wa_t.shape
    C = blocks * bw
    if u.shape[-1] != C or a.shape[-1] != C or b.shape[-1] != C or wi_t.shape != wa_t.shape or c.numel() != C:
        raise KernelError("rglru_gates: shapes disagree")
    kernel("diag_recurrence", "gg_rglru_gates")(_p(u), _p(wa_t), _p(wi_t), _p(ba), _p(bi), _p(c), _p(a), _p(b),
                                                 _p(seq_of_token), int(n_tokens), C, blocks, _stream())


def diag_scan(a: torch.Tensor, b: torch.Tensor, y: torch.Tensor, ybias: Optional[torch.Tensor], out: torch.Tensor,
              state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, seq_of_token: torch.Tensor,
              n_tokens: int, n_seqs: int) -> None:
    """S_t = a_t S_(t-1) + b_t per channel from and into state [slots, C] (float32); out[t] = S_t * gelu_tanh(y[t] +
    ybias) in the compute dtype (y [T, C] may be a column range of a wider buffer of that dtype)."""
    _need(a, torch.float32, "a")
    _need(b, torch.float32, "b")
    _need(state, torch.float32, "state")
    C = a.shape[-1]
    if y.stride(-1) != 1 or y.shape[-1] != C or not out.is_contiguous() or out.shape[-1] != C or state.shape[-1] != C:
        raise KernelError("diag_scan: shapes disagree")
    if ybias is not None:
        _need(ybias, torch.float32, "ybias")
    kernel("diag_recurrence", "gg_diag_scan")(_p(a), _p(b), _p(y), y.stride(0), dtype_code(y.dtype), dtype_code(out.dtype),
                                               _p(ybias), _p(out),
                                               _p(state), _p(cu_seqlens), _p(slots), _p(seq_of_token), int(n_tokens),
                                               int(n_seqs), C, _stream())


DIAG_CHUNK = 64               # rows per chunk of the many-thread form (DG_CHUNK in csrc/diag_recurrence.cu)


def diag_scan_chunks_scratch(n_tokens: int, n_seqs: int, C: int) -> int:
    """Floats of scratch `diag_scan_chunks` needs: two numbers per chunk and channel."""
    return (n_tokens // DIAG_CHUNK + n_seqs) * 2 * C


def diag_scan_chunks(a: torch.Tensor, b: torch.Tensor, y: torch.Tensor, ybias: Optional[torch.Tensor], out: torch.Tensor,
                     scratch: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor,
                     seq_of_token: torch.Tensor, n_tokens: int, n_seqs: int) -> None:
    """`diag_scan` for prompts, cut so that every chunk of 64 rows of every channel is a thread of its own: the
    chunks' products and sums, a walk over a sequence's chunks, the rows again from each chunk's starting state."""
    _need(a, torch.float32, "a")
    _need(b, torch.float32, "b")
    _need(state, torch.float32, "state")
    _need(scratch, torch.float32, "scratch")
    C = a.shape[-1]
    if y.stride(-1) != 1 or y.shape[-1] != C or not out.is_contiguous() or out.shape[-1] != C or state.shape[-1] != C:
        raise KernelError("diag_scan: shapes disagree")
    if scratch.numel() < diag_scan_chunks_scratch(n_tokens, n_seqs, C):
        raise KernelError("diag_scan: the scratch is too small")
    if ybias is not None:
        _need(ybias, torch.float32, "ybias")
    kernel("diag_recurrence", "gg_diag_scan_chunks")(_p(a), _p(b), _p(y), y.stride(0), dtype_code(y.dtype),
                                                      dtype_code(out.dtype), _p(ybias),
                                                      _p(out), _p(scratch), _p(state), _p(cu_seqlens), _p(slots),
                                                      _p(seq_of_token), int(n_tokens), int(n_seqs), C, _stream())


# ------------------------------------------------------------------------------- routed experts
def moe_router_logits(h: torch.Tensor, wr: torch.Tensor, z: torch.Tensor, n_tokens: int) -> None:
    """z[t, e] = wr[e] . h[t], float32 sums on the CUDA cores (the router is never computed in reduced precision)."""
    _need(z, torch.float32, "router logits")
    E, W = wr.shape
    if h.shape[-1] != W or z.shape[-1] != E or not h.is_contiguous() or not wr.is_contiguous():
        raise KernelError("moe_router_logits: shapes disagree")
    kernel("moe", "gg_moe_router_logits")(_p(h), dtype_code(h.dtype), _p(wr), dtype_code(wr.dtype), _p(z), int(n_tokens),
                                           W, E, _stream())


def moe_route(z: torch.Tensor, top: int, idx: torch.Tensor, wts: torch.Tensor, seq_of_token: Optional[torch.Tensor],
              softmax: bool = False, renormalize: bool = False, rows: Optional[int] = None,
              correction: Optional[torch.Tensor] = None, groups: int = 1, keep: int = 1, n_real: int = 0,
              scale: float = 1.0) -> None:
    """The `top` experts of every row of z and their weights.  correction (float32 [E], optional) is added to the
    scores for the choice only; with groups > 1 the experts form that many equal runs of neighbours and only the
    `keep` groups whose two best choice scores sum highest can be chosen from.  n_real (0: all): router outputs
    from n_real on stand for no expert, a choice of one is stored as index -1; scale multiplies the weights."""
    _need(z, torch.float32, "router logits")
    if correction is not None:
        _need(correction, torch.float32, "correction")
    _need(idx, torch.int32, "idx")
    _need(wts, torch.float32, "wts")
    T = z.shape[0] if rows is None else rows
    kernel("moe", "gg_moe_route")(_p(z), T, z.shape[-1], int(top), int(softmax), int(renormalize), _p(correction),
                                   int(groups), int(keep), int(n_real), float(scale), _p(idx), _p(wts), _p(seq_of_token),
                                   _stream())


def moe_gate_up(h: torch.Tensor, w_gu: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, y: torch.Tensor,
                n_tokens: int, top: int, weight_on_input: bool, limit: float, slope: float, out_scale: float,
                up_offset: float = 1.0) -> None:
    """y[t * top + k] = out_scale * act(Wg[e] x, Wu[e] x) for e = idx[t, k]; w_gu [E, 2, F, W]."""
    E, two, F, W = w_gu.shape
    if two != 2 or h.shape[-1] != W or not h.is_contiguous() or not w_gu.is_contiguous() or not y.is_contiguous():
        raise KernelError("moe_gate_up: shapes disagree")
    kernel("moe", "gg_moe_gate_up")(_p(h), dtype_code(h.dtype), _p(w_gu), dtype_code(w_gu.dtype), _p(idx), _p(wts),
                                     _p(y), dtype_code(y.dtype), n_tokens, W, F, int(top), int(weight_on_input),
                                     float(limit), float(slope), float(up_offset), float(out_scale), _stream())


def moe_down(y: torch.Tensor, w_d: torch.Tensor, idx: torch.Tensor, residual: torch.Tensor, n_tokens: int, top: int,
             seq_of_token: Optional[torch.Tensor]) -> None:
    """residual[t] += sum_k Wd[idx[t, k]] y[t * top + k]; w_d [E, W, F]."""
    E, W, F = w_d.shape
    _need(residual, torch.float32, "residual")
    if residual.shape[-1] != W or not w_d.is_contiguous() or not y.is_contiguous():
        raise KernelError("moe_down: shapes disagree")
    kernel("moe", "gg_moe_down")(_p(y), dtype_code(y.dtype), _p(w_d), dtype_code(w_d.dtype), _p(idx), _p(residual),
                                  n_tokens, W, F, int(top), _p(seq_of_token), _stream())


def moe_gather(h: torch.Tensor, wts: torch.Tensor, place: Optional[torch.Tensor], xs: torch.Tensor, n_pairs: int,
               top: int, weight_on_input: bool) -> None:
    """xs[place[p]] (xs[p] without `place`) = bfloat16(h[p // top] * (wts[p] if the weight sits on the input))."""
    _need(h, torch.bfloat16, "h")
    _need(xs, torch.bfloat16, "xs")
    kernel("moe", "gg_moe_gather")(_p(h), _p(wts), _p(place), _p(xs), int(n_pairs), h.shape[-1], int(top),
                                    int(weight_on_input), _stream())


def moe_combine(rows: torch.Tensor, place: Optional[torch.Tensor], residual: torch.Tensor, n_tokens: int, top: int,
                seq_of_token: Optional[torch.Tensor], idx: Optional[torch.Tensor] = None) -> None:
    """residual[t] += sum over k (in order) of rows[place[t * top + k]], or of rows[t * top + k] without `place`;
    with `idx`, pairs whose index is negative (a choice without an expert) are left out."""
    _need(rows, torch.float32, "rows")
    _need(residual, torch.float32, "residual")
    kernel("moe", "gg_moe_combine")(_p(rows), _p(place), _p(residual), int(n_tokens), residual.shape[-1], int(top),
                                     _p(seq_of_token), _p(idx), _stream())


def moe_identity(h: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, residual: torch.Tensor, n_tokens: int, top: int,
                 seq_of_token: Optional[torch.Tensor]) -> None:
    """residual[t] += (sum of wts[t, k] over the choices with idx[t, k] < 0) * h[t]: the identity experts."""
    _need(residual, torch.float32, "residual")
    _need(idx, torch.int32, "idx")
    _need(wts, torch.float32, "wts")
    if not h.is_contiguous() or h.shape[-1] != residual.shape[-1]:
        raise KernelError("moe_identity: shapes disagree")
    kernel("moe", "gg_moe_identity")(_p(h), dtype_code(h.dtype), _p(idx), _p(wts), _p(residual), int(n_tokens),
                                      residual.shape[-1], int(top), _p(seq_of_token), _stream())


MOE_MMA_MAX_PAIRS = 8192      # the most (token, choice) pairs the mma.sync experts kernel takes (csrc/moe.cu)


def moe_expert_mma(x: torch.Tensor, w: torch.Tensor, idx: torch.Tensor, n_pairs: int, out: torch.Tensor, gated: bool,
                   limit: float = 0.0, slope: float = 1.0, out_scale: float = 1.0,
                   wts: Optional[torch.Tensor] = None, up_offset: float = 1.0) -> None:
    """The experts' products on the tensor cores for up to 8,192 pairs, through the chosen index.  gated: x [P, K]
    against w [E, 2, N, K], out bfloat16 [P, N] = out_scale * act(gate, up) (* wts[p]); else w [E, N, K], out float32."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    _need(out, torch.bfloat16 if gated else torch.float32, "out")
    E, N, K = w.shape[0], w.shape[-2], w.shape[-1]
    if x.shape[-1] != K or out.shape[-1] != N or (gated and (w.dim() != 4 or w.shape[1] != 2)):
        raise KernelError("moe_expert_mma: shapes disagree")
    kernel("moe", "gg_moe_expert_mma")(_p(x), _p(w), _p(idx), int(n_pairs), E, _p(out), N, K, int(gated), float(limit),
                                        float(slope), float(up_offset), float(out_scale), _p(wts), _stream())


def wait_probe(limit_cycles: int, code: int, status: torch.Tensor) -> torch.Tensor:
    """Run the package's bounded wait on a barrier nothing arrives at (csrc/diagnostics.cu) and return the
    kernel's report (5 int32 on the device): both roles' return values, their elapsed cycles / 1024, the
    abort flag.  `status` is the int32 status word the code is to land in."""
    report = torch.full((5,), -1, dtype=torch.int32, device=status.device)
    kernel("diagnostics", "gg_wait_probe")(int(limit_cycles), int(code), _p(status), _p(report), _stream())
    return report


# ------------------------------------------------------------------------------- sampling
_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor, rows: Optional[int] = None) -> None:
    _need(logits, torch.float32, "logits")
    _need(out, torch.int32, "out")
    R = logits.shape[0] if rows is None else rows
    scratch = _argmax_scratch.get(logits.device)
    if scratch is None or scratch.numel() < R * 128:
        scratch = _argmax_scratch[logits.device] = torch.empty(max(R, 64) * 128, dtype=torch.int32,
                                                                device=logits.device)
    kernel("sampling", "gg_argmax")(_p(logits), logits.stride(0), _p(out), R, logits.shape[1],
                                     _p(scratch), scratch.numel(), _stream())


def repeat_penalty(logits: torch.Tensor, hist: torch.Tensor, hist_len: torch.Tensor, ring_rows: torch.Tensor,
                   penalty: float, rows: int) -> None:
    """In place on logits[:rows]: every distinct id in the sequences' rings is penalised once."""
    _need(logits, torch.float32, "logits")
    for t, n in ((hist, "hist"), (hist_len, "hist_len"), (ring_rows, "ring_rows")):
        _need(t, torch.int32, n)
    kernel("sampling", "gg_repeat_penalty")(_p(logits), logits.stride(0), rows, logits.shape[1], _p(hist), _p(hist_len),
                                             _p(ring_rows), hist.shape[1], float(penalty), _stream())


def history_append(tokens: torch.Tensor, ring_rows: torch.Tensor, hist: torch.Tensor, hist_len: torch.Tensor,
                   hist_pos: torch.Tensor, rows: int) -> None:
    """Append tokens[r] to the ring of sequence ring_rows[r]."""
    for t, n in ((tokens, "tokens"), (hist, "hist"), (hist_len, "hist_len"), (hist_pos, "hist_pos"), (ring_rows, "ring_rows")):
        _need(t, torch.int32, n)
    kernel("sampling", "gg_history_append")(_p(tokens), _p(ring_rows), _p(hist), _p(hist_len), _p(hist_pos),
                                             hist.shape[1], rows, _stream())


TOPK_MAX = 1024      # largest top-k the on-device chain takes (csrc/sampling.cu)


_topk_scratch = {}
_sample_scratch = {}


def sample_topk(logits: torch.Tensor, temp: float, top_k: int, top_p: float, min_p: float, uniforms: torch.Tensor,
                out: torch.Tensor, rows: Optional[int] = None) -> None:
    """The sampling chain with a top-k on the device: temperature, top-k, min-p, softmax, top-p, draw."""
    _need(logits, torch.float32, "logits")
    _need(uniforms, torch.float64, "uniforms")
    _need(out, torch.int32, "out")
    R = logits.shape[0] if rows is None else rows
    V = logits.shape[1]
    words = -(-V // 8192) * min(int(top_k), V) * R          # what gg_sample_topk_scratch_words says
    buf = _topk_scratch.get(logits.device)
    if buf is None or buf.numel() < words:
        buf = _topk_scratch[logits.device] = torch.empty(max(words, 1 << 16), dtype=torch.int64, device=logits.device)
    kernel("sampling", "gg_sample_topk")(_p(logits), logits.stride(0), float(temp), int(top_k), float(top_p),
                                          float(min_p), _p(uniforms), _p(out), R, V, _p(buf), buf.numel(), _stream())


_nucleus_scratch = {}


def sample_nucleus(logits: torch.Tensor, temp: float, top_p: float, min_p: float, uniforms: torch.Tensor,
                   out: torch.Tensor, flags: torch.Tensor, rows: Optional[int] = None) -> None:
    """Top-p and / or min-p without a top-k: candidates are each row's 1,024 largest logits, the softmax runs over
    the whole row; flags[r] = 1 where the answer may lie beyond the candidates (out[r] is then not to be used)."""
    _need(logits, torch.float32, "logits")
    _need(uniforms, torch.float64, "uniforms")
    _need(out, torch.int32, "out")
    _need(flags, torch.int32, "flags")
    R = logits.shape[0] if rows is None else rows
    V = logits.shape[1]
    slices = -(-V // 8192)
    nbytes = R * 128 * 4 + R * slices * 8 + R * slices * min(V, 1024) * 8
    buf = _nucleus_scratch.get(logits.device)
    if buf is None or buf.numel() * 8 < nbytes:
        buf = _nucleus_scratch[logits.device] = torch.empty(max(-(-nbytes // 8), 1 << 16), dtype=torch.int64,
                                                            device=logits.device)
    kernel("sampling", "gg_sample_nucleus")(_p(logits), logits.stride(0), float(temp), float(top_p), float(min_p),
                                             _p(uniforms), _p(out), _p(flags), R, V, _p(buf), buf.numel() * 8, _stream())


def sample(logits: torch.Tensor, temps: torch.Tensor, uniforms: torch.Tensor, out: torch.Tensor,
           rows: Optional[int] = None) -> None:
    _need(logits, torch.float32, "logits")
    _need(temps, torch.float32, "temps")
    _need(uniforms, torch.float64, "uniforms")
    _need(out, torch.int32, "out")
    R = logits.shape[0] if rows is None else rows
    V = logits.shape[1]
    words = R * 128 + 2 * R * (-(-V // 8192))
    scratch = _sample_scratch.get(logits.device)
    if scratch is None or scratch.numel() < words:
        scratch = _sample_scratch[logits.device] = torch.empty(max(words, 1 << 14), dtype=torch.int32, device=logits.device)
    kernel("sampling", "gg_sample")(_p(logits), logits.stride(0), _p(temps), _p(uniforms), _p(out), R, V,
                                     _p(scratch), scratch.numel(), _stream())
