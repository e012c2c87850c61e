"""Host side of the tensor-core latent attention kernels (csrc/latent_attention.cu): the per-head products
and the attention over the latent cache on mma.sync, for bfloat16."""
from __future__ import annotations

from typing import Optional

import torch

from .build import KernelError, kernel, module


def headwise_gemm_mma(x: torch.Tensor, ldx: int, hx: int, w: torch.Tensor, out: torch.Tensor, ldo: int, ho: int,
                      m: int, alpha: float = 1.0) -> None:
    """out[t, h, :] = alpha * w[h] @ x[t, h, :] on the tensor cores; bfloat16 x and w [H, N, K], K, ldx and hx
    multiples of 8, out bfloat16 or float32."""
    H, N, K = w.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous():
        raise KernelError("headwise_gemm_mma takes bfloat16 operands, the weights contiguous [H, N, K]")
    from .kernels import dtype_code
    kernel("latent_attention", "gg_headwise_gemm_mma")(
        x.data_ptr(), int(ldx), int(hx), w.data_ptr(), out.data_ptr(), dtype_code(out.dtype), int(ldo), int(ho),
        int(m), N, K, H, float(alpha), torch.cuda.current_stream().cuda_stream)


def latent_attention_mma(qcat: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, cu_seqlens: torch.Tensor,
                         positions: torch.Tensor, seq_of_token: torch.Tensor, page_table: torch.Tensor,
                         page_size: int, n_seqs: int, n_tokens: int, heads: int, R: int, r: int, scale: float,
                         window: int, splits: int = 1, part_o: Optional[torch.Tensor] = None,
                         part_ml: Optional[torch.Tensor] = None, max_new: Optional[int] = None,
                         sink: Optional[torch.Tensor] = None) -> None:
    """splits > 1 cuts every CTA's range of cached positions into that many shares (steps with few CTAs); part_o
    float32 [n_tokens * heads, splits, R] and part_ml [n_tokens * heads, splits, 2] take the partial results.
    max_new: the most new tokens any sequence brings (default: all could be one sequence's); a step of few rows
    per sequence keeps less shared memory for its queries."""
    for t in (qcat, pool, out):
        if t.dtype != torch.bfloat16:
            raise KernelError("latent_attention_mma takes bfloat16 queries, cache and output")
    from .tcgen05_gemm import status_word
    kernel("latent_attention", "gg_latent_attention_mma")(
        qcat.data_ptr(), pool.data_ptr(), pool.shape[-1], out.data_ptr(), cu_seqlens.data_ptr(), positions.data_ptr(),
        seq_of_token.data_ptr(), page_table.data_ptr(), page_table.shape[-1], int(page_size), pool.shape[0],
        int(n_seqs), int(n_tokens), heads, R, r, float(scale), int(window), int(splits),
        part_o.data_ptr() if part_o is not None else 0, part_ml.data_ptr() if part_ml is not None else 0,
        int(max_new) if max_new is not None else int(n_tokens), sink.data_ptr() if sink is not None else 0,
        status_word(qcat.device).data_ptr(),
        torch.cuda.current_stream().cuda_stream)


def mma_splits(n_seqs: int, n_tokens: int, heads: int, R: int, r: int, window: int, max_ctx: int) -> int:
    return int(module("latent_attention").lib.gg_latent_attention_mma_splits(
        int(n_seqs), int(n_tokens), heads, R, r, int(window), int(max_ctx)))


def latent_prompt_mma(qd: torch.Tensor, qcat: torch.Tensor, kv: torch.Tensor, ckr: torch.Tensor, av: torch.Tensor,
                      cu_seqlens: torch.Tensor, seq_of_token: torch.Tensor, n_seqs: int, n_tokens: int, heads: int,
                      d: int, r: int, dv: int, R: int, scale: float, window: int, out_scale: float = 1.0,
                      sink: Optional[torch.Tensor] = None) -> None:
    """Attention of a step whose sequences all start at position 0, in the expanded form: qd [T, >= heads (d + r)]
    (plain query parts), qcat [T, heads, R + r] (rotated parts at [..., R:]), kv [T, heads d + heads dv] (per-head
    plain keys, then values), ckr [T, R + r] (the shared rotated key part at [:, R:]); av [T, heads, dv] receives
    out_scale times the heads' outputs.  All bfloat16."""
    for t in (qd, qcat, kv, ckr, av):
        if t.dtype != torch.bfloat16 or t.stride(-1) != 1:
            raise KernelError("latent_prompt_mma takes bfloat16 rows")
    kernel("latent_attention", "gg_latent_prompt_mma")(
        qd.data_ptr(), qd.stride(0), qcat.data_ptr(), kv.data_ptr(), kv.stride(0), ckr.data_ptr(), ckr.stride(0),
        av.data_ptr(), cu_seqlens.data_ptr(), seq_of_token.data_ptr(), int(n_seqs), int(n_tokens), heads, d, r, dv, R,
        float(scale), int(window), float(out_scale), sink.data_ptr() if sink is not None else 0,
        torch.cuda.current_stream().cuda_stream)


def prompt_takes(d: int, r: int, dv: int) -> bool:
    return bool(module("latent_attention").lib.gg_latent_prompt_mma_takes(int(d), int(r), int(dv)))


def mma_takes(R: int, r: int) -> bool:
    return bool(module("latent_attention").lib.gg_latent_attention_mma_takes(int(R), int(r)))


class _Fast:
    def __init__(self, heads: int, R: int, r: int, scale: float, window: int, sink: Optional[torch.Tensor] = None):
        self.H, self.R, self.r, self.scale, self.window = heads, R, r, scale, window
        self.sink = sink            # float32 [heads] or None: a term of the softmax's denominator per head

    def absorb(self, qd: torch.Tensor, ldx: int, hx: int, uk_t: torch.Tensor, qcat: torch.Tensor, m: int) -> None:
        """qcat[t, h, :R] = Wuk_h^T q_plain[t, h]."""
        D = self.R + self.r
        headwise_gemm_mma(qd, ldx, hx, uk_t, qcat, self.H * D, D, m)

    def attention(self, qcat, pool, out, ctx, table, page_size: int) -> None:
        T, H, R = ctx.n_tokens, self.H, self.R
        # ctx.max_ctx is the longest sequence of the step (an upper bound under a captured graph)
        splits = mma_splits(ctx.n_seqs, T, H, R, self.r, self.window, max(int(ctx.max_ctx), 1))
        part_o = part_ml = None
        if splits > 1:
            part_o = ctx.ws.get("lat_part_o", (T * H, splits, R), torch.float32)
            part_ml = ctx.ws.get("lat_part_ml", (T * H, splits, 2), torch.float32)
        latent_attention_mma(qcat, pool, out, ctx.cu_seqlens, ctx.positions, ctx.seq_of_token, table, page_size,
                             ctx.n_seqs, T, H, R, self.r, self.scale, self.window, splits, part_o, part_ml,
                             max_new=max(int(ctx.max_new), 1), sink=self.sink)

    def expand(self, olat: torch.Tensor, uv: torch.Tensor, av: torch.Tensor, m: int, alpha: float) -> None:
        """av[t, h, :] = alpha * Wuv_h olat[t, h]."""
        dv = uv.shape[1]
        headwise_gemm_mma(olat, self.H * self.R, self.R, uv, av, self.H * dv, dv, m, alpha)


def try_make(heads: int, nope_dim: int, latent_dim: int, rope_dim: int, row_stride: int, scale: float,
             window: int, sink: Optional[torch.Tensor] = None) -> Optional[_Fast]:
    """The tensor-core forms for bfloat16, or None when the sizes are outside what they take (latent and rotated
    sizes multiples of 16, every row of the q / down product on a 16-byte boundary); the plain kernels then serve."""
    if nope_dim % 8 or (nope_dim + rope_dim) % 8 or row_stride % 8 or not mma_takes(latent_dim, rope_dim):
        return None
    return _Fast(heads, latent_dim, rope_dim, scale, window, sink)
