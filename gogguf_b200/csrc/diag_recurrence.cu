// Linear recurrences with a vector state: S_t = a_t * S_(t-1) + b_t, element by element, S [C] per sequence
// (float32, zero at a sequence's start, kept in the cache's per-slot state and carried from step to step).
//
// The real-gated linear recurrent unit makes a_t and b_t from its input u_t [C] (float32) with two gates whose
// matrices are block-diagonal: u is cut into `blocks` equal runs, and in run n
//     r = sigmoid(Wa[n] u_n + ba[n]),  i = sigmoid(Wi[n] u_n + bi[n])
//     log a = c * r  (c [C] <= 0: the stored decay parameter, made by the caller),  a = exp(log a)
//     b = sqrt(1 - a^2) * i * u          (1 - a^2 as -expm1(2 log a), which keeps its digits where a is near one)
// rglru_gates_kernel leaves a and b [T, C]; diag_scan_kernel walks every sequence's rows from the slot's state and
// into it and stores out_t = S_t * gelu(yproj_t + ybias) (the tanh form), the unit's second branch, in the compute
// dtype for the output product.  Everything here is float32 on the CUDA cores; a position's result does not
// depend on how its sequence was cut into steps or on what else is in the batch.
#include "common.cuh"

#define RG_TT 8            // tokens a block of the gates kernel holds
#define RG_THREADS 256

// grid (ceil(T / RG_TT), blocks).  wa_t, wi_t [blocks][bw (in)][bw (out)] float32: transposed when the model is
// built, so that neighbouring threads (outputs) read neighbouring words.  u, a, b [T, C] float32, C = blocks * bw.
__global__ void __launch_bounds__(RG_THREADS) rglru_gates_kernel(const float* u, const float* __restrict__ wa_t,
                                                                 const float* __restrict__ wi_t,
                                                                 const float* __restrict__ ba, const float* __restrict__ bi,
                                                                 const float* __restrict__ c, float* a, float* b,
                                                                 const int* __restrict__ seq_of_token, int T, int C, int bw) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float us[];                 // [RG_TT][bw]
    const int t0 = blockIdx.x * RG_TT, n = blockIdx.y;
    const int nt = min(RG_TT, T - t0);
    for (int idx = threadIdx.x; idx < RG_TT * bw; idx += blockDim.x) {
        const int tt = idx / bw, k = idx - tt * bw;
        us[idx] = tt < nt ? u[(size_t)(t0 + tt) * C + n * bw + k] : 0.f;
    }
    __syncthreads();
    const float* wa = wa_t + (size_t)n * bw * bw;
    const float* wi = wi_t + (size_t)n * bw * bw;
    for (int o = threadIdx.x; o < bw; o += blockDim.x) {
        float r[RG_TT], g[RG_TT];
#pragma unroll
        for (int tt = 0; tt < RG_TT; ++tt) { r[tt] = 0.f; g[tt] = 0.f; }
        for (int k = 0; k < bw; ++k) {
            const float x = wa[(size_t)k * bw + o], y = wi[(size_t)k * bw + o];
#pragma unroll
            for (int tt = 0; tt < RG_TT; ++tt) {
                const float uk = us[tt * bw + k];
                r[tt] = fmaf(x, uk, r[tt]);
                g[tt] = fmaf(y, uk, g[tt]);
            }
        }
        const int ch = n * bw + o;
        const float bra = ba[ch], bri = bi[ch], cc = c[ch];
#pragma unroll
        for (int tt = 0; tt < RG_TT; ++tt) {
            if (tt < nt) {
                const size_t at = (size_t)(t0 + tt) * C + ch;
                if (seq_of_token[t0 + tt] < 0) { a[at] = 1.f; b[at] = 0.f; continue; }
                const float rr = 1.0f / (1.0f + expf(-(r[tt] + bra)));
                const float ii = 1.0f / (1.0f + expf(-(g[tt] + bri)));
                const float la = cc * rr;
                a[at] = expf(la);
                b[at] = sqrtf(fmaxf(-expm1f(2.0f * la), 0.f)) * ii * us[tt * bw + o];
            }
        }
    }
}

GG_API gg_rglru_gates(const float* u, const float* wa_t, const float* wi_t, const float* ba, const float* bi, const float* c,
                      float* a, float* b, const int* seq_of_token, int ntok, int C, int blocks, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (C <= 0 || blocks <= 0 || C % blocks || blocks > 65535) return GG_ERR_ARG;
    const int bw = C / blocks;
    const size_t smem = (size_t)RG_TT * bw * sizeof(float);
    if (smem > 200 * 1024) return GG_ERR_ARG;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(rglru_gates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gg_launch(rglru_gates_kernel, dim3((ntok + RG_TT - 1) / RG_TT, blocks), dim3(RG_THREADS), smem, stream, 1, u, wa_t, wi_t,
              ba, bi, c, a, b, seq_of_token, ntok, C, bw);
    return gg_last_error();
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// grid (sequence, ceil(C / 256)): a thread owns one channel of one sequence and walks its rows.
// a, b [T, C] float32; y [T, ldy] the second branch's projection, float32 or the compute dtype (its C columns start at
// y), ybias [C] (may be null); out [T, C] in the compute dtype; state [slots][C] float32.
template <typename TY, typename T>
__global__ void __launch_bounds__(256) diag_scan_kernel(const float* a, const float* b, const TY* y, long long ldy,
                                                        const float* __restrict__ ybias, T* out, float* state,
                                                        const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                                        const int* __restrict__ seq_of_token, int C) {
    pdl_launch();
    pdl_wait();
    const int s = blockIdx.x;
    const int ch = blockIdx.y * blockDim.x + threadIdx.x;
    const int start = cu_seqlens[s], end = cu_seqlens[s + 1];
    if (ch >= C || end <= start) return;
    if (seq_of_token[start] < 0) {                 // a padding row of a replayed batch: zeros, the state untouched
        for (int t = start; t < end; ++t) out[(size_t)t * C + ch] = from_f<T>(0.f);
        return;
    }
    float* sp = state + (size_t)slots[s] * C + ch;
    float S = *sp;
    const float yb = ybias != nullptr ? ybias[ch] : 0.f;
#pragma unroll 4
    for (int t = start; t < end; ++t) {
        S = fmaf(a[(size_t)t * C + ch], S, b[(size_t)t * C + ch]);
        out[(size_t)t * C + ch] = from_f<T>(S * gelu_tanh_f(to_f<TY>(y[(size_t)t * ldy + ch]) + yb));
    }
    *sp = S;
}

// y_dtype: the dtype of y; dtype: that of out.
GG_API gg_diag_scan(const float* a, const float* b, const void* y, long long ldy, int y_dtype, int dtype, const float* ybias,
                    void* out, float* state, const int* cu_seqlens, const int* slots, const int* seq_of_token, int ntok,
                    int n_seqs, int C, cudaStream_t stream) {
    if (ntok <= 0 || n_seqs <= 0) return 0;
    if (C <= 0 || state == nullptr || ldy < C || (C + 255) / 256 > 65535) return GG_ERR_ARG;
    GG_DISPATCH_DTYPE(dtype, T,
        GG_DISPATCH_DTYPE(y_dtype, TY,
            gg_launch(diag_scan_kernel<TY, T>, dim3(n_seqs, (C + 255) / 256), dim3(256), 0, stream, 1, a, b, (const TY*)y, ldy,
                      ybias, (T*)out, state, cu_seqlens, slots, seq_of_token, C)));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- prompts in chunks
// The same recurrence cut into chunks of DG_CHUNK rows, every (chunk, channel) a thread of its own, in three
// kernels.  Inside a chunk that starts from S_in:  S_t = P_t S_in + L_t,  P_t = a_first ... a_t,  L_t the chunk's own
// scan from zero.
//   1. diag_chunk_sums_kernel:  A_c = P_last and B_c = L_last of every chunk
//   2. diag_chunk_walk_kernel:  S_in(c + 1) = A_c S_in(c) + B_c along a sequence's chunks, from the slot's state and
//                               into it; every chunk's S_in is left in scratch
//   3. diag_chunk_out_kernel:   the chunk's rows again from S_in, out_t = S_t * gelu(y_t + ybias)
// The sums are those of the row-by-row walk in another bracketing, so what a position gets does not depend on how
// its prompt was cut beyond rounding.  Chunks never cross sequences: chunk k of the step's list belongs to the
// sequence b whose chunks' running count passes k.
#define DG_CHUNK 64

__device__ __forceinline__ bool diag_find_chunk(const int* __restrict__ cu_seqlens, int n_seqs, int k, int& b, int& t0, int& t1) {
    for (b = 0; b < n_seqs; ++b) {
        const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
        const int nc = (n + DG_CHUNK - 1) / DG_CHUNK;
        if (k < nc) {
            t0 = start + k * DG_CHUNK;
            t1 = min(t0 + DG_CHUNK, start + n);
            return true;
        }
        k -= nc;
    }
    return false;
}

// grid (chunks, ceil(C / 256)); sums [chunks][2][C]
__global__ void __launch_bounds__(256) diag_chunk_sums_kernel(const float* a, const float* b, float* sums,
                                                              const int* __restrict__ cu_seqlens, int n_seqs, int C) {
    pdl_launch();
    pdl_wait();
    const int ch = blockIdx.y * blockDim.x + threadIdx.x;
    int sq, t0, t1;
    if (ch >= C || !diag_find_chunk(cu_seqlens, n_seqs, blockIdx.x, sq, t0, t1)) return;
    float A = 1.f, B = 0.f;
#pragma unroll 8
    for (int t = t0; t < t1; ++t) {
        const float at = a[(size_t)t * C + ch];
        B = fmaf(at, B, b[(size_t)t * C + ch]);
        A *= at;
    }
    sums[((size_t)blockIdx.x * 2) * C + ch] = A;
    sums[((size_t)blockIdx.x * 2 + 1) * C + ch] = B;
}

// grid (sequence, ceil(C / 256)); sums[k][0] is overwritten by the chunk's S_in
__global__ void __launch_bounds__(256) diag_chunk_walk_kernel(float* sums, float* state, const int* __restrict__ cu_seqlens,
                                                              const int* __restrict__ slots,
                                                              const int* __restrict__ seq_of_token, int C) {
    pdl_launch();
    pdl_wait();
    const int s = blockIdx.x;
    const int ch = blockIdx.y * blockDim.x + threadIdx.x;
    const int start = cu_seqlens[s], end = cu_seqlens[s + 1];
    if (ch >= C || end <= start || seq_of_token[start] < 0) return;
    int k0 = 0;
    for (int b = 0; b < s; ++b) k0 += (cu_seqlens[b + 1] - cu_seqlens[b] + DG_CHUNK - 1) / DG_CHUNK;
    const int nc = (end - start + DG_CHUNK - 1) / DG_CHUNK;
    float* sp = state + (size_t)slots[s] * C + ch;
    float S = *sp;
    for (int k = k0; k < k0 + nc; ++k) {
        const float A = sums[((size_t)k * 2) * C + ch], B = sums[((size_t)k * 2 + 1) * C + ch];
        sums[((size_t)k * 2) * C + ch] = S;
        S = fmaf(A, S, B);
    }
    *sp = S;
}

template <typename TY, typename T>
__global__ void __launch_bounds__(256) diag_chunk_out_kernel(const float* a, const float* b, const float* sums, const TY* y,
                                                             long long ldy, const float* __restrict__ ybias, T* out,
                                                             const int* __restrict__ cu_seqlens,
                                                             const int* __restrict__ seq_of_token, int n_seqs, int C) {
    pdl_launch();
    pdl_wait();
    const int ch = blockIdx.y * blockDim.x + threadIdx.x;
    int sq, t0, t1;
    if (ch >= C || !diag_find_chunk(cu_seqlens, n_seqs, blockIdx.x, sq, t0, t1)) return;
    if (seq_of_token[t0] < 0) {
        for (int t = t0; t < t1; ++t) out[(size_t)t * C + ch] = from_f<T>(0.f);
        return;
    }
    float S = sums[((size_t)blockIdx.x * 2) * C + ch];
    const float yb = ybias != nullptr ? ybias[ch] : 0.f;
#pragma unroll 8
    for (int t = t0; t < t1; ++t) {
        S = fmaf(a[(size_t)t * C + ch], S, b[(size_t)t * C + ch]);
        out[(size_t)t * C + ch] = from_f<T>(S * gelu_tanh_f(to_f<TY>(y[(size_t)t * ldy + ch]) + yb));
    }
}

// As gg_diag_scan; sums: scratch of (ntok / 64 + n_seqs) * 2 * C floats.
GG_API gg_diag_scan_chunks(const float* a, const float* b, const void* y, long long ldy, int y_dtype, int dtype,
                           const float* ybias, void* out, float* sums, float* state, const int* cu_seqlens, const int* slots,
                           const int* seq_of_token, int ntok, int n_seqs, int C, cudaStream_t stream) {
    if (ntok <= 0 || n_seqs <= 0) return 0;
    if (C <= 0 || state == nullptr || sums == nullptr || ldy < C || (C + 255) / 256 > 65535) return GG_ERR_ARG;
    const int chunks = ntok / DG_CHUNK + n_seqs;
    const dim3 cgrid(chunks, (C + 255) / 256);
    gg_launch(diag_chunk_sums_kernel, cgrid, dim3(256), 0, stream, 1, a, b, sums, cu_seqlens, n_seqs, C);
    gg_launch(diag_chunk_walk_kernel, dim3(n_seqs, (C + 255) / 256), dim3(256), 0, stream, 1, sums, state, cu_seqlens, slots,
              seq_of_token, C);
    GG_DISPATCH_DTYPE(dtype, T,
        GG_DISPATCH_DTYPE(y_dtype, TY,
            gg_launch(diag_chunk_out_kernel<TY, T>, cgrid, dim3(256), 0, stream, 1, a, b, (const float*)sums, (const TY*)y, ldy,
                      ybias, (T*)out, cu_seqlens, seq_of_token, n_seqs, C)));
    return gg_last_error();
}
