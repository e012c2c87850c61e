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
// a, b [T, C] float32; y [T, ldy] the second branch's projection in the compute dtype (its C columns start at y),
// ybias [C] (may be null); out [T, C] in the compute dtype; state [slots][C] float32.
template <typename T>
__global__ void __launch_bounds__(256) diag_scan_kernel(const float* a, const float* b, const T* y, long long ldy,
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
        out[(size_t)t * C + ch] = from_f<T>(S * gelu_tanh_f(to_f<T>(y[(size_t)t * ldy + ch]) + yb));
    }
    *sp = S;
}

GG_API gg_diag_scan(const float* a, const float* b, const void* y, long long ldy, int dtype, const float* ybias, void* out,
                    float* state, const int* cu_seqlens, const int* slots, const int* seq_of_token, int ntok, int n_seqs,
                    int C, cudaStream_t stream) {
    if (ntok <= 0 || n_seqs <= 0) return 0;
    if (C <= 0 || state == nullptr || ldy < C || (C + 255) / 256 > 65535) return GG_ERR_ARG;
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(diag_scan_kernel<T>, dim3(n_seqs, (C + 255) / 256), dim3(256), 0, stream, 1, a, b, (const T*)y, ldy, ybias,
                  (T*)out, state, cu_seqlens, slots, seq_of_token, C));
    return gg_last_error();
}
