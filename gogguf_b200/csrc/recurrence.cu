// Linear recurrences with a matrix state per head: S_t = diag(g_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t.
//
// S [d][dv] (float32, zero at a sequence's start) lives in the cache's per-slot state and is carried from step
// to step.  The step's projections arrive as one row per token, x [T, ld], with the q, k and v heads at column
// offsets; what enters the recurrence is made from them in float32 when a round of tokens is staged:
//   gate 0 (a fixed decay per head):    g_t = decay_h for every row;  k_t = act_k(x_k)
//   gate 1 (a forget gate per channel): f = low + (1 - low) sigmoid(x_k + bias);  g_t = f,  k_t = 1 - f
//   q_t = act_q(x_q), v_t = act_v(x_v), act: 0 identity, 1 silu
// The scan kernel leaves the raw outputs o_t in float32; the finish kernel norms them (every head by itself over
// dv with a weight [dv] the heads share, or all heads together over H dv with a weight [H dv]; eps inside the root),
// multiplies by an output gate made from another column block of x (none, sigmoid or silu) and by a factor, and
// stores the rows in the compute dtype for the output projection.  Everything between the projections' outputs
// and that store is float32, in both compute paths; the sums run in an order that does not depend on how the
// sequence was cut into steps or on what else is in the batch.
//
// The scan: grid (sequence, head, tile of 32 columns); thread (part, j) owns RPT rows of column j of the state in
// registers, tokens go by in rounds of REC_TB staged in shared memory.  Prompts and decode steps take the same
// kernel, so a position's result is the same however its sequence was cut.
#include "common.cuh"

#define REC_TB 8
#define REC_COLS 32

__device__ __forceinline__ float rec_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float rec_act(float z, int act) { return act == 1 ? z * rec_sigmoid(z) : z; }

template <typename T, int RPT, bool GATED>
__global__ void __launch_bounds__(256) gated_scan_kernel(
    const T* x, long long ld, int q_off, int k_off, int v_off, float* raw, float* state,
    const int* __restrict__ cu_seqlens, const int* __restrict__ slots, const int* __restrict__ seq_of_token,
    const float* __restrict__ decay, const float* __restrict__ fbias, const float* __restrict__ flow,
    int H, int d, int dv, int parts, int act_q, int act_k, int act_v) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    const int b = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * REC_COLS;
    const int ncols = min(REC_COLS, dv - j0);
    const int dp = parts * RPT;                 // d rounded up to the threads' shares; the tail holds zeros
    float* qs = sm;                             // [REC_TB][dp]
    float* ks = qs + REC_TB * dp;               // [REC_TB][dp]
    float* gs = ks + REC_TB * dp;               // [REC_TB][dp] (GATED only)
    float* vs = gs + (GATED ? REC_TB * dp : 0); // [REC_TB][REC_COLS]
    float* os = vs + REC_TB * REC_COLS;         // [REC_TB][parts][REC_COLS]
    const int start = cu_seqlens[b], end = cu_seqlens[b + 1];
    if (end <= start) return;
    const size_t HV = (size_t)H * dv;
    if (seq_of_token[start] < 0) {              // a padding row of a replayed batch: zeros, the state untouched
        for (int t = start; t < end; ++t)
            for (int j = threadIdx.x; j < ncols; j += blockDim.x) raw[(size_t)t * HV + h * dv + j0 + j] = 0.f;
        return;
    }
    const int part = threadIdx.x / REC_COLS, j = threadIdx.x - part * REC_COLS;
    const bool live = j < ncols;
    const int r0 = part * RPT;
    const float a = GATED ? 0.f : decay[h];
    float* sp = state + (((size_t)slots[b] * H + h) * d) * dv + j0 + j;
    float S[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) S[i] = (live && r0 + i < d) ? sp[(size_t)(r0 + i) * dv] : 0.f;
    if (dp > d)
        for (int idx = threadIdx.x; idx < REC_TB * (dp - d); idx += blockDim.x) {
            const int tt = idx / (dp - d), i = d + idx % (dp - d);
            qs[tt * dp + i] = 0.f;
            ks[tt * dp + i] = 0.f;
            if (GATED) gs[tt * dp + i] = 0.f;
        }
    for (int t0 = start; t0 < end; t0 += REC_TB) {
        const int nb = min(REC_TB, end - t0);
        for (int idx = threadIdx.x; idx < nb * d; idx += blockDim.x) {
            const int tt = idx / d, i = idx - tt * d;
            const T* row = x + (size_t)(t0 + tt) * ld;
            qs[tt * dp + i] = rec_act(to_f<T>(row[q_off + h * d + i]), act_q);
            const float kz = to_f<T>(row[k_off + h * d + i]);
            if (GATED) {
                const float lo = flow[h * d + i];
                const float f = lo + (1.0f - lo) * rec_sigmoid(kz + fbias[h * d + i]);
                gs[tt * dp + i] = f;
                ks[tt * dp + i] = 1.0f - f;
            } else {
                ks[tt * dp + i] = rec_act(kz, act_k);
            }
        }
        for (int idx = threadIdx.x; idx < nb * ncols; idx += blockDim.x) {
            const int tt = idx / ncols, c = idx - tt * ncols;
            vs[tt * REC_COLS + c] = rec_act(to_f<T>(x[(size_t)(t0 + tt) * ld + v_off + h * dv + j0 + c]), act_v);
        }
        __syncthreads();
        if (live) {
#pragma unroll 1
            for (int tt = 0; tt < nb; ++tt) {
                const float vj = vs[tt * REC_COLS + j];
                const float* kt = ks + tt * dp + r0;
                const float* qt = qs + tt * dp + r0;
                const float* gt = gs + tt * dp + r0;
                // (rows of the thread's share that lie beyond d hold zeros in k and q: no test in the loop)
                float o0 = 0.f, o1 = 0.f;
#pragma unroll
                for (int i = 0; i < RPT; i += 2) {
                    S[i] = fmaf(GATED ? gt[i] : a, S[i], kt[i] * vj);
                    S[i + 1] = fmaf(GATED ? gt[i + 1] : a, S[i + 1], kt[i + 1] * vj);
                    o0 = fmaf(S[i], qt[i], o0);
                    o1 = fmaf(S[i + 1], qt[i + 1], o1);
                }
                os[(tt * parts + part) * REC_COLS + j] = o0 + o1;
            }
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < nb * ncols; idx += blockDim.x) {
            const int tt = idx / ncols, c = idx - tt * ncols;
            float o = 0.f;
            for (int p = 0; p < parts; ++p) o += os[(tt * parts + p) * REC_COLS + c];
            raw[(size_t)(t0 + tt) * HV + h * dv + j0 + c] = o;
        }
        // the next round's loads touch qs / ks / gs / vs only, which no thread reads after the barrier above; its
        // outputs are written after its own first barrier, when every thread has left the loop over `os`
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i)
        if (live && r0 + i < d) sp[(size_t)(r0 + i) * dv] = S[i];
}

// x [T, ld] in `dtype`; q heads at q_off (H d columns), k heads (gate 0) or the forget gate's pre-activation
// (gate 1) at k_off, v heads at v_off (H dv columns).  raw [T, H dv] float32; state [slots][H][d][dv] float32.
// gate 0: decay [H]; gate 1: fbias and flow [H d].
GG_API gg_gated_scan(const void* x, int dtype, long long ld, int q_off, int k_off, int v_off, float* raw, float* state,
                     const int* cu_seqlens, const int* slots, const int* seq_of_token, const float* decay,
                     const float* fbias, const float* flow, int gate, int ntok, int n_seqs, int H, int d, int dv,
                     int act_q, int act_k, int act_v, cudaStream_t stream) {
    if (ntok <= 0 || n_seqs <= 0) return 0;
    if (H <= 0 || H > 65535 || d <= 0 || d > 256 || dv <= 0 || raw == nullptr || state == nullptr) return GG_ERR_ARG;
    if (gate == 0 ? decay == nullptr : (gate != 1 || fbias == nullptr || flow == nullptr)) return GG_ERR_ARG;
    const int rpt = d <= 64 ? 16 : 32;
    const int parts = (d + rpt - 1) / rpt;
    const int tiles = (dv + REC_COLS - 1) / REC_COLS;
    if (tiles > 65535) return GG_ERR_ARG;
    const size_t smem = ((size_t)(gate ? 3 : 2) * REC_TB * parts * rpt + (size_t)REC_TB * REC_COLS * (1 + parts)) * sizeof(float);
    if (smem > 200 * 1024) return GG_ERR_ARG;
#define GG_SCAN(T_, R_, G_)                                                                                          \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(gated_scan_kernel<T_, R_, G_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        gg_launch(gated_scan_kernel<T_, R_, G_>, dim3(n_seqs, H, tiles), dim3(parts * REC_COLS), smem, stream, 1,     \
                  (const T_*)x, ld, q_off, k_off, v_off, raw, state, cu_seqlens, slots, seq_of_token, decay, fbias,  \
                  flow, H, d, dv, parts, act_q, act_k, act_v);                                                       \
    } while (0)
    GG_DISPATCH_DTYPE(dtype, T,
        if (rpt == 16) { if (gate) GG_SCAN(T, 16, true); else GG_SCAN(T, 16, false); }
        else { if (gate) GG_SCAN(T, 32, true); else GG_SCAN(T, 32, false); });
#undef GG_SCAN
    return gg_last_error();
}

// ----------------------------------------------------------------------------- norm, output gate, store
// One block per token.  whole == 0: every head's dv outputs are divided by their own root mean square and
// multiplied by w[c] (w [dv], may be null); whole != 0: the token's H dv outputs by theirs, w [H dv].  Then
// gate 1: * sigmoid(x[g_off + c]), gate 2: * silu(x[g_off + c]); then * out_scale.
template <typename T>
__global__ void __launch_bounds__(256) scan_finish_kernel(const float* raw, const T* x, long long ld, int g_off, T* out,
                                                          const float* __restrict__ w, const int* __restrict__ seq_of_token,
                                                          int H, int dv, float eps, float out_scale, int whole, int gate) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int n = H * dv;
    const float* r = raw + (size_t)t * n;
    T* o = out + (size_t)t * n;
    if (seq_of_token[t] < 0) {
        for (int c = threadIdx.x; c < n; c += blockDim.x) o[c] = from_f<T>(0.f);
        return;
    }
    const T* gp = x + (size_t)t * ld + g_off;
    if (whole) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < n; c += blockDim.x) ss = fmaf(r[c], r[c], ss);
        ss = block_sum(ss, red);
        const float f = out_scale / sqrtf(ss / (float)n + eps);
        for (int c = threadIdx.x; c < n; c += blockDim.x) {
            float v = r[c] * f * (w != nullptr ? w[c] : 1.0f);
            if (gate == 1) v *= rec_sigmoid(to_f<T>(gp[c]));
            else if (gate == 2) { const float z = to_f<T>(gp[c]); v *= z * rec_sigmoid(z); }
            o[c] = from_f<T>(v);
        }
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int h = warp; h < H; h += nwarps) {
        const float* rh = r + h * dv;
        float ss = 0.f;
        for (int c = lane; c < dv; c += 32) ss = fmaf(rh[c], rh[c], ss);
        ss = warp_sum(ss);
        const float f = out_scale / sqrtf(ss / (float)dv + eps);
        for (int c = lane; c < dv; c += 32) {
            float v = rh[c] * f * (w != nullptr ? w[c] : 1.0f);
            if (gate == 1) v *= rec_sigmoid(to_f<T>(gp[h * dv + c]));
            else if (gate == 2) { const float z = to_f<T>(gp[h * dv + c]); v *= z * rec_sigmoid(z); }
            o[h * dv + c] = from_f<T>(v);
        }
    }
}

// The same with four neighbouring outputs a thread (16-byte reads of the float32 rows, 8- or 16-byte reads of the
// gate and stores), the row held in registers between the sum of squares and the store: rows of up to 4,096 numbers
// (whole) or heads of up to 512 (a warp a head), every extent a multiple of four.
template <typename T> struct Fin4;
template <> struct Fin4<float> {
    static __device__ __forceinline__ void load(const float* p, float* v) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* v) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Fin4<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float* v) {
        const uint2 a = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&a);
        const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]);
        v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y;
    }
    static __device__ __forceinline__ void store(bf16* p, const float* v) {
        uint2 a;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&a);
        h2[0] = __floats2bfloat162_rn(v[0], v[1]);
        h2[1] = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(p) = a;
    }
};

#define FIN_K 4
template <typename T>
__device__ __forceinline__ void fin_emit(const float* v, float f, const float* __restrict__ w, const T* gp, T* o, int c,
                                         int wc, int gate) {
    float r[4], g[4], wv[4] = {1.f, 1.f, 1.f, 1.f};
    if (w != nullptr) Fin4<float>::load(w + wc, wv);
    if (gate) Fin4<T>::load(gp + c, g);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        r[i] = v[i] * f * wv[i];
        if (gate == 1) r[i] *= rec_sigmoid(g[i]);
        else if (gate == 2) r[i] *= g[i] * rec_sigmoid(g[i]);
    }
    Fin4<T>::store(o + c, r);
}

template <typename T>
__global__ void __launch_bounds__(256) scan_finish_vec_kernel(const float* raw, const T* x, long long ld, int g_off, T* out,
                                                              const float* __restrict__ w,
                                                              const int* __restrict__ seq_of_token, int H, int dv, float eps,
                                                              float out_scale, int whole, int gate) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int n = H * dv;
    const float* r = raw + (size_t)t * n;
    T* o = out + (size_t)t * n;
    const float zero[4] = {0.f, 0.f, 0.f, 0.f};
    if (seq_of_token[t] < 0) {
        for (int c = 4 * threadIdx.x; c < n; c += 4 * blockDim.x) Fin4<T>::store(o + c, zero);
        return;
    }
    const T* gp = x + (size_t)t * ld + g_off;
    float v[FIN_K][4];
    if (whole) {
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < FIN_K; ++k) {
            const int c = 4 * (threadIdx.x + 256 * k);
            if (c < n) {
                Fin4<float>::load(r + c, v[k]);
                ss += v[k][0] * v[k][0] + v[k][1] * v[k][1] + v[k][2] * v[k][2] + v[k][3] * v[k][3];
            }
        }
        ss = block_sum(ss, red);
        const float f = out_scale / sqrtf(ss / (float)n + eps);
#pragma unroll
        for (int k = 0; k < FIN_K; ++k) {
            const int c = 4 * (threadIdx.x + 256 * k);
            if (c < n) fin_emit<T>(v[k], f, w, gp, o, c, c, gate);
        }
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int h = warp; h < H; h += 8) {
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < FIN_K; ++k) {
            const int c = 4 * (lane + 32 * k);
            if (c < dv) {
                Fin4<float>::load(r + h * dv + c, v[k]);
                ss += v[k][0] * v[k][0] + v[k][1] * v[k][1] + v[k][2] * v[k][2] + v[k][3] * v[k][3];
            }
        }
        ss = warp_sum(ss);
        const float f = out_scale / sqrtf(ss / (float)dv + eps);
#pragma unroll
        for (int k = 0; k < FIN_K; ++k) {
            const int c = 4 * (lane + 32 * k);
            if (c < dv) fin_emit<T>(v[k], f, w, gp, o, h * dv + c, c, gate);
        }
    }
}

GG_API gg_scan_finish(const float* raw, const void* x, int dtype, long long ld, int g_off, void* out, const float* w,
                      const int* seq_of_token, int ntok, int H, int dv, float eps, float out_scale, int whole, int gate,
                      cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (H <= 0 || dv <= 0 || gate < 0 || gate > 2 || (gate != 0 && x == nullptr)) return GG_ERR_ARG;
    const bool fits = dv % 4 == 0 && (whole ? (long long)H * dv <= 4 * 256 * FIN_K : dv <= 4 * 32 * FIN_K);
    const bool gate_ok = gate == 0 || (ld % 4 == 0 && g_off % 4 == 0 && ((uintptr_t)x & 15) == 0);
    const bool vec = fits && gate_ok && (((uintptr_t)raw | (uintptr_t)out | (uintptr_t)w) & 15) == 0;
    GG_DISPATCH_DTYPE(dtype, T,
        if (vec)
            gg_launch(scan_finish_vec_kernel<T>, dim3(ntok), dim3(256), 0, stream, 1, raw, (const T*)x, ld, g_off, (T*)out, w,
                      seq_of_token, H, dv, eps, out_scale, whole, gate);
        else
            gg_launch(scan_finish_kernel<T>, dim3(ntok), dim3(256), 0, stream, 1, raw, (const T*)x, ld, g_off, (T*)out, w,
                      seq_of_token, H, dv, eps, out_scale, whole, gate));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- prompts over many CTAs
// The same sums cut into chunks of REC_PC tokens, every (chunk, head) a CTA of its own, in three kernels.  With
// i, j counting a chunk's n tokens from 0 and G_i = g_0 g_1 ... g_i (per channel r, the row of the state):
//   1. what the chunk adds to the state:   U = sum_j diag(G_(n-1) / G_j) k_j v_j^T,   D = G_(n-1)
//   2. a walk over a sequence's chunks:    S_in(c + 1) = diag(D_c) S_in(c) + U_c, from the slot's state and into it
//   3. the outputs:   o_i = S_in^T (G_i * q_i) + sum_{j <= i} A_ij v_j,   A_ij = sum_r q_i[r] k_j[r] G_i[r] / G_j[r]
// A fixed decay makes every ratio a power of one number, so A is a product of q and k rows times decay^(i - j).
// With a forget gate per channel the ratios are formed as 2^(L_i[r] - L_j[r]) from running sums L of log2 g (each
// log2 held above REC_LOG2_FLOOR, far below what float32 tells from zero): never a quotient of two small numbers,
// and no ratio above one.  float32 on the CUDA cores; 16 x 16 threads with register tiles; d, dv <= REC_PMAX.
// The running sums lose about |L| ulps against the token-by-token form, which is rounding next to 16-bit
// projections; the 32-bit path keeps the scan above.
#define REC_PC 64
#define REC_PMAX 128
#define REC_LOG2_FLOOR -150.0f

// Which (sequence, chunk) is CTA `item`?  Chunks are numbered sequence after sequence, padding rows have none.
__device__ __forceinline__ bool rec_find_chunk(int item, const int* cu_seqlens, const int* seq_of_token, int n_seqs,
                                               int& b, int& t0, int& n) {
    for (int i = 0; i < n_seqs; ++i) {
        const int a = cu_seqlens[i], e = cu_seqlens[i + 1];
        if (e <= a || seq_of_token[a] < 0) continue;
        const int nc = (e - a + REC_PC - 1) / REC_PC;
        if (item < nc) { b = i; t0 = a + item * REC_PC; n = min(REC_PC, e - t0); return true; }
        item -= nc;
    }
    return false;
}

// q (if qs), k and, with a forget gate, log2 g (if ls) of head h for n tokens from row t0, float32, into shared
// memory.  q rows are qstride apart; k and log2 g rows kstride apart, element i of row tt in column
// i ^ (tt & 31) when swz (unpadded rows whose columns are then read from different banks by different rows).
template <typename T, bool GATED>
__device__ __forceinline__ void rec_stage_qk(const T* x, long long ld, int q_off, int k_off, int t0, int n, int h, int d,
                                             const float* __restrict__ fbias, const float* __restrict__ flow, int act_q,
                                             int act_k, float* qs, int qstride, float* ks, float* ls, int kstride, bool swz) {
    for (int idx = threadIdx.x; idx < n * d; idx += blockDim.x) {
        const int tt = idx / d, i = idx - tt * d;
        const T* row = x + (size_t)(t0 + tt) * ld;
        if (qs) qs[tt * qstride + i] = rec_act(to_f<T>(row[q_off + h * d + i]), act_q);
        const float kz = to_f<T>(row[k_off + h * d + i]);
        const int at = tt * kstride + (swz ? (i ^ (tt & 31)) : i);
        if (GATED) {
            const float lo = flow[h * d + i];
            const float f = lo + (1.0f - lo) * rec_sigmoid(kz + fbias[h * d + i]);
            ks[at] = 1.0f - f;
            if (ls) ls[at] = fmaxf(log2f(f), REC_LOG2_FLOOR);
        } else {
            ks[at] = rec_act(kz, act_k);
        }
    }
}

template <typename T>
__device__ __forceinline__ void rec_stage_v(const T* x, long long ld, int v_off, int t0, int n, int h, int dv, int act_v,
                                            float* vs) {
    for (int idx = threadIdx.x; idx < n * dv; idx += blockDim.x) {
        const int tt = idx / dv, j = idx - tt * dv;
        vs[tt * dv + j] = rec_act(to_f<T>(x[(size_t)(t0 + tt) * ld + v_off + h * dv + j]), act_v);
    }
}

// 1. U [chunk][H][d][dv] and D [chunk][H][d].
template <typename T, bool GATED>
__global__ void __launch_bounds__(256) rec_chunk_state_kernel(
    const T* x, long long ld, int q_off, int k_off, int v_off, float* U, float* D, const int* __restrict__ cu_seqlens,
    const int* __restrict__ seq_of_token, const float* __restrict__ decay, const float* __restrict__ fbias,
    const float* __restrict__ flow, int n_seqs, int H, int d, int dv, int act_k, int act_v) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    int b, t0, n;
    if (!rec_find_chunk(blockIdx.x, cu_seqlens, seq_of_token, n_seqs, b, t0, n)) return;
    const int h = blockIdx.y, ds = d + 1;
    float* ks = sm;                        // [PC][ds], in the end times G_(n-1) / G_j
    float* vs = ks + REC_PC * ds;          // [PC][dv]
    float* ls = vs + REC_PC * dv;          // [PC][ds] (GATED only)
    rec_stage_qk<T, GATED>(x, ld, q_off, k_off, t0, n, h, d, fbias, flow, 0, act_k, nullptr, 0, ks, GATED ? ls : nullptr,
                           ds, false);
    rec_stage_v<T>(x, ld, v_off, t0, n, h, dv, act_v, vs);
    __syncthreads();
    for (int r = threadIdx.x; r < d; r += blockDim.x) {      // a thread owns channel r of every token
        float* dp = D + ((size_t)blockIdx.x * H + h) * d;
        if (GATED) {
            float run = 0.f;
            for (int tt = 0; tt < n; ++tt) { run += ls[tt * ds + r]; ls[tt * ds + r] = run; }
            for (int tt = 0; tt < n; ++tt) ks[tt * ds + r] *= exp2f(run - ls[tt * ds + r]);
            dp[r] = exp2f(run);
        } else {
            const float a = decay[h];
            float p = 1.f;
            for (int tt = n - 1; tt >= 0; --tt) { ks[tt * ds + r] *= p; p *= a; }
            dp[r] = p;
        }
    }
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[REC_PMAX / 16][REC_PMAX / 16];
#pragma unroll
    for (int i = 0; i < REC_PMAX / 16; ++i)
#pragma unroll
        for (int j = 0; j < REC_PMAX / 16; ++j) acc[i][j] = 0.f;
#pragma unroll 4
    for (int j = 0; j < n; ++j) {
        float kr[REC_PMAX / 16], vc[REC_PMAX / 16];
#pragma unroll
        for (int i = 0; i < REC_PMAX / 16; ++i) {
            kr[i] = ty + 16 * i < d ? ks[j * ds + ty + 16 * i] : 0.f;
            vc[i] = tx + 16 * i < dv ? vs[j * dv + tx + 16 * i] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < REC_PMAX / 16; ++i)
#pragma unroll
            for (int c = 0; c < REC_PMAX / 16; ++c) acc[i][c] = fmaf(kr[i], vc[c], acc[i][c]);
    }
    float* up = U + ((size_t)blockIdx.x * H + h) * d * dv;
#pragma unroll
    for (int i = 0; i < REC_PMAX / 16; ++i)
#pragma unroll
        for (int c = 0; c < REC_PMAX / 16; ++c)
            if (ty + 16 * i < d && tx + 16 * c < dv) up[(size_t)(ty + 16 * i) * dv + tx + 16 * c] = acc[i][c];
}

// 2. The walk: U[c] becomes the state chunk c starts from, the slot's state the one after the last chunk.
__global__ void __launch_bounds__(256) rec_chunk_walk_kernel(
    float* U, const float* D, float* state, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
    const int* __restrict__ seq_of_token, int H, int d, int dv) {
    pdl_launch();
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    const int start = cu_seqlens[b], end = cu_seqlens[b + 1];
    if (e >= d * dv || end <= start || seq_of_token[start] < 0) return;
    int base = 0;
    for (int i = 0; i < b; ++i) {
        const int a0 = cu_seqlens[i], e0 = cu_seqlens[i + 1];
        if (e0 > a0 && seq_of_token[a0] >= 0) base += (e0 - a0 + REC_PC - 1) / REC_PC;
    }
    const int nch = (end - start + REC_PC - 1) / REC_PC;
    float* sp = state + (((size_t)slots[b] * H + h) * d) * dv + e;
    float s = *sp;
    const size_t step = (size_t)H * d * dv, dstep = (size_t)H * d;
    float* up = U + ((size_t)base * H + h) * d * dv + e;
    const float* dp = D + ((size_t)base * H + h) * d + e / dv;
    // eight chunks' terms are asked for at once: the walk itself is a chain of dependent multiply-adds only
    for (int c0 = 0; c0 < nch; c0 += 8) {
        float u[8], g[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            u[k] = c0 + k < nch ? up[(size_t)(c0 + k) * step] : 0.f;
            g[k] = c0 + k < nch ? dp[(size_t)(c0 + k) * dstep] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (c0 + k < nch) {
                up[(size_t)(c0 + k) * step] = s;
                s = fmaf(s, g[k], u[k]);
            }
        }
    }
    *sp = s;
}

// 3. The outputs of a chunk from the state it starts with (Sin, what the walk left in U) and its own tokens.
// Shared memory is cut so that two CTAs share an SM at 128 x 128 heads: q rows unpadded (read as broadcasts), k
// (and log2 g) rows unpadded with swizzled columns where d is a multiple of 32 (else padded by one); with a
// forget gate the v rows arrive in the place of the running sums once A is made.
template <typename T, bool GATED>
__global__ void __launch_bounds__(256, 2) rec_chunk_out_kernel(
    const T* x, long long ld, int q_off, int k_off, int v_off, float* raw, const float* Sin,
    const int* __restrict__ cu_seqlens, const int* __restrict__ seq_of_token, const float* __restrict__ decay,
    const float* __restrict__ fbias, const float* __restrict__ flow, int n_seqs, int H, int d, int dv, int act_q,
    int act_k, int act_v) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    int b, t0, n;
    if (!rec_find_chunk(blockIdx.x, cu_seqlens, seq_of_token, n_seqs, b, t0, n)) return;
    const bool swz = (d & 31) == 0;
    const int h = blockIdx.y, ds = swz ? d : d + 1;
    float* qs = sm;                                   // [PC][d]
    float* ks = qs + REC_PC * d;                      // [PC][ds]
    float* vs = ks + REC_PC * ds;                     // [PC][max(ds, dv)]: v rows; GATED: first the running sums
    float* ls = vs;
    float* A = vs + REC_PC * max(ds, dv);             // [PC][PC]
    float* pw = A + REC_PC * REC_PC;                  // [PC + 1]: powers of the decay (not GATED)
    if (!GATED && threadIdx.x <= REC_PC) {
        const float a = decay[h];
        float p = 1.f;
        for (int i = 0; i < (int)threadIdx.x; ++i) p *= a;
        pw[threadIdx.x] = p;
    }
    rec_stage_qk<T, GATED>(x, ld, q_off, k_off, t0, n, h, d, fbias, flow, act_q, act_k, qs, d, ks, GATED ? ls : nullptr, ds,
                           swz);
    if (!GATED) rec_stage_v<T>(x, ld, v_off, t0, n, h, dv, act_v, vs);
    __syncthreads();
    if (GATED) {
        for (int r = threadIdx.x; r < d; r += blockDim.x) {
            float run = 0.f;
            for (int tt = 0; tt < n; ++tt) {
                const int at = tt * ds + (swz ? (r ^ (tt & 31)) : r);
                run += ls[at];
                ls[at] = run;
            }
        }
        __syncthreads();
    }
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    {   // A[i][j] for j <= i < n, else 0; rows i = ty + 16 a, columns j = tx + 16 b; b > a lies above the diagonal
        float acc[REC_PC / 16][REC_PC / 16];
#pragma unroll
        for (int i = 0; i < REC_PC / 16; ++i)
#pragma unroll
            for (int j = 0; j < REC_PC / 16; ++j) acc[i][j] = 0.f;
#pragma unroll 2
        for (int r = 0; r < d; ++r) {
            float qv[REC_PC / 16], kv[REC_PC / 16], lq[REC_PC / 16], lk[REC_PC / 16];
#pragma unroll
            for (int i = 0; i < REC_PC / 16; ++i) {
                const int qi = ty + 16 * i, kj = tx + 16 * i;
                qv[i] = qi < n ? qs[qi * d + r] : 0.f;
                kv[i] = kj < n ? ks[kj * ds + (swz ? (r ^ (kj & 31)) : r)] : 0.f;
                if (GATED) {
                    lq[i] = qi < n ? ls[qi * ds + (swz ? (r ^ (qi & 31)) : r)] : 0.f;
                    lk[i] = kj < n ? ls[kj * ds + (swz ? (r ^ (kj & 31)) : r)] : 0.f;
                }
            }
#pragma unroll
            for (int i = 0; i < REC_PC / 16; ++i)
#pragma unroll
                for (int j = 0; j < REC_PC / 16; ++j) {
                    if (GATED) {
                        if (j <= i) acc[i][j] = fmaf(qv[i] * kv[j], exp2f(fminf(lq[i] - lk[j], 0.f)), acc[i][j]);
                    } else {
                        acc[i][j] = fmaf(qv[i], kv[j], acc[i][j]);
                    }
                }
        }
        __syncthreads();                          // every thread is done with the q rows and the running sums as they are
#pragma unroll
        for (int i = 0; i < REC_PC / 16; ++i)
#pragma unroll
            for (int j = 0; j < REC_PC / 16; ++j) {
                const int qi = ty + 16 * i, kj = tx + 16 * j;
                const float wgt = GATED ? 1.f : pw[max(qi - kj, 0)];
                A[qi * REC_PC + kj] = (kj <= qi && qi < n) ? acc[i][j] * wgt : 0.f;
            }
    }
    // q_i times G_i, in place
    for (int idx = threadIdx.x; idx < n * d; idx += blockDim.x) {
        const int tt = idx / d, i = idx - tt * d;
        qs[idx] *= GATED ? exp2f(ls[tt * ds + (swz ? (i ^ (tt & 31)) : i)]) : pw[tt + 1];
    }
    __syncthreads();
    if (GATED) rec_stage_v<T>(x, ld, v_off, t0, n, h, dv, act_v, vs);
    // o[i][c]: rows i = ty + 16 a, columns c = tx + 16 b
    float o[REC_PC / 16][REC_PMAX / 16];
#pragma unroll
    for (int i = 0; i < REC_PC / 16; ++i)
#pragma unroll
        for (int c = 0; c < REC_PMAX / 16; ++c) o[i][c] = 0.f;
    const float* S = Sin + ((size_t)blockIdx.x * H + h) * d * dv;
#pragma unroll 4
    for (int r = 0; r < d; ++r) {
        float qv[REC_PC / 16], sv[REC_PMAX / 16];
#pragma unroll
        for (int i = 0; i < REC_PC / 16; ++i) qv[i] = ty + 16 * i < n ? qs[(ty + 16 * i) * d + r] : 0.f;
#pragma unroll
        for (int c = 0; c < REC_PMAX / 16; ++c) sv[c] = tx + 16 * c < dv ? S[(size_t)r * dv + tx + 16 * c] : 0.f;
#pragma unroll
        for (int i = 0; i < REC_PC / 16; ++i)
#pragma unroll
            for (int c = 0; c < REC_PMAX / 16; ++c) o[i][c] = fmaf(qv[i], sv[c], o[i][c]);
    }
    __syncthreads();                              // the v rows are whole (and so is A)
#pragma unroll 4
    for (int j = 0; j < n; ++j) {
        float av[REC_PC / 16], vv[REC_PMAX / 16];
#pragma unroll
        for (int i = 0; i < REC_PC / 16; ++i) av[i] = A[(ty + 16 * i) * REC_PC + j];
#pragma unroll
        for (int c = 0; c < REC_PMAX / 16; ++c) vv[c] = tx + 16 * c < dv ? vs[j * dv + tx + 16 * c] : 0.f;
#pragma unroll
        for (int i = 0; i < REC_PC / 16; ++i)
#pragma unroll
            for (int c = 0; c < REC_PMAX / 16; ++c) o[i][c] = fmaf(av[i], vv[c], o[i][c]);
    }
    const size_t HV = (size_t)H * dv;
#pragma unroll
    for (int i = 0; i < REC_PC / 16; ++i)
#pragma unroll
        for (int c = 0; c < REC_PMAX / 16; ++c)
            if (ty + 16 * i < n && tx + 16 * c < dv) raw[(size_t)(t0 + ty + 16 * i) * HV + h * dv + tx + 16 * c] = o[i][c];
}

static inline size_t rec_chunk_smem_state(int d, int dv, int gate) {
    return ((size_t)REC_PC * ((gate ? 2 : 1) * (d + 1) + dv)) * sizeof(float);
}
static inline size_t rec_chunk_smem_out(int d, int dv) {
    const int ds = (d & 31) == 0 ? d : d + 1;
    return ((size_t)REC_PC * (d + ds + (ds > dv ? ds : dv) + REC_PC) + REC_PC + 1) * sizeof(float);
}

// The chunked form of gg_gated_scan for steps that bring prompts: the same arguments, and scratch of
// (ntok / 64 + n_seqs) * H * d * (dv + 1) floats (a state and a decay per chunk and head).  d, dv <= 128.
GG_API gg_gated_scan_chunks(const void* x, int dtype, long long ld, int q_off, int k_off, int v_off, float* raw,
                            float* scratch, float* state, const int* cu_seqlens, const int* slots, const int* seq_of_token,
                            const float* decay, const float* fbias, const float* flow, int gate, int ntok, int n_seqs, int H,
                            int d, int dv, int act_q, int act_k, int act_v, cudaStream_t stream) {
    if (ntok <= 0 || n_seqs <= 0) return 0;
    if (H <= 0 || H > 65535 || d <= 0 || dv <= 0 || d > REC_PMAX || dv > REC_PMAX || raw == nullptr || state == nullptr ||
        scratch == nullptr) return GG_ERR_ARG;
    if (gate == 0 ? decay == nullptr : (gate != 1 || fbias == nullptr || flow == nullptr)) return GG_ERR_ARG;
    const int chunks = ntok / REC_PC + n_seqs;
    float* U = scratch;
    float* D = scratch + (size_t)chunks * H * d * dv;
    const size_t smem_a = rec_chunk_smem_state(d, dv, gate), smem_c = rec_chunk_smem_out(d, dv);
#define GG_CHUNKS(T_, G_)                                                                                              \
    do {                                                                                                               \
        if (smem_a > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(rec_chunk_state_kernel<T_, G_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a); \
        if (smem_c > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(rec_chunk_out_kernel<T_, G_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_c);  \
        gg_launch(rec_chunk_state_kernel<T_, G_>, dim3(chunks, H), dim3(256), smem_a, stream, 1, (const T_*)x, ld, q_off,  \
                  k_off, v_off, U, D, cu_seqlens, seq_of_token, decay, fbias, flow, n_seqs, H, d, dv, act_k, act_v);       \
        gg_launch(rec_chunk_walk_kernel, dim3(n_seqs, H, (d * dv + 255) / 256), dim3(256), 0, stream, 1, U,               \
                  (const float*)D, state, cu_seqlens, slots, seq_of_token, H, d, dv);                                     \
        gg_launch(rec_chunk_out_kernel<T_, G_>, dim3(chunks, H), dim3(256), smem_c, stream, 1, (const T_*)x, ld, q_off,    \
                  k_off, v_off, raw, (const float*)U, cu_seqlens, seq_of_token, decay, fbias, flow, n_seqs, H, d, dv,     \
                  act_q, act_k, act_v);                                                                                   \
    } while (0)
    GG_DISPATCH_DTYPE(dtype, T, if (gate) GG_CHUNKS(T, true); else GG_CHUNKS(T, false));
#undef GG_CHUNKS
    return gg_last_error();
}

// ----------------------------------------------------------------------------- a step size per head (state-space form)
// The same matrix state with a gate that is one number per head and token, made from a step size:
//     dt = softplus(x_dt + dt_bias_h),   g_t = exp(neg_a_h * dt)   (neg_a_h = -exp(A_log_h) <= 0, made by the caller)
//     S_t = g_t S_(t-1) + (dt B_t) v_t^T,   o_t = S_t^T C_t
// S [d][dv] with d the state size and dv the head's value size.  B and C [groups][d] are shared by the heads of a
// group (head h reads group h / (H / groups)).  v, B and C arrive as float32 columns of one row per token
// (xc [T, ldc]: v heads at column 0, B at b_off, C at c_off: a convolution's output); x_dt as column dt_off + h of
// the projection's row in the compute dtype (xd [T, ldd]).  The structure is gated_scan_kernel's: grid (sequence,
// head, tile of 32 columns), thread (part, j) owns RPT rows of column j of the state, rounds of REC_TB tokens.
__device__ __forceinline__ float rec_softplus(float z) { return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.f); }

template <typename T, int RPT>
__global__ void __launch_bounds__(256) stepsize_scan_kernel(
    const float* xc, long long ldc, int b_off, int c_off, const T* xd, long long ldd, int dt_off, float* raw, float* state,
    const int* __restrict__ cu_seqlens, const int* __restrict__ slots, const int* __restrict__ seq_of_token,
    const float* __restrict__ dt_bias, const float* __restrict__ neg_a, int H, int d, int dv, int parts, int hpg,
    int phase, int chunk, int n_seqs, float* chunk_state, float* chunk_decay) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    const int h = blockIdx.y, j0 = blockIdx.z * REC_COLS;
    // phase 0: blockIdx.x is a sequence, walked whole from the slot's state and into it.  Phases 1 and 2: blockIdx.x
    // is a chunk of `chunk` rows of some sequence (the chunks of the step in order, never across sequences); phase 1
    // starts from zero and leaves what the chunk adds to the state and the product of its gates, phase 2 starts
    // from the state the walk between the two left for the chunk and makes the outputs.
    int b = blockIdx.x, start, end;
    if (phase == 0) {
        start = cu_seqlens[b];
        end = cu_seqlens[b + 1];
    } else {
        int k = blockIdx.x;
        bool found = false;
        for (b = 0; b < n_seqs; ++b) {
            const int s0 = cu_seqlens[b], n = cu_seqlens[b + 1] - s0;
            const int nc = (n + chunk - 1) / chunk;
            if (k < nc) { start = s0 + k * chunk; end = min(start + chunk, s0 + n); found = true; break; }
            k -= nc;
        }
        if (!found) return;
    }
    const bool emit = phase != 1;
    const int ncols = min(REC_COLS, dv - j0);
    const int dp = parts * RPT;
    float* qs = sm;                             // [REC_TB][dp]  C_t
    float* ks = qs + REC_TB * dp;               // [REC_TB][dp]  dt B_t
    float* vs = ks + REC_TB * dp;               // [REC_TB][REC_COLS]
    float* os = vs + REC_TB * REC_COLS;         // [REC_TB][parts][REC_COLS]
    float* dts = os + REC_TB * parts * REC_COLS;  // [REC_TB] dt
    float* gs = dts + REC_TB;                   // [REC_TB] g
    if (end <= start) return;
    const size_t HV = (size_t)H * dv;
    if (seq_of_token[start] < 0) {
        if (emit)
            for (int t = start; t < end; ++t)
                for (int j = threadIdx.x; j < ncols; j += blockDim.x) raw[(size_t)t * HV + h * dv + j0 + j] = 0.f;
        return;
    }
    const int part = threadIdx.x / REC_COLS, j = threadIdx.x - part * REC_COLS;
    const bool live = j < ncols;
    const int r0 = part * RPT;
    const int grp = h / hpg;
    const float bias = dt_bias[h], na = neg_a[h];
    float* sp = (phase == 0 ? state + (((size_t)slots[b] * H + h) * d) * dv
                            : chunk_state + (((size_t)blockIdx.x * H + h) * d) * dv) + j0 + j;
    float S[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) S[i] = (phase != 1 && live && r0 + i < d) ? sp[(size_t)(r0 + i) * dv] : 0.f;
    if (dp > d)
        for (int idx = threadIdx.x; idx < REC_TB * (dp - d); idx += blockDim.x) {
            const int tt = idx / (dp - d), i = d + idx % (dp - d);
            qs[tt * dp + i] = 0.f;
            ks[tt * dp + i] = 0.f;
        }
    float gprod = 1.f;                          // (thread 0, phase 1) the product of the chunk's gates
    for (int t0 = start; t0 < end; t0 += REC_TB) {
        const int nb = min(REC_TB, end - t0);
        if (threadIdx.x < nb) {
            const float dt = rec_softplus(to_f<T>(xd[(size_t)(t0 + threadIdx.x) * ldd + dt_off + h]) + bias);
            dts[threadIdx.x] = dt;
            gs[threadIdx.x] = expf(na * dt);
        }
        __syncthreads();
        if (phase == 1 && threadIdx.x == 0)
            for (int tt = 0; tt < nb; ++tt) gprod *= gs[tt];
        for (int idx = threadIdx.x; idx < nb * d; idx += blockDim.x) {
            const int tt = idx / d, i = idx - tt * d;
            const float* row = xc + (size_t)(t0 + tt) * ldc;
            qs[tt * dp + i] = row[c_off + grp * d + i];
            ks[tt * dp + i] = dts[tt] * row[b_off + grp * d + i];
        }
        for (int idx = threadIdx.x; idx < nb * ncols; idx += blockDim.x) {
            const int tt = idx / ncols, c = idx - tt * ncols;
            vs[tt * REC_COLS + c] = xc[(size_t)(t0 + tt) * ldc + h * dv + j0 + c];
        }
        __syncthreads();
        if (live) {
#pragma unroll 1
            for (int tt = 0; tt < nb; ++tt) {
                const float vj = vs[tt * REC_COLS + j], g = gs[tt];
                const float* kt = ks + tt * dp + r0;
                const float* qt = qs + tt * dp + r0;
                float o0 = 0.f, o1 = 0.f;
#pragma unroll
                for (int i = 0; i < RPT; i += 2) {
                    S[i] = fmaf(g, S[i], kt[i] * vj);
                    S[i + 1] = fmaf(g, S[i + 1], kt[i + 1] * vj);
                    if (emit) {
                        o0 = fmaf(S[i], qt[i], o0);
                        o1 = fmaf(S[i + 1], qt[i + 1], o1);
                    }
                }
                if (emit) os[(tt * parts + part) * REC_COLS + j] = o0 + o1;
            }
        }
        __syncthreads();
        if (emit)
            for (int idx = threadIdx.x; idx < nb * ncols; idx += blockDim.x) {
                const int tt = idx / ncols, c = idx - tt * ncols;
                float o = 0.f;
                for (int p = 0; p < parts; ++p) o += os[(tt * parts + p) * REC_COLS + c];
                raw[(size_t)(t0 + tt) * HV + h * dv + j0 + c] = o;
            }
        // (the next round writes dts / gs before its first barrier: every thread has read gs in the loop above, which
        // ends before the barrier that precedes these stores)
    }
    if (phase == 2) return;
#pragma unroll
    for (int i = 0; i < RPT; ++i)
        if (live && r0 + i < d) sp[(size_t)(r0 + i) * dv] = S[i];
    if (phase == 1 && threadIdx.x == 0 && blockIdx.z == 0) chunk_decay[(size_t)blockIdx.x * H + h] = gprod;
}

// The walk between the two chunked phases: along a sequence's chunks S_in(c + 1) = D_c S_in(c) + U_c, from the slot's
// state and into it; every chunk's U is replaced by its S_in.  grid (sequence, head, ceil(d dv / 256)).
__global__ void __launch_bounds__(256) stepsize_chunk_walk_kernel(float* chunk_state, const float* chunk_decay, float* state,
                                                                  const int* __restrict__ cu_seqlens,
                                                                  const int* __restrict__ slots,
                                                                  const int* __restrict__ seq_of_token, int H, int ddv,
                                                                  int chunk) {
    pdl_launch();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    const int start = cu_seqlens[s], end = cu_seqlens[s + 1];
    if (e >= ddv || end <= start || seq_of_token[start] < 0) return;
    int k0 = 0;
    for (int b = 0; b < s; ++b) k0 += (cu_seqlens[b + 1] - cu_seqlens[b] + chunk - 1) / chunk;
    const int nc = (end - start + chunk - 1) / chunk;
    float* sp = state + ((size_t)slots[s] * H + h) * ddv + e;
    float S = *sp;
    for (int k = k0; k < k0 + nc; k += 8) {              // eight chunks' loads in flight, then the chain
        float U[8], D[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (k + i < k0 + nc) {
                U[i] = chunk_state[((size_t)(k + i) * H + h) * ddv + e];
                D[i] = chunk_decay[(size_t)(k + i) * H + h];
            }
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (k + i < k0 + nc) {
                chunk_state[((size_t)(k + i) * H + h) * ddv + e] = S;
                S = fmaf(D[i], S, U[i]);
            }
    }
    *sp = S;
}

// xc [T, ldc] float32; xd [T, ldd] in `dtype`; raw [T, H dv] float32; state [slots][H][d][dv] float32;
// dt_bias, neg_a [H]; groups divides H.
// chunk > 0 (prompts): the three-launch form over chunks of that many rows, with scratch of
// (ntok / chunk + n_seqs) * H * (d * dv + 1) floats; chunk == 0: every sequence walked whole by its own CTAs.
GG_API gg_stepsize_scan(const float* xc, long long ldc, int b_off, int c_off, const void* xd, int dtype, long long ldd,
                        int dt_off, float* raw, float* state, const int* cu_seqlens, const int* slots,
                        const int* seq_of_token, const float* dt_bias, const float* neg_a, int ntok, int n_seqs, int H,
                        int groups, int d, int dv, int chunk, float* scratch, cudaStream_t stream) {
    if (ntok <= 0 || n_seqs <= 0) return 0;
    if (chunk < 0 || (chunk > 0 && scratch == nullptr)) return GG_ERR_ARG;
    if (H <= 0 || H > 65535 || groups <= 0 || H % groups || d <= 0 || d > 256 || dv <= 0 || raw == nullptr ||
        state == nullptr || dt_bias == nullptr || neg_a == nullptr)
        return GG_ERR_ARG;
    const int rpt = d <= 64 ? 16 : 32;
    const int parts = (d + rpt - 1) / rpt;
    const int tiles = (dv + REC_COLS - 1) / REC_COLS;
    if (tiles > 65535) return GG_ERR_ARG;
    const size_t smem = ((size_t)2 * REC_TB * parts * rpt + (size_t)REC_TB * REC_COLS * (1 + parts) + 2 * REC_TB) * sizeof(float);
    if (smem > 200 * 1024) return GG_ERR_ARG;
#define GG_SSCAN(T_, R_)                                                                                             \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(stepsize_scan_kernel<T_, R_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (chunk == 0) {                                                                                            \
            gg_launch(stepsize_scan_kernel<T_, R_>, dim3(n_seqs, H, tiles), dim3(parts * REC_COLS), smem, stream, 1, xc, ldc, \
                      b_off, c_off, (const T_*)xd, ldd, dt_off, raw, state, cu_seqlens, slots, seq_of_token, dt_bias, neg_a, \
                      H, d, dv, parts, H / groups, 0, 0, n_seqs, (float*)nullptr, (float*)nullptr);                  \
        } else {                                                                                                     \
            const int chunks = ntok / chunk + n_seqs;                                                                \
            float* cs = scratch;                                                                                     \
            float* cd = scratch + (size_t)chunks * H * d * dv;                                                       \
            gg_launch(stepsize_scan_kernel<T_, R_>, dim3(chunks, H, tiles), dim3(parts * REC_COLS), smem, stream, 1, xc, ldc, \
                      b_off, c_off, (const T_*)xd, ldd, dt_off, raw, state, cu_seqlens, slots, seq_of_token, dt_bias, neg_a, \
                      H, d, dv, parts, H / groups, 1, chunk, n_seqs, cs, cd);                                        \
            gg_launch(stepsize_chunk_walk_kernel, dim3(n_seqs, H, (d * dv + 255) / 256), dim3(256), 0, stream, 1, cs,   \
                      (const float*)cd, state, cu_seqlens, slots, seq_of_token, H, d * dv, chunk);                   \
            gg_launch(stepsize_scan_kernel<T_, R_>, dim3(chunks, H, tiles), dim3(parts * REC_COLS), smem, stream, 1, xc, ldc, \
                      b_off, c_off, (const T_*)xd, ldd, dt_off, raw, state, cu_seqlens, slots, seq_of_token, dt_bias, neg_a, \
                      H, d, dv, parts, H / groups, 2, chunk, n_seqs, cs, cd);                                        \
        }                                                                                                            \
    } while (0)
    GG_DISPATCH_DTYPE(dtype, T, if (rpt == 16) GG_SSCAN(T, 16); else GG_SSCAN(T, 32));
#undef GG_SSCAN
    return gg_last_error();
}

// The finish of that form, one block per token: val = (raw + skip_h * v) * silu(z), with v the head's input row
// (xc, float32) and z the gate's columns of the projection (xd, float32 or the compute dtype); the row of H dv numbers is then cut
// into `norm_groups` equal runs, each divided by its own sqrt(mean(run^2) + eps), times w [H dv]; stored in the
// compute dtype.  The gate comes before the norm.
template <typename TX, typename T>
__global__ void __launch_bounds__(256) stepsize_finish_kernel(const float* raw, const float* xc, long long ldc, const TX* xd,
                                                              long long ldd, int z_off, const float* __restrict__ skip,
                                                              const float* __restrict__ w, T* out,
                                                              const int* __restrict__ seq_of_token, int H, int dv,
                                                              int norm_groups, float eps) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int n = H * dv;
    T* o = out + (size_t)t * n;
    if (seq_of_token[t] < 0) {
        for (int c = threadIdx.x; c < n; c += blockDim.x) o[c] = from_f<T>(0.f);
        return;
    }
    const float* r = raw + (size_t)t * n;
    const float* v = xc + (size_t)t * ldc;
    const TX* z = xd + (size_t)t * ldd + z_off;
    const int gs = n / norm_groups;
    auto val = [&](int c) {
        const float zz = to_f<TX>(z[c]);
        return (r[c] + skip[c / dv] * v[c]) * (zz * rec_sigmoid(zz));
    };
    for (int g = 0; g < norm_groups; ++g) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < gs; i += blockDim.x) { const float a = val(g * gs + i); ss = fmaf(a, a, ss); }
        ss = block_sum(ss, red);
        const float f = 1.0f / sqrtf(ss / (float)gs + eps);
        for (int i = threadIdx.x; i < gs; i += blockDim.x) {
            const int c = g * gs + i;
            o[c] = from_f<T>(val(c) * f * w[c]);
        }
    }
}

// x_dtype: the dtype of xd; dtype: that of out.
GG_API gg_stepsize_finish(const float* raw, const float* xc, long long ldc, const void* xd, int x_dtype, int dtype,
                          long long ldd, int z_off, const float* skip, const float* w, void* out, const int* seq_of_token, int ntok, int H,
                          int dv, int norm_groups, float eps, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (H <= 0 || dv <= 0 || norm_groups <= 0 || (H * dv) % norm_groups || skip == nullptr || w == nullptr) return GG_ERR_ARG;
    GG_DISPATCH_DTYPE(dtype, T,
        GG_DISPATCH_DTYPE(x_dtype, TX,
            gg_launch(stepsize_finish_kernel<TX, T>, dim3(ntok), dim3(256), 0, stream, 1, raw, xc, ldc, (const TX*)xd, ldd, z_off,
                      skip, w, (T*)out, seq_of_token, H, dv, norm_groups, eps)));
    return gg_last_error();
}
