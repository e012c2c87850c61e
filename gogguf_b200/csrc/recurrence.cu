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

GG_API gg_scan_finish(const float* raw, const void* x, int dtype, long long ld, int g_off, void* out, const float* w,
                      const int* seq_of_token, int ntok, int H, int dv, float eps, float out_scale, int whole, int gate,
                      cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (H <= 0 || dv <= 0 || gate < 0 || gate > 2 || (gate != 0 && x == nullptr)) return GG_ERR_ARG;
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(scan_finish_kernel<T>, dim3(ntok), dim3(256), 0, stream, 1, raw, (const T*)x, ld, g_off, (T*)out, w,
                  seq_of_token, H, dv, eps, out_scale, whole, gate));
    return gg_last_error();
}
