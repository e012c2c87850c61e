// Differential attention over the paged cache: every query head holds two maps, each an attention of its own over
// the same values; the maps' outputs are subtracted, out = a1 - lambda a2, the difference is divided by its root
// mean square over the head's values and multiplied by a factor.
//
// Layout.  A token's projection row holds q as [head][map][d], then (where the layer makes keys and values) k as
// [kv head][map][d] and v as [kv head][dv].  The cache's key pool keeps the two maps of a kv head side by side,
// k [page][kv head][page_size][2 d], the value pool v [page][kv head][page_size][dv].  Query head h reads kv head
// h / (heads / kv_heads).
//
// Preparation (diff_qk_prep_kernel): every (head, map) run of d elements of q and k is divided by its root mean
// square and multiplied by a weight of size d that heads and maps share, then the pairs (2i, 2i + 1) of its first
// `rot` elements are turned by the step's cos / sin tables (column i is pair i); q goes to q_out, k and v into the
// pools at the token's position.  A layer that reads another layer's keys and values passes no pools and a row
// that holds q alone.
//
// Attention (diff_attention_kernel): one block per (token, head), the keys 0..position (or the last `window`) spread
// over the warps; score = q . k * scale, then cap * tanh(score / cap) where cap > 0; an online softmax per map.
// Everything between the loads and the store is float32.
#include "common.cuh"

#define DA_WARPS 4
#define DA_MAXDV 256

template <typename T>
__global__ void __launch_bounds__(256) diff_qk_prep_kernel(
    const T* qkv, long long ld, T* q_out, const float* __restrict__ qw, const float* __restrict__ kw, float eps,
    const float* cosv, const float* sinv, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ page_table, int max_pages, int page_size, T* k_pool, T* v_pool,
    int H, int G, int d, int dv, int rot, const PageBounds pb) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    const int t = blockIdx.x;
    const bool has_kv = k_pool != nullptr;
    const int nq = 2 * H, nk = has_kv ? 2 * G : 0;     // runs of d elements
    const int nqk = (nq + nk) * d;
    float* buf = sm;                 // [nqk]
    float* hs = sm + nqk;            // [nq + nk] one factor per run
    const int b = seq_of_token[t];
    const T* src = qkv + (size_t)t * ld;
    for (int i = threadIdx.x; i < nqk; i += blockDim.x) buf[i] = to_f<T>(src[i]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int r = warp; r < nq + nk; r += nwarps) {
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) { const float v = buf[r * d + i]; ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        if (lane == 0) hs[r] = 1.0f / sqrtf(ss / (float)d + eps);
    }
    __syncthreads();
    int page = -1, slot_in_page = 0;
    if (has_kv && b >= 0) {
        const int pos = positions[t];
        page = gg_page_w(page_table + (size_t)b * max_pages, pos / page_size, max_pages, pb, 50);
        slot_in_page = pos % page_size;
    }
    const int half = rot >> 1;
    const float* c = cosv + (size_t)t * half;
    const float* s = sinv + (size_t)t * half;
    for (int idx = threadIdx.x; idx < nqk; idx += blockDim.x) {
        const int r = idx / d, i = idx - r * d;
        const bool is_q = r < nq;
        if (!is_q && page < 0) continue;
        const float* w = is_q ? qw : kw;
        const float f = hs[r];
        auto val = [&](int j) { return buf[r * d + j] * f * w[j]; };
        float o;
        if (i < rot) {
            const int p = i >> 1;
            o = (i & 1) ? val(i) * c[p] + val(i - 1) * s[p] : val(i) * c[p] - val(i + 1) * s[p];
        } else {
            o = val(i);
        }
        if (is_q) {
            q_out[(size_t)t * nq * d + idx] = from_f<T>(o);
        } else {
            const int rk = r - nq, g = rk >> 1, m = rk & 1;
            k_pool[(((size_t)page * G + g) * page_size + slot_in_page) * (2 * d) + m * d + i] = from_f<T>(o);
        }
    }
    if (page >= 0) {
        for (int idx = threadIdx.x; idx < G * dv; idx += blockDim.x) {
            const int g = idx / dv, i = idx - g * dv;
            v_pool[(((size_t)page * G + g) * page_size + slot_in_page) * dv + i] = src[nqk + idx];
        }
    }
}

// qkv [T, ld] in `dtype`: q (H * 2 * d columns), then, with pools, k (G * 2 * d) and v (G * dv).  q_out [T, H, 2, d].
// k_pool and v_pool both null: the row holds q alone and nothing is written to a cache.
GG_API gg_diff_qk_prep(const void* qkv, long long ld, int dtype, void* q_out, const float* qw, const float* kw, float eps,
                       const float* cosv, const float* sinv, const int* positions, const int* seq_of_token,
                       const int* page_table, int max_pages, int page_size, int n_pages, void* k_pool, void* v_pool,
                       int ntok, int H, int G, int d, int dv, int rot, int* status, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (H <= 0 || G <= 0 || d <= 0 || dv <= 0 || rot < 0 || rot > d || (rot & 1) || page_size <= 0 || qw == nullptr ||
        (k_pool == nullptr) != (v_pool == nullptr) || (k_pool != nullptr && kw == nullptr) || (rot > 0 && (cosv == nullptr || sinv == nullptr)))
        return GG_ERR_ARG;
    const int runs = 2 * H + (k_pool != nullptr ? 2 * G : 0);
    const size_t smem = ((size_t)runs * d + runs) * sizeof(float);
    if (smem > 200 * 1024) return GG_ERR_ARG;
    GG_DISPATCH_DTYPE(dtype, T,
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(diff_qk_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gg_launch(diff_qk_prep_kernel<T>, dim3(ntok), dim3(256), smem, stream, 1, (const T*)qkv, ld, (T*)q_out, qw, kw, eps,
                  cosv, sinv, positions, seq_of_token, page_table, max_pages, page_size, (T*)k_pool, (T*)v_pool, H, G, d, dv,
                  rot, PageBounds{n_pages, status}));
    return gg_last_error();
}

template <typename T>
__global__ void __launch_bounds__(DA_WARPS * 32) diff_attention_kernel(
    const T* q, const T* k_pool, const T* v_pool, T* out, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ page_table, int max_pages, int page_size,
    int H, int G, int d, int dv, float scale, float cap, int window, float lambda, float eps, float out_scale,
    const PageBounds pb) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    float* qs = sm;                               // [2][d]
    float* accs = qs + 2 * d;                     // [DA_WARPS][2][dv]
    float* ml = accs + DA_WARPS * 2 * dv;         // [DA_WARPS][4]: m1, l1, m2, l2
    float* red = ml + DA_WARPS * 4;               // [33]
    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    T* o = out + ((size_t)t * H + h) * dv;
    const int b = seq_of_token[t];
    if (b < 0) {
        for (int i = threadIdx.x; i < dv; i += blockDim.x) o[i] = from_f<T>(0.f);
        return;
    }
    const int pos = positions[t];
    const int g = h / (H / G);
    int lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    const T* qp = q + ((size_t)t * H + h) * 2 * d;
    for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) qs[i] = to_f<T>(qp[i]);
    __syncthreads();

    float acc1[DA_MAXDV / 32], acc2[DA_MAXDV / 32];
#pragma unroll
    for (int j = 0; j < DA_MAXDV / 32; ++j) { acc1[j] = 0.f; acc2[j] = 0.f; }
    float m1 = -INFINITY, l1 = 0.f, m2 = -INFINITY, l2 = 0.f;
    const int* pt = page_table + (size_t)b * max_pages;
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
    for (int j = lo + warp; j <= pos; j += DA_WARPS) {
        const int page = gg_page(pt, j / page_size, max_pages, pb, 51);
        const size_t base = ((size_t)page * G + g) * page_size + (j % page_size);
        const T* kp = k_pool + base * 2 * d;
        const T* vp = v_pool + base * dv;
        float s1 = 0.f, s2 = 0.f;
        for (int i = lane; i < d; i += 32) {
            s1 = fmaf(qs[i], to_f<T>(kp[i]), s1);
            s2 = fmaf(qs[d + i], to_f<T>(kp[d + i]), s2);
        }
        s1 = warp_sum(s1) * scale;
        s2 = warp_sum(s2) * scale;
        if (cap > 0.f) { s1 = cap * tanhf(s1 * inv_cap); s2 = cap * tanhf(s2 * inv_cap); }
        const float n1 = fmaxf(m1, s1), n2 = fmaxf(m2, s2);
        const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);
        const float p1 = expf(s1 - n1), p2 = expf(s2 - n2);
        l1 = l1 * c1 + p1;
        l2 = l2 * c2 + p2;
#pragma unroll
        for (int jj = 0; jj < DA_MAXDV / 32; ++jj) {
            const int i = lane + 32 * jj;
            if (i < dv) {
                const float v = to_f<T>(vp[i]);
                acc1[jj] = acc1[jj] * c1 + p1 * v;
                acc2[jj] = acc2[jj] * c2 + p2 * v;
            }
        }
        m1 = n1;
        m2 = n2;
    }
#pragma unroll
    for (int jj = 0; jj < DA_MAXDV / 32; ++jj) {
        const int i = lane + 32 * jj;
        if (i < dv) { accs[(warp * 2) * dv + i] = acc1[jj]; accs[(warp * 2 + 1) * dv + i] = acc2[jj]; }
    }
    if (lane == 0) { ml[warp * 4] = m1; ml[warp * 4 + 1] = l1; ml[warp * 4 + 2] = m2; ml[warp * 4 + 3] = l2; }
    __syncthreads();
    float f1[DA_WARPS], f2[DA_WARPS];
    float M1 = -INFINITY, M2 = -INFINITY, L1 = 0.f, L2 = 0.f;
    for (int w = 0; w < DA_WARPS; ++w) { M1 = fmaxf(M1, ml[w * 4]); M2 = fmaxf(M2, ml[w * 4 + 2]); }
    for (int w = 0; w < DA_WARPS; ++w) {
        f1[w] = ml[w * 4] == -INFINITY ? 0.f : expf(ml[w * 4] - M1);
        f2[w] = ml[w * 4 + 2] == -INFINITY ? 0.f : expf(ml[w * 4 + 2] - M2);
        L1 += ml[w * 4 + 1] * f1[w];
        L2 += ml[w * 4 + 3] * f2[w];
    }
    const float i1 = 1.0f / L1, i2 = lambda / L2;
    // the difference of the maps, kept in the first map's area of warp 0, and its mean square
    float ss = 0.f;
    for (int i = threadIdx.x; i < dv; i += blockDim.x) {
        float a1 = 0.f, a2 = 0.f;
        for (int w = 0; w < DA_WARPS; ++w) { a1 += accs[(w * 2) * dv + i] * f1[w]; a2 += accs[(w * 2 + 1) * dv + i] * f2[w]; }
        const float df = a1 * i1 - a2 * i2;
        accs[i] = df;                             // (each thread rewrites only elements it alone has just read)
        ss = fmaf(df, df, ss);
    }
    ss = block_sum(ss, red);
    const float f = out_scale / sqrtf(ss / (float)dv + eps);
    for (int i = threadIdx.x; i < dv; i += blockDim.x) o[i] = from_f<T>(accs[i] * f);
}

// q [T, H, 2, d] and out [T, H, dv] in `dtype`; pools k [page][G][page_size][2 d], v [page][G][page_size][dv] in
// `dtype`, n_pages of them.  cap <= 0: the scores are not bounded; window <= 0: every earlier position is seen.
GG_API gg_diff_attention(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype, const int* positions,
                         const int* seq_of_token, const int* page_table, int max_pages, int page_size, int n_pages, int ntok,
                         int H, int G, int d, int dv, float scale, float cap, int window, float lambda, float eps,
                         float out_scale, int* status, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (d <= 0 || dv <= 0 || dv > DA_MAXDV || d > 4096 || H <= 0 || G <= 0 || H % G || H > 65535 || page_size <= 0)
        return GG_ERR_ARG;
    const size_t smem = ((size_t)2 * d + (size_t)DA_WARPS * 2 * dv + 4 * DA_WARPS + 33) * sizeof(float);
    if (smem > 200 * 1024) return GG_ERR_ARG;
    GG_DISPATCH_DTYPE(dtype, T,
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(diff_attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gg_launch(diff_attention_kernel<T>, dim3(ntok, H), dim3(DA_WARPS * 32), smem, stream, 1, (const T*)q,
                  (const T*)k_pool, (const T*)v_pool, (T*)out, positions, seq_of_token, page_table, max_pages, page_size, H, G,
                  d, dv, scale, cap, window, lambda, eps, out_scale, PageBounds{n_pages, status}));
    return gg_last_error();
}

// 1 if this library was built with checked page tables (the debug build), else 0.
GG_API gg_diff_attention_checked() { return gg_debug_bounds(); }
