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
#define DA_MAXDV 512

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

// ----------------------------------------------------------------------------- the same on the tensor cores (bfloat16)
// A CTA of four warps takes 64 query rows: the hpg = heads / kv_heads query heads of one kv head for tpt = 64 / hpg
// consecutive tokens of one sequence (row r: token r / hpg, head r % hpg), so the keys and values of a page are
// read once for all heads that share them.  The key tiles are the sequence's pages (64 positions: [64][2 d] keys
// with both maps side by side, [64][dv] values), brought into shared memory by cp.async in two stages.  Per tile
// and map: S = Q_m K_m^T (mma.sync m16n8k16, fragments by ldmatrix), scale, bound and mask in float32, an online
// softmax per row and map in float32, P as the A operand of O_m += P V in two bfloat16 terms (its rounding and
// what the rounding left out, so that the weights enter with sixteen bits and more; V fragments by ldmatrix.trans).  At the end out = out_scale * unit(O_1 / l_1 - lambda O_2 / l_2) per row.  Prompts, portions
// and decode steps take this kernel; page_size must be 64, d and dv one of 32, 64, 128.
__device__ __forceinline__ void da_ldsm4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void da_ldsm4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void da_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void da_cp16(void* dst, const void* src) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(a), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t da_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// (x, y) as a pair of bfloat16 numbers `hi` and the pair `lo` of what that rounding left out
__device__ __forceinline__ void da_split(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const float2 hf = __bfloat1622float2(h);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = da_pack(x - hf.x, y - hf.y);
}
__device__ __forceinline__ float da_quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float da_quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

#define DA_ROWS 64
#define DA_KEYS 64

// WK (tiles of at most 16 rows: decode steps): the four warps all hold the tile's rows and take 16 of a page's 64 keys
// each; at the end their maxima, sums and weighted values are put together in shared memory.
template <int D, int DV, bool WK>
__global__ void __launch_bounds__(128) diff_attention_mma_kernel(
    const bf16* q, const bf16* k_pool, const bf16* v_pool, bf16* out, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens, const int* __restrict__ page_table,
    int max_pages, int n_seqs, int H, int G, int hpg, int tpt, float scale, float cap, int window, float lambda,
    float eps, float out_scale, int nsplit, float* partial, const PageBounds pb) {
    pdl_wait();
    constexpr int QS = 2 * D + 8, KS = 2 * D + 8, VS = DV + 8;     // row strides in elements (16 bytes of padding)
    extern __shared__ __align__(16) unsigned char da_smem[];
    bf16* Qs = reinterpret_cast<bf16*>(da_smem);                    // [64][QS]
    bf16* Ks = Qs + DA_ROWS * QS;                                   // [2][64][KS]
    bf16* Vs = Ks + 2 * DA_KEYS * KS;                               // [2][64][VS]
    __shared__ int info[3];
    const int g = blockIdx.y;
    if (threadIdx.x == 0) {
        // (the step's last tiles first: a sequence's late tiles read the most keys, and the CTAs that start first
        // should be the long ones)
        int tile = (int)gridDim.x - 1 - (int)blockIdx.x, b = 0, found = 0;
        for (; b < n_seqs; ++b) {
            const int n = cu_seqlens[b + 1] - cu_seqlens[b];
            const int nt = (n + tpt - 1) / tpt;
            if (tile < nt) { found = 1; break; }
            tile -= nt;
        }
        info[0] = found ? b : -1;
        info[1] = found ? cu_seqlens[b] + tile * tpt : 0;
        info[2] = found ? min(tpt, cu_seqlens[b + 1] - (cu_seqlens[b] + tile * tpt)) : 0;
    }
    __syncthreads();
    const int b = info[0], t0 = info[1], ntok = info[2];
    if (b < 0) return;
    const int nrows = ntok * hpg;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (seq_of_token[t0] < 0) {                                     // padding rows of a replayed batch: zeros
        if (nsplit > 1) return;                                     // (the kernel that merges the shares writes them)
        for (int idx = threadIdx.x; idx < nrows * DV; idx += blockDim.x) {
            const int r = idx / DV, c = idx - r * DV;
            out[((size_t)(t0 + r / hpg) * H + g * hpg + r % hpg) * DV + c] = __float2bfloat16_rn(0.f);
        }
        return;
    }
    // the query rows, both maps side by side
    for (int idx = threadIdx.x; idx < DA_ROWS * (2 * D / 8); idx += blockDim.x) {
        const int r = idx / (2 * D / 8), c8 = idx - r * (2 * D / 8);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < nrows)
            v = *reinterpret_cast<const uint4*>(q + ((size_t)(t0 + r / hpg) * H + g * hpg + r % hpg) * (2 * D) + c8 * 8);
        *reinterpret_cast<uint4*>(Qs + r * QS + c8 * 8) = v;
    }
    const int pos0 = positions[t0];
    const int pos_last = pos0 + ntok - 1;
    const int lo_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    int j_lo = lo_key / DA_KEYS, j_hi = pos_last / DA_KEYS;
    if (nsplit > 1) {                                               // this CTA's share of the tiles (it may be empty)
        const int per = (j_hi - j_lo + nsplit) / nsplit;
        j_lo += (int)blockIdx.z * per;
        j_hi = min(j_hi, j_lo + per - 1);
    }
    const int* pt = page_table + (size_t)b * max_pages;

    auto load_tile = [&](int j, int stage) {
        const int page = gg_page(pt, j, max_pages, pb, 51);
        const bf16* kp = k_pool + ((size_t)page * G + g) * DA_KEYS * (2 * D);
        const bf16* vp = v_pool + ((size_t)page * G + g) * DA_KEYS * DV;
        bf16* kd = Ks + stage * DA_KEYS * KS;
        bf16* vd = Vs + stage * DA_KEYS * VS;
        for (int idx = threadIdx.x; idx < DA_KEYS * (2 * D / 8); idx += blockDim.x) {
            const int r = idx / (2 * D / 8), c8 = idx - r * (2 * D / 8);
            da_cp16(kd + r * KS + c8 * 8, kp + (size_t)r * (2 * D) + c8 * 8);
        }
        for (int idx = threadIdx.x; idx < DA_KEYS * (DV / 8); idx += blockDim.x) {
            const int r = idx / (DV / 8), c8 = idx - r * (DV / 8);
            da_cp16(vd + r * VS + c8 * 8, vp + (size_t)r * DV + c8 * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // this thread's two rows of its warp's sixteen
    const int gq = lane >> 2, t4 = lane & 3;
    const int rbase = WK ? 0 : warp * 16;                          // the warp's first row of the tile
    const int kbase = WK ? warp * 16 : 0;                          // the warp's first key of a page
    constexpr int NP = WK ? 1 : 4;                                  // runs of 16 keys the warp takes of a page
    const int rA = rbase + gq, rB = rA + 8;
    const int posA = rA < nrows ? pos0 + rA / hpg : -1, posB = rB < nrows ? pos0 + rB / hpg : -1;
    const int loA = window > 0 ? posA - window + 1 : 0, loB = window > 0 ? posB - window + 1 : 0;
    const int wlast = min(rbase + 15, nrows - 1);
    const int wmax = rbase < nrows ? pos0 + wlast / hpg : -1;       // the warp's largest position (-1: no rows)
    float O[2][DV / 8][4];
    float mrun[2][2], lrun[2][2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        mrun[m][0] = mrun[m][1] = -INFINITY;
        lrun[m][0] = lrun[m][1] = 0.f;
#pragma unroll
        for (int n = 0; n < DV / 8; ++n) { O[m][n][0] = O[m][n][1] = O[m][n][2] = O[m][n][3] = 0.f; }
    }
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;

    if (j_lo <= j_hi) load_tile(j_lo, 0);
    for (int j = j_lo; j <= j_hi; ++j) {
        const int stage = (j - j_lo) & 1;
        if (j < j_hi) {
            load_tile(j + 1, stage ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const int key0 = j * DA_KEYS;
        if (key0 <= wmax) {
            const bf16* Kt = Ks + stage * DA_KEYS * KS;
            const bf16* Vt = Vs + stage * DA_KEYS * VS;
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                float s[2 * NP][4];
#pragma unroll
                for (int n = 0; n < 2 * NP; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    uint32_t a0, a1, a2, a3;
                    da_ldsm4(a0, a1, a2, a3, Qs + (rbase + (lane & 7) + ((lane >> 3) & 1) * 8) * QS + m * D + ks * 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int np = 0; np < NP; ++np) {
                        uint32_t b0, b1, b2, b3;
                        da_ldsm4(b0, b1, b2, b3, Kt + (kbase + np * 16 + (lane & 7) + (lane >> 4) * 8) * KS + m * D + ks * 16 + ((lane >> 3) & 1) * 8);
                        da_mma(s[2 * np], a0, a1, a2, a3, b0, b1);
                        da_mma(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
                    }
                }
                float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
                for (int n = 0; n < 2 * NP; ++n) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + kbase + n * 8 + 2 * t4 + (e & 1);
                        float v = s[n][e] * scale;
                        if (cap > 0.f) v = cap * tanhf(v * inv_cap);
                        const bool ok = e < 2 ? (key <= posA && key >= loA) : (key <= posB && key >= loB);
                        v = ok ? v : -INFINITY;
                        s[n][e] = v;
                        if (e < 2) mxA = fmaxf(mxA, v); else mxB = fmaxf(mxB, v);
                    }
                }
                mxA = da_quad_max(mxA);
                mxB = da_quad_max(mxB);
                const float nA = fmaxf(mrun[m][0], mxA), nB = fmaxf(mrun[m][1], mxB);
                const float uA = nA == -INFINITY ? 0.f : nA, uB = nB == -INFINITY ? 0.f : nB;
                const float cA = expf(mrun[m][0] - uA), cB = expf(mrun[m][1] - uB);
                mrun[m][0] = nA;
                mrun[m][1] = nB;
                float sumA = 0.f, sumB = 0.f;
#pragma unroll
                for (int n = 0; n < 2 * NP; ++n) {
                    s[n][0] = expf(s[n][0] - uA); s[n][1] = expf(s[n][1] - uA);
                    s[n][2] = expf(s[n][2] - uB); s[n][3] = expf(s[n][3] - uB);
                    sumA += s[n][0] + s[n][1];
                    sumB += s[n][2] + s[n][3];
                }
                lrun[m][0] = lrun[m][0] * cA + sumA;
                lrun[m][1] = lrun[m][1] * cB + sumB;
#pragma unroll
                for (int n = 0; n < DV / 8; ++n) { O[m][n][0] *= cA; O[m][n][1] *= cA; O[m][n][2] *= cB; O[m][n][3] *= cB; }
#pragma unroll
                for (int kk = 0; kk < NP; ++kk) {
                    // the weights as two bfloat16 terms, p = hi + lo, so that the product with the values takes them
                    // to sixteen bits and more
                    uint32_t ah[4], al[4];
                    da_split(s[2 * kk][0], s[2 * kk][1], ah[0], al[0]);
                    da_split(s[2 * kk][2], s[2 * kk][3], ah[1], al[1]);
                    da_split(s[2 * kk + 1][0], s[2 * kk + 1][1], ah[2], al[2]);
                    da_split(s[2 * kk + 1][2], s[2 * kk + 1][3], ah[3], al[3]);
#pragma unroll
                    for (int np = 0; np < DV / 16; ++np) {
                        uint32_t b0, b1, b2, b3;
                        da_ldsm4_t(b0, b1, b2, b3, Vt + (kbase + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + np * 16 + (lane >> 4) * 8);
                        da_mma(O[m][2 * np], ah[0], ah[1], ah[2], ah[3], b0, b1);
                        da_mma(O[m][2 * np + 1], ah[0], ah[1], ah[2], ah[3], b2, b3);
                        da_mma(O[m][2 * np], al[0], al[1], al[2], al[3], b0, b1);
                        da_mma(O[m][2 * np + 1], al[0], al[1], al[2], al[3], b2, b3);
                    }
                }
            }
        }
        __syncthreads();
    }
    // the difference of the maps, its root mean square over the head's values, the store
    const float l1A = da_quad_sum(lrun[0][0]), l1B = da_quad_sum(lrun[0][1]);
    const float l2A = da_quad_sum(lrun[1][0]), l2B = da_quad_sum(lrun[1][1]);
    if (WK) {
        // the four warps' shares of the keys, put together in shared memory (the pipeline's stages are free now)
        float* mg = reinterpret_cast<float*>(da_smem);               // [warp][16 rows][map][2 + DV]
        __syncthreads();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = half ? rB : rA;
            if ((half ? posB : posA) < 0) continue;
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                float* pm = mg + ((size_t)(warp * 16 + r) * 2 + m) * (2 + DV);
                if (t4 == 0) { pm[0] = mrun[m][half]; pm[1] = half ? (m ? l2B : l1B) : (m ? l2A : l1A); }
#pragma unroll
                for (int n = 0; n < DV / 8; ++n) {
                    pm[2 + n * 8 + 2 * t4] = O[m][n][2 * half];
                    pm[2 + n * 8 + 2 * t4 + 1] = O[m][n][2 * half + 1];
                }
            }
        }
        __syncthreads();
        for (int r = warp; r < nrows; r += 4) {                     // a warp a row
            float M[2], L[2], f[2][4];
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                M[m] = -INFINITY;
                L[m] = 0.f;
#pragma unroll
                for (int w = 0; w < 4; ++w) M[m] = fmaxf(M[m], mg[((size_t)(w * 16 + r) * 2 + m) * (2 + DV)]);
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const float* pm = mg + ((size_t)(w * 16 + r) * 2 + m) * (2 + DV);
                    f[m][w] = pm[0] == -INFINITY ? 0.f : expf(pm[0] - M[m]);
                    L[m] += pm[1] * f[m][w];
                }
            }
            const int tok = t0 + r / hpg, head = g * hpg + r % hpg;
            float df[DV / 32];
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < DV / 32; ++k) {
                const int c = lane + 32 * k;
                float a[2] = {0.f, 0.f};
#pragma unroll
                for (int m = 0; m < 2; ++m)
#pragma unroll
                    for (int w = 0; w < 4; ++w) a[m] += mg[((size_t)(w * 16 + r) * 2 + m) * (2 + DV) + 2 + c] * f[m][w];
                if (nsplit > 1) {
                    float* base = partial + (((size_t)tok * H + head) * nsplit + blockIdx.z) * 2 * (2 + DV);
                    base[2 + c] = a[0];
                    base[(2 + DV) + 2 + c] = a[1];
                } else {
                    df[k] = a[0] / L[0] - lambda * a[1] / L[1];
                    ss = fmaf(df[k], df[k], ss);
                }
            }
            if (nsplit > 1) {
                if (lane < 2) {
                    float* base = partial + (((size_t)tok * H + head) * nsplit + blockIdx.z) * 2 * (2 + DV) + lane * (2 + DV);
                    base[0] = M[lane];
                    base[1] = L[lane];
                }
            } else {
                ss = warp_sum(ss);
                const float fn = out_scale / sqrtf(ss / (float)DV + eps);
                bf16* o = out + ((size_t)tok * H + head) * DV;
#pragma unroll
                for (int k = 0; k < DV / 32; ++k) o[lane + 32 * k] = __float2bfloat16_rn(df[k] * fn);
            }
        }
        return;
    }
    if (nsplit > 1) {
        // a share of the keys: each row's running maximum, sum and weighted values per map go to scratch
        // [row of the step][head][share][map][2 + DV]; diff_attention_merge_kernel puts the shares together
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = half ? rB : rA;
            if ((half ? posB : posA) < 0) continue;
            float* base = partial + (((size_t)(t0 + r / hpg) * H + g * hpg + r % hpg) * nsplit + blockIdx.z) * 2 * (2 + DV);
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                float* pm = base + m * (2 + DV);
                if (t4 == 0) { pm[0] = mrun[m][half]; pm[1] = half ? (m ? l2B : l1B) : (m ? l2A : l1A); }
#pragma unroll
                for (int n = 0; n < DV / 8; ++n)
                    *reinterpret_cast<float2*>(pm + 2 + n * 8 + 2 * t4) = make_float2(O[m][n][2 * half], O[m][n][2 * half + 1]);
            }
        }
        return;
    }
    const float i1A = posA >= 0 ? 1.0f / l1A : 0.f, i1B = posB >= 0 ? 1.0f / l1B : 0.f;
    const float i2A = posA >= 0 ? lambda / l2A : 0.f, i2B = posB >= 0 ? lambda / l2B : 0.f;
    float ssA = 0.f, ssB = 0.f;
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
        O[0][n][0] = O[0][n][0] * i1A - O[1][n][0] * i2A;
        O[0][n][1] = O[0][n][1] * i1A - O[1][n][1] * i2A;
        O[0][n][2] = O[0][n][2] * i1B - O[1][n][2] * i2B;
        O[0][n][3] = O[0][n][3] * i1B - O[1][n][3] * i2B;
        ssA += O[0][n][0] * O[0][n][0] + O[0][n][1] * O[0][n][1];
        ssB += O[0][n][2] * O[0][n][2] + O[0][n][3] * O[0][n][3];
    }
    ssA = da_quad_sum(ssA);
    ssB = da_quad_sum(ssB);
    const float fA = out_scale / sqrtf(ssA / (float)DV + eps), fB = out_scale / sqrtf(ssB / (float)DV + eps);
    if (posA >= 0) {
        bf16* o = out + ((size_t)(t0 + rA / hpg) * H + g * hpg + rA % hpg) * DV;
#pragma unroll
        for (int n = 0; n < DV / 8; ++n)
            *reinterpret_cast<uint32_t*>(o + n * 8 + 2 * t4) = da_pack(O[0][n][0] * fA, O[0][n][1] * fA);
    }
    if (posB >= 0) {
        bf16* o = out + ((size_t)(t0 + rB / hpg) * H + g * hpg + rB % hpg) * DV;
#pragma unroll
        for (int n = 0; n < DV / 8; ++n)
            *reinterpret_cast<uint32_t*>(o + n * 8 + 2 * t4) = da_pack(O[0][n][2] * fB, O[0][n][3] * fB);
    }
}

// One block per (row of the step, head): the shares' maxima, sums and weighted values per map are put together, then
// out = out_scale * unit(a1 - lambda a2) as in the kernels above.  partial [T][H][nsplit][2][2 + dv] float32.
__global__ void __launch_bounds__(128) diff_attention_merge_kernel(const float* partial, bf16* out,
                                                                   const int* __restrict__ seq_of_token, int H, int dv,
                                                                   int nsplit, float lambda, float eps, float out_scale) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x, h = blockIdx.y;
    bf16* o = out + ((size_t)t * H + h) * dv;
    if (seq_of_token[t] < 0) {
        for (int i = threadIdx.x; i < dv; i += blockDim.x) o[i] = __float2bfloat16_rn(0.f);
        return;
    }
    const float* base = partial + ((size_t)t * H + h) * nsplit * 2 * (2 + dv);
    float M[2] = {-INFINITY, -INFINITY}, L[2] = {0.f, 0.f};
    for (int m = 0; m < 2; ++m) {
        for (int z = 0; z < nsplit; ++z) M[m] = fmaxf(M[m], base[(z * 2 + m) * (2 + dv)]);
        for (int z = 0; z < nsplit; ++z) {
            const float mz = base[(z * 2 + m) * (2 + dv)];
            if (mz != -INFINITY) L[m] += base[(z * 2 + m) * (2 + dv) + 1] * expf(mz - M[m]);
        }
    }
    // (dv <= 128 = the block: a thread owns one value)
    const int i = threadIdx.x;
    float df = 0.f;
    if (i < dv) {
        float a[2] = {0.f, 0.f};
        for (int m = 0; m < 2; ++m)
            for (int z = 0; z < nsplit; ++z) {
                const float mz = base[(z * 2 + m) * (2 + dv)];
                if (mz != -INFINITY) a[m] += base[(z * 2 + m) * (2 + dv) + 2 + i] * expf(mz - M[m]);
            }
        df = a[0] / L[0] - lambda * a[1] / L[1];
    }
    const float ss = block_sum(df * df, red);
    if (i < dv) o[i] = __float2bfloat16_rn(df * out_scale / sqrtf(ss / (float)dv + eps));
}

template <int D, int DV, bool WK>
static int da_mma_launch(const bf16* q, const bf16* k_pool, const bf16* v_pool, bf16* out, const int* positions,
                         const int* seq_of_token, const int* cu_seqlens, const int* page_table, int max_pages, int n_pages,
                         int ntok, int n_seqs, int H, int G, float scale, float cap, int window, float lambda, float eps,
                         float out_scale, int nsplit, float* partial, int* status, cudaStream_t stream) {
    const int hpg = H / G;
    const int tpt = (WK ? 16 : DA_ROWS) / hpg;
    size_t smem = ((size_t)DA_ROWS * (2 * D + 8) + 2 * DA_KEYS * (2 * D + 8) + 2 * DA_KEYS * (DV + 8)) * sizeof(bf16);
    if (WK) smem = max(smem, (size_t)4 * 16 * 2 * (2 + DV) * sizeof(float));      // the warps' shares, put together
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(diff_attention_mma_kernel<D, DV, WK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int tiles = (ntok + tpt - 1) / tpt + n_seqs;             // an upper bound on the sequences' tiles
    const int rc = gg_launch(diff_attention_mma_kernel<D, DV, WK>, dim3(tiles, G, nsplit), dim3(128), smem, stream, 1, q, k_pool,
                             v_pool, out, positions, seq_of_token, cu_seqlens, page_table, max_pages, n_seqs, H, G, hpg, tpt,
                             scale, cap, window, lambda, eps, out_scale, nsplit, partial, PageBounds{n_pages, status});
    if (rc != 0 || nsplit <= 1) return rc;
    return gg_launch(diff_attention_merge_kernel, dim3(ntok, H), dim3(128), 0, stream, 1, (const float*)partial, out,
                     seq_of_token, H, DV, nsplit, lambda, eps, out_scale);
}

// 1 if the tensor-core form takes these sizes (bfloat16 only), else 0.
GG_API gg_diff_attention_mma_takes(int H, int G, int d, int dv, int page_size) {
    const bool dims = (d == 32 || d == 64 || d == 128) && (dv == 32 || dv == 64 || dv == 128);
    return (dims && page_size == DA_KEYS && G > 0 && H % G == 0 && H / G <= DA_ROWS && G <= 65535) ? 1 : 0;
}

// As gg_diff_attention for bfloat16 tensors, with the step's cu_seqlens [n_seqs + 1].  max_new: the most rows one
// sequence brings (0: not known); where max_new * (H / G) <= 16 a tile holds 16 rows and its four warps share out every
// page's keys.  nsplit > 1 (steps of few
// rows and long contexts): every (tile, kv head) is the work of nsplit CTAs, each with a share of the key tiles, and a
// second kernel merges them; partial is scratch of ntok * H * nsplit * 2 * (2 + dv) floats.
GG_API gg_diff_attention_mma(const void* q, const void* k_pool, const void* v_pool, void* out, const int* positions,
                             const int* seq_of_token, const int* cu_seqlens, const int* page_table, int max_pages,
                             int page_size, int n_pages, int ntok, int n_seqs, int H, int G, int d, int dv, float scale,
                             float cap, int window, float lambda, float eps, float out_scale, int nsplit, float* partial,
                             int max_new, int* status, cudaStream_t stream) {
    if (ntok <= 0 || n_seqs <= 0) return 0;
    if (!gg_diff_attention_mma_takes(H, G, d, dv, page_size)) return GG_ERR_ARG;
    if (nsplit < 1 || nsplit > 64 || (nsplit > 1 && partial == nullptr)) return GG_ERR_ARG;
    const bool wk = max_new > 0 && max_new * (H / G) <= 16;
#define DA_ARGS (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out, positions, seq_of_token, cu_seqlens, \
        page_table, max_pages, n_pages, ntok, n_seqs, H, G, scale, cap, window, lambda, eps, out_scale, nsplit, partial, status, stream
#define DA_GO(D_, V_) return wk ? da_mma_launch<D_, V_, true>(DA_ARGS) : da_mma_launch<D_, V_, false>(DA_ARGS)
    if (d == 32) { if (dv == 32) DA_GO(32, 32); if (dv == 64) DA_GO(32, 64); DA_GO(32, 128); }
    if (d == 64) { if (dv == 32) DA_GO(64, 32); if (dv == 64) DA_GO(64, 64); DA_GO(64, 128); }
    if (dv == 32) DA_GO(128, 32);
    if (dv == 64) DA_GO(128, 64);
    DA_GO(128, 128);
#undef DA_GO
#undef DA_ARGS
}

// 1 if this library was built with checked page tables (the debug build), else 0.
GG_API gg_diff_attention_checked() { return gg_debug_bounds(); }
