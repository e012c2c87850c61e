// Latent attention over a paged cache of one vector per position.
//
// A layer of this kind caches, per position, a latent c (R elements, RMS-normed) and one rotated key part
// k_r (r elements) that all heads share: the row [c | k_r] of the pool.  Per head h the key is
// [W_uk,h c | k_r] and the value W_uv,h c.  Because both are linear in c, a query never needs them:
//
//   score(i, j) = scale * ( (W_uk,h^T q_plain,i) . c_j  +  q_rot,i . k_r,j )
//   out_h(i)    = W_uv,h * sum_j p(i, j) c_j
//
// so a step runs   prep (norm, rotation, cache write)  ->  absorb (q_lat = W_uk,h^T q_plain, a product per head)
// ->  attention over the rows of the pool with queries [q_lat | q_rot] of R + r elements, whose weighted sum of
// the rows' first R elements is the latent output  ->  expand (W_uv,h on the latent output, a product per head).
// Every head reads the same rows: one pass over a window of the cache serves all heads, in a prompt and in
// decoding alike, and the result does not depend on how a prompt was cut into steps.
//
// Kernels here: latent_prep, headwise_gemm (the per-head products, CUDA cores, any dtype mix),
// latent_attention_plain (one block per token and head, float32 arithmetic: the 32-bit path and the twin of
// the tensor-core kernel), latent_attention_mma (bfloat16, mma.sync, 64 query rows per CTA), and
// latent_prompt_mma: whole prompts in the expanded form (per-head keys and values built by a product).
// Scores, softmax, the norm and the rotation are float32 in all of them.
#include "common.cuh"

// ----------------------------------------------------------------------------- prep
// One block per token.  dkv[t] = [latent (R) | key part (r)] as the down projection left it; q[t] holds H heads
// of [plain (d) | rot (r)].  Writes pool row [rms(latent) * w | rotate(key part)] and qcat[t, h, R : R + r] =
// rotate(q rot part).  The rotation pairs element 2i with 2i+1 for i < dims / 2 and leaves the rest as it is;
// cos/sin[t, i] are the step's tables.  Padding tokens (seq_of_token < 0) write zeros to qcat and no cache.
template <typename T, typename TQ>
__global__ void __launch_bounds__(256) latent_prep_kernel(
    const T* q, long long ldq, const T* dkv, long long lddkv, const float* __restrict__ normw, float eps,
    const float* cosv, const float* sinv, int dims, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ page_table, int max_pages, int page_size,
    T* pool, int pool_row, TQ* qcat, int H, int d, int r, int R, const PageBounds pb, T* dense) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int b = seq_of_token[t];
    const int half = dims >> 1;
    TQ* qc = qcat + (size_t)t * H * (R + r);
    if (b < 0) {
        for (int i = threadIdx.x; i < H * r; i += blockDim.x) qc[(size_t)(i / r) * (R + r) + R + (i % r)] = from_f<TQ>(0.f);
        return;
    }
    const float* cs = cosv + (size_t)t * half;
    const float* sn = sinv + (size_t)t * half;
    // rotated part of every query head
    const T* qt = q + (size_t)t * ldq;
    for (int i = threadIdx.x; i < H * r; i += blockDim.x) {
        const int h = i / r, e = i % r;
        const T* src = qt + (size_t)h * (d + r) + d;
        float v = to_f<T>(src[e]);
        if (e < dims) {
            const float o = to_f<T>(src[e ^ 1]);
            const float c = cs[e >> 1], s = sn[e >> 1];
            v = (e & 1) ? v * c + o * s : v * c - o * s;
        }
        qc[(size_t)h * (R + r) + R + e] = from_f<TQ>(v);
    }
    if (pool == nullptr && dense == nullptr) return;
    const T* dk = dkv + (size_t)t * lddkv;
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) { const float v = to_f<T>(dk[i]); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float f = 1.0f / sqrtf(ss / (float)R + eps);
    const int pos = positions[t];
    T* row = nullptr;
    if (pool != nullptr) {
        const int page = gg_page_w(page_table + (size_t)b * max_pages, pos / page_size, max_pages, pb, 49);
        if (page >= 0) row = pool + ((size_t)page * page_size + (pos % page_size)) * pool_row;
    }
    T* drow = dense != nullptr ? dense + (size_t)t * (R + r) : nullptr;      // the same row, token by token
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const T v = from_f<T>(to_f<T>(dk[i]) * f * normw[i]);
        if (row != nullptr) row[i] = v;
        if (drow != nullptr) drow[i] = v;
    }
    for (int e = threadIdx.x; e < r; e += blockDim.x) {
        float v = to_f<T>(dk[R + e]);
        if (e < dims) {
            const float o = to_f<T>(dk[R + (e ^ 1)]);
            const float c = cs[e >> 1], s = sn[e >> 1];
            v = (e & 1) ? v * c + o * s : v * c - o * s;
        }
        if (row != nullptr) row[R + e] = from_f<T>(v);
        if (drow != nullptr) drow[R + e] = from_f<T>(v);
    }
}

// q, dkv and the pool share `dtype`; qcat has `q_dtype`.  pool may be null (a layer that reads another's cache).
// dense (may be null): [T, R + r] in `dtype`, the rows the cache gets, token by token.
GG_API gg_latent_prep(const void* q, long long ldq, const void* dkv, long long lddkv, int dtype, const float* normw,
                      float eps, const float* cosv, const float* sinv, int dims, const int* positions,
                      const int* seq_of_token, const int* page_table, int max_pages, int page_size, int n_pages,
                      void* pool, int pool_row, void* qcat, int q_dtype, int ntok, int H, int d, int r, int R,
                      void* dense, int* status, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (H <= 0 || d <= 0 || r < 0 || R <= 0 || dims < 0 || dims > r || (dims & 1) || pool_row < R + r || page_size <= 0)
        return GG_ERR_ARG;
    const PageBounds pb{n_pages, status};
#define GG_PREP(T, TQ) gg_launch(latent_prep_kernel<T, TQ>, dim3(ntok), dim3(256), 0, stream, 1, (const T*)q, ldq, \
        (const T*)dkv, lddkv, normw, eps, cosv, sinv, dims, positions, seq_of_token, page_table, max_pages, page_size, \
        (T*)pool, pool_row, (TQ*)qcat, H, d, r, R, pb, (T*)dense)
    if (dtype == GG_F32 && q_dtype == GG_F32) GG_PREP(float, float);
    else if (dtype == GG_BF16 && q_dtype == GG_F32) GG_PREP(bf16, float);
    else if (dtype == GG_BF16 && q_dtype == GG_BF16) GG_PREP(bf16, bf16);
    else return GG_ERR_DTYPE;
#undef GG_PREP
    return gg_last_error();
}

// ----------------------------------------------------------------------------- per-head products
// out[t, h, n] = alpha * sum_k x[t, h, k] * w[h, n, k] for h < H: H small products that share the token axis.
// x[t, h, k] is at x + t * ldx + h * hx + k, out[t, h, n] at out + t * ldo + h * ho + n, w[h] is [N, K] row-major.
// The sum over k runs in a fixed order that does not depend on the number of tokens.
#define HB 64
#define HK 16
template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256) headwise_gemm_kernel(const TX* x, long long ldx, long long hx,
                                                            const TW* __restrict__ w, TO* out, long long ldo,
                                                            long long ho, int M, int N, int K, float alpha) {
    pdl_launch();
    pdl_wait();
    __shared__ float xs[HK][HB + 1];
    __shared__ float ws[HK][HB + 1];
    const int h = blockIdx.z;
    const int m0 = blockIdx.y * HB, n0 = blockIdx.x * HB;
    const int tid = threadIdx.x;
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    const TX* xh = x + (size_t)h * hx;
    const TW* wh = w + (size_t)h * N * K;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int rr = idx / HK, kk = idx % HK;
            const int gk = k0 + kk;
            float xv = 0.f, wv = 0.f;
            if (gk < K) {
                if (m0 + rr < M) xv = to_f<TX>(xh[(size_t)(m0 + rr) * ldx + gk]);
                if (n0 + rr < N) wv = to_f<TW>(wh[(size_t)(n0 + rr) * K + gk]);
            }
            xs[kk][rr] = xv;
            ws[kk][rr] = wv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HK; ++kk) {
            float a[4], bq[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][tm + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bq[j] = ws[kk][tn + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bq[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n < N) out[(size_t)m * ldo + (size_t)h * ho + n] = from_f<TO>(acc[i][j] * alpha);
        }
    }
}

GG_API gg_headwise_gemm(const void* x, int x_dtype, long long ldx, long long hx, const void* w, int w_dtype,
                        void* out, int out_dtype, long long ldo, long long ho, int M, int N, int K, int H,
                        float alpha, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || H <= 0) return 0;
    if (K <= 0 || H > 65535 || (M + HB - 1) / HB > 65535) return GG_ERR_ARG;
    dim3 grid((N + HB - 1) / HB, (M + HB - 1) / HB, H);
#define GG_HW(TX, TW, TO) gg_launch(headwise_gemm_kernel<TX, TW, TO>, dim3(grid), dim3(256), 0, stream, 1, \
        (const TX*)x, ldx, hx, (const TW*)w, (TO*)out, ldo, ho, M, N, K, alpha)
    const int code = x_dtype * 4 + w_dtype * 2 + out_dtype;
    switch (code) {
        case 0: GG_HW(float, float, float); break;
        case 1: GG_HW(float, float, bf16); break;
        case 2: GG_HW(float, bf16, float); break;
        case 3: GG_HW(float, bf16, bf16); break;
        case 4: GG_HW(bf16, float, float); break;
        case 5: GG_HW(bf16, float, bf16); break;
        case 6: GG_HW(bf16, bf16, float); break;
        case 7: GG_HW(bf16, bf16, bf16); break;
        default: return GG_ERR_DTYPE;
    }
#undef GG_HW
    return gg_last_error();
}

// ----------------------------------------------------------------------------- attention, plain
// One block per (token, head).  The token at position p of sequence b reads the pool rows of positions lo..p,
// lo = max(0, p - window + 1) for a windowed layer (itself included: its row was written by latent_prep).
#define LAT_WARPS 4
#define LAT_MAXR 2048

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(LAT_WARPS * 32) latent_attention_plain_kernel(
    const TQ* qcat, const TC* pool, int pool_row, TO* out, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ page_table, int max_pages, int page_size,
    int H, int R, int r, float scale, int window, const PageBounds pb, const float* __restrict__ sink) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    const int D = R + r;
    float* qs = sm;                       // [D]
    float* accs = sm + D;                 // [LAT_WARPS][R]
    float* ml = accs + LAT_WARPS * R;     // [LAT_WARPS][2]
    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    TO* o = out + ((size_t)t * H + h) * R;
    const int b = seq_of_token[t];
    if (b < 0) {
        for (int i = threadIdx.x; i < R; i += blockDim.x) o[i] = from_f<TO>(0.f);
        return;
    }
    const int pos = positions[t];
    int lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    const TQ* qp = qcat + ((size_t)t * H + h) * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) qs[i] = to_f<TQ>(qp[i]);
    __syncthreads();
    float acc[LAT_MAXR / 32];
#pragma unroll
    for (int j = 0; j < LAT_MAXR / 32; ++j) acc[j] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int* pt = page_table + (size_t)b * max_pages;
    for (int j = lo + warp; j <= pos; j += LAT_WARPS) {
        const int page = gg_page(pt, j / page_size, max_pages, pb, 50);
        const TC* row = pool + ((size_t)page * page_size + (j % page_size)) * pool_row;
        float dot = 0.f;
        for (int i = lane; i < D; i += 32) dot = fmaf(qs[i], to_f<TC>(row[i]), dot);
        dot = warp_sum(dot) * scale;
        const float mn = fmaxf(m, dot);
        const float corr = expf(m - mn);
        const float p = expf(dot - mn);
        l = l * corr + p;
#pragma unroll
        for (int jj = 0; jj < LAT_MAXR / 32; ++jj) {
            const int i = lane + 32 * jj;
            if (i < R) acc[jj] = acc[jj] * corr + p * to_f<TC>(row[i]);
        }
        m = mn;
    }
#pragma unroll
    for (int jj = 0; jj < LAT_MAXR / 32; ++jj) {
        const int i = lane + 32 * jj;
        if (i < R) accs[warp * R + i] = acc[jj];
    }
    if (lane == 0) { ml[warp * 2] = m; ml[warp * 2 + 1] = l; }
    __syncthreads();
    float Mx = -INFINITY;
    for (int w = 0; w < LAT_WARPS; ++w) Mx = fmaxf(Mx, ml[w * 2]);
    if (sink != nullptr) Mx = fmaxf(Mx, sink[h]);
    float L = 0.f;
    float f[LAT_WARPS];
    for (int w = 0; w < LAT_WARPS; ++w) {
        f[w] = ml[w * 2] == -INFINITY ? 0.f : expf(ml[w * 2] - Mx);
        L += ml[w * 2 + 1] * f[w];
    }
    if (sink != nullptr) L += expf(sink[h] - Mx);         // the sink: one more term of the denominator, no value
    const float inv = 1.0f / L;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        float s = 0.f;
        for (int w = 0; w < LAT_WARPS; ++w) s += accs[w * R + i] * f[w];
        o[i] = from_f<TO>(s * inv);
    }
}

// qcat [T, H, R + r] in q_dtype, pool [page][page_size][pool_row] in c_dtype, out [T, H, R] in o_dtype.
GG_API gg_latent_attention_plain(const void* qcat, int q_dtype, const void* pool, int c_dtype, int pool_row, void* out,
                                 int o_dtype, const int* positions, const int* seq_of_token, const int* page_table,
                                 int max_pages, int page_size, int n_pages, int ntok, int H, int R, int r, float scale,
                                 int window, const float* sink, int* status, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (H <= 0 || H > 65535 || R <= 0 || R > LAT_MAXR || r < 0 || pool_row < R + r || page_size <= 0) return GG_ERR_ARG;
    const size_t smem = ((size_t)(R + r) + (size_t)LAT_WARPS * R + 2 * LAT_WARPS) * sizeof(float);
    if (smem > 48 * 1024) return GG_ERR_ARG;
    const PageBounds pb{n_pages, status};
    dim3 grid(ntok, H);
#define GG_LAP(TQ, TC, TO) gg_launch(latent_attention_plain_kernel<TQ, TC, TO>, dim3(grid), dim3(LAT_WARPS * 32), smem, \
        stream, 1, (const TQ*)qcat, (const TC*)pool, pool_row, (TO*)out, positions, seq_of_token, page_table, max_pages, \
        page_size, H, R, r, scale, window, pb, sink)
    if (q_dtype == GG_F32 && c_dtype == GG_F32 && o_dtype == GG_F32) GG_LAP(float, float, float);
    else if (q_dtype == GG_F32 && c_dtype == GG_BF16 && o_dtype == GG_F32) GG_LAP(float, bf16, float);
    else if (q_dtype == GG_BF16 && c_dtype == GG_BF16 && o_dtype == GG_BF16) GG_LAP(bf16, bf16, bf16);
    else return GG_ERR_DTYPE;
#undef GG_LAP
    return gg_last_error();
}

// ----------------------------------------------------------------------------- tensor-core helpers (mma.sync)
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void zero16(void* smem) { *reinterpret_cast<uint4*>(smem) = make_uint4(0u, 0u, 0u, 0u); }

// ----------------------------------------------------------------------------- per-head products on mma.sync
// The same contract as headwise_gemm_kernel for bfloat16 operands whose rows start on 16-byte boundaries
// (K, ldx and hx multiples of 8).  A CTA computes 64 tokens x 64 outputs of one head; x and w rows are staged
// 64 columns of k at a time (rows padded by 8 elements, so ldmatrix reads without bank conflicts).
#define HM_KS 64
#define HM_LD (HM_KS + 8)
template <typename TO>
__global__ void __launch_bounds__(128) headwise_mma_kernel(const bf16* x, long long ldx, long long hx,
                                                           const bf16* __restrict__ w, TO* out, long long ldo,
                                                           long long ho, int M, int N, int K, float alpha) {
    pdl_launch();
    __shared__ __align__(16) bf16 xs[64 * HM_LD];
    __shared__ __align__(16) bf16 ws[64 * HM_LD];
    const int h = blockIdx.z, m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bf16* xh = x + (size_t)h * hx;
    const bf16* wh = w + (size_t)h * N * K;
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    pdl_wait();
    for (int k0 = 0; k0 < K; k0 += HM_KS) {
        for (int c = tid; c < 64 * (HM_KS / 8); c += 128) {
            const int row = c / (HM_KS / 8), kc = (c % (HM_KS / 8)) * 8;
            bf16* dx = xs + row * HM_LD + kc;
            bf16* dw = ws + row * HM_LD + kc;
            if (m0 + row < M && k0 + kc < K) cp_async16(dx, xh + (size_t)(m0 + row) * ldx + k0 + kc); else zero16(dx);
            if (n0 + row < N && k0 + kc < K) cp_async16(dw, wh + (size_t)(n0 + row) * K + k0 + kc); else zero16(dw);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < HM_KS / 16; ++ks) {
            uint32_t a[4];
            ldsm_x4(a, xs + (warp * 16 + (lane & 15)) * HM_LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                ldsm_x4(b, ws + (np * 16 + (lane & 7) + (lane >> 4) * 8) * HM_LD + ks * 16 + ((lane >> 3) & 1) * 8);
                mma16816(acc[2 * np], a, b[0], b[1]);
                mma16816(acc[2 * np + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    const int g = lane >> 2, q4 = lane & 3;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        const int n = n0 + nt * 8 + 2 * q4;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int m = m0 + warp * 16 + g + half * 8;
            if (m >= M) continue;
            TO* o = out + (size_t)m * ldo + (size_t)h * ho + n;
            if (n < N) o[0] = from_f<TO>(acc[nt][2 * half] * alpha);
            if (n + 1 < N) o[1] = from_f<TO>(acc[nt][2 * half + 1] * alpha);
        }
    }
}

GG_API gg_headwise_gemm_mma(const void* x, long long ldx, long long hx, const void* w, void* out, int out_dtype,
                            long long ldo, long long ho, int M, int N, int K, int H, float alpha, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || H <= 0) return 0;
    if (K <= 0 || (K % 8) || (ldx % 8) || (hx % 8) || (((uintptr_t)x) & 15) || (((uintptr_t)w) & 15) || H > 65535 ||
        (M + 63) / 64 > 65535)
        return GG_ERR_ARG;
    dim3 grid((N + 63) / 64, (M + 63) / 64, H);
    GG_DISPATCH_DTYPE(out_dtype, TO,
        gg_launch(headwise_mma_kernel<TO>, dim3(grid), dim3(128), 0, stream, 1, (const bf16*)x, ldx, hx,
                  (const bf16*)w, (TO*)out, ldo, ho, M, N, K, alpha));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- attention on mma.sync
// A CTA of four warps takes 64 consecutive rows of one sequence's new (token, head) pairs, head fastest, so its
// rows belong to a few consecutive tokens and share one range of cached positions: from the first token's
// window start to the last token's own position.  That range is streamed in tiles of KT positions (cp.async, two
// stages); per tile S = Q K^T over all R + r columns (Q in shared memory, fragments by ldmatrix), the causal and
// window mask per row, an online softmax in float32, and O += P V where V is the first R columns of the very
// tile K was read from.  A CTA keeps RC columns of O in registers; a latent wider than RC is covered by
// gridDim.y CTAs that repeat the scores and own RC columns each.  Rows past the sequence's pairs are not written.
template <int KT, int RC>
__global__ void __launch_bounds__(128) latent_attention_mma_kernel(
    const bf16* qcat, const bf16* pool, int pool_row, bf16* out, const int* __restrict__ cu_seqlens,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ page_table,
    int max_pages, int page_size, int n_seqs, int H, int R, int r, float scale_log2, int window, const PageBounds pb,
    float* part_o, float* part_ml, int q_rows, const float* __restrict__ sink) {
    pdl_launch();
    extern __shared__ __align__(16) unsigned char smraw[];
    const int D = R + r, LD = D + 8;
    // q_rows (a multiple of 16, at most 64): the most rows a CTA of this launch can have; a decode step of few
    // heads keeps less shared memory for queries, so that more CTAs share an SM
    bf16* qs = reinterpret_cast<bf16*>(smraw);          // [q_rows][LD]
    bf16* ks = qs + q_rows * LD;                        // [2][KT][LD]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // which sequence and which 64 rows of it
    int b = 0, chunk = blockIdx.x, t0 = 0, n_new = 0;
    for (; b < n_seqs; ++b) {
        t0 = cu_seqlens[b];
        n_new = cu_seqlens[b + 1] - t0;
        const int chunks = (n_new * H + 63) / 64;
        if (chunk < chunks) break;
        chunk -= chunks;
    }
    if (b >= n_seqs) return;
    const int rows_total = n_new * H;
    const int f0 = chunk * 64;
    const int rows_here = min(64, rows_total - f0);
    const int z0 = blockIdx.y * RC;                      // first latent column of this CTA's share of O
    bf16* orow0 = out + ((size_t)t0 * H + f0) * R;
    pdl_wait();                                          // nothing is written, and no activation read, before this
    if (seq_of_token[t0] < 0) {                          // a padding sequence: zero rows
        for (int i = tid; i < rows_here * RC; i += 128) {
            const int c = z0 + i % RC;
            if (c < R) orow0[(size_t)(i / RC) * R + c] = __float2bfloat16_rn(0.f);
        }
        return;
    }
    const int tl0 = f0 / H, tl1 = (f0 + rows_here - 1) / H;
    const int pos0 = positions[t0 + tl0], pos1 = pos0 + (tl1 - tl0);
    int key_lo = 0;
    if (window > 0 && pos0 - window + 1 > 0) key_lo = pos0 - window + 1;
    int tile0 = key_lo / KT, ntiles = pos1 / KT - tile0 + 1;
    // gridDim.z > 1: the CTAs of one (rows, columns) share the range of tiles between them and leave partial sums
    const int splits = gridDim.z, split = blockIdx.z;
    if (splits > 1) {
        const int per = (ntiles + splits - 1) / splits;
        tile0 += split * per;
        ntiles = max(0, min(per, ntiles - split * per));
    }
    const int* pt = page_table + (size_t)b * max_pages;
    const int chunks_per_row = D / 8;

    // a warp copies whole rows (one page look-up per row and lane), its lanes the rows' 16-byte pieces
    auto load_keys = [&](int tile, int stage) {
        bf16* dst = ks + (size_t)stage * KT * LD;
        const int j0 = tile * KT;
        for (int kk = warp; kk < KT; kk += 4) {
            const int j = j0 + kk;
            bf16* d = dst + kk * LD;
            if (j <= pos1) {
                const int page = gg_page(pt, j / page_size, max_pages, pb, 51);
                const bf16* src = pool + ((size_t)page * page_size + (j % page_size)) * pool_row;
                for (int c = lane; c < chunks_per_row; c += 32) cp_async16(d + c * 8, src + c * 8);
            } else {
                for (int c = lane; c < chunks_per_row; c += 32) zero16(d + c * 8);
            }
        }
    };
    {   // the queries of this CTA: rows_here consecutive rows of qcat
        const bf16* qsrc = qcat + ((size_t)t0 * H + f0) * D;
        for (int row = warp; row < q_rows; row += 4) {
            bf16* d = qs + row * LD;
            if (row < rows_here) {
                for (int c = lane; c < chunks_per_row; c += 32) cp_async16(d + c * 8, qsrc + (size_t)row * D + c * 8);
            } else {
                for (int c = lane; c < chunks_per_row; c += 32) zero16(d + c * 8);
            }
        }
    }
    if (ntiles > 0) load_keys(tile0, 0);
    cp_async_commit();

    const int g = lane >> 2, q4 = lane & 3;
    int prow[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int f = f0 + warp * 16 + g + 8 * i;
        valid[i] = f < rows_total;
        prow[i] = pos0 + (f / H - tl0);
    }
    float o[RC / 8][4];
#pragma unroll
    for (int i = 0; i < RC / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
    const int ksteps = D / 16;
    const int ocols = min(RC, R - z0);                   // columns of O this CTA owns (a multiple of 16)

    for (int it = 0; it < ntiles; ++it) {
        if (it + 1 < ntiles) {
            load_keys(tile0 + it + 1, (it + 1) & 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* kt = ks + (size_t)(it & 1) * KT * LD;
        if (warp * 16 < rows_here) {                     // a warp without rows (decode steps of few heads) only copies
        float s[KT / 8][4];
#pragma unroll
        for (int i = 0; i < KT / 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
        for (int kk = 0; kk < ksteps; ++kk) {
            uint32_t a[4];
            ldsm_x4(a, qs + (warp * 16 + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int np = 0; np < KT / 16; ++np) {
                uint32_t bb[4];
                ldsm_x4(bb, kt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
                mma16816(s[2 * np], a, bb[0], bb[1]);
                mma16816(s[2 * np + 1], a, bb[2], bb[3]);
            }
        }
        // mask, running maximum and sum (two rows per thread; a row's 4 threads hold its KT scores)
        const int j0 = (tile0 + it) * KT;
        float mnew[2] = {mrow[0], mrow[1]};
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = e >> 1;
                const int j = j0 + nt * 8 + 2 * q4 + (e & 1);
                const bool see = valid[i] && j <= prow[i] && (window <= 0 || j > prow[i] - window);
                const float v = see ? s[nt][e] * scale_log2 : -INFINITY;
                s[nt][e] = v;
                mnew[i] = fmaxf(mnew[i], v);
            }
        float corr[2], muse[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mnew[i] = fmaxf(mnew[i], __shfl_xor_sync(0xffffffffu, mnew[i], 1));
            mnew[i] = fmaxf(mnew[i], __shfl_xor_sync(0xffffffffu, mnew[i], 2));
            muse[i] = mnew[i] == -INFINITY ? 0.f : mnew[i];
            corr[i] = exp2f(mrow[i] - muse[i]);          // 0 while the row has seen nothing
            mrow[i] = mnew[i];
            lrow[i] *= corr[i];
        }
        uint32_t pfrag[KT / 16][4];
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt) {
            const float p0 = exp2f(s[nt][0] - muse[0]), p1 = exp2f(s[nt][1] - muse[0]);
            const float p2 = exp2f(s[nt][2] - muse[1]), p3 = exp2f(s[nt][3] - muse[1]);
            lrow[0] += p0 + p1;
            lrow[1] += p2 + p3;
            // the C fragments of two neighbouring 8-key tiles are the A fragment of one 16-key step
            pfrag[nt >> 1][(nt & 1) * 2] = pack_bf16(p0, p1);
            pfrag[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int i = 0; i < RC / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        // O += P V, V[key][col] = tile[key][z0 + col]
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
#pragma unroll
            for (int np = 0; np < RC / 16; ++np) {
                if (np * 16 < ocols) {
                    uint32_t bb[4];
                    ldsm_x4_trans(bb, kt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + z0 + np * 16 + (lane >> 4) * 8);
                    mma16816(o[2 * np], pfrag[kk], bb[0], bb[1]);
                    mma16816(o[2 * np + 1], pfrag[kk], bb[2], bb[3]);
                }
            }
        }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    // the row sums live in the 4 threads of a row
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 1);
        lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 2);
    }
    if (splits > 1) {
        // partial result of this share of the keys: unnormalised sums, the running maximum (log2 units) and the sum
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (!valid[i]) continue;
            const size_t row = (size_t)t0 * H + f0 + warp * 16 + g + 8 * i;
            float* po = part_o + (row * splits + split) * R + z0;
#pragma unroll
            for (int nt = 0; nt < RC / 8; ++nt) {
                const int c = nt * 8 + 2 * q4;
                if (c < ocols) *reinterpret_cast<float2*>(po + c) = make_float2(o[nt][2 * i], o[nt][2 * i + 1]);
            }
            if (q4 == 0 && blockIdx.y == 0) {
                part_ml[(row * splits + split) * 2] = mrow[i];
                part_ml[(row * splits + split) * 2 + 1] = lrow[i];
            }
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (!valid[i]) continue;
        if (sink != nullptr)             // the sink joins the denominator (scores are in log2 units here)
            lrow[i] += exp2f(sink[(f0 + warp * 16 + g + 8 * i) % H] * 1.4426950408889634f - mrow[i]);
        const float inv = 1.0f / lrow[i];
        bf16* orow = orow0 + (size_t)(warp * 16 + g + 8 * i) * R + z0;
#pragma unroll
        for (int nt = 0; nt < RC / 8; ++nt) {
            const int c = nt * 8 + 2 * q4;
            if (c < ocols)
                *reinterpret_cast<uint32_t*>(orow + c) = pack_bf16(o[nt][2 * i] * inv, o[nt][2 * i + 1] * inv);
        }
    }
}

template <int KT, int RC>
static int launch_latent_mma(const void* qcat, const void* pool, int pool_row, void* out, const int* cu_seqlens,
                             const int* positions, const int* seq_of_token, const int* page_table, int max_pages,
                             int page_size, int n_seqs, int ntok, int H, int R, int r, float scale, int window,
                             const PageBounds pb, int splits, float* part_o, float* part_ml, int q_rows, const float* sink,
                             cudaStream_t stream) {
    const size_t smem = (size_t)(q_rows + 2 * KT) * (R + r + 8) * sizeof(bf16);
    auto kern = latent_attention_mma_kernel<KT, RC>;
    static bool attr_set = false;                        // per instantiation
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    const long long chunks = ((long long)ntok * H + 63) / 64 + n_seqs;
    dim3 grid((unsigned)chunks, (R + RC - 1) / RC, splits);
    return gg_launch(kern, dim3(grid), dim3(128), smem, stream, 1, (const bf16*)qcat, (const bf16*)pool, pool_row,
                     (bf16*)out, cu_seqlens, positions, seq_of_token, page_table, max_pages, page_size, n_seqs, H, R, r,
                     scale * 1.4426950408889634f, window, pb, part_o, part_ml, q_rows, sink);
}

// Merge of the partial results of a split: one block per (token, head) row.
__global__ void __launch_bounds__(128) latent_combine_kernel(const float* part_o, const float* part_ml, bf16* out,
                                                             const int* __restrict__ seq_of_token, int H, int R, int splits,
                                                             const float* __restrict__ sink) {
    pdl_launch();
    pdl_wait();
    const size_t row = blockIdx.x;
    if (seq_of_token[row / H] < 0) return;               // the attention kernel wrote the zero rows of padding itself
    const float* ml = part_ml + row * splits * 2;
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, ml[2 * s]);
    const float sk = sink != nullptr ? sink[row % H] * 1.4426950408889634f : -INFINITY;
    M = fmaxf(M, sk);
    float L = sink != nullptr ? exp2f(sk - M) : 0.f;
    for (int s = 0; s < splits; ++s) L += ml[2 * s] == -INFINITY ? 0.f : exp2f(ml[2 * s] - M) * ml[2 * s + 1];
    const float inv = 1.0f / L;
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float m = ml[2 * s];
            if (m != -INFINITY) acc = fmaf(exp2f(m - M), part_o[(row * splits + s) * R + c], acc);
        }
        out[row * R + c] = __float2bfloat16_rn(acc * inv);
    }
}

// How many shares of the keys a step's attention is cut into: 1 unless the step has too few CTAs to fill the
// GPU (decode steps of small batches); bounded by the tiles a window holds and by `max_splits`.
GG_API gg_latent_attention_mma_splits(int n_seqs, int ntok, int H, int R, int r, int window, int max_ctx) {
    // CTAs that have rows: a decode step (one token a sequence) has ceil(H / 64) per sequence, a prompt about
    // ntok * H / 64; each times the CTAs that share a wide latent's columns
    const long long row_ctas = ntok == n_seqs ? (long long)n_seqs * ((H + 63) / 64) : ((long long)ntok * H + 63) / 64;
    const long long ctas = row_ctas * ((R + 255) / 256);
    const bool wide = (size_t)(64 + 2 * 64) * (R + r + 8) * sizeof(bf16) <= 200 * 1024;
    const int kt = wide ? 64 : 32;
    const int keys = window > 0 && window < max_ctx ? window + 1 : max_ctx;
    const int tiles = (keys + kt - 1) / kt + 1;
    static int target = -1;                              // CTAs a step should have; GOGGUF_B200_LATENT_SPLIT_CTAS overrides
    if (target < 0) {
        const char* e = getenv("GOGGUF_B200_LATENT_SPLIT_CTAS");
        target = e != nullptr && atoi(e) > 0 ? atoi(e) : 3 * 148 / 2;       // measured best of 1.5, 2, 3 and 4 per SM
    }
    if (ctas >= target) return 1;
    long long s = (target + ctas - 1) / ctas;
    if (s > tiles) s = tiles;
    if (s > 32) s = 32;
    return s < 1 ? 1 : (int)s;
}

// Does the tensor-core kernel take these sizes?  R and r multiples of 16, the staged tiles within shared memory.
GG_API gg_latent_attention_mma_takes(int R, int r) {
    if (R <= 0 || r < 0 || (R % 16) || (r % 16)) return 0;
    return (size_t)(64 + 2 * 32) * (R + r + 8) * sizeof(bf16) <= 200 * 1024 ? 1 : 0;
}

// qcat [T, H, R + r], pool [page][page_size][pool_row], out [T, H, R], all bfloat16; cu_seqlens [n_seqs + 1].
// splits > 1: part_o [T * H, splits, R] and part_ml [T * H, splits, 2] (float32) take the shares' partial results
// and a second kernel merges them.  max_new: the most new tokens any sequence of the step brings.
GG_API gg_latent_attention_mma(const void* qcat, const void* pool, int pool_row, void* out, const int* cu_seqlens,
                               const int* positions, const int* seq_of_token, const int* page_table, int max_pages,
                               int page_size, int n_pages, int n_seqs, int ntok, int H, int R, int r, float scale,
                               int window, int splits, float* part_o, float* part_ml, int max_new, const float* sink,
                               int* status, cudaStream_t stream) {
    if (ntok <= 0 || n_seqs <= 0) return 0;
    if (!gg_latent_attention_mma_takes(R, r) || H <= 0 || (pool_row % 8) || pool_row < R + r || page_size <= 0 ||
        (page_size % 64) || (((uintptr_t)qcat | (uintptr_t)pool | (uintptr_t)out) & 15))
        return GG_ERR_ARG;
    const PageBounds pb{n_pages, status};
    const bool wide = (size_t)(64 + 2 * 64) * (R + r + 8) * sizeof(bf16) <= 200 * 1024;     // room for 64-key tiles
#define GG_LM(KT, RC) launch_latent_mma<KT, RC>(qcat, pool, pool_row, out, cu_seqlens, positions, seq_of_token, page_table, \
        max_pages, page_size, n_seqs, ntok, H, R, r, scale, window, pb, splits, part_o, part_ml, q_rows, sink, stream)
    if (splits < 1 || (splits > 1 && (part_o == nullptr || part_ml == nullptr)) || max_new < 1) return GG_ERR_ARG;
    // the most rows one CTA can have: 64, or all (token, head) pairs of the longest new stretch if those are fewer
    const long long most = (long long)max_new * H;
    const int q_rows = most >= 64 ? 64 : (int)((most + 15) / 16 * 16);
    int rc;
    if (R <= 64) rc = wide ? GG_LM(64, 64) : GG_LM(32, 64);
    else if (R <= 128) rc = wide ? GG_LM(64, 128) : GG_LM(32, 128);
    else rc = wide ? GG_LM(64, 256) : GG_LM(32, 256);
#undef GG_LM
    if (rc != 0 || splits == 1) return rc;
    return gg_launch(latent_combine_kernel, dim3((unsigned)(ntok * H)), dim3(128), 0, stream, 1, (const float*)part_o,
                     (const float*)part_ml, (bf16*)out, seq_of_token, H, R, splits, sink);
}

// ----------------------------------------------------------------------------- attention of whole prompts, expanded
// A step in which every sequence starts at position 0 holds all the keys it reads among its own tokens, so the
// per-head keys [W_uk,h c | k_r] and values W_uv,h c can be made once by a product (kv[t] = [all heads' plain keys |
// all heads' values]) and attention runs in the ordinary form: per (query, key, head) d + r + dv multiply-adds
// instead of 2 R + r, and O is only dv wide, so many warps share an SM.  A CTA takes 64 consecutive tokens of one
// sequence and one head; key tiles of 64 tokens come from the step's own rows (no page table), the rotated key part
// from the dense copy latent_prep leaves.  Scores, softmax and sums in float32; the output is written per head into
// av[t, h, :] already multiplied by `out_scale`.
template <int DVT>
__global__ void __launch_bounds__(128) latent_prompt_mma_kernel(
    const bf16* qd, long long ldq, const bf16* qcat, const bf16* kv, long long ldkv, const bf16* ckr, long long ldc,
    bf16* av, const int* __restrict__ cu_seqlens, const int* __restrict__ seq_of_token, int n_seqs, int H, int d, int r,
    int dv, int R, float scale_log2, int window, float out_scale, const float* __restrict__ sink) {
    pdl_launch();
    extern __shared__ __align__(16) unsigned char smraw[];
    constexpr int KT = 64;
    const int dq = d + r, LQ = dq + 8, LV = dv + 8;
    bf16* qs = reinterpret_cast<bf16*>(smraw);          // [64][LQ]
    bf16* ks = qs + 64 * LQ;                            // [2][KT][LQ]
    bf16* vs = ks + 2 * KT * LQ;                        // [2][KT][LV]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y;
    int b = 0, chunk = blockIdx.x, t0 = 0, n_new = 0;
    for (; b < n_seqs; ++b) {
        t0 = cu_seqlens[b];
        n_new = cu_seqlens[b + 1] - t0;
        const int chunks = (n_new + 63) / 64;
        if (chunk < chunks) break;
        chunk -= chunks;
    }
    if (b >= n_seqs) return;
    const int p0 = chunk * 64;                           // first position of this CTA's queries (positions start at 0)
    const int rows_here = min(64, n_new - p0);
    pdl_wait();
    if (seq_of_token[t0] < 0) {                          // a padding sequence: zero rows
        for (int i = tid; i < rows_here * dv; i += 128)
            av[((size_t)(t0 + p0 + i / dv) * H + h) * dv + i % dv] = __float2bfloat16_rn(0.f);
        return;
    }
    const int p1 = p0 + rows_here - 1;
    int key_lo = 0;
    if (window > 0 && p0 - window + 1 > 0) key_lo = p0 - window + 1;
    const int tile0 = key_lo / KT, ntiles = p1 / KT - tile0 + 1;
    const int cq_plain = d / 8, cq = dq / 8, cv = dv / 8;

    auto load_keys = [&](int tile, int stage) {
        bf16* kd = ks + (size_t)stage * KT * LQ;
        bf16* vd = vs + (size_t)stage * KT * LV;
        const int j0 = tile * KT;
        for (int kk = warp; kk < KT; kk += 4) {
            const int j = j0 + kk;
            bf16* dk = kd + kk * LQ;
            bf16* dvp = vd + kk * LV;
            if (j <= p1) {
                const bf16* kp = kv + (size_t)(t0 + j) * ldkv + (size_t)h * d;           // this head's plain key
                const bf16* kr = ckr + (size_t)(t0 + j) * ldc + R;                       // the shared rotated part
                const bf16* vp = kv + (size_t)(t0 + j) * ldkv + (size_t)H * d + (size_t)h * dv;
                for (int c = lane; c < cq; c += 32)
                    cp_async16(dk + c * 8, c < cq_plain ? kp + c * 8 : kr + (c - cq_plain) * 8);
                for (int c = lane; c < cv; c += 32) cp_async16(dvp + c * 8, vp + c * 8);
            } else {
                for (int c = lane; c < cq; c += 32) zero16(dk + c * 8);
                for (int c = lane; c < cv; c += 32) zero16(dvp + c * 8);
            }
        }
    };
    for (int row = warp; row < 64; row += 4) {           // queries: plain part from the product, rotated part from prep
        bf16* dst = qs + row * LQ;
        if (row < rows_here) {
            const bf16* qp = qd + (size_t)(t0 + p0 + row) * ldq + (size_t)h * dq;
            const bf16* qr = qcat + ((size_t)(t0 + p0 + row) * H + h) * (R + r) + R;
            for (int c = lane; c < cq; c += 32) cp_async16(dst + c * 8, c < cq_plain ? qp + c * 8 : qr + (c - cq_plain) * 8);
        } else {
            for (int c = lane; c < cq; c += 32) zero16(dst + c * 8);
        }
    }
    load_keys(tile0, 0);
    cp_async_commit();

    const int g = lane >> 2, q4 = lane & 3;
    int prow[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int rr = warp * 16 + g + 8 * i;
        valid[i] = rr < rows_here;
        prow[i] = p0 + rr;
    }
    float o[DVT / 8][4];
#pragma unroll
    for (int i = 0; i < DVT / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
    const int ksteps = dq / 16;

    for (int it = 0; it < ntiles; ++it) {
        if (it + 1 < ntiles) {
            load_keys(tile0 + it + 1, (it + 1) & 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (warp * 16 < rows_here) {
            const bf16* kt = ks + (size_t)(it & 1) * KT * LQ;
            const bf16* vt = vs + (size_t)(it & 1) * KT * LV;
            float s[KT / 8][4];
#pragma unroll
            for (int i = 0; i < KT / 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
            for (int kk = 0; kk < ksteps; ++kk) {
                uint32_t a[4];
                ldsm_x4(a, qs + (warp * 16 + (lane & 15)) * LQ + kk * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int np = 0; np < KT / 16; ++np) {
                    uint32_t bb[4];
                    ldsm_x4(bb, kt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LQ + kk * 16 + ((lane >> 3) & 1) * 8);
                    mma16816(s[2 * np], a, bb[0], bb[1]);
                    mma16816(s[2 * np + 1], a, bb[2], bb[3]);
                }
            }
            const int j0 = (tile0 + it) * KT;
            float mnew[2] = {mrow[0], mrow[1]};
#pragma unroll
            for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1;
                    const int j = j0 + nt * 8 + 2 * q4 + (e & 1);
                    const bool see = valid[i] && j <= prow[i] && (window <= 0 || j > prow[i] - window);
                    const float v = see ? s[nt][e] * scale_log2 : -INFINITY;
                    s[nt][e] = v;
                    mnew[i] = fmaxf(mnew[i], v);
                }
            float corr[2], muse[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mnew[i] = fmaxf(mnew[i], __shfl_xor_sync(0xffffffffu, mnew[i], 1));
                mnew[i] = fmaxf(mnew[i], __shfl_xor_sync(0xffffffffu, mnew[i], 2));
                muse[i] = mnew[i] == -INFINITY ? 0.f : mnew[i];
                corr[i] = exp2f(mrow[i] - muse[i]);
                mrow[i] = mnew[i];
                lrow[i] *= corr[i];
            }
            uint32_t pfrag[KT / 16][4];
#pragma unroll
            for (int nt = 0; nt < KT / 8; ++nt) {
                const float p0f = exp2f(s[nt][0] - muse[0]), p1f = exp2f(s[nt][1] - muse[0]);
                const float p2f = exp2f(s[nt][2] - muse[1]), p3f = exp2f(s[nt][3] - muse[1]);
                lrow[0] += p0f + p1f;
                lrow[1] += p2f + p3f;
                pfrag[nt >> 1][(nt & 1) * 2] = pack_bf16(p0f, p1f);
                pfrag[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2f, p3f);
            }
#pragma unroll
            for (int i = 0; i < DVT / 8; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
#pragma unroll
            for (int kk = 0; kk < KT / 16; ++kk) {
#pragma unroll
                for (int np = 0; np < DVT / 16; ++np) {
                    if (np * 16 < dv) {
                        uint32_t bb[4];
                        ldsm_x4_trans(bb, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LV + np * 16 + (lane >> 4) * 8);
                        mma16816(o[2 * np], pfrag[kk], bb[0], bb[1]);
                        mma16816(o[2 * np + 1], pfrag[kk], bb[2], bb[3]);
                    }
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 1);
        lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 2);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (!valid[i]) continue;
        if (sink != nullptr) lrow[i] += exp2f(sink[h] * 1.4426950408889634f - mrow[i]);
        const float inv = out_scale / lrow[i];
        bf16* orow = av + ((size_t)(t0 + prow[i]) * H + h) * dv;
#pragma unroll
        for (int nt = 0; nt < DVT / 8; ++nt) {
            const int c = nt * 8 + 2 * q4;
            if (c < dv) *reinterpret_cast<uint32_t*>(orow + c) = pack_bf16(o[nt][2 * i] * inv, o[nt][2 * i + 1] * inv);
        }
    }
}

// Does the expanded prompt kernel take these sizes?  Plain, rotated and value sizes whose rows and split points fall
// on 16-byte boundaries, d + r and dv multiples of 16, dv at most 128, d + r at most 256.
GG_API gg_latent_prompt_mma_takes(int d, int r, int dv) {
    return (d > 0 && r >= 0 && dv > 0 && d % 8 == 0 && r % 8 == 0 && (d + r) % 16 == 0 && dv % 16 == 0 && dv <= 128 &&
            d + r <= 256) ? 1 : 0;
}

// qd [T, >= H (d + r)] (row stride ldq; head h's plain query at h (d + r)), qcat [T, H, R + r] (rotated query parts
// at [..., R:]), kv [T, H d + H dv] (row stride ldkv), ckr [T, R + r] (row stride ldc; rotated key part at R),
// av [T, H, dv]; every sequence of the step starts at position 0.
GG_API gg_latent_prompt_mma(const void* qd, long long ldq, const void* qcat, const void* kv, long long ldkv,
                            const void* ckr, long long ldc, void* av, const int* cu_seqlens, const int* seq_of_token,
                            int n_seqs, int ntok, int H, int d, int r, int dv, int R, float scale, int window,
                            float out_scale, const float* sink, cudaStream_t stream) {
    if (ntok <= 0 || n_seqs <= 0) return 0;
    if (!gg_latent_prompt_mma_takes(d, r, dv) || H <= 0 || H > 65535 || (ldq % 8) || (ldkv % 8) || (ldc % 8) ||
        ((R + r) % 8) || (R % 8) || ((H * d) % 8) ||
        (((uintptr_t)qd | (uintptr_t)qcat | (uintptr_t)kv | (uintptr_t)ckr | (uintptr_t)av) & 15))
        return GG_ERR_ARG;
    const size_t smem = ((size_t)(64 + 2 * 64) * (d + r + 8) + (size_t)2 * 64 * (dv + 8)) * sizeof(bf16);
    dim3 grid((unsigned)(ntok / 64 + n_seqs), H);
    const float sl2 = scale * 1.4426950408889634f;
    if (dv <= 64) {
        auto kern = latent_prompt_mma_kernel<64>;
        static bool set = false;
        if (!set) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            if (e != cudaSuccess) return (int)e;
            set = true;
        }
        return gg_launch(kern, dim3(grid), dim3(128), smem, stream, 1, (const bf16*)qd, ldq, (const bf16*)qcat, (const bf16*)kv,
                         ldkv, (const bf16*)ckr, ldc, (bf16*)av, cu_seqlens, seq_of_token, n_seqs, H, d, r, dv, R, sl2, window,
                         out_scale, sink);
    }
    auto kern = latent_prompt_mma_kernel<128>;
    static bool set2 = false;
    if (!set2) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (e != cudaSuccess) return (int)e;
        set2 = true;
    }
    return gg_launch(kern, dim3(grid), dim3(128), smem, stream, 1, (const bf16*)qd, ldq, (const bf16*)qcat, (const bf16*)kv, ldkv,
                     (const bf16*)ckr, ldc, (bf16*)av, cu_seqlens, seq_of_token, n_seqs, H, d, r, dv, R, sl2, window, out_scale, sink);
}

GG_API gg_latent_attention_checked() { return gg_debug_bounds(); }
