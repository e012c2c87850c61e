// Row-wise and element-wise kernels: embedding gather, RMSNorm, rotary tables,
// fused per-head QK-norm + rotary + cache write, SwiGLU, residual add, row statistics.
//
// They replace the reference's rmsnorm / rope_heads / swiglu / add_inplace PTX
// kernels (pkg/gpu/cuda/ptx.go:428-496, 498-564, 634-677, 891-924), which run
// one vector per launch; these run every token of a step in one launch.
// Reductions, the inverse root, the rotation and the SiLU are done in float32
// (angles in float64); the residual stream is float32 in both precisions.
#include "common.cuh"

// ----------------------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* tokens,
                                    float* __restrict__ out, int H, int V, float scale) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const int tok = tokens[t];
    float* o = out + (size_t)t * H;
    if (tok < 0 || tok >= V) {  // padding row
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const TW* r = table + (size_t)tok * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f<TW>(r[i]) * scale;
}

GG_API gg_embed_gather(const void* table, int table_dtype, const int* tokens, float* out,
                       int T, int H, int V, float scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || V <= 0) return GG_ERR_ARG;
    GG_DISPATCH_DTYPE(table_dtype, TW,
        gg_launch(embed_gather_kernel<TW>, dim3(T), dim3(256), 0, stream, 1, (const TW*)table, tokens, out, H, V, scale));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- RMSNorm
// out[r,:] = x[src(r),:] * (1/sqrt(mean(x^2)+eps)) * w ; src(r) = rows ? rows[r] : r.
// x is the float32 residual stream.  A negative source row gives a zero row.
template <typename TO>
__global__ void rmsnorm_kernel(const float* x, const int* __restrict__ rows,
                               const float* __restrict__ w, TO* __restrict__ out, int H, float eps) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    TO* o = out + (size_t)r * H;
    if (src < 0) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f<TO>(0.f);
        return;
    }
    const float* xr = x + (size_t)src * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { float v = xr[i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f<TO>(xr[i] * scale * w[i]);
}

// Same result for rows of up to 8192 floats whose length is a multiple of 4: the row is read once with
// 16-byte loads that are all in flight together and kept in registers for the second pass.  In a
// decode step only a few rows exist, so the kernel's time is one memory latency, not two loops of them.
template <typename TO, int VPT /* float4 per thread */>
__global__ void __launch_bounds__(256) rmsnorm_vec_kernel(const float* x, const int* __restrict__ rows,
                                                          const float* __restrict__ w, TO* __restrict__ out, int H, float eps) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    TO* o = out + (size_t)r * H;
    const int nvec = H >> 2;
    float4 v[VPT];
    float ss = 0.f;
    if (src >= 0) {
        const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * H);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = threadIdx.x + j * 256;
            v[j] = i < nvec ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
            ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
        }
    } else {
#pragma unroll
        for (int j = 0; j < VPT; ++j) v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    ss = block_sum(ss, red);
    const float scale = src >= 0 ? 1.0f / sqrtf(ss / (float)H + eps) : 0.f;
    const float4* wr = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i < nvec) {
            const float4 ww = wr[i];
            const float a = v[j].x * scale * ww.x, b = v[j].y * scale * ww.y;
            const float c = v[j].z * scale * ww.z, d = v[j].w * scale * ww.w;
            if (sizeof(TO) == 4) {
                reinterpret_cast<float4*>(o)[i] = make_float4(a, b, c, d);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo);
                pk.y = *reinterpret_cast<uint32_t*>(&hi);
                reinterpret_cast<uint2*>(o)[i] = pk;
            }
        }
    }
}

GG_API gg_rmsnorm(const float* x, const int* rows, const float* w, void* out, int out_dtype,
                  int R, int H, float eps, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (H <= 0) return GG_ERR_ARG;
    const bool aligned = (H % 4 == 0) && ((((uintptr_t)x) & 15) == 0) && ((((uintptr_t)w) & 15) == 0) &&
                         ((((uintptr_t)out) & 15) == 0);
    if (aligned && H <= 8192) {
        const int vpt = (H / 4 + 255) / 256;     // 1..8
        GG_DISPATCH_DTYPE(out_dtype, TO, {
            if (vpt <= 1) gg_launch(rmsnorm_vec_kernel<TO, 1>, dim3(R), dim3(256), 0, stream, 1, x, rows, w, (TO*)out, H, eps);
            else if (vpt <= 2) gg_launch(rmsnorm_vec_kernel<TO, 2>, dim3(R), dim3(256), 0, stream, 1, x, rows, w, (TO*)out, H, eps);
            else if (vpt <= 4) gg_launch(rmsnorm_vec_kernel<TO, 4>, dim3(R), dim3(256), 0, stream, 1, x, rows, w, (TO*)out, H, eps);
            else gg_launch(rmsnorm_vec_kernel<TO, 8>, dim3(R), dim3(256), 0, stream, 1, x, rows, w, (TO*)out, H, eps);
        });
        return gg_last_error();
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    GG_DISPATCH_DTYPE(out_dtype, TO,
        gg_launch(rmsnorm_kernel<TO>, dim3(R), dim3(threads), 0, stream, 1, x, rows, w, (TO*)out, H, eps));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- row statistics
// What a product with a folded RMSNorm reads instead of the normalised rows: xhat = bfloat16(x) and,
// per row, the sums of squares over blocks of 128 columns (ceil(H / 128) partial sums).  The products
// that add into the residual stream write both themselves; this kernel makes them where no such
// product came before (after the embedding, after a part that does not emit them).
__global__ void __launch_bounds__(128) row_stats_kernel(const float* x, bf16* __restrict__ xhat,
                                                        float* __restrict__ ssq, int H, int parts) {
    pdl_launch();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int part = blockIdx.y * 4 + (threadIdx.x >> 5);
    const int t = blockIdx.x;
    if (part >= parts) return;
    const int c0 = part * 128 + lane * 4;
    const float* xr = x + (size_t)t * H + c0;
    bf16* hr = xhat + (size_t)t * H + c0;
    float ss = 0.f;
    if (c0 + 4 <= H && ((((uintptr_t)xr) & 15) == 0) && ((((uintptr_t)hr) & 7) == 0)) {
        const float4 v = *reinterpret_cast<const float4*>(xr);
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(hr) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
    } else {
        for (int j = 0; j < 4; ++j)
            if (c0 + j < H) { const float v = xr[j]; ss = fmaf(v, v, ss); hr[j] = __float2bfloat16_rn(v); }
    }
    ss = warp_sum(ss);
    if (lane == 0) ssq[(size_t)t * parts + part] = ss;
}

GG_API gg_row_stats(const float* x, void* xhat, float* ssq, int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || H > 128 * 4 * 65535) return GG_ERR_ARG;
    const int parts = (H + 127) / 128;
    gg_launch(row_stats_kernel, dim3(T, (parts + 3) / 4), dim3(128), 0, stream, 1, x, (bf16*)xhat, ssq, H, parts);
    return gg_last_error();
}

// ----------------------------------------------------------------------------- rotary tables
// cos/sin[t, i] of angle = pos[t] * inv_freq[i], computed in float64 (the reference computes
// its tables in float64 too, pkg/ops/rope_tables.go:6-20) and stored as float32.  `mag` multiplies both
// tables (encodings that lengthen the rotated pairs; 1 for a plain rotation).
__global__ void rope_tables_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                   float* __restrict__ cosv, float* __restrict__ sinv, int T, int half, double mag) {
    pdl_launch();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    const int t = idx / half, i = idx - t * half;
    int p = positions[t];
    if (p < 0) p = 0;
    double s, c;
    sincos((double)p * inv_freq[i], &s, &c);
    cosv[idx] = (float)(c * mag);
    sinv[idx] = (float)(s * mag);
}

GG_API gg_rope_tables(const int* positions, const double* inv_freq, float* cosv, float* sinv,
                      int T, int half, double mag, cudaStream_t stream) {
    if (T <= 0 || half <= 0) return 0;
    const int n = T * half;
    gg_launch(rope_tables_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, 1, positions, inv_freq, cosv, sinv, T, half, mag);
    return gg_last_error();
}

// ----------------------------------------------------------------------------- QK-norm + rotary + cache write
// One warp per (token, head) of the fused projection output qkv[T, (nq + 2 nkv) * d]:
//   q heads: optional RMSNorm over d with weight qw, rotary, written to q_out[T, nq, d];
//   k heads: optional RMSNorm with kw, rotary, written into the paged key pool;
//   v heads: copied into the paged value pool.
// Order as in the reference: norm first, rotation after (pkg/model/qwen3/model.go:227-236).
// Pool layout: [page][kv_head][page_size][d]; the page of position p of sequence b is
// page_table[b * max_pages + p / page_size].  Pools may be null (a layer that reads another
// layer's cache writes none); then k and v heads are skipped.
template <typename T>
__global__ void qk_norm_rope_cache_kernel(
    const T* qkv, T* __restrict__ q_out,
    const float* __restrict__ qw, const float* __restrict__ kw, float eps,
    const float* cosv, const float* sinv,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ page_table, int max_pages, int page_size,
    T* __restrict__ k_pool, T* __restrict__ v_pool,
    int ntok, int nq, int nkv, int d, int rot, const PageBounds pb) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nheads = nq + 2 * nkv;
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (wid >= (long long)ntok * nheads) return;
    const int t = (int)(wid / nheads), h = (int)(wid - (long long)t * nheads);
    const int b = seq_of_token[t];
    const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
    if (!is_q && (k_pool == nullptr || b < 0)) return;
    float* buf = sm + warp * d;
    const T* src = qkv + ((size_t)t * nheads + h) * d;
    T* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * nq + h) * d;
    } else {
        const int pos = positions[t];
        const int page = gg_page_w(page_table + (size_t)b * max_pages, pos / page_size, max_pages, pb, 46);
        if (page < 0) return;            // (debug build) outside the pool: nothing is written
        const int kvh = is_k ? h - nq : h - nq - nkv;
        T* pool = is_k ? k_pool : v_pool;
        dst = pool + (((size_t)page * nkv + kvh) * page_size + (pos % page_size)) * d;
    }
    if (!is_q && !is_k) {  // value head: plain copy
        for (int i = lane; i < d; i += 32) dst[i] = src[i];
        return;
    }
    const float* w = is_q ? qw : kw;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) { float v = to_f<T>(src[i]); buf[i] = v; ss = fmaf(v, v, ss); }
    float scale = 1.f;
    if (w != nullptr) {
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / (float)d + eps);
    }
    __syncwarp();
    const int half = rot >> 1;
    const float* c = cosv + (size_t)t * half;
    const float* s = sinv + (size_t)t * half;
    for (int i = lane; i < d; i += 32) {
        float v = buf[i] * scale * (w ? w[i] : 1.f);
        float o;
        if (i < half) {
            const float p = buf[i + half] * scale * (w ? w[i + half] : 1.f);
            o = v * c[i] - p * s[i];
        } else if (i < rot) {
            const int j = i - half;
            const float p = buf[j] * scale * (w ? w[j] : 1.f);
            o = p * s[j] + v * c[j];
        } else {
            o = v;
        }
        dst[i] = from_f<T>(o);
    }
}

// bfloat16 form for a full rotation (rot == d) and d = 64, 128 or 256.  D / 16 lanes share one head: a lane
// owns eight pairs (i, i + d/2), i = 8 * sub .. + 8, so both halves of a pair sit in the same thread and
// every access to the head is 16 bytes wide; a warp handles 32 / (D / 16) heads at once (four of size 128),
// which keeps 1 KB in flight per warp.  The head's sum of squares is added over its lanes by shuffles.
template <int D>
__global__ void __launch_bounds__(128) qk_norm_rope_cache_vec_kernel(
    const bf16* qkv, bf16* __restrict__ q_out,
    const float* __restrict__ qw, const float* __restrict__ kw, float eps,
    const float* cosv, const float* sinv,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ page_table, int max_pages, int page_size,
    bf16* __restrict__ k_pool, bf16* __restrict__ v_pool, int ntok, int nq, int nkv, const PageBounds pb) {
    pdl_launch();
    pdl_wait();
    constexpr int HALF = D / 2, LPH = D / 16, HPW = 32 / LPH;      // lanes per head, heads per warp
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nheads = nq + 2 * nkv;
    const long long item = ((long long)blockIdx.x * (blockDim.x >> 5) + warp) * HPW + lane / LPH;
    const int sub = lane % LPH;
    const bool in_range = item < (long long)ntok * nheads;
    const int t = in_range ? (int)(item / nheads) : 0, h = in_range ? (int)(item - (long long)t * nheads) : 0;
    const int b = in_range ? seq_of_token[t] : -1;
    const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
    bool live = in_range && (is_q || (k_pool != nullptr && b >= 0));     // every lane stays for the shuffles
    const bf16* src = qkv + ((size_t)t * nheads + h) * D;
    bf16* dst = nullptr;
    if (live) {
        if (is_q) {
            dst = q_out + ((size_t)t * nq + h) * D;
        } else {
            const int pos = positions[t];
            const int page = gg_page_w(page_table + (size_t)b * max_pages, pos / page_size, max_pages, pb, 47);
            const int kvh = is_k ? h - nq : h - nq - nkv;
            if (page < 0) live = false;      // (debug build) outside the pool: nothing is written
            else dst = (is_k ? k_pool : v_pool) + (((size_t)page * nkv + kvh) * page_size + (pos % page_size)) * D;
        }
    }
    const int i0 = sub * 8;             // first index of this lane in the low half
    uint4 lo4 = make_uint4(0, 0, 0, 0), hi4 = make_uint4(0, 0, 0, 0);
    if (live) {
        lo4 = *reinterpret_cast<const uint4*>(src + i0);
        hi4 = *reinterpret_cast<const uint4*>(src + i0 + HALF);
    }
    if (live && !is_q && !is_k) {       // value head: plain copy
        *reinterpret_cast<uint4*>(dst + i0) = lo4;
        *reinterpret_cast<uint4*>(dst + i0 + HALF) = hi4;
    }
    const bool rotate = live && (is_q || is_k);
    const float* w = is_q ? qw : kw;
    float4 cs[2], sn[2], wl[2], wh[2];
    if (rotate) {                       // asked for before the sum of squares is known
        const float4* cp = reinterpret_cast<const float4*>(cosv + (size_t)t * HALF + i0);
        const float4* sp = reinterpret_cast<const float4*>(sinv + (size_t)t * HALF + i0);
        cs[0] = cp[0]; cs[1] = cp[1]; sn[0] = sp[0]; sn[1] = sp[1];
        if (w != nullptr) {
            wl[0] = reinterpret_cast<const float4*>(w + i0)[0]; wl[1] = reinterpret_cast<const float4*>(w + i0)[1];
            wh[0] = reinterpret_cast<const float4*>(w + i0 + HALF)[0]; wh[1] = reinterpret_cast<const float4*>(w + i0 + HALF)[1];
        }
    }
    const bf16* lo = reinterpret_cast<const bf16*>(&lo4);
    const bf16* hi = reinterpret_cast<const bf16*>(&hi4);
    float a[8], c[8], ss = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        a[k] = __bfloat162float(lo[k]); c[k] = __bfloat162float(hi[k]);
        ss = fmaf(a[k], a[k], ss); ss = fmaf(c[k], c[k], ss);
    }
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!rotate) return;
    const float scale = w != nullptr ? 1.0f / sqrtf(ss / (float)D + eps) : 1.f;
    const float* csf = reinterpret_cast<const float*>(cs);
    const float* snf = reinterpret_cast<const float*>(sn);
    const float* wlf = reinterpret_cast<const float*>(wl);
    const float* whf = reinterpret_cast<const float*>(wh);
    uint4 olo, ohi;
    bf16* ol = reinterpret_cast<bf16*>(&olo);
    bf16* oh = reinterpret_cast<bf16*>(&ohi);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float x0 = a[k] * scale * (w != nullptr ? wlf[k] : 1.f);
        const float x1 = c[k] * scale * (w != nullptr ? whf[k] : 1.f);
        ol[k] = __float2bfloat16_rn(x0 * csf[k] - x1 * snf[k]);
        oh[k] = __float2bfloat16_rn(x0 * snf[k] + x1 * csf[k]);
    }
    *reinterpret_cast<uint4*>(dst + i0) = olo;
    *reinterpret_cast<uint4*>(dst + i0 + HALF) = ohi;
}

GG_API gg_qk_norm_rope_cache(const void* qkv, int dtype, void* q_out, const float* qw, const float* kw, float eps,
                             const float* cosv, const float* sinv, const int* positions, const int* seq_of_token,
                             const int* page_table, int max_pages, int page_size, int n_pages, void* k_pool, void* v_pool,
                             int ntok, int nq, int nkv, int d, int rot, int* status, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (d <= 0 || d > 1024 || rot < 0 || rot > d || (rot & 1) || nq <= 0 || nkv <= 0 || page_size <= 0) return GG_ERR_ARG;
    const int warps = 4;
    const long long total = (long long)ntok * (nq + 2 * nkv);
    const unsigned grid = (unsigned)((total + warps - 1) / warps);
    const bool al = ((((uintptr_t)qkv) | ((uintptr_t)q_out) | ((uintptr_t)k_pool) | ((uintptr_t)v_pool) |
                      ((uintptr_t)cosv) | ((uintptr_t)sinv) | ((uintptr_t)qw) | ((uintptr_t)kw)) & 15) == 0;
    if (dtype == GG_BF16 && rot == d && al && (d == 64 || d == 128 || d == 256)) {
        const int per_block = warps * (32 / (d / 16));          // heads a block of four warps handles
        const unsigned vgrid = (unsigned)((total + per_block - 1) / per_block);
#define GG_QK_VEC(D_) gg_launch(qk_norm_rope_cache_vec_kernel<D_>, dim3(vgrid), dim3(warps * 32), 0, stream, 1,  \
            (const bf16*)qkv, (bf16*)q_out, qw, kw, eps, cosv, sinv, positions, seq_of_token, page_table, max_pages, \
            page_size, (bf16*)k_pool, (bf16*)v_pool, ntok, nq, nkv, PageBounds{n_pages, status})
        if (d == 64) GG_QK_VEC(64); else if (d == 128) GG_QK_VEC(128); else GG_QK_VEC(256);
#undef GG_QK_VEC
        return gg_last_error();
    }
    const size_t smem = (size_t)warps * d * sizeof(float);
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(qk_norm_rope_cache_kernel<T>, dim3(grid), dim3(warps * 32), smem, stream, 1, 
            (const T*)qkv, (T*)q_out, qw, kw, eps, cosv, sinv, positions, seq_of_token, page_table, max_pages,
            page_size, (T*)k_pool, (T*)v_pool, ntok, nq, nkv, d, rot, PageBounds{n_pages, status}));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- q/k/v preparation, general form
// One block per token of the fused projection output qkv[T, nq*d + nkv*d + nkv*dv] (q heads, k heads, v heads):
//   norm_mode 0: no q/k norm; 1: every q and k head normed over its d elements with one weight of size d;
//   2: q normed over all its nq*d elements at once with a weight of that size, k over its nkv*d alike;
//   then the rotation of the pairs (i, i + rot/2) of the first `rot` elements of every q and k head;
//   q to q_out[T, nq, d], k into the paged key pool [page][kv_head][page_size][d], v (untouched) into the paged
//   value pool [page][kv_head][page_size][dv].  The key and value head sizes may differ.  All arithmetic float32.
template <typename T>
__global__ void __launch_bounds__(256) qkv_prep_kernel(
    const T* qkv, T* __restrict__ q_out,
    const float* __restrict__ qw, const float* __restrict__ kw, float eps, int norm_mode,
    const float* cosv, const float* sinv,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ page_table, int max_pages, int page_size,
    T* __restrict__ k_pool, T* __restrict__ v_pool,
    int nq, int nkv, int d, int dv, int rot, const PageBounds pb) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    const int t = blockIdx.x;
    const int nqk = (nq + nkv) * d, row = nqk + nkv * dv;
    float* buf = sm;                 // [nqk] q and k as float
    float* hs = sm + nqk;            // [nq + nkv] one factor per head
    float* red = hs + nq + nkv;      // [33]
    const int b = seq_of_token[t];
    const T* src = qkv + (size_t)t * row;
    const bool write_kv = k_pool != nullptr && b >= 0;
    for (int i = threadIdx.x; i < nqk; i += blockDim.x) buf[i] = to_f<T>(src[i]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    if (norm_mode == 1) {
        for (int h = warp; h < nq + nkv; h += nwarps) {
            float ss = 0.f;
            for (int i = lane; i < d; i += 32) { const float v = buf[h * d + i]; ss = fmaf(v, v, ss); }
            ss = warp_sum(ss);
            if (lane == 0) hs[h] = 1.0f / sqrtf(ss / (float)d + eps);
        }
    } else if (norm_mode == 2) {
        float sq = 0.f, sk = 0.f;
        for (int i = threadIdx.x; i < nq * d; i += blockDim.x) { const float v = buf[i]; sq = fmaf(v, v, sq); }
        for (int i = nq * d + threadIdx.x; i < nqk; i += blockDim.x) { const float v = buf[i]; sk = fmaf(v, v, sk); }
        sq = block_sum(sq, red);
        sk = block_sum(sk, red);
        const float fq = 1.0f / sqrtf(sq / (float)(nq * d) + eps), fk = 1.0f / sqrtf(sk / (float)(nkv * d) + eps);
        for (int h = threadIdx.x; h < nq + nkv; h += blockDim.x) hs[h] = h < nq ? fq : fk;
    }
    __syncthreads();
    int page = -1, slot_in_page = 0;
    if (write_kv) {
        const int pos = positions[t];
        page = gg_page_w(page_table + (size_t)b * max_pages, pos / page_size, max_pages, pb, 46);
        slot_in_page = pos % page_size;
    }
    const int half = rot >> 1;
    const float* c = cosv + (size_t)t * half;
    const float* s = sinv + (size_t)t * half;
    for (int idx = threadIdx.x; idx < nqk; idx += blockDim.x) {
        const int h = idx / d, i = idx - h * d;
        const bool is_q = h < nq;
        if (!is_q && page < 0) continue;
        const float* w = is_q ? qw : kw;
        // weight index: per head (mode 1) or over the whole projection (mode 2)
        const int wbase = norm_mode == 2 ? (is_q ? h * d : (h - nq) * d) : 0;
        const float f = norm_mode ? hs[h] : 1.f;
        auto val = [&](int j) { return buf[h * d + j] * f * (norm_mode ? w[wbase + j] : 1.f); };
        float o;
        if (i < half) o = val(i) * c[i] - val(i + half) * s[i];
        else if (i < rot) o = val(i - half) * s[i - half] + val(i) * c[i - half];
        else o = val(i);
        if (is_q) q_out[(size_t)t * nq * d + idx] = from_f<T>(o);
        else k_pool[(((size_t)page * nkv + (h - nq)) * page_size + slot_in_page) * d + i] = from_f<T>(o);
    }
    if (page >= 0) {
        for (int idx = threadIdx.x; idx < nkv * dv; idx += blockDim.x) {
            const int h = idx / dv, i = idx - h * dv;
            v_pool[(((size_t)page * nkv + h) * page_size + slot_in_page) * dv + i] = src[nqk + idx];
        }
    }
}

GG_API gg_qkv_prep(const void* qkv, int dtype, void* q_out, const float* qw, const float* kw, float eps, int norm_mode,
                   const float* cosv, const float* sinv, const int* positions, const int* seq_of_token,
                   const int* page_table, int max_pages, int page_size, int n_pages, void* k_pool, void* v_pool,
                   int ntok, int nq, int nkv, int d, int dv, int rot, int* status, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (d <= 0 || dv <= 0 || rot < 0 || rot > d || (rot & 1) || nq <= 0 || nkv <= 0 || page_size <= 0 ||
        norm_mode < 0 || norm_mode > 2 || (norm_mode && (qw == nullptr || kw == nullptr))) return GG_ERR_ARG;
    const size_t smem = ((size_t)(nq + nkv) * d + nq + nkv + 33) * sizeof(float);
    if (smem > 200 * 1024) return GG_ERR_ARG;
    GG_DISPATCH_DTYPE(dtype, T,
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(qkv_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gg_launch(qkv_prep_kernel<T>, dim3(ntok), dim3(256), smem, stream, 1,
            (const T*)qkv, (T*)q_out, qw, kw, eps, norm_mode, cosv, sinv, positions, seq_of_token, page_table, max_pages,
            page_size, (T*)k_pool, (T*)v_pool, nq, nkv, d, dv, rot, PageBounds{n_pages, status}));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- norm of a part's output, added
// x[r, :] += y[r, :] / sqrt(mean(y[r, :]^2) + eps) * w: the norm that follows a part in a block with norms on
// both sides of its parts, and the add into the residual stream, in one pass.  All float32; one block per row.
// With xhat and ssq it also leaves what a product with a folded norm reads of the updated row: its bfloat16 copy
// and the sums of its squares over blocks of 128 columns (see row_stats_kernel), so the norm before the next
// part needs no kernel of its own.
__global__ void __launch_bounds__(256) rmsnorm_add_kernel(float* x, float* y, const float* __restrict__ w,
                                                          int H, float eps, bf16* __restrict__ xhat,
                                                          float* __restrict__ ssq, int parts, int zero_y,
                                                          const float* gate, const float* __restrict__ gate_bias) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    extern __shared__ float psum[];          // [parts][4]: a 128-column block is four warps' 32 columns
    const size_t r = blockIdx.x;
    float* yr = y + r * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = yr[i];
        if (gate != nullptr) {               // the gated row replaces the raw one: the second pass reads it back
            v *= 1.0f / (1.0f + expf(-(gate[r * H + i] + (gate_bias != nullptr ? gate_bias[i] : 0.f))));
            yr[i] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float f = 1.0f / sqrtf(ss / (float)H + eps);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i0 = 0; i0 < H; i0 += blockDim.x) {
        const int i = i0 + threadIdx.x;
        float v = 0.f;
        if (i < H) {
            v = x[r * H + i] + yr[i] * f * w[i];
            x[r * H + i] = v;
            if (zero_y) yr[i] = 0.f;
            if (xhat != nullptr) xhat[r * H + i] = __float2bfloat16_rn(v);
        }
        if (ssq != nullptr) {
            const float q = warp_sum(v * v);
            const int part = (i0 >> 7) + (warp >> 2);
            if (lane == 0 && part < parts) psum[part * 4 + (warp & 3)] = q;
        }
    }
    if (ssq != nullptr) {
        __syncthreads();
        for (int p = threadIdx.x; p < parts; p += blockDim.x)
            ssq[r * parts + p] = (psum[p * 4] + psum[p * 4 + 1]) + (psum[p * 4 + 2] + psum[p * 4 + 3]);
    }
}

// The same with 16-byte accesses (H a multiple of 4, rows on 16-byte boundaries): a thread owns four columns, a
// warp the 128 columns of one block of the sums of squares, so those need no shared memory.
__device__ __forceinline__ float gate_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

__global__ void __launch_bounds__(1024) rmsnorm_add_vec_kernel(float* x, float* y, const float* __restrict__ w,
                                                               int H, float eps, bf16* __restrict__ xhat,
                                                               float* __restrict__ ssq, int parts, int zero_y,
                                                               const float* gate, const float* __restrict__ gate_bias) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    float4* yr = reinterpret_cast<float4*>(y + r * H);
    const float4* wr = reinterpret_cast<const float4*>(w);
    float4* xr = reinterpret_cast<float4*>(x + r * H);
    const int n4 = H >> 2;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
        float4 v = yr[i];
        if (gate != nullptr) {               // the gated row replaces the raw one: the second pass reads it back
            float4 g = reinterpret_cast<const float4*>(gate + r * H)[i];
            if (gate_bias != nullptr) {
                const float4 gb = reinterpret_cast<const float4*>(gate_bias)[i];
                g.x += gb.x; g.y += gb.y; g.z += gb.z; g.w += gb.w;
            }
            v.x *= gate_sigmoid(g.x); v.y *= gate_sigmoid(g.y); v.z *= gate_sigmoid(g.z); v.w *= gate_sigmoid(g.w);
            yr[i] = v;
        }
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    ss = block_sum(ss, red);
    const float f = 1.0f / sqrtf(ss / (float)H + eps);
    const int lane = threadIdx.x & 31;
    for (int i0 = 0; i0 < n4; i0 += blockDim.x) {
        const int i = i0 + threadIdx.x;
        float q = 0.f;
        if (i < n4) {
            const float4 a = xr[i], b = yr[i], c = wr[i];
            float4 v;
            v.x = a.x + b.x * f * c.x; v.y = a.y + b.y * f * c.y; v.z = a.z + b.z * f * c.z; v.w = a.w + b.w * f * c.w;
            xr[i] = v;
            if (zero_y) yr[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (xhat != nullptr) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                *reinterpret_cast<uint2*>(xhat + r * H + 4 * (size_t)i) =
                    make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            }
            q = (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        }
        if (ssq != nullptr) {
            q = warp_sum(q);
            const int part = (i - lane) >> 5;             // the warp's first column / 128
            if (lane == 0 && part < parts) ssq[r * parts + part] = q;
        }
    }
}

// xhat (bfloat16 [rows, H]) and ssq (float32 [rows, ceil(H / 128)]) may both be null.  zero_y != 0: y is left
// zeroed (the buffer the next part of the block adds its output into, without a fill of its own).  gate (float32
// [rows, H], may be null) with gate_bias ([H], may be null): y is first multiplied by sigmoid(gate + gate_bias),
// element by element, and the norm is taken of the product.
GG_API gg_rmsnorm_add(float* x, float* y, const float* w, int rows, int H, float eps, void* xhat, float* ssq,
                      int zero_y, const float* gate, const float* gate_bias, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H <= 0 || (xhat == nullptr) != (ssq == nullptr)) return GG_ERR_ARG;
    const int parts = (H + 127) / 128;
    if ((H & 3) == 0 && (((uintptr_t)x | (uintptr_t)y | (uintptr_t)w | (uintptr_t)gate | (uintptr_t)gate_bias) & 15) == 0 &&
        (((uintptr_t)xhat) & 7) == 0) {
        // few rows (decode steps): as many threads as the row has groups of four columns, up to 1,024
        int threads = ((H >> 2) + 31) / 32 * 32;
        if (threads > 1024 || rows >= 512) threads = threads > 256 ? 256 : threads;
        gg_launch(rmsnorm_add_vec_kernel, dim3(rows), dim3(threads), 0, stream, 1, x, y, w, H, eps, (bf16*)xhat, ssq, parts, zero_y,
                  gate, gate_bias);
        return gg_last_error();
    }
    // (a block of 128 columns whose tail lies beyond H gets zeros from the warps that have no column)
    const size_t smem = ssq != nullptr ? ((size_t)(parts + 1) * 4) * sizeof(float) : 0;
    if (smem > 48 * 1024) return GG_ERR_ARG;
    gg_launch(rmsnorm_add_kernel, dim3(rows), dim3(256), smem, stream, 1, x, y, w, H, eps, (bf16*)xhat, ssq, parts, zero_y,
              gate, gate_bias);
    return gg_last_error();
}

// ----------------------------------------------------------------------------- SwiGLU
// out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(z) = z / (1 + exp(-z)) (pkg/ops/ops.go:316-318).
template <typename T>
__global__ void swiglu_kernel(const T* gu, T* __restrict__ out, long long n, int I) {
    pdl_launch();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const long long t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_f<T>(gu[t * 2 * I + i]);
    const float u = to_f<T>(gu[t * 2 * I + I + i]);
    out[idx] = from_f<T>(g / (1.0f + expf(-g)) * u);
}

// Eight elements per thread with 16-byte accesses (rows of I elements, I a multiple of 8).
__global__ void swiglu_vec8_kernel(const bf16* gu, bf16* __restrict__ out, long long nvec, int I8) {
    pdl_launch();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= nvec) return;
    const long long t = idx / I8;
    const int c = (int)(idx - t * I8);
    const uint4 gv = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + c) * 8);
    const uint4 uv = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + I8 + c) * 8);
    const uint32_t* gw = reinterpret_cast<const uint32_t*>(&gv);
    const uint32_t* uw = reinterpret_cast<const uint32_t*>(&uv);
    uint32_t ow[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const __nv_bfloat162 g2 = *reinterpret_cast<const __nv_bfloat162*>(&gw[k]);
        const __nv_bfloat162 u2 = *reinterpret_cast<const __nv_bfloat162*>(&uw[k]);
        const float g0 = __low2float(g2), g1 = __high2float(g2);
        const float r0 = g0 / (1.0f + expf(-g0)) * __low2float(u2);
        const float r1 = g1 / (1.0f + expf(-g1)) * __high2float(u2);
        const __nv_bfloat162 r = __floats2bfloat162_rn(r0, r1);
        ow[k] = *reinterpret_cast<const uint32_t*>(&r);
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

GG_API gg_swiglu(const void* gu, int dtype, void* out, int ntok, int I, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (I <= 0) return GG_ERR_ARG;
    const long long n = (long long)ntok * I;
    if (dtype == GG_BF16 && I % 8 == 0 && ((((uintptr_t)gu) | ((uintptr_t)out)) & 15) == 0) {
        const long long nvec = n / 8;
        gg_launch(swiglu_vec8_kernel, dim3((unsigned)((nvec + 255) / 256)), dim3(256), 0, stream, 1, (const bf16*)gu, (bf16*)out, nvec, I / 8);
        return gg_last_error();
    }
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(swiglu_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, (const T*)gu, (T*)out, n, I));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- residual add
// x (float32) += delta.  The fast path folds this into the producing product's epilogue;
// this is the stand-alone form (pkg/gpu/cuda/ptx.go:891-924 add_inplace).
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ x, const T* delta, long long n) {
    pdl_launch();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) x[idx] += to_f<T>(delta[idx]);
}

GG_API gg_residual_add(float* x, const void* delta, int dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(residual_add_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, x, (const T*)delta, n));
    return gg_last_error();
}

// x (float32) += alpha * delta: what an arrangement with a factor on its parts' outputs adds when a part
// could not take the factor into its own last product.
template <typename T>
__global__ void residual_axpy_kernel(float* __restrict__ x, const T* delta, float alpha, long long n) {
    pdl_launch();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) x[idx] = fmaf(alpha, to_f<T>(delta[idx]), x[idx]);
}

GG_API gg_residual_axpy(float* x, const void* delta, int dtype, float alpha, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(residual_axpy_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, x, (const T*)delta, alpha, n));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- xIELU
// out = out_scale * f(z), f(z) = ap z^2 + z / 2 for z > 0 and aq (exp(z) - 1 - z) + z / 2 otherwise; ap and aq are
// the activation's two coefficients as the host derived them from its stored scalars (ap = softplus(p),
// aq = 1/2 + softplus(q)).  float32 arithmetic; expm1f keeps exp(z) - 1 exact near zero.
template <typename T>
__global__ void xielu_kernel(const T* z, T* out, float ap, float aq, float out_scale, long long n) {
    pdl_launch();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const float v = to_f<T>(z[idx]);
    const float f = v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(aq, expm1f(v) - v, 0.5f * v);
    out[idx] = from_f<T>(f * out_scale);
}

// The same for bfloat16 with eight elements (16 bytes) per thread.
__global__ void __launch_bounds__(256) xielu_vec8_kernel(const bf16* z, bf16* out, float ap, float aq, float out_scale,
                                                         long long nvec) {
    pdl_launch();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nvec) return;
    uint4 raw = reinterpret_cast<const uint4*>(z)[i];
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float2 v = __bfloat1622float2(h2[j]);
        v.x = (v.x > 0.f ? fmaf(ap * v.x, v.x, 0.5f * v.x) : fmaf(aq, expm1f(v.x) - v.x, 0.5f * v.x)) * out_scale;
        v.y = (v.y > 0.f ? fmaf(ap * v.y, v.y, 0.5f * v.y) : fmaf(aq, expm1f(v.y) - v.y, 0.5f * v.y)) * out_scale;
        h2[j] = __floats2bfloat162_rn(v.x, v.y);
    }
    reinterpret_cast<uint4*>(out)[i] = raw;
}

GG_API gg_xielu(const void* z, int dtype, void* out, float ap, float aq, float out_scale, long long n,
                cudaStream_t stream) {
    if (n <= 0) return 0;
    if (dtype == GG_BF16 && (n % 8) == 0 && ((((uintptr_t)z) | ((uintptr_t)out)) & 15) == 0) {
        const long long nvec = n / 8;
        gg_launch(xielu_vec8_kernel, dim3((unsigned)((nvec + 255) / 256)), dim3(256), 0, stream, 1, (const bf16*)z, (bf16*)out,
                  ap, aq, out_scale, nvec);
        return gg_last_error();
    }
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(xielu_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, (const T*)z, (T*)out, ap, aq, out_scale, n));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- token feed
// tokens[i] = sampled[src[i]] where src[i] >= 0: lets a decode step take the ids that the previous
// step's sampling kernel left on the device, without a round trip through the host.
__global__ void feed_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ src,
                                   const int* sampled, int n) {
    pdl_launch();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && src[i] >= 0) tokens[i] = sampled[src[i]];
}

GG_API gg_feed_tokens(int* tokens, const int* src, const int* sampled, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    return gg_launch(feed_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, 1, tokens, src, sampled, n);
}

// ----------------------------------------------------------------------------- short causal convolution over time
// out[t, c] = h[t, c] * keep + sum_j w[j, c] * h[t - taps + 1 + j, c] (j < taps; the last tap meets the token
// itself), per channel, inside each sequence; keep = 1 adds the convolution to its input.  Rows before the step's
// first token come from the sequence's state [slot][taps - 1][W] (float32: the last taps - 1 input rows of the
// sequence in order, zeros at its start).  Blocks (token, 256 channels).  The state is not written here: other blocks of
// the same sequence still read it (short_conv_state_kernel moves it on afterwards).
template <typename T>
__global__ void __launch_bounds__(256) short_conv_kernel(const T* h, T* out, const float* __restrict__ w,
                                                         const float* state, const int* __restrict__ cu_seqlens,
                                                         const int* __restrict__ slots, const int* __restrict__ seq_of_token,
                                                         int W, int taps, float keep) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const int b = seq_of_token[t];
    T* o = out + (size_t)t * W;
    if (b < 0) {
        for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < W; c += gridDim.y * blockDim.x) o[c] = from_f<T>(0.f);
        return;
    }
    const int start = cu_seqlens[b];
    const int R = taps - 1;
    const float* st = state + (size_t)slots[b] * R * W;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < W; c += gridDim.y * blockDim.x) {
        const float* wc = w + c;                       // tap j of channel c at wc[j * W]
        float acc = to_f<T>(h[(size_t)t * W + c]) * (keep + wc[(size_t)R * W]);
        for (int j = 0; j < R; ++j) {
            const int s = t - R + j;
            const float v = s >= start ? to_f<T>(h[(size_t)s * W + c]) : st[(size_t)(R + (s - start)) * W + c];
            acc = fmaf(wc[(size_t)j * W], v, acc);
        }
        o[c] = from_f<T>(acc);
    }
}

// The state after the step: the last taps - 1 input rows of every sequence (rows of the step where it brought
// that many, else the old state moved up).  Blocks (sequence, 256 channels); a thread reads all it needs of a channel
// before it writes.  Padding sequences (seq_of_token < 0 at their first row) are left alone.
#define CONV_MAX_TAPS 16
template <typename T>
__global__ void __launch_bounds__(256) short_conv_state_kernel(const T* h, float* state, const int* __restrict__ cu_seqlens,
                                                               const int* __restrict__ slots,
                                                               const int* __restrict__ seq_of_token, int W, int taps) {
    pdl_launch();
    pdl_wait();
    const int b = blockIdx.x;
    const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
    if (n <= 0 || seq_of_token[start] < 0) return;
    const int R = taps - 1;
    float* st = state + (size_t)slots[b] * R * W;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < W; c += gridDim.y * blockDim.x) {
        float keep[CONV_MAX_TAPS];
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j) {
            if (j < R) {
                const int rel = n - R + j;
                keep[j] = rel >= 0 ? to_f<T>(h[(size_t)(start + rel) * W + c]) : st[(size_t)(R + rel) * W + c];
            }
        }
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j)
            if (j < R) st[(size_t)j * W + c] = keep[j];
    }
}

// The 16-byte form: a thread makes V = 16 / sizeof(T) neighbouring channels of one token (W a multiple of V) with
// the tap count known at compile time; its loads of earlier rows meet other threads' in L1 and L2.  one_each != 0:
// no sequence brings more than one token, so the thread that makes a token's channels is the only one that reads
// its sequence's state there, and it moves the state on itself (no second launch).
template <typename T> struct ConvRow;
template <> struct ConvRow<float> {
    static __device__ __forceinline__ void unpack(const uint4& a, float* v) {
        v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y); v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
    }
    static __device__ __forceinline__ uint4 pack(const float* v) {
        return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
    }
};
template <> struct ConvRow<bf16> {
    static __device__ __forceinline__ void unpack(const uint4& a, float* v) {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h2[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ uint4 pack(const float* v) {
        uint4 a;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&a);
#pragma unroll
        for (int i = 0; i < 4; ++i) h2[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        return a;
    }
};
static __device__ __forceinline__ void conv_load4(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
static __device__ __forceinline__ void conv_store4(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}

// A thread makes V channels of TT consecutive rows of the step.  The TT rows and the taps - 1 rows before them are
// asked for before anything is known of the tokens' sequences (they are rows of this step's h whatever sequence
// they belong to), so that one round of memory latency serves them, the weights and the sequences' bounds together;
// a row from before a sequence's start in this step is then replaced by the state's.  Blocks (TT rows, 128 x V
// channels).
template <typename T, int TAPS, int TT>
__global__ void __launch_bounds__(128) short_conv_vec_kernel(const T* h, T* out, const float* __restrict__ w, float* state,
                                                             const int* __restrict__ cu_seqlens,
                                                             const int* __restrict__ slots,
                                                             const int* __restrict__ seq_of_token, int W, int ntok,
                                                             float keep, int one_each) {
    pdl_launch();
    pdl_wait();
    constexpr int V = 16 / (int)sizeof(T);
    constexpr int R = TAPS - 1;
    const int c0 = (blockIdx.y * 128 + threadIdx.x) * V;
    if (c0 >= W) return;
    const int t0 = blockIdx.x * TT;
    uint4 row[R + TT];                                    // rows t0 - R .. t0 + TT - 1 of h
#pragma unroll
    for (int i = 0; i < R + TT; ++i) {
        const int s = t0 - R + i;
        row[i] = (s >= 0 && s < ntok) ? *reinterpret_cast<const uint4*>(h + (size_t)s * W + c0) : make_uint4(0u, 0u, 0u, 0u);
    }
    int seq[TT];
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) seq[tt] = t0 + tt < ntok ? seq_of_token[t0 + tt] : -1;
    float wr[TAPS * V];                                   // tap j of channel c0 + v at [j * V + v]
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
#pragma unroll
        for (int v = 0; v < V; v += 4) conv_load4(w + (size_t)j * W + c0 + v, wr + j * V + v);
    }
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
        const int t = t0 + tt;
        if (t >= ntok) break;
        T* o = out + (size_t)t * W + c0;
        const int b = seq[tt];
        if (b < 0) {
            *reinterpret_cast<uint4*>(o) = make_uint4(0u, 0u, 0u, 0u);
            continue;
        }
        float acc[V], x[V];
        ConvRow<T>::unpack(row[R + tt], x);
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = x[v] * (keep + wr[R * V + v]);
        if (R > 0) {
            const int start = cu_seqlens[b];
            float* st = t - R < start ? state + (size_t)slots[b] * R * W + c0 : nullptr;
#pragma unroll
            for (int j = 0; j < R; ++j) {
                const int s = t - R + j;
                float prev[V];
                if (s >= start) {
                    ConvRow<T>::unpack(row[tt + j], prev);
                } else {
                    const float* sr = st + (size_t)(R + (s - start)) * W;
#pragma unroll
                    for (int v = 0; v < V; v += 4) conv_load4(sr + v, prev + v);
                }
#pragma unroll
                for (int v = 0; v < V; ++v) acc[v] = fmaf(wr[j * V + v], prev[v], acc[v]);
                // one token of this sequence: row j of the old state was just read (s - start = j - R); it is row
                // j - 1 of the new one, which this thread read in the round before
                if (one_each && j >= 1) {
#pragma unroll
                    for (int v = 0; v < V; v += 4) conv_store4(st + (size_t)(j - 1) * W + v, prev + v);
                }
            }
            if (one_each) {
#pragma unroll
                for (int v = 0; v < V; v += 4) conv_store4(st + (size_t)(R - 1) * W + v, x + v);
            }
        }
        *reinterpret_cast<uint4*>(o) = ConvRow<T>::pack(acc);
    }
}

// Few rows (decode steps): a row a thread, so that the step fills more of the GPU; else four.
template <typename T, int TAPS>
static int short_conv_vec_launch(const T* h, T* out, const float* w, float* state, const int* cu_seqlens, const int* slots,
                                 const int* seq_of_token, int ntok, int W, float keep, int one_each, cudaStream_t stream) {
    constexpr int V = 16 / (int)sizeof(T);
    const unsigned cb = (unsigned)((W / V + 127) / 128);
    if (ntok < 1024)
        return gg_launch(short_conv_vec_kernel<T, TAPS, 1>, dim3((unsigned)ntok, cb), dim3(128), 0, stream, 1, h, out, w,
                         state, cu_seqlens, slots, seq_of_token, W, ntok, keep, one_each);
    return gg_launch(short_conv_vec_kernel<T, TAPS, 4>, dim3((unsigned)((ntok + 3) / 4), cb), dim3(128), 0, stream, 1, h, out,
                     w, state, cu_seqlens, slots, seq_of_token, W, ntok, keep, one_each);
}

#define CONV_VEC_MAX_TAPS 8
template <typename T>
static int short_conv_vec(int taps, const T* h, T* out, const float* w, float* state, const int* cu_seqlens,
                          const int* slots, const int* seq_of_token, int ntok, int W, float keep, int one_each,
                          cudaStream_t stream) {
#define CONV_CASE(N) case N: return short_conv_vec_launch<T, N>(h, out, w, state, cu_seqlens, slots, seq_of_token, ntok, W, \
                                                                keep, one_each, stream);
    switch (taps) { CONV_CASE(1) CONV_CASE(2) CONV_CASE(3) CONV_CASE(4) CONV_CASE(5) CONV_CASE(6) CONV_CASE(7) CONV_CASE(8) }
#undef CONV_CASE
    return GG_ERR_ARG;
}

// h and out [T, W] in `dtype` (they may not overlap), w [taps][W] float32 (a tap's weights side by side), state [slots][taps - 1][W] float32.
// max_new: the most tokens one sequence brings (0: not known).
GG_API gg_short_conv(const void* h, void* out, int dtype, const float* w, float* state, const int* cu_seqlens,
                     const int* slots, const int* seq_of_token, int ntok, int n_seqs, int W, int taps, float keep,
                     int max_new, cudaStream_t stream) {
    if (ntok <= 0 || n_seqs <= 0) return 0;
    if (W <= 0 || taps < 1 || taps > CONV_MAX_TAPS || (taps > 1 && state == nullptr)) return GG_ERR_ARG;
    const int cb = min((W + 255) / 256, 65535);
    const int one_each = max_new == 1;
    GG_DISPATCH_DTYPE(dtype, T,
        const bool vec = taps <= CONV_VEC_MAX_TAPS && W / 4 <= 65535 * 128 && W % (16 / (int)sizeof(T)) == 0 && ((uintptr_t)h | (uintptr_t)out | (uintptr_t)w |
                                                                          (uintptr_t)state) % 16 == 0;
        if (vec) {
            short_conv_vec<T>(taps, (const T*)h, (T*)out, w, state, cu_seqlens, slots, seq_of_token, ntok, W, keep, one_each,
                              stream);
        } else {
            // a thread per channel: blocks of 256 channels side by side
            gg_launch(short_conv_kernel<T>, dim3(ntok, cb), dim3(256), 0, stream, 1, (const T*)h, (T*)out, w,
                      (const float*)state, cu_seqlens, slots, seq_of_token, W, taps, keep);
        }
        if (taps > 1 && !(vec && one_each))
            gg_launch(short_conv_state_kernel<T>, dim3(n_seqs, cb), dim3(256), 0, stream, 1, (const T*)h, state, cu_seqlens,
                      slots, seq_of_token, W, taps));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- RMS norm of strided rows
// out[t, :n] = x[t, :n] / sqrt(mean(x[t, :n]^2) + eps) * w, rows of x ldx apart and of out ldo apart; the sums in
// float32.  One block per row (the latent of a projection's output, normed before the next projection).
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const T* x, long long ldx, const float* __restrict__ w, T* out,
                                                           long long ldo, int n, float eps) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const T* xr = x + (size_t)blockIdx.x * ldx;
    T* o = out + (size_t)blockIdx.x * ldo;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = to_f<T>(xr[i]); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float f = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = from_f<T>(to_f<T>(xr[i]) * f * w[i]);
}

GG_API gg_rmsnorm_rows(const void* x, long long ldx, int dtype, const float* w, void* out, long long ldo, int rows, int n,
                       float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (n <= 0 || ldx < n || ldo < n) return GG_ERR_ARG;
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(rmsnorm_rows_kernel<T>, dim3(rows), dim3(256), 0, stream, 1, (const T*)x, ldx, w, (T*)out, ldo, n, eps));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- soft cap
// z <- cap * tanh(z / cap), in place, float32 (logits that are bounded smoothly).
__global__ void softcap_kernel(float* z, float cap, long long n) {
    pdl_launch();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) z[i] = cap * tanhf(z[i] / cap);
}

GG_API gg_softcap(float* z, float cap, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return GG_ERR_ARG;
    return gg_launch(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, z, cap, n);
}

// ----------------------------------------------------------------------------- RMS norm in groups
// A row of H numbers is cut into `groups` equal consecutive runs; each run is divided by its own
// sqrt(mean(run^2) + eps) and the whole is multiplied by w [H].  groups = 1 is the plain RMS norm.
// Norm of gathered float32 rows into the compute dtype (the model's last norm): one block per row.
template <typename T>
__global__ void __launch_bounds__(256) group_rmsnorm_kernel(const float* x, const int* __restrict__ rows,
                                                            const float* __restrict__ w, T* out, int H, int groups, float eps) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int src = rows != nullptr ? rows[r] : r;
    T* o = out + (size_t)r * H;
    if (src < 0) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f<T>(0.f);
        return;
    }
    const float* xr = x + (size_t)src * H;
    const int gs = H / groups;
    for (int g = 0; g < groups; ++g) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < gs; i += blockDim.x) { const float v = xr[g * gs + i]; ss = fmaf(v, v, ss); }
        ss = block_sum(ss, red);
        const float f = 1.0f / sqrtf(ss / (float)gs + eps);
        for (int i = threadIdx.x; i < gs; i += blockDim.x) o[g * gs + i] = from_f<T>(xr[g * gs + i] * f * w[g * gs + i]);
    }
}

GG_API gg_group_rmsnorm(const float* x, const int* rows, const float* w, void* out, int out_dtype, int R, int H, int groups,
                        float eps, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (H <= 0 || groups <= 0 || H % groups) return GG_ERR_ARG;
    GG_DISPATCH_DTYPE(out_dtype, T,
        gg_launch(group_rmsnorm_kernel<T>, dim3(R), dim3(256), 0, stream, 1, x, rows, w, (T*)out, H, groups, eps));
    return gg_last_error();
}

// x[r, :] += groupnorm(y[r, :]) * w: the norm that follows a part and the add into the stream, all float32.
// zero_y != 0: y is left zeroed.  One block per row.  Runs of up to 4,096 numbers are a warp's work each (no block
// barrier: the warp sums its run, norms it and adds it); longer runs take the whole block, a run at a time.
__global__ void __launch_bounds__(256) group_rmsnorm_add_kernel(float* x, float* y, const float* __restrict__ w, int H,
                                                                int groups, float eps, int zero_y) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    float* yr = y + r * H;
    float* xr = x + r * H;
    const int gs = H / groups;
    if (gs <= 4096) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
        for (int g = warp; g < groups; g += nwarps) {
            float ss = 0.f;
            for (int i = lane; i < gs; i += 32) { const float v = yr[g * gs + i]; ss = fmaf(v, v, ss); }
            ss = warp_sum(ss);
            const float f = 1.0f / sqrtf(ss / (float)gs + eps);
            for (int i = lane; i < gs; i += 32) {
                const int c = g * gs + i;
                xr[c] += yr[c] * f * w[c];
                if (zero_y) yr[c] = 0.f;
            }
        }
        return;
    }
    for (int g = 0; g < groups; ++g) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < gs; i += blockDim.x) { const float v = yr[g * gs + i]; ss = fmaf(v, v, ss); }
        ss = block_sum(ss, red);
        const float f = 1.0f / sqrtf(ss / (float)gs + eps);
        for (int i = threadIdx.x; i < gs; i += blockDim.x) {
            const int c = g * gs + i;
            xr[c] += yr[c] * f * w[c];
            if (zero_y) yr[c] = 0.f;
        }
    }
}

GG_API gg_group_rmsnorm_add(float* x, float* y, const float* w, int rows, int H, int groups, float eps, int zero_y,
                            cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H <= 0 || groups <= 0 || H % groups) return GG_ERR_ARG;
    // few rows (decode steps) of few runs: no more warps than runs, so that a block is not mostly idle
    const int gs = H / groups;
    int threads = 256;
    if (gs <= 4096 && groups < 8) threads = 32 * groups;
    gg_launch(group_rmsnorm_add_kernel, dim3(rows), dim3(threads), 0, stream, 1, x, y, w, H, groups, eps, zero_y);
    return gg_last_error();
}

// ----------------------------------------------------------------------------- token shift
// out[t, c] = x[t, c] + (prev[c] - x[t, c]) * mu[c], prev the row before t in its sequence: row t - 1 of the step,
// or, for a sequence's first row of the step, state[slot] (float32 [slots][W]: the sequence's last row of the step
// before, zeros at its start).  x is float32, out the compute dtype.  one_each != 0: no sequence brings more than
// one row, so the thread that makes a channel is the only one that reads its state and moves it on itself;
// otherwise token_shift_state_kernel moves the states on once every block has read them.
template <typename T>
__global__ void __launch_bounds__(256) token_shift_kernel(const float* x, T* out, const float* __restrict__ mu, float* state,
                                                          const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                                          const int* __restrict__ seq_of_token, int W, int one_each) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const int b = seq_of_token[t];
    T* o = out + (size_t)t * W;
    if (b < 0) {
        for (int c = threadIdx.x; c < W; c += blockDim.x) o[c] = from_f<T>(0.f);
        return;
    }
    const bool first = t == cu_seqlens[b];
    float* st = state + (size_t)slots[b] * W;
    const float* prev = first ? st : x + (size_t)(t - 1) * W;
    const float* xr = x + (size_t)t * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = xr[c], p = prev[c];
        o[c] = from_f<T>(v + (p - v) * mu[c]);
        if (one_each) st[c] = v;
    }
}

__global__ void __launch_bounds__(256) token_shift_state_kernel(const float* x, float* state, const int* __restrict__ cu_seqlens,
                                                                const int* __restrict__ slots,
                                                                const int* __restrict__ seq_of_token, int W) {
    pdl_launch();
    pdl_wait();
    const int b = blockIdx.x;
    const int start = cu_seqlens[b], end = cu_seqlens[b + 1];
    if (end <= start || seq_of_token[start] < 0) return;
    float* st = state + (size_t)slots[b] * W;
    const float* last = x + (size_t)(end - 1) * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) st[c] = last[c];
}

GG_API gg_token_shift(const float* x, void* out, int out_dtype, const float* mu, float* state, const int* cu_seqlens,
                      const int* slots, const int* seq_of_token, int ntok, int n_seqs, int W, int max_new,
                      cudaStream_t stream) {
    if (ntok <= 0 || n_seqs <= 0) return 0;
    if (W <= 0 || state == nullptr) return GG_ERR_ARG;
    const int one_each = max_new == 1;
    GG_DISPATCH_DTYPE(out_dtype, T,
        gg_launch(token_shift_kernel<T>, dim3(ntok), dim3(256), 0, stream, 1, x, (T*)out, mu, state, cu_seqlens, slots,
                  seq_of_token, W, one_each));
    if (!one_each)
        gg_launch(token_shift_state_kernel, dim3(n_seqs), dim3(256), 0, stream, 1, x, state, cu_seqlens, slots, seq_of_token, W);
    return gg_last_error();
}

// ----------------------------------------------------------------------------- weighted sum over depth
// hist [slots_of_depth][n] float32 keeps what every layer left; this stores x as hist[store_at] and then, if
// n_terms > 0, replaces x by sum_{j < n_terms} coeff[j] * hist[j] (j ascending; hist[store_at] is x itself).
__global__ void __launch_bounds__(256) depth_mix_kernel(float* hist, float* x, const float* __restrict__ coeff, int store_at,
                                                        int n_terms, long long n) {
    pdl_launch();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = x[i];
    hist[(size_t)store_at * n + i] = v;
    if (n_terms <= 0) return;
    float acc = 0.f;
    for (int j = 0; j < n_terms; ++j) acc = fmaf(coeff[j], j == store_at ? v : hist[(size_t)j * n + i], acc);
    x[i] = acc;
}

// The same with 16-byte accesses (n a multiple of four, buffers on 16-byte boundaries).
__global__ void __launch_bounds__(256) depth_mix_vec_kernel(float4* hist, float4* x, const float* __restrict__ coeff,
                                                            int store_at, int n_terms, long long n4) {
    pdl_launch();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 v = x[i];
    hist[(size_t)store_at * n4 + i] = v;
    if (n_terms <= 0) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < n_terms; ++j) {
        const float cj = coeff[j];
        const float4 hj = j == store_at ? v : hist[(size_t)j * n4 + i];
        acc.x = fmaf(cj, hj.x, acc.x); acc.y = fmaf(cj, hj.y, acc.y); acc.z = fmaf(cj, hj.z, acc.z); acc.w = fmaf(cj, hj.w, acc.w);
    }
    x[i] = acc;
}

GG_API gg_depth_mix(float* hist, float* x, const float* coeff, int store_at, int n_terms, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (store_at < 0 || n_terms < 0 || (n_terms > 0 && coeff == nullptr)) return GG_ERR_ARG;
    if ((n & 3) == 0 && (((uintptr_t)hist | (uintptr_t)x) & 15) == 0) {
        gg_launch(depth_mix_vec_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, stream, 1, (float4*)hist, (float4*)x,
                  coeff, store_at, n_terms, n / 4);
        return gg_last_error();
    }
    gg_launch(depth_mix_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, hist, x, coeff, store_at, n_terms, n);
    return gg_last_error();
}

// ----------------------------------------------------------------------------- float32 rows into the compute dtype
template <typename T>
__global__ void cast_rows_kernel(const float* x, T* out, long long n) {
    pdl_launch();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f<T>(x[i]);
}

GG_API gg_cast_rows(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    GG_DISPATCH_DTYPE(out_dtype, T,
        gg_launch(cast_rows_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, x, (T*)out, n));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- GELU
// out = z Phi(z), exactly (erf) or in the tanh form 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))); float32
// arithmetic, in place allowed.
__device__ __forceinline__ float gelu_value(float z, int tanh_form) {
    if (tanh_form) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f));
}

template <typename T>
__global__ void gelu_kernel(const T* z, T* out, int tanh_form, long long n) {
    pdl_launch();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f<T>(gelu_value(to_f<T>(z[i]), tanh_form));
}

GG_API gg_gelu(const void* z, void* out, int dtype, int tanh_form, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(gelu_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, (const T*)z, (T*)out, tanh_form, n));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- a gate per row
// act[t, :] *= sigmoid(g . h[t, :]): one number per token, made from the token's input row h [T, W] and a stored
// vector g [W] (float32 sum), multiplies the token's activation row act [T, F] (float32 product, rounded to the
// dtype of act).  One block per token.
template <typename T>
__global__ void __launch_bounds__(256) row_gate_kernel(T* act, int F, const T* h, int W, const float* __restrict__ g,
                                                       const int* __restrict__ seq_of_token) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x;
    if (seq_of_token != nullptr && seq_of_token[t] < 0) return;
    const T* hr = h + (size_t)t * W;
    float s = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) s = fmaf(g[i], to_f<T>(hr[i]), s);
    s = block_sum(s, red);
    const float f = 1.0f / (1.0f + expf(-s));
    T* a = act + (size_t)t * F;
    for (int i = threadIdx.x; i < F; i += blockDim.x) a[i] = from_f<T>(to_f<T>(a[i]) * f);
}

GG_API gg_row_gate(void* act, int F, const void* h, int W, int dtype, const float* g, const int* seq_of_token, int ntok,
                   cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (F <= 0 || W <= 0 || g == nullptr) return GG_ERR_ARG;
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(row_gate_kernel<T>, dim3(ntok), dim3(256), 0, stream, 1, (T*)act, F, (const T*)h, W, g, seq_of_token));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- convolution of a projection's columns
// out[t, c] = act( bias[c] + sum_j w[j, c] * v[t - taps + 1 + j, c] ), v[s, c] = h[s, c] + in_bias[c] for rows of the
// sequence (the last tap meets the token itself), zeros before its start; rows from before the step come from
// state [slot][taps - 1][C] (float32: the sequence's last taps - 1 values of v).  h holds C columns of a wider
// buffer (rows ldh apart, the compute dtype); out is float32, rows ldo apart.  act 0: none, 1: silu.  bias and
// in_bias may be null.  Blocks (token, 256 channels).  one_each != 0: no sequence brings more than one row, so the
// thread of a channel is the only one that reads its state and moves it on itself; otherwise
// column_conv_state_kernel does that once every block has read the old state.
template <typename T>
__global__ void __launch_bounds__(256) column_conv_kernel(const T* h, long long ldh, float* out, long long ldo,
                                                          const float* __restrict__ w, const float* __restrict__ bias,
                                                          const float* __restrict__ in_bias, float* state,
                                                          const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                                          const int* __restrict__ seq_of_token, int C, int taps, int act,
                                                          int one_each) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const int b = seq_of_token[t];
    float* o = out + (size_t)t * ldo;
    if (b < 0) {
        for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) o[c] = 0.f;
        return;
    }
    const int start = cu_seqlens[b];
    const int R = taps - 1;
    float* st = state + (size_t)slots[b] * R * C;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        const float ib = in_bias != nullptr ? in_bias[c] : 0.f;
        const float cur = to_f<T>(h[(size_t)t * ldh + c]) + ib;
        float acc = (bias != nullptr ? bias[c] : 0.f) + w[(size_t)R * C + c] * cur;
        float carry = cur;                                 // one_each: the value that moves into the row above
        for (int j = R - 1; j >= 0; --j) {
            const int s = t - R + j;
            const float v = s >= start ? to_f<T>(h[(size_t)s * ldh + c]) + ib : st[(size_t)(R + (s - start)) * C + c];
            acc = fmaf(w[(size_t)j * C + c], v, acc);
            if (one_each) { st[(size_t)j * C + c] = carry; carry = v; }
        }
        o[c] = act == 1 ? acc / (1.0f + expf(-acc)) : acc;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) column_conv_state_kernel(const T* h, long long ldh, const float* __restrict__ in_bias,
                                                                float* state, const int* __restrict__ cu_seqlens,
                                                                const int* __restrict__ slots,
                                                                const int* __restrict__ seq_of_token, int C, int taps) {
    pdl_launch();
    pdl_wait();
    const int b = blockIdx.x;
    const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
    if (n <= 0 || seq_of_token[start] < 0) return;
    const int R = taps - 1;
    float* st = state + (size_t)slots[b] * R * C;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        const float ib = in_bias != nullptr ? in_bias[c] : 0.f;
        float keep[CONV_MAX_TAPS];
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j) {
            if (j < R) {
                const int rel = n - R + j;
                keep[j] = rel >= 0 ? to_f<T>(h[(size_t)(start + rel) * ldh + c]) + ib : st[(size_t)(R + rel) * C + c];
            }
        }
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j)
            if (j < R) st[(size_t)j * C + c] = keep[j];
    }
}

// The same for up to eight taps, a thread walking TT consecutive rows of one channel with the window of earlier values
// in registers, so that a row of h is read once instead of once per tap; the window is filled again (from the
// step's rows or the sequence's state) where a new sequence starts among the rows.  Blocks (TT rows, 256 channels).
template <typename T, int TAPS, int TT>
__global__ void __launch_bounds__(256) column_conv_tile_kernel(const T* h, long long ldh, float* out, long long ldo,
                                                               const float* __restrict__ w, const float* __restrict__ bias,
                                                               const float* __restrict__ in_bias, float* state,
                                                               const int* __restrict__ cu_seqlens,
                                                               const int* __restrict__ slots,
                                                               const int* __restrict__ seq_of_token, int C, int ntok, int act,
                                                               int one_each) {
    pdl_launch();
    pdl_wait();
    constexpr int R = TAPS - 1;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float wr[TAPS];
#pragma unroll
    for (int j = 0; j < TAPS; ++j) wr[j] = w[(size_t)j * C + c];
    const float ob = bias != nullptr ? bias[c] : 0.f, ib = in_bias != nullptr ? in_bias[c] : 0.f;
    float win[R > 0 ? R : 1];
    const int t0 = blockIdx.x * TT;
    int prev_b = -2;
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
        const int t = t0 + tt;
        if (t >= ntok) break;
        const int b = seq_of_token[t];
        if (b < 0) { out[(size_t)t * ldo + c] = 0.f; prev_b = -2; continue; }
        float* st = state + (size_t)slots[b] * R * C + c;
        if (b != prev_b) {
            const int start = cu_seqlens[b];
#pragma unroll
            for (int j = 0; j < R; ++j) {
                const int s = t - R + j;
                win[j] = s >= start ? to_f<T>(h[(size_t)s * ldh + c]) + ib : st[(size_t)(R + (s - start)) * C];
            }
            prev_b = b;
        }
        const float cur = to_f<T>(h[(size_t)t * ldh + c]) + ib;
        float acc = fmaf(wr[R], cur, ob);
#pragma unroll
        for (int j = 0; j < R; ++j) acc = fmaf(wr[j], win[j], acc);
        out[(size_t)t * ldo + c] = act == 1 ? acc / (1.0f + expf(-acc)) : acc;
#pragma unroll
        for (int j = 0; j + 1 < R; ++j) win[j] = win[j + 1];
        if (R > 0) win[R - 1] = cur;
        if (one_each) {                                   // the sequence's only row of the step: its state moves on
#pragma unroll
            for (int j = 0; j < R; ++j) st[(size_t)j * C] = win[j];
        }
    }
}

template <typename T, int TAPS>
static int column_conv_tile_launch(const T* h, long long ldh, float* out, long long ldo, const float* w, const float* bias,
                                   const float* in_bias, float* state, const int* cu_seqlens, const int* slots,
                                   const int* seq_of_token, int ntok, int C, int act, int one_each, cudaStream_t stream) {
    const unsigned cb = (unsigned)((C + 255) / 256);
    if (ntok < 1024 || one_each)       // few rows, or a row a sequence: a row a thread, so that the step fills more of the GPU
        return gg_launch(column_conv_tile_kernel<T, TAPS, 1>, dim3((unsigned)ntok, cb), dim3(256), 0, stream, 1, h, ldh, out, ldo,
                         w, bias, in_bias, state, cu_seqlens, slots, seq_of_token, C, ntok, act, one_each);
    return gg_launch(column_conv_tile_kernel<T, TAPS, 8>, dim3((unsigned)((ntok + 7) / 8), cb), dim3(256), 0, stream, 1, h, ldh,
                     out, ldo, w, bias, in_bias, state, cu_seqlens, slots, seq_of_token, C, ntok, act, one_each);
}

template <typename T>
static int column_conv_tile(int taps, const T* h, long long ldh, float* out, long long ldo, const float* w, const float* bias,
                            const float* in_bias, float* state, const int* cu_seqlens, const int* slots,
                            const int* seq_of_token, int ntok, int C, int act, int one_each, cudaStream_t stream) {
#define CC_CASE(N) case N: return column_conv_tile_launch<T, N>(h, ldh, out, ldo, w, bias, in_bias, state, cu_seqlens, slots, \
                                                                seq_of_token, ntok, C, act, one_each, stream);
    switch (taps) { CC_CASE(1) CC_CASE(2) CC_CASE(3) CC_CASE(4) CC_CASE(5) CC_CASE(6) CC_CASE(7) CC_CASE(8) }
#undef CC_CASE
    return GG_ERR_ARG;
}

// w [taps][C] float32 (a tap's weights side by side); state [slots][taps - 1][C] float32 (null only for one tap).
GG_API gg_column_conv(const void* h, long long ldh, int dtype, float* out, long long ldo, const float* w, const float* bias,
                      const float* in_bias, float* state, const int* cu_seqlens, const int* slots, const int* seq_of_token,
                      int ntok, int n_seqs, int C, int taps, int act, int max_new, cudaStream_t stream) {
    if (ntok <= 0 || n_seqs <= 0) return 0;
    if (C <= 0 || taps < 1 || taps > CONV_MAX_TAPS || (taps > 1 && state == nullptr) || act < 0 || act > 1 || ldh < C || ldo < C)
        return GG_ERR_ARG;
    const int cb = min((C + 255) / 256, 65535);
    const int one_each = max_new == 1;
    GG_DISPATCH_DTYPE(dtype, T,
        if (taps <= 8 && cb <= 65535) {
            column_conv_tile<T>(taps, (const T*)h, ldh, out, ldo, w, bias, in_bias, state, cu_seqlens, slots, seq_of_token, ntok,
                                C, act, one_each, stream);
        } else {
            gg_launch(column_conv_kernel<T>, dim3(ntok, cb), dim3(256), 0, stream, 1, (const T*)h, ldh, out, ldo, w, bias, in_bias,
                      state, cu_seqlens, slots, seq_of_token, C, taps, act, one_each);
        }
        if (taps > 1 && !one_each)
            gg_launch(column_conv_state_kernel<T>, dim3(n_seqs, cb), dim3(256), 0, stream, 1, (const T*)h, ldh, in_bias, state,
                      cu_seqlens, slots, seq_of_token, C, taps));
    return gg_last_error();
}

// 1 if this library was built with checked page tables (the debug build), else 0.
GG_API gg_elementwise_checked() { return gg_debug_bounds(); }
