// Routed experts: the router's choice, and the experts' products through an index (no sorting, no host
// round trip), for steps of few tokens and for the 32-bit path.
//
//   route:    s = score(z) per expert (sigmoid, or softmax over all experts); the `top` largest are chosen
//             (ties go to the lower index); weights are the chosen scores, optionally divided by their sum.
//   gate_up:  for pair p = (token t, choice k) with expert e: x = h[t] (times the weight if the weight sits on
//             the expert's input); g = Wg[e] x, u = Wu[e] x; y[p] = out_scale * act(g, u) (times the weight if
//             it sits on the output).
//   down:     residual[t] += sum_k Wd[e(t, k)] y[t, k]  (k in order: the sum does not depend on the batch).
//
// act "clamped glu": g' = min(g, L), u' = clamp(u, -L, L), g' * sigmoid(slope g') * (u' + up_offset); the plain gated unit silu(g) u is L = infinity, slope 1, offset 0.
// Router scores, the choice, the weights and all sums are float32.
#include "common.cuh"

// ----------------------------------------------------------------------------- router logits
// z[t, e] = Wr[e] . h[t] in float32: a warp per (token, expert), the token's row in shared memory.  A product of so
// few output columns would be one or two CTAs of the tiled kernels; this one has a CTA per token and 8 experts.
template <typename TX, typename TW>
__global__ void __launch_bounds__(256) moe_router_logits_kernel(const TX* h, const TW* __restrict__ wr, float* z, int W, int E) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float rx[];
    const int t = blockIdx.x;
    const TX* ht = h + (size_t)t * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) rx[i] = to_f<TX>(ht[i]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.y * 8 + warp;
    if (e >= E) return;
    const TW* w = wr + (size_t)e * W;
    float s = 0.f;
    for (int i = lane; i < W; i += 32) s = fmaf(to_f<TW>(w[i]), rx[i], s);
    s = warp_sum(s);
    if (lane == 0) z[(size_t)t * E + e] = s;
}

GG_API gg_moe_router_logits(const void* h, int h_dtype, const void* wr, int w_dtype, float* z, int T, int W, int E,
                            cudaStream_t stream) {
    if (T <= 0) return 0;
    if (W <= 0 || E <= 0 || (size_t)W * 4 > 48 * 1024 || (E + 7) / 8 > 65535) return GG_ERR_ARG;
    dim3 grid(T, (E + 7) / 8);
    const size_t smem = (size_t)W * sizeof(float);
#define GG_RL(TX, TW) gg_launch(moe_router_logits_kernel<TX, TW>, dim3(grid), dim3(256), smem, stream, 1, (const TX*)h, \
        (const TW*)wr, z, W, E)
    if (h_dtype == GG_F32 && w_dtype == GG_F32) GG_RL(float, float);
    else if (h_dtype == GG_BF16 && w_dtype == GG_BF16) GG_RL(bf16, bf16);
    else if (h_dtype == GG_BF16 && w_dtype == GG_F32) GG_RL(bf16, float);
    else if (h_dtype == GG_F32 && w_dtype == GG_BF16) GG_RL(float, bf16);
    else return GG_ERR_DTYPE;
#undef GG_RL
    return gg_last_error();
}

// ----------------------------------------------------------------------------- route
// One warp per token.  z [T, E] float32 logits.  softmax != 0: scores are softmax(z), else sigmoid(z).
__global__ void __launch_bounds__(32) moe_route_kernel(const float* z, int E, int top, int softmax, int renorm,
                                                       int n_real, float scale,
                                                       int* idx, float* wts, const int* __restrict__ seq_of_token) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x;
    const float* zt = z + (size_t)t * E;
    if (seq_of_token != nullptr && seq_of_token[t] < 0) {      // padding: expert 0 with weight 0
        for (int k = lane; k < top; k += 32) { idx[(size_t)t * top + k] = 0; wts[(size_t)t * top + k] = 0.f; }
        return;
    }
    float mx = -INFINITY, den = 1.f;
    if (softmax) {
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zt[e]);
        mx = warp_max(mx);
        float s = 0.f;
        for (int e = lane; e < E; e += 32) s += expf(zt[e] - mx);
        den = warp_sum(s);
    }
    float total = 0.f;
    float prev_v = INFINITY;
    int prev_i = -1;
    for (int k = 0; k < top; ++k) {
        // the largest logit after (prev_v, prev_i) in the order (value descending, index ascending)
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = zt[e];
            const bool after = v < prev_v || (v == prev_v && e > prev_i);
            if (after && (v > bv || (v == bv && e < bi))) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        const float s = softmax ? expf(bv - mx) / den : 1.0f / (1.0f + expf(-bv));
        if (lane == 0) { idx[(size_t)t * top + k] = bi < n_real ? bi : -1; wts[(size_t)t * top + k] = s; }
        total += s;
        prev_v = bv;
        prev_i = bi;
    }
    if (renorm || scale != 1.0f) {
        __syncwarp();
        const float f = renorm ? scale / (total + 1e-20f) : scale;
        for (int k = lane; k < top; k += 32) wts[(size_t)t * top + k] *= f;
    }
}

// The same choice with a correction and groups: scores s = sigmoid(z) (or softmax); the choice scores are
// s + correction[e] (correction may be null); the experts form `groups` equal runs of neighbours, a group's score
// is the sum of its two largest choice scores, and only experts of the `keep` best groups can be chosen (the others
// count as minus infinity).  The `top` largest choice scores are chosen (ties to the lower index); the weights are
// the chosen experts' scores s without the correction.  One warp per token; scores in shared memory.
__global__ void __launch_bounds__(32) moe_route_grouped_kernel(const float* z, int E, int top, int softmax, int renorm,
                                                               const float* __restrict__ correction, int groups, int keep,
                                                               int n_real, float scale,
                                                               int* idx, float* wts, const int* __restrict__ seq_of_token) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float rsm[];
    float* sc = rsm;                 // [E] scores
    float* ch = sc + E;              // [E] choice scores (minus infinity once chosen or outside the kept groups)
    float* gsc = ch + E;             // [groups]
    const int t = blockIdx.x, lane = threadIdx.x;
    const float* zt = z + (size_t)t * E;
    if (seq_of_token != nullptr && seq_of_token[t] < 0) {      // padding: expert 0 with weight 0
        for (int k = lane; k < top; k += 32) { idx[(size_t)t * top + k] = 0; wts[(size_t)t * top + k] = 0.f; }
        return;
    }
    float mx = -INFINITY, den = 1.f;
    if (softmax) {
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zt[e]);
        mx = warp_max(mx);
        float s = 0.f;
        for (int e = lane; e < E; e += 32) s += expf(zt[e] - mx);
        den = warp_sum(s);
    }
    for (int e = lane; e < E; e += 32) {
        const float s = softmax ? expf(zt[e] - mx) / den : 1.0f / (1.0f + expf(-zt[e]));
        sc[e] = s;
        ch[e] = s + (correction != nullptr ? correction[e] : 0.f);
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float a = -INFINITY, b2 = -INFINITY;             // the two largest of the group
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = ch[e];
                if (v > a) { b2 = a; a = v; } else if (v > b2) b2 = v;
            }
            gsc[g] = per > 1 ? a + b2 : a;
        }
        __syncwarp();
        // drop the groups - keep worst groups: the worst is the lowest score, ties to the higher index
        for (int k = 0; k < groups - keep; ++k) {
            float wv = INFINITY;
            int wi = -1;
            for (int g = lane; g < groups; g += 32) {
                const float v = gsc[g];
                if (v != INFINITY && (v < wv || (v == wv && g > wi))) { wv = v; wi = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, wv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
                if (oi >= 0 && (wi < 0 || ov < wv || (ov == wv && oi > wi))) { wv = ov; wi = oi; }
            }
            if (wi < 0) break;
            for (int e = wi * per + lane; e < (wi + 1) * per; e += 32) ch[e] = -INFINITY;
            if (lane == 0) gsc[wi] = INFINITY;                // marks a dropped group
            __syncwarp();
        }
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = ch[e];
            if (v > bv || (v == bv && e < bi && v != -INFINITY)) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi >= E) bi = 0;                                  // fewer candidates than `top` (refused by the launcher)
        const float s = sc[bi];
        if (lane == 0) {
            idx[(size_t)t * top + k] = bi < n_real ? bi : -1;
            wts[(size_t)t * top + k] = bv == -INFINITY ? 0.f : s;
            ch[bi] = -INFINITY;
        }
        total += s;
        __syncwarp();
    }
    if (renorm || scale != 1.0f) {
        const float f = renorm ? scale / (total + 1e-20f) : scale;
        for (int k = lane; k < top; k += 32) wts[(size_t)t * top + k] *= f;
    }
}

// correction [E] (may be null); groups >= 1 equal runs of neighbouring experts of which `keep` can be chosen from.
// n_real (0: all E): router outputs from n_real on have no expert behind them (identity experts: the caller adds
// weight times the token's own row); a choice of one is stored as index -1 with its weight.  scale multiplies the
// weights after the renormalisation (which divides by the chosen scores' sum + 1e-20).
GG_API gg_moe_route(const float* z, int T, int E, int top, int softmax, int renorm, const float* correction, int groups,
                    int keep, int n_real, float scale, int* idx, float* wts, const int* seq_of_token, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || n_real < 0 || n_real > E) return GG_ERR_ARG;
    if (n_real == 0) n_real = E;
    if (groups < 1) groups = 1;
    if (keep < 1 || keep > groups) keep = groups;
    if (correction == nullptr && keep == groups) {
        gg_launch(moe_route_kernel, dim3(T), dim3(32), 0, stream, 1, z, E, top, softmax, renorm, n_real, scale, idx, wts, seq_of_token);
        return gg_last_error();
    }
    if (E % groups || top > (E / groups) * keep) return GG_ERR_ARG;
    const size_t smem = ((size_t)2 * E + groups) * sizeof(float);
    if (smem > 48 * 1024) return GG_ERR_ARG;
    gg_launch(moe_route_grouped_kernel, dim3(T), dim3(32), smem, stream, 1, z, E, top, softmax, renorm, correction, groups,
              keep, n_real, scale, idx, wts, seq_of_token);
    return gg_last_error();
}

// ----------------------------------------------------------------------------- activation
__device__ __forceinline__ float clamped_glu(float g, float u, float limit, float slope, float up_offset) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-slope * g)) * (u + up_offset);
}

// ----------------------------------------------------------------------------- gate and up through the index
// grid (pairs, ceil(F / 8)); 8 warps, one feature each: the two rows Wg[e][f], Wu[e][f] against x in shared memory.
// w_gu [E][2][F][W]: an expert's gate rows, then its up rows.
template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256) moe_gate_up_kernel(const TX* h, const TW* __restrict__ w_gu, const int* idx,
                                                          const float* wts, TY* y, int W, int F, int top,
                                                          int weight_on_input, float limit, float slope, float up_offset, float out_scale) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float xs[];
    const int p = blockIdx.x, t = p / top;
    const int e = idx[p];
    if (e < 0) return;                                   // a choice without an expert: nothing reads its row
    const float wt = wts[p];
    const float xin = weight_on_input ? wt : 1.0f;
    const TX* ht = h + (size_t)t * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) xs[i] = to_f<TX>(ht[i]) * xin;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f = blockIdx.y * 8 + warp;
    if (f >= F) return;
    const TW* wg = w_gu + ((size_t)e * 2 * F + f) * W;
    const TW* wu = wg + (size_t)F * W;
    float g = 0.f, u = 0.f;
    for (int i = lane; i < W; i += 32) {
        const float x = xs[i];
        g = fmaf(to_f<TW>(wg[i]), x, g);
        u = fmaf(to_f<TW>(wu[i]), x, u);
    }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) {
        float a = clamped_glu(g, u, limit, slope, up_offset) * out_scale;
        if (!weight_on_input) a *= wt;
        y[(size_t)p * F + f] = from_f<TY>(a);
    }
}

GG_API gg_moe_gate_up(const void* h, int h_dtype, const void* w_gu, int w_dtype, const int* idx, const float* wts,
                      void* y, int y_dtype, int T, int W, int F, int top, int weight_on_input, float limit,
                      float slope, float up_offset, float out_scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (W <= 0 || F <= 0 || top <= 0 || (size_t)W * 4 > 48 * 1024 || (F + 7) / 8 > 65535) return GG_ERR_ARG;
    dim3 grid(T * top, (F + 7) / 8);
    const size_t smem = (size_t)W * sizeof(float);
#define GG_GU(TX, TW, TY) gg_launch(moe_gate_up_kernel<TX, TW, TY>, dim3(grid), dim3(256), smem, stream, 1, (const TX*)h, \
        (const TW*)w_gu, idx, wts, (TY*)y, W, F, top, weight_on_input, limit, slope, up_offset, out_scale)
    if (h_dtype == GG_F32 && w_dtype == GG_F32 && y_dtype == GG_F32) GG_GU(float, float, float);
    else if (h_dtype == GG_BF16 && w_dtype == GG_BF16 && y_dtype == GG_F32) GG_GU(bf16, bf16, float);
    else if (h_dtype == GG_BF16 && w_dtype == GG_BF16 && y_dtype == GG_BF16) GG_GU(bf16, bf16, bf16);
    else return GG_ERR_DTYPE;
#undef GG_GU
    return gg_last_error();
}

// ----------------------------------------------------------------------------- down through the index
// grid (tokens, ceil(W / 8)); one warp per output element of the token; y[t, k] in shared memory, k by k.
// w_d [E][W][F].
template <typename TY, typename TW>
__global__ void __launch_bounds__(256) moe_down_kernel(const TY* y, const TW* __restrict__ w_d, const int* idx,
                                                       float* residual, int W, int F, int top,
                                                       const int* __restrict__ seq_of_token) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float ys[];
    const int t = blockIdx.x;
    if (seq_of_token != nullptr && seq_of_token[t] < 0) return;
    const TY* yt = y + (size_t)t * top * F;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.y * 8 + warp;
    float total = 0.f;
    for (int k = 0; k < top; ++k) {                      // one choice's row at a time in shared memory
        __syncthreads();
        for (int i = threadIdx.x; i < F; i += blockDim.x) ys[i] = to_f<TY>(yt[(size_t)k * F + i]);
        __syncthreads();
        if (n < W) {
            const int e = idx[(size_t)t * top + k];
            if (e < 0) continue;                         // a choice without an expert
            const TW* wr = w_d + ((size_t)e * W + n) * F;
            float s = 0.f;
            for (int i = lane; i < F; i += 32) s = fmaf(to_f<TW>(wr[i]), ys[i], s);
            total += warp_sum(s);
        }
    }
    if (n < W && lane == 0) residual[(size_t)t * W + n] += total;
}

GG_API gg_moe_down(const void* y, int y_dtype, const void* w_d, int w_dtype, const int* idx, float* residual, int T,
                   int W, int F, int top, const int* seq_of_token, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (W <= 0 || F <= 0 || top <= 0 || (size_t)F * 4 > 48 * 1024 || (W + 7) / 8 > 65535) return GG_ERR_ARG;
    dim3 grid(T, (W + 7) / 8);
    const size_t smem = (size_t)F * sizeof(float);
#define GG_DN(TY, TW) gg_launch(moe_down_kernel<TY, TW>, dim3(grid), dim3(256), smem, stream, 1, (const TY*)y, \
        (const TW*)w_d, idx, residual, W, F, top, seq_of_token)
    if (y_dtype == GG_F32 && w_dtype == GG_F32) GG_DN(float, float);
    else if (y_dtype == GG_F32 && w_dtype == GG_BF16) GG_DN(float, bf16);
    else if (y_dtype == GG_BF16 && w_dtype == GG_BF16) GG_DN(bf16, bf16);
    else return GG_ERR_DTYPE;
#undef GG_DN
    return gg_last_error();
}

// ----------------------------------------------------------------------------- sorted form (steps of many tokens)
// The (token, choice) pairs are grouped by expert so that each expert's rows are consecutive and one tensor-core
// product per expert serves them:  sort (counts, offsets, a place for every pair)  ->  gather (row of place i =
// the pair's token row, times its weight if the weight sits on the input)  ->  per expert: gate/up product,
// activation, down product (float32 rows)  ->  combine (residual[t] += the rows of the token's pairs, k in order).
// A row's result does not depend on its place, so the order of pairs inside an expert's range is free.

// One block.  offsets[E + 1] (exclusive prefix sums of the experts' counts), place[p] for every pair.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* idx, int P, int E, int* offsets, int* place,
                                                        int* cursor /* [E] scratch */) {
    pdl_launch();
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) cursor[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&cursor[idx[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) { const int c = cursor[e]; offsets[e] = run; cursor[e] = run; run += c; }
        offsets[E] = run;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) place[p] = atomicAdd(&cursor[idx[p]], 1);
}

GG_API gg_moe_sort(const int* idx, int P, int E, int* offsets, int* place, int* cursor, cudaStream_t stream) {
    if (P <= 0) return 0;
    if (E <= 0) return GG_ERR_ARG;
    gg_launch(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, 1, idx, P, E, offsets, place, cursor);
    return gg_last_error();
}

// xs[place[p]] (xs[p] without `place`) = bfloat16(h[p / top] * (weight_on_input ? wts[p] : 1)); one block per pair.
__global__ void __launch_bounds__(128) moe_gather_kernel(const bf16* h, const float* wts, const int* place, bf16* xs,
                                                         int W, int top, int weight_on_input) {
    pdl_launch();
    pdl_wait();
    const int p = blockIdx.x;
    const float f = weight_on_input ? wts[p] : 1.0f;
    const bf16* src = h + (size_t)(p / top) * W;
    bf16* dst = xs + (size_t)(place != nullptr ? place[p] : p) * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) dst[i] = __float2bfloat16_rn(__bfloat162float(src[i]) * f);
}

GG_API gg_moe_gather(const void* h, const float* wts, const int* place, void* xs, int P, int W, int top,
                     int weight_on_input, cudaStream_t stream) {
    if (P <= 0) return 0;
    gg_launch(moe_gather_kernel, dim3(P), dim3(128), 0, stream, 1, (const bf16*)h, wts, place, (bf16*)xs, W, top,
              weight_on_input);
    return gg_last_error();
}

// y[i, f] = out_scale * act(gu[i, f], gu[i, F + f]) (times the pair's weight if it sits on the output), rows in
// sorted order; pair_of[i] is the pair at place i (only read when the weight is on the output).
__global__ void moe_glu_rows_kernel(const bf16* gu, bf16* y, long long n, int F, float limit, float slope, float up_offset, float out_scale,
                                    const float* wts, const int* pair_of) {
    pdl_launch();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long row = i / F;
    const int f = (int)(i % F);
    float a = clamped_glu(__bfloat162float(gu[row * 2 * F + f]), __bfloat162float(gu[row * 2 * F + F + f]), limit, slope, up_offset) * out_scale;
    if (pair_of != nullptr) a *= wts[pair_of[row]];
    y[i] = __float2bfloat16_rn(a);
}

GG_API gg_moe_glu_rows(const void* gu, void* y, int P, int F, float limit, float slope, float up_offset, float out_scale,
                       const float* wts, const int* pair_of, cudaStream_t stream) {
    if (P <= 0) return 0;
    const long long n = (long long)P * F;
    gg_launch(moe_glu_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, (const bf16*)gu, (bf16*)y, n, F,
              limit, slope, up_offset, out_scale, wts, pair_of);
    return gg_last_error();
}

// pair_of[place[p]] = p
__global__ void moe_invert_kernel(const int* place, int* pair_of, int P) {
    pdl_launch();
    pdl_wait();
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p < P) pair_of[place[p]] = p;
}

GG_API gg_moe_invert(const int* place, int* pair_of, int P, cudaStream_t stream) {
    if (P <= 0) return 0;
    gg_launch(moe_invert_kernel, dim3((P + 255) / 256), dim3(256), 0, stream, 1, place, pair_of, P);
    return gg_last_error();
}

// residual[t, :] += sum_k rows[place[t * top + k], :]  (without `place`: the rows are in pair order)
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* rows, const int* place, float* residual, int W,
                                                          int top, const int* __restrict__ seq_of_token, const int* idx) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    if (seq_of_token != nullptr && seq_of_token[t] < 0) return;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const size_t p = (size_t)t * top + k;
            if (idx != nullptr && idx[p] < 0) continue;      // a choice without an expert left no row
            s += rows[(place != nullptr ? (size_t)place[p] : p) * W + i];
        }
        residual[(size_t)t * W + i] += s;
    }
}

// idx (may be null): the pairs' expert indices; pairs whose index is negative are left out.
GG_API gg_moe_combine(const float* rows, const int* place, float* residual, int T, int W, int top,
                      const int* seq_of_token, const int* idx, cudaStream_t stream) {
    if (T <= 0) return 0;
    gg_launch(moe_combine_kernel, dim3(T), dim3(256), 0, stream, 1, rows, place, residual, W, top, seq_of_token, idx);
    return gg_last_error();
}

// ----------------------------------------------------------------------------- identity experts
// residual[t, :] += sum over the choices k of token t whose index is negative of wts[t, k] * h[t, :]: an identity
// expert gives back its input, times the router's weight.  One block per token.
template <typename TX>
__global__ void __launch_bounds__(256) moe_identity_kernel(const TX* h, const int* idx, const float* wts, float* residual,
                                                           int W, int top, const int* __restrict__ seq_of_token) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    if (seq_of_token != nullptr && seq_of_token[t] < 0) return;
    float f = 0.f;
    for (int k = 0; k < top; ++k)
        if (idx[(size_t)t * top + k] < 0) f += wts[(size_t)t * top + k];
    if (f == 0.f) return;
    for (int i = threadIdx.x; i < W; i += blockDim.x) residual[(size_t)t * W + i] += f * to_f<TX>(h[(size_t)t * W + i]);
}

GG_API gg_moe_identity(const void* h, int h_dtype, const int* idx, const float* wts, float* residual, int T, int W, int top,
                       const int* seq_of_token, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (W <= 0 || top <= 0) return GG_ERR_ARG;
    GG_DISPATCH_DTYPE(h_dtype, TX,
        gg_launch(moe_identity_kernel<TX>, dim3(T), dim3(256), 0, stream, 1, (const TX*)h, idx, wts, residual, W, top,
                  seq_of_token));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- the experts on mma.sync (few pairs)
// Decode steps and short prompts in bfloat16: a CTA belongs to one expert and 64 of its output rows (features of
// gate and up, or elements of the down projection).  It collects the pairs that chose its expert (none: it leaves
// without touching a weight), takes their input rows as the 16-row operand of m16n8k16 and streams its weight rows
// once, 64 columns of k at a time through two cp.async stages.  x [P, K] in pair order (gate/up: the token's row
// times the weight where the weight sits on the input; down: the activation rows).  GATED: w [E][2][N][K], out[p, n] =
// out_scale * act(gate, up) (* wts[p] where given) as bfloat16; else w [E][N][K] and out[p, n] the float32 sum.
__device__ __forceinline__ void mx_mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mx_cp16(void* smem, const void* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void mx_ldsm(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
#define MX_KS 64
#define MX_LD (MX_KS + 8)
#define MX_MAXP 8192

template <bool GATED>
__global__ void __launch_bounds__(128) moe_expert_mma_kernel(const bf16* x, const bf16* __restrict__ w, const int* idx, int P,
                                                             void* out, int N, int K, float limit, float slope, float up_offset,
                                                             float out_scale, const float* wts) {
    pdl_launch();
    extern __shared__ __align__(16) unsigned char mx_raw[];
    constexpr int TILES = GATED ? 3 : 2;                 // x, gate (or the one matrix), up
    bf16* stage0 = reinterpret_cast<bf16*>(mx_raw);      // [2 stages][TILES][64][MX_LD]
    int* list = reinterpret_cast<int*>(mx_raw + (size_t)2 * TILES * 64 * MX_LD * sizeof(bf16));
    __shared__ int count;
    const int e = blockIdx.x, n0 = blockIdx.y * 64;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) count = 0;
    __syncthreads();
    pdl_wait();
    for (int p = tid; p < P; p += 128)
        if (idx[p] == e) list[atomicAdd(&count, 1)] = p;
    __syncthreads();
    const int cnt = count;
    if (cnt == 0) return;
    const bf16* wg = w + ((size_t)e * (GATED ? 2 : 1) * N + n0) * K;
    const bf16* wu = wg + (size_t)N * K;
    const int ksteps = (K + MX_KS - 1) / MX_KS;
    const int g = lane >> 2, q4 = lane & 3;
    for (int m0 = 0; m0 < cnt; m0 += 64) {
        const int rows = min(64, cnt - m0);
        auto load = [&](int kc, int st) {
            bf16* xs = stage0 + (size_t)st * TILES * 64 * MX_LD;
            bf16* gs = xs + 64 * MX_LD;
            bf16* us = gs + 64 * MX_LD;
            const int k0 = kc * MX_KS;
            for (int c = tid; c < 64 * (MX_KS / 8); c += 128) {
                const int row = c / (MX_KS / 8), kk = (c % (MX_KS / 8)) * 8;
                const bool kin = k0 + kk < K;
                bf16* dx = xs + row * MX_LD + kk;
                if (row < rows && kin) mx_cp16(dx, x + (size_t)list[m0 + row] * K + k0 + kk);
                else *reinterpret_cast<uint4*>(dx) = make_uint4(0u, 0u, 0u, 0u);
                bf16* dg = gs + row * MX_LD + kk;
                if (n0 + row < N && kin) mx_cp16(dg, wg + (size_t)row * K + k0 + kk);
                else *reinterpret_cast<uint4*>(dg) = make_uint4(0u, 0u, 0u, 0u);
                if (GATED) {
                    bf16* du = us + row * MX_LD + kk;
                    if (n0 + row < N && kin) mx_cp16(du, wu + (size_t)row * K + k0 + kk);
                    else *reinterpret_cast<uint4*>(du) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        float ag[8][4], au[GATED ? 8 : 1][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) { ag[i][j] = 0.f; if (GATED) au[i][j] = 0.f; }
        load(0, 0);
        for (int kc = 0; kc < ksteps; ++kc) {
            if (kc + 1 < ksteps) {
                load(kc + 1, (kc + 1) & 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncthreads();
            if (warp * 16 < rows) {                      // warps without pairs only copy
                const bf16* xs = stage0 + (size_t)(kc & 1) * TILES * 64 * MX_LD;
                const bf16* gs = xs + 64 * MX_LD;
                const bf16* us = gs + 64 * MX_LD;
#pragma unroll
                for (int ks = 0; ks < MX_KS / 16; ++ks) {
                    uint32_t a[4];
                    mx_ldsm(a, xs + (warp * 16 + (lane & 15)) * MX_LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int np = 0; np < 4; ++np) {
                        const int off = (np * 16 + (lane & 7) + (lane >> 4) * 8) * MX_LD + ks * 16 + ((lane >> 3) & 1) * 8;
                        uint32_t b[4];
                        mx_ldsm(b, gs + off);
                        mx_mma16816(ag[2 * np], a, b[0], b[1]);
                        mx_mma16816(ag[2 * np + 1], a, b[2], b[3]);
                        if (GATED) {
                            mx_ldsm(b, us + off);
                            mx_mma16816(au[2 * np], a, b[0], b[1]);
                            mx_mma16816(au[2 * np + 1], a, b[2], b[3]);
                        }
                    }
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = warp * 16 + g + half * 8;
            if (row >= rows) continue;
            const int p = list[m0 + row];
            const float f = GATED ? out_scale * (wts != nullptr ? wts[p] : 1.0f) : 1.0f;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int n = n0 + nt * 8 + 2 * q4 + j;
                    if (n >= N) continue;
                    if (GATED)
                        reinterpret_cast<bf16*>(out)[(size_t)p * N + n] =
                            __float2bfloat16_rn(clamped_glu(ag[nt][2 * half + j], au[nt][2 * half + j], limit, slope, up_offset) * f);
                    else
                        reinterpret_cast<float*>(out)[(size_t)p * N + n] = ag[nt][2 * half + j];
                }
        }
        __syncthreads();
    }
}

// gated != 0: x [P, K], w [E, 2, N, K], out bfloat16 [P, N]; else w [E, N, K], out float32 [P, N].  P <= 8,192 pairs.
GG_API gg_moe_expert_mma(const void* x, const void* w, const int* idx, int P, int E, void* out, int N, int K, int gated,
                         float limit, float slope, float up_offset, float out_scale, const float* wts, cudaStream_t stream) {
    if (P <= 0) return 0;
    if (E <= 0 || N <= 0 || K <= 0 || (K % 8) || P > MX_MAXP || (N + 63) / 64 > 65535 ||
        (((uintptr_t)x | (uintptr_t)w) & 15))
        return GG_ERR_ARG;
    dim3 grid(E, (N + 63) / 64);
    const size_t smem = (size_t)2 * (gated ? 3 : 2) * 64 * MX_LD * sizeof(bf16) + MX_MAXP * sizeof(int);
    static bool set_g = false, set_p = false;
    if (gated) {
        if (!set_g) {
            cudaError_t er = cudaFuncSetAttribute(moe_expert_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
            if (er != cudaSuccess) return (int)er;
            set_g = true;
        }
        return gg_launch(moe_expert_mma_kernel<true>, dim3(grid), dim3(128), smem, stream, 1, (const bf16*)x, (const bf16*)w, idx, P,
                         out, N, K, limit, slope, up_offset, out_scale, wts);
    }
    if (!set_p) {
        cudaError_t er = cudaFuncSetAttribute(moe_expert_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (er != cudaSuccess) return (int)er;
        set_p = true;
    }
    return gg_launch(moe_expert_mma_kernel<false>, dim3(grid), dim3(128), smem, stream, 1, (const bf16*)x, (const bf16*)w, idx, P,
                     out, N, K, limit, slope, up_offset, out_scale, wts);
}
