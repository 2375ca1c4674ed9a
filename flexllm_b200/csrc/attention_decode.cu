// Decode attention over a paged int8 KV cache (one new token per sequence, GQA).
//
// Cache layout, per layer (pool of `n_pages` pages of PAGE = 64 tokens, any page order):
//   K   [n_pages][HKV][PAGE][64] s8    one 64-byte row per token
//   Ks  [n_pages][HKV][PAGE]     f32   per-token-per-head scale
//   V^T [n_pages][HKV][64][PAGE] s8    transposed inside the page: for each of the 64 dims the
//                                       page's 64 tokens are contiguous, so P.V runs as dp4a over keys
//   Vs  [n_pages][HKV][PAGE]     f32
// (the reference keeps K token-major and V dimension-major for the same reason: Modules/MHA.h:85-90,
// :311-316; its caches are contiguous, Modules/MHA.h:447-559, :741-851 -- paging is new here.)
//
// One step for B sequences on one layer = the oracle's composition (decode graph order,
// SpinQuant_Llama_32_1B/MHA_i8xi8.h:1072-1111):
//   1. append : q,k -> dequant, RoPE(ctx), FHT-64/8, per-head int8 quant; k,v written at slot ctx
//   2. scores : x[h][j] = (((float)(q.k_j) * qs) * ks_j) * 0.125 for j <= ctx, per-split row max
//   3. softmax: row max, e = exp(x - max) (kept in place of x), the four ordered partial sums over
//               j mod 4, r = 1 / ((p0+p1)+(p2+p3))        -- one thread per chain, sequential adds
//   4. pv     : U_j = min(round(((e_j * r) * vs_j) / a_s), 255); O[d] += U_j * v_j[d] in int32,
//               partial sums of key ranges combined with integer atomics (exact, order-free)
//   5. out    : (float)O * a_s
// HBM-bound on the K and V pages (read once each); scores cost 2 x 4 bytes per (head, key).
#include <new>

#include "common.cuh"
#include "attention_decode.cuh"

namespace flexllm {

int* device_error_flag();

static inline KvLayer kv_layer(const flexllm_kv_cache* c, int layer) {
    KvLayer l;
    l.k = c->k + (size_t)layer * c->page_bytes;
    l.v = c->v + (size_t)layer * c->page_bytes;
    l.ks = c->ks + (size_t)layer * (c->scale_bytes / 4);
    l.vs = c->vs + (size_t)layer * (c->scale_bytes / 4);
    return l;
}

// ---- 1. append ---------------------------------------------------------------------------------
// One warp per (sequence, head). Heads [0,HQ) are query heads, [HQ, HQ+HKV) key heads,
// [HQ+HKV, HQ+2*HKV) value heads.
// With IN_F32 the inputs are one fp32 row [ (HQ+2*HKV)*64 ] per sequence (q heads, k heads, v heads,
// the output of the fused q/k/v projection); value heads are then quantised per head here.
template <bool IN_F32>
__global__ void __launch_bounds__(256) dec_append_kernel(const int8_t* __restrict__ q, const float* __restrict__ qs,
                                                         const int8_t* __restrict__ k, const float* __restrict__ ks,
                                                         const int8_t* __restrict__ v, const float* __restrict__ vs,
                                                         const float* __restrict__ qkv_f32,
                                                         const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                         KvLayer cache, const int32_t* __restrict__ page_table, int max_pages,
                                                         const int32_t* __restrict__ ctx, int B, int HQ, int HKV,
                                                         int8_t* __restrict__ q2, float* __restrict__ qs2, int max_pos,
                                                         int* error_flag) {
    const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int heads = HQ + 2 * HKV;
    if (w >= B * heads) return;
    const int b = w / heads, h = w % heads;
    const int pos = dec_guarded_pos(ctx, b, max_pos, error_flag);
    const long pg = page_table[(long)b * max_pages + pos / PAGE];
    const int slot = pos % PAGE;
    if (h >= HQ + HKV) {   // value head: into the transposed page
        const int hv = h - HQ - HKV;
        int8_t* dst = cache.v + (pg * HKV + hv) * (long)(64 * PAGE);
        if (IN_F32) {
            const float* src = qkv_f32 + (long)b * heads * 64 + (long)h * 64;
            const float a = src[lane], bb = src[lane + 32];
            const float mx = warp_max(fmaxf(a, bb)), mn = warp_min(fminf(a, bb));
            const float sc = sym_scale_from(mx, mn);
            dst[(long)lane * PAGE + slot] = quant_s8(a, sc);
            dst[(long)(lane + 32) * PAGE + slot] = quant_s8(bb, sc);
            if (lane == 0) cache.vs[(pg * HKV + hv) * PAGE + slot] = sc;
        } else {
            const int8_t* src = v + ((long)b * HKV + hv) * 64;
            dst[(long)lane * PAGE + slot] = src[lane];
            dst[(long)(lane + 32) * PAGE + slot] = src[lane + 32];
            if (lane == 0) cache.vs[(pg * HKV + hv) * PAGE + slot] = vs[(long)b * HKV + hv];
        }
        return;
    }
    const bool is_q = h < HQ;
    const int hh = is_q ? h : h - HQ;
    float x0, x1;
    if (IN_F32) {
        const float* src = qkv_f32 + (long)b * heads * 64 + (long)h * 64;
        x0 = src[lane]; x1 = src[lane + 32];
    } else {
        const int8_t* src = is_q ? q + ((long)b * HQ + hh) * 64 : k + ((long)b * HKV + hh) * 64;
        const float sc_in = is_q ? qs[(long)b * HQ + hh] : ks[(long)b * HKV + hh];
        x0 = (float)src[lane] * sc_in;
        x1 = (float)src[lane + 32] * sc_in;
    }
    const float c = cos_t[(long)pos * 32 + lane], sn = sin_t[(long)pos * 32 + lane];
    float a = x0 * c - x1 * sn;
    float bb = x0 * sn + x1 * c;
    auto lane_stage = [&](int bit) {
        float pa = __shfl_xor_sync(0xffffffffu, a, 1 << bit);
        float pb = __shfl_xor_sync(0xffffffffu, bb, 1 << bit);
        if (lane & (1 << bit)) { a = pa - a; bb = pb - bb; }
        else { a = a + pa; bb = bb + pb; }
    };
    lane_stage(1); lane_stage(2); lane_stage(3); lane_stage(4);
    { float lo = a, hi = bb; a = lo + hi; bb = lo - hi; }
    lane_stage(0);
    a = a / 8.0f;
    bb = bb / 8.0f;
    const float mx = warp_max(fmaxf(a, bb)), mn = warp_min(fminf(a, bb));
    const float sc = sym_scale_from(mx, mn);
    int8_t* dst;
    if (is_q) {
        dst = q2 + ((long)b * HQ + hh) * 64;
        if (lane == 0) qs2[(long)b * HQ + hh] = sc;
    } else {
        dst = cache.k + ((pg * HKV + hh) * PAGE + slot) * 64L;
        if (lane == 0) cache.ks[(pg * HKV + hh) * PAGE + slot] = sc;
    }
    dst[lane] = quant_s8(a, sc);
    dst[lane + 32] = quant_s8(bb, sc);
}

// Append only: the int8 K and V heads of one new token per sequence (already rotated / quantised by the caller) go to
// slot ctx[b] of the sequence's current page. One warp per (sequence, K or V head).
__global__ void __launch_bounds__(256) kv_append_kernel(const int8_t* __restrict__ k, const float* __restrict__ ks,
                                                        const int8_t* __restrict__ v, const float* __restrict__ vs, KvLayer cache,
                                                        const int32_t* __restrict__ page_table, int max_pages,
                                                        const int32_t* __restrict__ ctx, int B, int HKV, int max_pos, int* error_flag) {
    const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= B * 2 * HKV) return;
    const int b = w / (2 * HKV), h = w % (2 * HKV);
    const int pos = dec_guarded_pos(ctx, b, max_pos, error_flag);
    const long pg = page_table[(long)b * max_pages + pos / PAGE];
    const int slot = pos % PAGE;
    if (h < HKV) {
        const int8_t* src = k + ((long)b * HKV + h) * 64;
        int8_t* dst = cache.k + ((pg * HKV + h) * PAGE + slot) * 64L;
        dst[lane] = src[lane]; dst[lane + 32] = src[lane + 32];
        if (lane == 0) cache.ks[(pg * HKV + h) * PAGE + slot] = ks[(long)b * HKV + h];
    } else {
        const int hv = h - HKV;
        const int8_t* src = v + ((long)b * HKV + hv) * 64;
        int8_t* dst = cache.v + (pg * HKV + hv) * (long)(64 * PAGE);
        dst[(long)lane * PAGE + slot] = src[lane];
        dst[(long)(lane + 32) * PAGE + slot] = src[lane + 32];
        if (lane == 0) cache.vs[(pg * HKV + hv) * PAGE + slot] = vs[(long)b * HKV + hv];
    }
}

// ---- 2. scores ---------------------------------------------------------------------------------
// grid (splits, HKV, B), 256 threads: one key per thread per iteration (4 pages at a time),
// the G = HQ/HKV query heads of the group against each key.
template <int G>
__global__ void __launch_bounds__(256) dec_scores_kernel(const int8_t* __restrict__ q2, const float* __restrict__ qs2,
                                                         KvLayer cache, const int32_t* __restrict__ page_table, int max_pages,
                                                         const int32_t* __restrict__ ctx, int HQ, int HKV, int ctx_stride,
                                                         int nsplit, float* __restrict__ scores, float* __restrict__ smax, int max_pos) {
    const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
    const int nk = dec_guarded_pos(ctx, b, max_pos, nullptr) + 1;
    const int k_begin = split * KEYS_PER_CTA;
    __shared__ int qsm[G][16];
    __shared__ float red[G][8];
    if (threadIdx.x < G * 16) {
        const int g = threadIdx.x / 16, i = threadIdx.x % 16;
        qsm[g][i] = reinterpret_cast<const int*>(q2 + ((long)b * HQ + hkv * G + g) * 64)[i];
    }
    __syncthreads();
    float qsc[G];
    float mx[G];
#pragma unroll
    for (int g = 0; g < G; g++) { qsc[g] = qs2[(long)b * HQ + hkv * G + g]; mx[g] = -1e32f; }
    if (k_begin < nk) {
        const int k_end = min(nk, k_begin + KEYS_PER_CTA);
        for (int key = k_begin + threadIdx.x; key < k_end; key += 256) {
            const long pg = page_table[(long)b * max_pages + key / PAGE];
            const long row = (pg * HKV + hkv) * PAGE + (key % PAGE);
            const int4* kp = reinterpret_cast<const int4*>(cache.k + row * 64);
            const int4 k0 = kp[0], k1 = kp[1], k2 = kp[2], k3 = kp[3];
            const float ksc = cache.ks[row];
#pragma unroll
            for (int g = 0; g < G; g++) {
                int acc = 0;
                acc = __dp4a(qsm[g][0], k0.x, acc); acc = __dp4a(qsm[g][1], k0.y, acc);
                acc = __dp4a(qsm[g][2], k0.z, acc); acc = __dp4a(qsm[g][3], k0.w, acc);
                acc = __dp4a(qsm[g][4], k1.x, acc); acc = __dp4a(qsm[g][5], k1.y, acc);
                acc = __dp4a(qsm[g][6], k1.z, acc); acc = __dp4a(qsm[g][7], k1.w, acc);
                acc = __dp4a(qsm[g][8], k2.x, acc); acc = __dp4a(qsm[g][9], k2.y, acc);
                acc = __dp4a(qsm[g][10], k2.z, acc); acc = __dp4a(qsm[g][11], k2.w, acc);
                acc = __dp4a(qsm[g][12], k3.x, acc); acc = __dp4a(qsm[g][13], k3.y, acc);
                acc = __dp4a(qsm[g][14], k3.z, acc); acc = __dp4a(qsm[g][15], k3.w, acc);
                const float x = (((float)acc * qsc[g]) * ksc) * 0.125f;
                scores[((long)b * HQ + hkv * G + g) * ctx_stride + key] = x;
                mx[g] = x > mx[g] ? x : mx[g];
            }
        }
    }
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int g = 0; g < G; g++) {
        const float m = warp_max(mx[g]);
        if (lane == 0) red[g][w] = m;
    }
    __syncthreads();
    if (threadIdx.x < G) {
        float m = red[threadIdx.x][0];
        for (int i = 1; i < 8; i++) m = fmaxf(m, red[threadIdx.x][i]);
        smax[((long)b * HQ + hkv * G + threadIdx.x) * nsplit + split] = m;
    }
}

// ---- 3. softmax statistics ---------------------------------------------------------------------
// One CTA (128 threads) per (sequence, query head) row. e = exp(x - max) replaces x; the four
// chains k mod 4 are summed by four threads in increasing k (Softmax.h:514-553), staged through
// shared memory in chunks.
__global__ void __launch_bounds__(128) dec_softmax_kernel(const int32_t* __restrict__ ctx, int HQ, int ctx_stride, int nsplit,
                                                          float* __restrict__ scores, const float* __restrict__ smax,
                                                          float* __restrict__ rinv, int max_pos) {
    constexpr int CH = 2048;
    __shared__ float e_sm[CH];
    __shared__ float part[4];
    const int row = blockIdx.x;
    const int b = row / HQ;
    const int nk = dec_guarded_pos(ctx, b, max_pos, nullptr) + 1;
    float* x = scores + (long)row * ctx_stride;
    float mx = -1e32f;
    const int used = (nk + KEYS_PER_CTA - 1) / KEYS_PER_CTA;
    for (int i = 0; i < used; i++) mx = fmaxf(mx, smax[(long)row * nsplit + i]);
    float ps = 0.0f;
    for (int c0 = 0; c0 < nk; c0 += CH) {
        const int n = min(CH, nk - c0);
        for (int i = threadIdx.x; i < n; i += 128) {
            const float e = ref_expf(x[c0 + i] - mx);
            e_sm[i] = e;
            x[c0 + i] = e;
        }
        __syncthreads();
        if (threadIdx.x < 4) {
#pragma unroll 8
            for (int i = threadIdx.x; i < n; i += 4) ps += e_sm[i];   // c0 is a multiple of 4
        }
        __syncthreads();
    }
    if (threadIdx.x < 4) part[threadIdx.x] = ps;
    __syncthreads();
    if (threadIdx.x == 0) rinv[row] = 1.0f / ((part[0] + part[1]) + (part[2] + part[3]));
}

// ---- 4. P.V ------------------------------------------------------------------------------------
// grid (splits, HKV, B), 256 threads = G(4) heads x 64. Per page: thread (g, key) quantises its
// probability to u8 into shared memory; then thread (g, d) runs 16 dp4a over the page's 64 keys
// against row d of the transposed V page.
template <int G>
__global__ void __launch_bounds__(64 * G) dec_pv_kernel(KvLayer cache, const int32_t* __restrict__ page_table, int max_pages,
                                                        const int32_t* __restrict__ ctx, int HQ, int HKV, int ctx_stride,
                                                        const float* __restrict__ scores, const float* __restrict__ rinv,
                                                        const float* __restrict__ a_s, int32_t* __restrict__ oacc, int max_pos) {
    const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
    const int nk = dec_guarded_pos(ctx, b, max_pos, nullptr) + 1;
    const int k_begin = split * KEYS_PER_CTA;
    if (k_begin >= nk) return;
    const int k_end = min(nk, k_begin + KEYS_PER_CTA);
    __shared__ __align__(16) uint8_t u_sm[G][PAGE];
    const int g = threadIdx.x / 64, t = threadIdx.x % 64;
    const int hq = hkv * G + g;
    const float r = rinv[(long)b * HQ + hq];
    const float as = a_s[hq];
    const float* e = scores + ((long)b * HQ + hq) * ctx_stride;
    int acc = 0;
    for (int p0 = k_begin; p0 < k_end; p0 += PAGE) {
        const long pg = page_table[(long)b * max_pages + p0 / PAGE];
        const long prow = (pg * HKV + hkv) * PAGE;
        const int key = p0 + t;
        uint8_t u = 0;
        if (key < k_end) {
            const float p = e[key] * r;
            const float tt = (p * cache.vs[prow + t]) / as;
            int q = round_half_away_to_int(tt);
            q = q > 255 ? 255 : q;
            u = (uint8_t)q;
        }
        // this thread's V^T row for the page (issued before the barrier to overlap the latency)
        const int4* vp = reinterpret_cast<const int4*>(cache.v + (prow * 64) + (long)t * PAGE);
        const int4 v0 = vp[0], v1 = vp[1], v2 = vp[2], v3 = vp[3];
        __syncthreads();   // previous page's u_sm fully consumed
        u_sm[g][t] = u;
        __syncthreads();
        const int4* up = reinterpret_cast<const int4*>(u_sm[g]);
        const int4 u0 = up[0], u1 = up[1], u2 = up[2], u3 = up[3];
        // u is unsigned, v signed: mixed-sign dp4a
        acc = dp4a_u8s8((unsigned)u0.x, v0.x, acc); acc = dp4a_u8s8((unsigned)u0.y, v0.y, acc);
        acc = dp4a_u8s8((unsigned)u0.z, v0.z, acc); acc = dp4a_u8s8((unsigned)u0.w, v0.w, acc);
        acc = dp4a_u8s8((unsigned)u1.x, v1.x, acc); acc = dp4a_u8s8((unsigned)u1.y, v1.y, acc);
        acc = dp4a_u8s8((unsigned)u1.z, v1.z, acc); acc = dp4a_u8s8((unsigned)u1.w, v1.w, acc);
        acc = dp4a_u8s8((unsigned)u2.x, v2.x, acc); acc = dp4a_u8s8((unsigned)u2.y, v2.y, acc);
        acc = dp4a_u8s8((unsigned)u2.z, v2.z, acc); acc = dp4a_u8s8((unsigned)u2.w, v2.w, acc);
        acc = dp4a_u8s8((unsigned)u3.x, v3.x, acc); acc = dp4a_u8s8((unsigned)u3.y, v3.y, acc);
        acc = dp4a_u8s8((unsigned)u3.z, v3.z, acc); acc = dp4a_u8s8((unsigned)u3.w, v3.w, acc);
    }
    atomicAdd(oacc + ((long)b * HQ + hq) * 64 + t, acc);
}

// ---- fused single-kernel path (body in attention_decode.cuh) ----------------------------------------
template <bool IN_F32, int NT>
__global__ void __launch_bounds__(NT) dec_attn_fused_kernel(const int8_t* __restrict__ q, const float* __restrict__ qs,
                                                             const int8_t* __restrict__ k, const float* __restrict__ ks,
                                                             const int8_t* __restrict__ v, const float* __restrict__ vs,
                                                             const float* __restrict__ qkv_f32, const float* __restrict__ cos_t,
                                                             const float* __restrict__ sin_t, const float* __restrict__ a_s,
                                                             KvLayer cache, const int32_t* __restrict__ page_table, int max_pages,
                                                             const int32_t* __restrict__ ctx, int HQ, int HKV, int cs,
                                                             float* __restrict__ out, int32_t* __restrict__ oacc, int max_pos,
                                                             int* error_flag) {
    extern __shared__ __align__(16) uint8_t dsm[];
    __shared__ DecAttnSmem sm;
    pdl_sync();
    DecAttnIn in;
    in.q = q; in.qs = qs; in.k = k; in.ks = ks; in.v = v; in.vs = vs; in.qkv_f32 = qkv_f32;
    in.qkv_acc = nullptr; in.tok_scale = nullptr; in.ch_scale = nullptr; in.n_slabs = 0; in.slab_stride = 0;
    in.max_pos = max_pos; in.error_flag = error_flag;
    dec_attn_fused_body<IN_F32 ? 1 : 0, NT>(in, cos_t, sin_t, a_s, cache, page_table, max_pages, ctx, HQ, HKV, cs, out, oacc,
                                               (int)blockIdx.x, (int)blockIdx.y, dsm, sm, (int)threadIdx.x, 0);
}

// ---- 5. out ------------------------------------------------------------------------------------
__global__ void dec_out_kernel(const int32_t* __restrict__ oacc, const float* __restrict__ a_s, int B, int HQ,
                               float* __restrict__ out, int32_t* __restrict__ oacc_out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= B * HQ * 64) return;
    const int hq = (i / 64) % HQ;
    const int v = oacc[i];
    out[i] = (float)v * a_s[hq];
    if (oacc_out) oacc_out[i] = v;
}

}  // namespace flexllm

using namespace flexllm;

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

extern "C" int flexllm_kv_cache_create(flexllm_kv_cache** out, int layers, int n_pages, int hkv, int page) {
    FLEXLLM_REQUIRE(out && layers > 0 && n_pages > 0 && hkv > 0);
    if (page != PAGE) return FLEXLLM_ENOTSUP;
    flexllm_kv_cache* c = new (std::nothrow) flexllm_kv_cache();
    if (!c) return FLEXLLM_ENOMEM;
    c->layers = layers; c->n_pages = n_pages; c->hkv = hkv; c->page = page;
    c->page_bytes = (size_t)n_pages * hkv * PAGE * 64;
    c->scale_bytes = (size_t)n_pages * hkv * PAGE * sizeof(float);
    c->k = c->v = nullptr; c->ks = c->vs = nullptr;
    cudaError_t e = cudaMalloc(&c->k, c->page_bytes * layers);
    if (e == cudaSuccess) e = cudaMalloc(&c->v, c->page_bytes * layers);
    if (e == cudaSuccess) e = cudaMalloc(&c->ks, c->scale_bytes * layers);
    if (e == cudaSuccess) e = cudaMalloc(&c->vs, c->scale_bytes * layers);
    if (e != cudaSuccess) {
        flexllm_kv_cache_destroy(c);
        g_last_cuda_error = (int)e;
        return e == cudaErrorMemoryAllocation ? FLEXLLM_ENOMEM : FLEXLLM_ECUDA;
    }
    *out = c;
    return flexllm_kv_cache_reset(c, nullptr);
}

extern "C" int flexllm_kv_cache_destroy(flexllm_kv_cache* c) {
    if (!c) return FLEXLLM_OK;
    cudaFree(c->k); cudaFree(c->v); cudaFree(c->ks); cudaFree(c->vs);
    delete c;
    return FLEXLLM_OK;
}

extern "C" int flexllm_kv_cache_reset(flexllm_kv_cache* c, void* stream) {
    FLEXLLM_REQUIRE(c);
    cudaStream_t st = (cudaStream_t)stream;
    FLEXLLM_CHECK_CUDA(cudaMemsetAsync(c->k, 0, c->page_bytes * c->layers, st));
    FLEXLLM_CHECK_CUDA(cudaMemsetAsync(c->v, 0, c->page_bytes * c->layers, st));
    FLEXLLM_CHECK_CUDA(cudaMemsetAsync(c->ks, 0, c->scale_bytes * c->layers, st));
    FLEXLLM_CHECK_CUDA(cudaMemsetAsync(c->vs, 0, c->scale_bytes * c->layers, st));
    return FLEXLLM_OK;
}

extern "C" int flexllm_kv_cache_pools(flexllm_kv_cache* c, int layer, int8_t** k, float** ks, int8_t** v, float** vs) {
    FLEXLLM_REQUIRE(c && layer >= 0 && layer < c->layers);
    KvLayer l = kv_layer(c, layer);
    if (k) *k = l.k;
    if (ks) *ks = l.ks;
    if (v) *v = l.v;
    if (vs) *vs = l.vs;
    return FLEXLLM_OK;
}

extern "C" size_t flexllm_mha_decode_workspace(int B, int HQ, int max_ctx) {
    if (B <= 0 || HQ <= 0 || max_ctx < 0) return 0;
    const size_t ctx_stride = align_up((size_t)max_ctx + 1, 64);
    const size_t nsplit = (ctx_stride + KEYS_PER_CTA - 1) / KEYS_PER_CTA;
    size_t n = 0;
    n += align_up((size_t)B * HQ * 64, 256);                 // q2
    n += align_up((size_t)B * HQ * 4, 256);                  // qs2
    n += align_up((size_t)B * HQ * ctx_stride * 4, 256);     // scores / e
    n += align_up((size_t)B * HQ * nsplit * 4, 256);         // per-split max
    n += align_up((size_t)B * HQ * 4, 256);                  // 1 / sum
    n += align_up((size_t)B * HQ * 64 * 4, 256);             // int32 accumulators
    return n + 256;
}

namespace flexllm {
// Shared body of the int8 and fp32 front ends (qkv_f32 != nullptr selects the latter).
int mha_decode_run(flexllm_kv_cache* c, int layer, const int8_t* q, const float* qs, const int8_t* k, const float* ks,
                   const int8_t* v, const float* vs, const float* qkv_f32, const float* cos_t, const float* sin_t,
                   const float* a_s, const int32_t* page_table, int max_pages, const int32_t* ctx, int max_ctx, int B, int HQ,
                   float* out, int32_t* oacc, void* workspace, cudaStream_t st);

}  // namespace flexllm

// The cache managers' append on its own (dec_K_cache_manager_template / dec_V_cache_manager_template,
// Modules/MHA.h:484-513, :773-801): store the new token's K and V heads at position ctx[b], nothing else.
extern "C" int flexllm_kv_append(flexllm_kv_cache* c, int layer, const int8_t* k, const float* ks, const int8_t* v, const float* vs,
                                 const int32_t* page_table, int max_pages, const int32_t* ctx, int max_ctx, int B, void* stream) {
    FLEXLLM_REQUIRE(c && layer >= 0 && layer < c->layers && B >= 0 && max_ctx >= 0 && max_pages > 0);
    if (B == 0) return FLEXLLM_OK;
    FLEXLLM_REQUIRE(k && ks && v && vs && page_table && ctx);
    FLEXLLM_REQUIRE((long)max_pages * PAGE > max_ctx);
    const int warps = B * 2 * c->hkv;
    kv_append_kernel<<<(warps + 7) / 8, 256, 0, (cudaStream_t)stream>>>(k, ks, v, vs, kv_layer(c, layer), page_table, max_pages, ctx, B, c->hkv,
                                                                         max_ctx, device_error_flag());
    return launch_status();
}

extern "C" int flexllm_mha_i8xi8_decode(flexllm_kv_cache* c, int layer, const int8_t* q, const float* qs,
                                        const int8_t* k, const float* ks, const int8_t* v, const float* vs,
                                        const float* cos_t, const float* sin_t, const float* a_s,
                                        const int32_t* page_table, int max_pages, const int32_t* ctx, int max_ctx,
                                        int B, int HQ, float* out, int32_t* oacc, void* workspace,
                                        size_t workspace_bytes, void* stream) {
    FLEXLLM_REQUIRE(c && layer >= 0 && layer < c->layers && B >= 0 && HQ > 0 && max_ctx >= 0 && max_pages > 0);
    if (B == 0) return FLEXLLM_OK;
    FLEXLLM_REQUIRE(q && qs && k && ks && v && vs && cos_t && sin_t && a_s && page_table && ctx && out && workspace);
    FLEXLLM_REQUIRE(HQ % c->hkv == 0);
    if (HQ / c->hkv != 4) return FLEXLLM_ENOTSUP;
    FLEXLLM_REQUIRE((long)max_pages * PAGE > max_ctx);
    FLEXLLM_REQUIRE(workspace_bytes >= flexllm_mha_decode_workspace(B, HQ, max_ctx));
    return mha_decode_run(c, layer, q, qs, k, ks, v, vs, nullptr, cos_t, sin_t, a_s, page_table, max_pages, ctx, max_ctx, B,
                          HQ, out, oacc, workspace, (cudaStream_t)stream);
}

int flexllm::mha_decode_run(flexllm_kv_cache* c, int layer, const int8_t* q, const float* qs, const int8_t* k, const float* ks,
                            const int8_t* v, const float* vs, const float* qkv_f32, const float* cos_t, const float* sin_t,
                            const float* a_s, const int32_t* page_table, int max_pages, const int32_t* ctx, int max_ctx, int B,
                            int HQ, float* out, int32_t* oacc, void* workspace, cudaStream_t st) {
    const int HKV = c->hkv;
    const int ctx_stride = (int)align_up((size_t)max_ctx + 1, 64);
    const int nsplit = (ctx_stride + KEYS_PER_CTA - 1) / KEYS_PER_CTA;
    uint8_t* w = (uint8_t*)align_up((size_t)workspace, 256);
    int8_t* q2 = (int8_t*)w; w += align_up((size_t)B * HQ * 64, 256);
    float* qs2 = (float*)w; w += align_up((size_t)B * HQ * 4, 256);
    float* scores = (float*)w; w += align_up((size_t)B * HQ * ctx_stride * 4, 256);
    float* smax = (float*)w; w += align_up((size_t)B * HQ * nsplit * 4, 256);
    float* rinv = (float*)w; w += align_up((size_t)B * HQ * 4, 256);
    int32_t* acc = (int32_t*)w;
    KvLayer L = kv_layer(c, layer);
    int* err = device_error_flag();     // raised (and the length clamped) when a ctx[] entry lies beyond max_ctx

    // enough (sequence, head) pairs, or short rows: one fused kernel; otherwise the split kernels
    const size_t fused_smem = (size_t)20 * ctx_stride < 4096 ? 4096 : (size_t)20 * ctx_stride;
    if (fused_smem <= 200 * 1024 && (B * HKV >= 64 || max_ctx <= 2048)) {
        dim3 fg(HKV, B);
        if (qkv_f32) {
            auto kern = dec_attn_fused_kernel<true, 512>;
            if (fused_smem > 48 * 1024) FLEXLLM_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fused_smem));
            launch_k(kern, fg, dim3(512), fused_smem, st, q, qs, k, ks, v, vs, qkv_f32, cos_t, sin_t, a_s, L, page_table, max_pages, ctx,
                     HQ, HKV, ctx_stride, out, oacc, max_ctx, err);
        } else {
            auto kern = dec_attn_fused_kernel<false, 512>;
            if (fused_smem > 48 * 1024) FLEXLLM_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fused_smem));
            launch_k(kern, fg, dim3(512), fused_smem, st, q, qs, k, ks, v, vs, (const float*)nullptr, cos_t, sin_t, a_s, L, page_table,
                     max_pages, ctx, HQ, HKV, ctx_stride, out, oacc, max_ctx, err);
        }
        return launch_status(1);
    }
    const int warps = B * (HQ + 2 * HKV);
    if (qkv_f32)
        dec_append_kernel<true><<<(warps + 7) / 8, 256, 0, st>>>(q, qs, k, ks, v, vs, qkv_f32, cos_t, sin_t, L, page_table,
                                                                 max_pages, ctx, B, HQ, HKV, q2, qs2, max_ctx, err);
    else
        dec_append_kernel<false><<<(warps + 7) / 8, 256, 0, st>>>(q, qs, k, ks, v, vs, nullptr, cos_t, sin_t, L, page_table,
                                                                  max_pages, ctx, B, HQ, HKV, q2, qs2, max_ctx, err);
    dim3 grid(nsplit, HKV, B);
    dec_scores_kernel<4><<<grid, 256, 0, st>>>(q2, qs2, L, page_table, max_pages, ctx, HQ, HKV, ctx_stride, nsplit, scores, smax, max_ctx);
    dec_softmax_kernel<<<B * HQ, 128, 0, st>>>(ctx, HQ, ctx_stride, nsplit, scores, smax, rinv, max_ctx);
    FLEXLLM_CHECK_CUDA(cudaMemsetAsync(acc, 0, (size_t)B * HQ * 64 * 4, st));
    dec_pv_kernel<4><<<grid, 256, 0, st>>>(L, page_table, max_pages, ctx, HQ, HKV, ctx_stride, scores, rinv, a_s, acc, max_ctx);
    dec_out_kernel<<<(B * HQ * 64 + 255) / 256, 256, 0, st>>>(acc, a_s, B, HQ, out, oacc);
    return launch_status(5);
}
