// Device code shared by the decode attention kernel and the persistent decode-step kernel: the
// paged KV-cache view and the fused per-(sequence, KV head) attention step.
#pragma once
#include "common.cuh"
#include "tc_common.cuh"

// Paged int8 KV cache, all layers (layout at the top of attention_decode.cu).
struct flexllm_kv_cache {
    int layers, n_pages, hkv, page;
    int8_t* k; float* ks; int8_t* v; float* vs;   // [layers][...]
    size_t page_bytes, scale_bytes;               // per layer
};

namespace flexllm {

// d = c + sum_i a.u8[i] * b.s8[i]
__device__ __forceinline__ int dp4a_u8s8(unsigned a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Development aid (compiled in only with -DFLEXLLM_ATT_TRACE): thread 0 of the item (sequence 0, KV head 0)
// stamps the global timer at the boundaries of the fused attention step; read back with flexllm_att_trace().
#ifdef FLEXLLM_ATT_TRACE
static __device__ unsigned long long g_att_ts[32];
#define ATT_TS(i) do { if (b == 0 && hkv == 0 && tid == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); g_att_ts[i] = t_; } } while (0)
#else
#define ATT_TS(i) do { } while (0)
#endif

constexpr int PAGE = 64;
constexpr int KEYS_PER_CTA = 512;   // 8 pages per CTA in the score and P.V kernels

struct KvLayer { int8_t* k; float* ks; int8_t* v; float* vs; };


// Inputs of the new token, one of three forms (MODE): 0 = int8 heads with per-head scales,
// 1 = one fp32 row [(HQ + 2 HKV) * 64] per sequence, 2 = the int32 split-K partial sums of the fused q|k|v
// projection with the per-token and per-channel scales (summed and dequantised here).
struct DecAttnIn {
    const int8_t *q, *k, *v; const float *qs, *ks, *vs;
    const float* qkv_f32;
    const int32_t* qkv_acc; const float* tok_scale; const float* ch_scale;
    int n_slabs; long slab_stride;     // MODE 2: split-K partial sums, slab s at qkv_acc + s * slab_stride
    int max_pos;                       // largest context length the tables, the page-table rows and the score rows cover
    int* error_flag;                   // raised when a sequence's ctx[] lies beyond max_pos (optional)
};

// Context length of sequence b as the kernels use it: ctx[] is device data the host cannot vet, so a
// value outside [0, max_pos] is clamped (every index derived from it then stays inside the page-table
// row, the RoPE tables and the score row) and reported through the error word.
__device__ __forceinline__ int dec_guarded_pos(const int32_t* __restrict__ ctx, int b, int max_pos, int* error_flag) {
    int pos = ctx[b];
    if (pos < 0 || pos > max_pos) {
        if (error_flag) atomicOr(error_flag, 2);
        pos = pos < 0 ? 0 : max_pos;
    }
    return pos;
}

// Asks L2 for everything one (sequence, KV head) item will read: its K and V pages (4 KB each) and
// their scale rows. `n_threads` threads (index `t`) share the work. Pure hint: no data is returned.
__device__ __forceinline__ void dec_attn_prefetch_l2(const KvLayer& cache, const int32_t* __restrict__ page_table, int max_pages,
                                                     const int32_t* __restrict__ ctx, int HKV, int hkv, int b, int t, int n_threads) {
    int npages = (ctx[b] + 1 + PAGE - 1) / PAGE;
    npages = npages < 0 ? 0 : (npages > max_pages ? max_pages : npages);     // a hint only, but it indexes the page table
    // per page: 32 lines of K, 32 lines of V, 2 lines of K scales, 2 lines of V scales (128 bytes each)
    for (int i = t; i < npages * 68; i += n_threads) {
        const int p = i / 68, j = i - p * 68;
        const long pg = page_table[(long)b * max_pages + p];
        const long base = pg * HKV + hkv;
        const void* line;
        if (j < 32) line = cache.k + base * (long)(64 * PAGE) + (long)j * 128;
        else if (j < 64) line = cache.v + base * (long)(64 * PAGE) + (long)(j - 32) * 128;
        else if (j < 66) line = cache.ks + base * PAGE + (j - 64) * 32;
        else line = cache.vs + base * PAGE + (j - 66) * 32;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
    }
}

// The same hint issued by a group of 128 threads (index `t`) with ONE dependent load per thread: thread t takes the lines
// t % 6, t % 6 + 6, ... of page t / 6 (+ 21, + 42, ...), so that its page-table entry is read once and the prefetches
// follow without further waits. Several groups of a CTA can serve different items side by side.
__device__ __forceinline__ void dec_attn_prefetch_l2_g128(const KvLayer& cache, const int32_t* __restrict__ page_table, int max_pages,
                                                          const int32_t* __restrict__ ctx, int HKV, int hkv, int b, int t) {
    int npages = (ctx[b] + 1 + PAGE - 1) / PAGE;
    npages = npages < 0 ? 0 : (npages > max_pages ? max_pages : npages);
    const int sub = t % 6;
    for (int p = t / 6; p < npages; p += 21) {
        if (t >= 126) break;                                   // threads 126, 127 have no page in this layout
        const long pg = page_table[(long)b * max_pages + p];
        const long base = pg * HKV + hkv;
        for (int j = sub; j < 68; j += 6) {
            const void* line;
            if (j < 32) line = cache.k + base * (long)(64 * PAGE) + (long)j * 128;
            else if (j < 64) line = cache.v + base * (long)(64 * PAGE) + (long)(j - 32) * 128;
            else if (j < 66) line = cache.ks + base * PAGE + (j - 64) * 32;
            else line = cache.vs + base * PAGE + (j - 66) * 32;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
        }
    }
}

// Small per-call shared-memory state of dec_attn_fused_body (one per group of threads that runs it).
struct DecAttnSmem {
    __align__(16) int8_t q_sm[4][64];
    float q_scale[4], red[4][16], row_max[4], row_rinv[4], part[4][4];
    int pt_sm[160];
    int last;           // scratch flag for callers (e.g. "this item completed its sequence")
};

// One call by a group of NT threads per (sequence b, KV head hkv) does the whole step for its GQA group of 4 query
// heads: Q/K/V preparation and cache append, scores, max, exp, the ordered partial sums, the u8
// quantiser and P.V, with the score row kept in shared memory (`dsm`: 20 bytes per key, at least
// 4096 bytes). The group's NT threads (256 or 512; `tid` = index in the group) synchronise on named
// barrier `bar`.
template <int MODE, int NT>
__device__ __forceinline__ void dec_attn_fused_body(const DecAttnIn& in, const float* __restrict__ cos_t,
                                                    const float* __restrict__ sin_t, const float* __restrict__ a_s,
                                                    const KvLayer& cache, const int32_t* __restrict__ page_table, int max_pages,
                                                    const int32_t* __restrict__ ctx, int HQ, int HKV, int cs,
                                                    float* __restrict__ out, int32_t* __restrict__ oacc,
                                                    const int hkv, const int b, uint8_t* dsm, DecAttnSmem& sm, const int tid,
                                                    const int bar) {
    constexpr int G = 4;
    float* sc = reinterpret_cast<float*>(dsm);                       // [G][cs]
    uint8_t* u_sm = dsm + (size_t)G * cs * 4;                        // [G][cs]
    int8_t (*q_sm)[64] = sm.q_sm;
    float* q_scale = sm.q_scale; float (*red)[16] = sm.red; float* row_max = sm.row_max; float* row_rinv = sm.row_rinv;
    float (*part)[4] = sm.part;
    int* pt_sm = sm.pt_sm;                                            // this sequence's page-table row
    named_sync_id<NT>(bar);   // a CTA may run several (sequence, head) items back to back
    ATT_TS(0);
    const int w = tid >> 5, lane = tid & 31;
    const int heads = HQ + 2 * HKV;
    // MODE 2: the split-K partial sums of this warp's head do not depend on the context length, so
    // their loads go out first and overlap the context / page-table round trips below
    int a0 = 0, a1 = 0;
    if (MODE == 2 && w < 6) {
        const int h = w < 4 ? hkv * G + w : (w == 4 ? HQ + hkv : HQ + HKV + hkv);
        const int32_t* src = in.qkv_acc + (long)b * heads * 64 + (long)h * 64 + lane;
#pragma unroll 1
        for (int sl = 0; sl < in.n_slabs; sl += 4) {
            int p0[4], p1[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const bool on = sl + i < in.n_slabs;
                p0[i] = on ? __ldcg(src + (sl + i) * in.slab_stride) : 0;
                p1[i] = on ? __ldcg(src + (sl + i) * in.slab_stride + 32) : 0;
            }
            a0 += (p0[0] + p0[1]) + (p0[2] + p0[3]);
            a1 += (p1[0] + p1[1]) + (p1[2] + p1[3]);
        }
    }
    const int pos = dec_guarded_pos(ctx, b, in.max_pos, in.error_flag);
    const int nk = pos + 1;
    const int npages_all = (nk + PAGE - 1) / PAGE;
    const bool pt_cached = npages_all <= 160;
    if (pt_cached)
        for (int i = tid; i < npages_all; i += NT) pt_sm[i] = page_table[(long)b * max_pages + i];
    // warm L2 with this head's V pages while the scores are computed (V is first needed in step G);
    // the persistent kernel (MODE 2) has asked for them a phase earlier
    if (MODE != 2)
    for (int i = tid; i < npages_all * 32; i += NT) {
        const long pg = page_table[(long)b * max_pages + (i >> 5)];
        const int8_t* line = cache.v + (pg * HKV + hkv) * (long)(64 * PAGE) + (long)(i & 31) * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
    }

    ATT_TS(1);
    // ---- A. prepare: warps 0..3 the query heads, warp 4 the key head, warp 5 the value head
    if (w < 6) {
        const long pg = page_table[(long)b * max_pages + pos / PAGE];
        const int slot = pos % PAGE;
        const int h = w < 4 ? hkv * G + w : (w == 4 ? HQ + hkv : HQ + HKV + hkv);   // index in the fused row
        float x0, x1;
        if (MODE == 2) {
            // int32 partial sums of the fused q|k|v projection (one slab per K split), added up above
            // (integers: exact in any order); dequantise here
            const float st = __ldcg(in.tok_scale + b);
            x0 = ((float)a0 * st) * in.ch_scale[h * 64 + lane];
            x1 = ((float)a1 * st) * in.ch_scale[h * 64 + lane + 32];
        } else if (MODE == 1) {
            const float* src = in.qkv_f32 + (long)b * heads * 64 + (long)h * 64;
            x0 = src[lane]; x1 = src[lane + 32];
        } else {
            const int8_t* src = w < 4 ? in.q + ((long)b * HQ + hkv * G + w) * 64 : (w == 4 ? in.k : in.v) + ((long)b * HKV + hkv) * 64;
            const float sc_in = w < 4 ? in.qs[(long)b * HQ + hkv * G + w] : (w == 4 ? in.ks : in.vs)[(long)b * HKV + hkv];
            x0 = (float)src[lane]; x1 = (float)src[lane + 32];
            if (w < 5) { x0 = x0 * sc_in; x1 = x1 * sc_in; }
            if (w == 5) {   // int8 value head: plain copy
                int8_t* dst = cache.v + (pg * HKV + hkv) * (long)(64 * PAGE);
                dst[(long)lane * PAGE + slot] = src[lane];
                dst[(long)(lane + 32) * PAGE + slot] = src[lane + 32];
                if (lane == 0) cache.vs[(pg * HKV + hkv) * PAGE + slot] = sc_in;
            }
        }
        if (MODE != 0 || w < 5) {
            float a = x0, bb = x1;
            if (w < 5) {
                const float c = cos_t[(long)pos * 32 + lane], sn = sin_t[(long)pos * 32 + lane];
                a = x0 * c - x1 * sn;
                bb = x0 * sn + x1 * c;
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
            }
            const float mx = warp_max(fmaxf(a, bb)), mn = warp_min(fminf(a, bb));
            const float s2 = sym_scale_from(mx, mn);
            const int8_t qa = quant_s8(a, s2), qb = quant_s8(bb, s2);
            if (w < 4) {
                q_sm[w][lane] = qa; q_sm[w][lane + 32] = qb;
                if (lane == 0) q_scale[w] = s2;
            } else if (w == 4) {
                int8_t* dst = cache.k + ((pg * HKV + hkv) * PAGE + slot) * 64L;
                dst[lane] = qa; dst[lane + 32] = qb;
                if (lane == 0) cache.ks[(pg * HKV + hkv) * PAGE + slot] = s2;
            } else {
                int8_t* dst = cache.v + (pg * HKV + hkv) * (long)(64 * PAGE);
                dst[(long)lane * PAGE + slot] = qa;
                dst[(long)(lane + 32) * PAGE + slot] = qb;
                if (lane == 0) cache.vs[(pg * HKV + hkv) * PAGE + slot] = s2;
            }
        }
    }
    named_sync_id<NT>(bar);
    ATT_TS(2);

    // ---- B. scores: four lanes share one key (16 bytes of its row each), NT/4 keys per iteration
    const int l4 = tid & 3, slot = tid >> 2;
    int qreg[G][4];
    float qsc[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
#pragma unroll
        for (int i = 0; i < 4; i++) qreg[g][i] = reinterpret_cast<const int*>(q_sm[g])[l4 * 4 + i];
        qsc[g] = q_scale[g];
    }
    float mymax = -1e32f;                      // lane l4 tracks the maximum of head g = l4
    // batches of UB iterations: all of a batch's K rows and scales are requested before any is used
    // (the stores into the score row would otherwise keep the next iteration's loads from starting)
    constexpr int UB = 4;
#pragma unroll 1
    for (int key0 = 0; key0 < nk; key0 += UB * (NT / 4)) {
        int4 kv4[UB];
        float ksc[UB];
#pragma unroll
        for (int u = 0; u < UB; u++) {
            const int key = key0 + u * (NT / 4) + slot;
            const int kk = key < nk ? key : nk - 1;
            const long pg = pt_cached ? pt_sm[kk / PAGE] : page_table[(long)b * max_pages + kk / PAGE];
            const long row = (pg * HKV + hkv) * PAGE + (kk % PAGE);
            kv4[u] = *reinterpret_cast<const int4*>(cache.k + row * 64 + l4 * 16);
            ksc[u] = cache.ks[row];
        }
#pragma unroll
        for (int u = 0; u < UB; u++) {
            const int key = key0 + u * (NT / 4) + slot;
            float xg = 0.0f;
#pragma unroll
            for (int g = 0; g < G; g++) {
                int acc = __dp4a(qreg[g][0], kv4[u].x, 0);
                acc = __dp4a(qreg[g][1], kv4[u].y, acc); acc = __dp4a(qreg[g][2], kv4[u].z, acc); acc = __dp4a(qreg[g][3], kv4[u].w, acc);
                acc += __shfl_xor_sync(0xffffffffu, acc, 1);
                acc += __shfl_xor_sync(0xffffffffu, acc, 2);
                const float x = (((float)acc * qsc[g]) * ksc[u]) * 0.125f;
                if (g == l4) xg = x;
            }
            if (key < nk) {
                sc[l4 * cs + key] = xg;
                mymax = xg > mymax ? xg : mymax;
            }
        }
    }
    ATT_TS(3);
    // maximum over the lanes with the same l4 (xor 4, 8, 16), then over the warps
    mymax = fmaxf(mymax, __shfl_xor_sync(0xffffffffu, mymax, 4));
    mymax = fmaxf(mymax, __shfl_xor_sync(0xffffffffu, mymax, 8));
    mymax = fmaxf(mymax, __shfl_xor_sync(0xffffffffu, mymax, 16));
    if (lane < 4) red[lane][w] = mymax;
    named_sync_id<NT>(bar);
    if (tid < G) {
        float m = red[tid][0];
        for (int i = 1; i < NT / 32; i++) m = fmaxf(m, red[tid][i]);
        row_max[tid] = m;
    }
    named_sync_id<NT>(bar);
    // the V scales of this thread's first UF keys (step F) are requested now: their latency hides behind
    // the exponentials and the ordered sums
    constexpr int UF = 6;
    float vsc_pre[UF];
#pragma unroll
    for (int u = 0; u < UF; u++) {
        const int key = tid + u * NT;
        vsc_pre[u] = 0.0f;
        if (key < nk) {
            const long pg = pt_cached ? pt_sm[key / PAGE] : page_table[(long)b * max_pages + key / PAGE];
            vsc_pre[u] = cache.vs[(pg * HKV + hkv) * PAGE + (key % PAGE)];
        }
    }
    ATT_TS(4);
    // ---- D. e = exp(x - max), in place: the four heads of a key together (four independent evaluations in flight)
    {
        const float m0 = row_max[0], m1 = row_max[1], m2 = row_max[2], m3 = row_max[3];
        for (int key = tid; key < nk; key += NT) {
            const float x0 = sc[key] - m0, x1 = sc[cs + key] - m1, x2 = sc[2 * cs + key] - m2, x3 = sc[3 * cs + key] - m3;
            const float e0 = ref_expf(x0), e1 = ref_expf(x1), e2 = ref_expf(x2), e3 = ref_expf(x3);
            sc[key] = e0; sc[cs + key] = e1; sc[2 * cs + key] = e2; sc[3 * cs + key] = e3;
        }
    }
    named_sync_id<NT>(bar);
    ATT_TS(5);
    // ---- E. the four ordered chains of each row (Softmax.h:514-553): one thread per chain
    if (tid < 4 * G) {
        const int g = tid >> 2, j = tid & 3;
        const float* e = sc + g * cs;
        float ps = 0.0f;
#pragma unroll 8
        for (int i = j; i < nk; i += 4) ps += e[i];
        part[g][j] = ps;
    }
    named_sync_id<NT>(bar);
    if (tid < G) row_rinv[tid] = 1.0f / ((part[tid][0] + part[tid][1]) + (part[tid][2] + part[tid][3]));
    named_sync_id<NT>(bar);
    ATT_TS(6);
    // ---- F. u8 probabilities (zero beyond the last key up to the page boundary)
    const int nk_pad = (nk + PAGE - 1) / PAGE * PAGE;
    {
        float rinv_g[G];
        DivBy as_g[G];
#pragma unroll
        for (int g = 0; g < G; g++) { rinv_g[g] = row_rinv[g]; as_g[g] = div_by(a_s[hkv * G + g]); }
        auto quantise_key = [&](int key, float vsc) {
#pragma unroll
            for (int g = 0; g < G; g++) {
                uint8_t uq = 0;
                if (key < nk) {
                    const float p = sc[g * cs + key] * rinv_g[g];
                    const float tt = div_for_rounding(p * vsc, as_g[g]);
                    int r = round_half_away_to_int(tt);
                    r = r > 255 ? 255 : r;
                    uq = (uint8_t)r;
                }
                u_sm[g * cs + key] = uq;
            }
        };
#pragma unroll
        for (int u = 0; u < UF; u++) {
            const int key = tid + u * NT;
            if (key < nk_pad) quantise_key(key, vsc_pre[u]);
        }
        for (int key = tid + UF * NT; key < nk_pad; key += NT) {      // contexts beyond UF * NT keys
            float vsc = 0.0f;
            if (key < nk) {
                const long pg = pt_cached ? pt_sm[key / PAGE] : page_table[(long)b * max_pages + key / PAGE];
                vsc = cache.vs[(pg * HKV + hkv) * PAGE + (key % PAGE)];
            }
            quantise_key(key, vsc);
        }
    }
    named_sync_id<NT>(bar);
    ATT_TS(7);
    // ---- G. P.V: four lanes share one V^T row (16 keys of the page each); thread = (page slot, d, quarter)
    {
        const int d = (tid >> 2) & 63, ps = tid >> 8;     // ps: which of the NT/256 pages of an iteration
        int acc[G] = {0, 0, 0, 0};
        const int npages = nk_pad / PAGE;
#pragma unroll 8
        for (int p = ps; p < npages; p += NT / 256) {
            const long pg = pt_cached ? pt_sm[p] : page_table[(long)b * max_pages + p];
            const int4 v4 = *reinterpret_cast<const int4*>(cache.v + ((pg * HKV + hkv) * 64L + d) * PAGE + l4 * 16);
#pragma unroll
            for (int g = 0; g < G; g++) {
                const int4 u4 = *reinterpret_cast<const int4*>(u_sm + g * cs + p * PAGE + l4 * 16);
                int a = acc[g];
                a = dp4a_u8s8((unsigned)u4.x, v4.x, a); a = dp4a_u8s8((unsigned)u4.y, v4.y, a);
                a = dp4a_u8s8((unsigned)u4.z, v4.z, a); a = dp4a_u8s8((unsigned)u4.w, v4.w, a);
                acc[g] = a;
            }
        }
        ATT_TS(8);
        int mine = 0;
#pragma unroll
        for (int g = 0; g < G; g++) {
            int a = acc[g];
            a += __shfl_xor_sync(0xffffffffu, a, 1);
            a += __shfl_xor_sync(0xffffffffu, a, 2);
            if (g == l4) mine = a;
        }
        // combine the NT/256 page slots through shared memory (integer adds: exact)
        int* pv_sm = reinterpret_cast<int*>(sc);          // scores are no longer needed: reuse [NT/256][G][64]
        named_sync_id<NT>(bar);
        pv_sm[(ps * G + l4) * 64 + d] = mine;
        named_sync_id<NT>(bar);
        if (ps == 0) {
            int tot = 0;
            for (int i = 0; i < NT / 256; i++) tot += pv_sm[(i * G + l4) * 64 + d];
            const int hq = hkv * G + l4;
            const long o = ((long)b * HQ + hq) * 64 + d;
            out[o] = (float)tot * a_s[hq];
            if (oacc) oacc[o] = tot;
        }
        ATT_TS(9);
    }
}


// ---- staged variant (persistent decode kernel) ---------------------------------------------------------
// The same step with the K pages, and after them the V pages, of the item brought into shared memory by bulk
// asynchronous copies (one 4 KB copy per page, all in flight at once, completion on an mbarrier) instead of
// per-thread global loads in dependent batches: the copies are issued before the new token is prepared, so the
// scores start from shared memory as soon as the query is ready, and the V pages arrive while the softmax runs.
// Needs (ctx + 1) keys <= cap_pages * 64; the caller falls back to dec_attn_fused_body otherwise. Same arithmetic
// in the same order, hence the same bits.
struct DecAttnStage {
    uint8_t* kv;              // cap_pages * 4096 bytes of shared memory (128-byte aligned): K pages, later V^T pages
    uint32_t bar_k, bar_v;    // shared-memory addresses of two mbarriers (arrival count 1)
    uint32_t parity;          // their phase parity for this item (each is used once per item)
    int cap_pages;
    volatile int* abort_flag; // the CTA's "a bounded wait ran out" flag
};

__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Warp-level integer tensor-core product D (16 x 8, s32) += A (16 x 32, row-major) * B (32 x 8, column-major).
// Fragments (lane = 4 * g + t): a0 = A[g][4t..4t+3], a1 = A[g+8][4t..], a2 = A[g][16+4t..], a3 = A[g+8][16+4t..];
// b0 = B[4t..4t+3][g], b1 = B[16+4t..][g]; d0 = D[g][2t], d1 = D[g][2t+1], d2 = D[g+8][2t], d3 = D[g+8][2t+1].
// Integer accumulation: exact, the same sums as the dp4a path in any order.
__device__ __forceinline__ void mma_s8s8(int (&d)[4], const int (&a)[4], const int (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// the same with unsigned B (u8 probabilities against s8 values)
__device__ __forceinline__ void mma_s8u8(int (&d)[4], const int (&a)[4], const int (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Returns false when a bounded wait ran out (the same verdict for all NT threads).
template <int NT>
__device__ __forceinline__ bool dec_attn_staged_body(const DecAttnIn& in, const float* __restrict__ cos_t,
                                                     const float* __restrict__ sin_t, const float* __restrict__ a_s,
                                                     const KvLayer& cache, const int32_t* __restrict__ page_table, int max_pages,
                                                     int HQ, int HKV, int cs, float* __restrict__ out, const int hkv, const int b,
                                                     const int pos, uint8_t* dsm, DecAttnSmem& sm, const DecAttnStage& st,
                                                     const int tid, const int bar) {
    constexpr int G = 4;
    float* sc = reinterpret_cast<float*>(dsm);                       // [G][cs]
    uint8_t* u_sm = dsm + (size_t)G * cs * 4;                        // [G][cs]
    int8_t (*q_sm)[64] = sm.q_sm;
    float* q_scale = sm.q_scale; float (*red)[16] = sm.red; float* row_max = sm.row_max; float* row_rinv = sm.row_rinv;
    float (*part)[4] = sm.part;
    int* pt_sm = sm.pt_sm;
    named_sync_id<NT>(bar);   // the previous item of this group is done with the staging area and the score rows
    ATT_TS(0);
    const int w = tid >> 5, lane = tid & 31;
    const int heads = HQ + 2 * HKV;
    const int nk = pos + 1;
    const int npages = (nk + PAGE - 1) / PAGE;
    const uint32_t stage_addr = tc::smem_u32(st.kv);
    // warp 7: one bulk copy per K page, all in flight
    if (w == NT / 32 - 1) {
        if (lane == 0) tc::mbar_expect_tx(st.bar_k, (uint32_t)npages * 4096u);
        __syncwarp();
        for (int p = lane; p < npages; p += 32) {
            const long pg = page_table[(long)b * max_pages + p];
            bulk_g2s(stage_addr + p * 4096, cache.k + (pg * HKV + hkv) * (long)(64 * PAGE), 4096u, st.bar_k);
        }
    }
    // split-K partial sums of this warp's head (independent of the context): loads first
    int a0 = 0, a1 = 0;
    if (w < 6) {
        const int h = w < 4 ? hkv * G + w : (w == 4 ? HQ + hkv : HQ + HKV + hkv);
        const int32_t* src = in.qkv_acc + (long)b * heads * 64 + (long)h * 64 + lane;
#pragma unroll 1
        for (int sl = 0; sl < in.n_slabs; sl += 4) {
            int p0[4], p1[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const bool on = sl + i < in.n_slabs;
                p0[i] = on ? __ldcg(src + (sl + i) * in.slab_stride) : 0;
                p1[i] = on ? __ldcg(src + (sl + i) * in.slab_stride + 32) : 0;
            }
            a0 += (p0[0] + p0[1]) + (p0[2] + p0[3]);
            a1 += (p1[0] + p1[1]) + (p1[2] + p1[3]);
        }
    }
    for (int i = tid; i < npages; i += NT) pt_sm[i] = page_table[(long)b * max_pages + i];
    // K scales of this thread's keys (tid + u * NT) into registers; the new token's own scale comes from its preparation
    constexpr int UK = 5;                                             // 5 * NT keys >= the staging capacity (20 / 32 pages)
    float ks_pre[UK];
#pragma unroll
    for (int u = 0; u < UK; u++) {
        const int key = tid + u * NT;
        ks_pre[u] = 0.0f;
        if (key < pos) {
            const long pg = page_table[(long)b * max_pages + key / PAGE];
            ks_pre[u] = cache.ks[(pg * HKV + hkv) * PAGE + (key % PAGE)];
        }
    }
    ATT_TS(1);
    // ---- A. prepare: warps 0..3 the query heads, warp 4 the key head, warp 5 the value head
    int8_t new_a = 0, new_b = 0; float new_s = 0.0f;                  // warps 4 / 5: the new token's quantised head, for the staging patch
    if (w < 6) {
        const long pg = page_table[(long)b * max_pages + pos / PAGE];
        const int slot = pos % PAGE;
        const int h = w < 4 ? hkv * G + w : (w == 4 ? HQ + hkv : HQ + HKV + hkv);
        const float stk = __ldcg(in.tok_scale + b);
        const float x0 = ((float)a0 * stk) * in.ch_scale[h * 64 + lane];
        const float x1 = ((float)a1 * stk) * in.ch_scale[h * 64 + lane + 32];
        float a = x0, bb = x1;
        if (w < 5) {
            const float c = cos_t[(long)pos * 32 + lane], sn = sin_t[(long)pos * 32 + lane];
            a = x0 * c - x1 * sn;
            bb = x0 * sn + x1 * c;
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
        }
        const float mx = warp_max(fmaxf(a, bb)), mn = warp_min(fminf(a, bb));
        const float s2 = sym_scale_from(mx, mn);
        const int8_t qa = quant_s8(a, s2), qb = quant_s8(bb, s2);
        new_a = qa; new_b = qb; new_s = s2;
        if (w < 4) {
            q_sm[w][lane] = qa; q_sm[w][lane + 32] = qb;
            if (lane == 0) q_scale[w] = s2;
        } else if (w == 4) {
            int8_t* dst = cache.k + ((pg * HKV + hkv) * PAGE + slot) * 64L;
            dst[lane] = qa; dst[lane + 32] = qb;
            if (lane == 0) cache.ks[(pg * HKV + hkv) * PAGE + slot] = s2;
        } else {
            int8_t* dst = cache.v + (pg * HKV + hkv) * (long)(64 * PAGE);
            dst[(long)lane * PAGE + slot] = qa;
            dst[(long)(lane + 32) * PAGE + slot] = qb;
            if (lane == 0) cache.vs[(pg * HKV + hkv) * PAGE + slot] = s2;
        }
    }
    // K scales into row 0 of the score buffer (each is read by its key's four lanes right before lane 0 overwrites it)
#pragma unroll
    for (int u = 0; u < UK; u++) {
        const int key = tid + u * NT;
        if (key < pos) sc[key] = ks_pre[u];
    }
    // warp 4 waits for the K pages, then puts the new token's row (the copy may or may not have seen the append) and scale in place
    if (w == 4) {
        int ok = lane == 0 ? (tc::mbar_wait(st.bar_k, st.parity, st.abort_flag) ? 1 : 0) : 1;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok) {
            int8_t* row = reinterpret_cast<int8_t*>(st.kv) + (size_t)pos * 64;
            row[lane] = new_a; row[lane + 32] = new_b;
            if (lane == 0) sc[pos] = new_s;
        }
        if (lane == 0) sm.last = ok;
    }
    named_sync_id<NT>(bar);
    if (!sm.last) return false;
    ATT_TS(2);

    // ---- B. scores on the tensor cores: a warp takes blocks of 16 keys; A = 16 key rows x 32 dims from the staging area,
    //         B = 32 dims x the 4 query heads (columns 4..7 are zero), two steps for the 64 dims
    const int gi = lane >> 2, ti = lane & 3;
    int bq[2][2];
#pragma unroll
    for (int ks = 0; ks < 2; ks++) {
        bq[ks][0] = gi < G ? *reinterpret_cast<const int*>(&q_sm[gi][ks * 32 + ti * 4]) : 0;
        bq[ks][1] = gi < G ? *reinterpret_cast<const int*>(&q_sm[gi][ks * 32 + 16 + ti * 4]) : 0;
    }
    // lanes ti < 2 receive the sums of heads 2 ti and 2 ti + 1 for the keys gi and gi + 8 of the block
    const float qs0 = q_scale[(2 * ti) & 3], qs1 = q_scale[(2 * ti + 1) & 3];
    float mx0 = -1e32f, mx1 = -1e32f;
    const int nblk = (nk + 15) >> 4;
    for (int blk = w; blk < nblk; blk += NT / 32) {
        const uint8_t* rows = st.kv + (size_t)(blk * 16 + gi) * 64 + ti * 4;
        int d[4] = {0, 0, 0, 0};
#pragma unroll
        for (int ks = 0; ks < 2; ks++) {
            int af[4];
            af[0] = *reinterpret_cast<const int*>(rows + ks * 32);
            af[1] = *reinterpret_cast<const int*>(rows + 8 * 64 + ks * 32);
            af[2] = *reinterpret_cast<const int*>(rows + ks * 32 + 16);
            af[3] = *reinterpret_cast<const int*>(rows + 8 * 64 + ks * 32 + 16);
            mma_s8s8(d, af, bq[ks]);
        }
        const int kA = blk * 16 + gi, kB = kA + 8;
        const float ksA = sc[kA < nk ? kA : nk - 1], ksB = sc[kB < nk ? kB : nk - 1];
        __syncwarp();                            // every lane has read its keys' scales before row 0 is overwritten below
        if (ti < 2) {
            const int h0 = 2 * ti, h1 = h0 + 1;
            if (kA < nk) {
                const float x0 = (((float)d[0] * qs0) * ksA) * 0.125f, x1 = (((float)d[1] * qs1) * ksA) * 0.125f;
                sc[h0 * cs + kA] = x0; sc[h1 * cs + kA] = x1;
                mx0 = x0 > mx0 ? x0 : mx0; mx1 = x1 > mx1 ? x1 : mx1;
            }
            if (kB < nk) {
                const float x0 = (((float)d[2] * qs0) * ksB) * 0.125f, x1 = (((float)d[3] * qs1) * ksB) * 0.125f;
                sc[h0 * cs + kB] = x0; sc[h1 * cs + kB] = x1;
                mx0 = x0 > mx0 ? x0 : mx0; mx1 = x1 > mx1 ? x1 : mx1;
            }
        }
    }
    ATT_TS(3);
    // maximum over the lanes with the same ti (xor 4, 8, 16): lanes 0 and 1 then hold heads (0, 1) and (2, 3) of this warp
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
    }
    if (lane < 2) { red[2 * lane][w] = mx0; red[2 * lane + 1][w] = mx1; }
    tc::fence_proxy_async_smem();               // this thread's reads / writes of the staging area, before the V copies overwrite it
    named_sync_id<NT>(bar);
    // warp 7: the V^T pages into the staging area
    if (w == NT / 32 - 1) {
        if (lane == 0) tc::mbar_expect_tx(st.bar_v, (uint32_t)npages * 4096u);
        __syncwarp();
        for (int p = lane; p < npages; p += 32)
            bulk_g2s(stage_addr + p * 4096, cache.v + ((long)pt_sm[p] * HKV + hkv) * (long)(64 * PAGE), 4096u, st.bar_v);
    }
    if (tid < G) {
        float m = red[tid][0];
        for (int i = 1; i < NT / 32; i++) m = fmaxf(m, red[tid][i]);
        row_max[tid] = m;
    }
    // V scales of this thread's keys (step F): requested now, used after the exponentials and the ordered sums
    constexpr int UF = UK;
    float vsc_pre[UF];
#pragma unroll
    for (int u = 0; u < UF; u++) {
        const int key = tid + u * NT;
        vsc_pre[u] = 0.0f;
        if (key < nk) vsc_pre[u] = cache.vs[((long)pt_sm[key / PAGE] * HKV + hkv) * PAGE + (key % PAGE)];
    }
    named_sync_id<NT>(bar);
    ATT_TS(4);
    // ---- D. e = exp(x - max), in place: the four heads of a key together (four independent evaluations in flight)
    {
        const float m0 = row_max[0], m1 = row_max[1], m2 = row_max[2], m3 = row_max[3];
        for (int key = tid; key < nk; key += NT) {
            const float x0 = sc[key] - m0, x1 = sc[cs + key] - m1, x2 = sc[2 * cs + key] - m2, x3 = sc[3 * cs + key] - m3;
            const float e0 = ref_expf(x0), e1 = ref_expf(x1), e2 = ref_expf(x2), e3 = ref_expf(x3);
            sc[key] = e0; sc[cs + key] = e1; sc[2 * cs + key] = e2; sc[3 * cs + key] = e3;
        }
    }
    named_sync_id<NT>(bar);
    ATT_TS(5);
    // ---- E. the four ordered chains of each row (Softmax.h:514-553): one thread per chain; the next eight terms are
    //         fetched while the current eight are added (the adds are one dependent chain, the loads are not)
    if (tid < 4 * G) {
        const int g = tid >> 2, j = tid & 3;
        const float* e = sc + g * cs + j;
        const int n = (nk - j + 3) >> 2;                 // terms of this chain: keys j, j + 4, ...
        float ps = 0.0f;
        float cur[8], nxt[8];
#pragma unroll
        for (int i = 0; i < 8; i++) cur[i] = i < n ? e[4 * i] : 0.0f;
        int i0 = 0;
        for (; i0 + 8 < n; i0 += 8) {
#pragma unroll
            for (int i = 0; i < 8; i++) nxt[i] = i0 + 8 + i < n ? e[4 * (i0 + 8 + i)] : 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) ps += cur[i];
#pragma unroll
            for (int i = 0; i < 8; i++) cur[i] = nxt[i];
        }
#pragma unroll
        for (int i = 0; i < 8; i++) if (i0 + i < n) ps += cur[i];
        part[g][j] = ps;
    }
    named_sync_id<NT>(bar);
    if (tid < G) row_rinv[tid] = 1.0f / ((part[tid][0] + part[tid][1]) + (part[tid][2] + part[tid][3]));
    named_sync_id<NT>(bar);
    ATT_TS(6);
    // ---- F. u8 probabilities (zero beyond the last key up to the page boundary)
    const int nk_pad = npages * PAGE;
    {
        float rinv_g[G];
        DivBy as_g[G];
#pragma unroll
        for (int g = 0; g < G; g++) { rinv_g[g] = row_rinv[g]; as_g[g] = div_by(a_s[hkv * G + g]); }
#pragma unroll
        for (int u = 0; u < UF; u++) {
            const int key = tid + u * NT;
            if (key < nk_pad) {
#pragma unroll
                for (int g = 0; g < G; g++) {
                    int r = 0;
                    if (key < nk) {
                        const float p = sc[g * cs + key] * rinv_g[g];
                        r = round_half_away_to_int(div_for_rounding(p * vsc_pre[u], as_g[g]));
                        r = r > 255 ? 255 : r;
                    }
                    u_sm[g * cs + key] = (uint8_t)r;
                }
            }
        }
    }
    // warp 5 waits for the V pages and puts the new token's column in place
    if (w == 5) {
        int ok = lane == 0 ? (tc::mbar_wait(st.bar_v, st.parity, st.abort_flag) ? 1 : 0) : 1;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok) {
            int8_t* pg = reinterpret_cast<int8_t*>(st.kv) + (size_t)(pos / PAGE) * 4096 + (pos % PAGE);
            pg[lane * PAGE] = new_a; pg[(lane + 32) * PAGE] = new_b;
        }
        if (lane == 0) sm.last = ok;
    }
    named_sync_id<NT>(bar);
    if (!sm.last) return false;
    ATT_TS(7);
    // ---- G. P.V on the tensor cores: A = 16 dims x 32 keys of the V^T page, B = 32 keys x the 4 heads' u8 probabilities.
    //         Warp w: dims 16 (w & 3) .. +15, pages (w >> 2), (w >> 2) + NT / 128, ...; the partial sums per dim block are
    //         added through shared memory (integers: exact)
    {
        constexpr int NPS = NT / 128;                     // page sets: 2 (eight warps) or 4 (sixteen warps)
        static_assert(NT == 256 || NT == 512, "four dim blocks x NT / 128 page sets");
        const int dblk = w & 3, pset = w >> 2;
        int d[4] = {0, 0, 0, 0};
        for (int p = pset; p < npages; p += NPS) {
            const uint8_t* rows = st.kv + (size_t)p * 4096 + (size_t)(dblk * 16 + gi) * PAGE + ti * 4;
            const uint8_t* ucol = u_sm + (gi & 3) * cs + p * PAGE + ti * 4;
#pragma unroll
            for (int ks = 0; ks < 2; ks++) {
                int af[4], bu[2];
                af[0] = *reinterpret_cast<const int*>(rows + ks * 32);
                af[1] = *reinterpret_cast<const int*>(rows + 8 * PAGE + ks * 32);
                af[2] = *reinterpret_cast<const int*>(rows + ks * 32 + 16);
                af[3] = *reinterpret_cast<const int*>(rows + 8 * PAGE + ks * 32 + 16);
                bu[0] = gi < G ? *reinterpret_cast<const int*>(ucol + ks * 32) : 0;
                bu[1] = gi < G ? *reinterpret_cast<const int*>(ucol + ks * 32 + 16) : 0;
                mma_s8u8(d, af, bu);
            }
        }
        ATT_TS(8);
        // the exponentials and the u8 rows are no longer needed: [NPS - 1][G][64] sums of page sets 1 .. NPS - 1 (at most
        // 3 KB of the item's scratch, which holds at least 4 KB)
        int* pv_sm = reinterpret_cast<int*>(dsm);
        named_sync_id<NT>(bar);
        if (pset > 0 && ti < 2) {
            int* dst = pv_sm + (pset - 1) * (G * 64);
            dst[(2 * ti) * 64 + dblk * 16 + gi] = d[0]; dst[(2 * ti + 1) * 64 + dblk * 16 + gi] = d[1];
            dst[(2 * ti) * 64 + dblk * 16 + gi + 8] = d[2]; dst[(2 * ti + 1) * 64 + dblk * 16 + gi + 8] = d[3];
        }
        named_sync_id<NT>(bar);
        if (pset == 0 && ti < 2) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int hd = 2 * ti + (i & 1), dim = dblk * 16 + gi + (i >> 1) * 8;
                int tot = d[i];
#pragma unroll
                for (int ps = 0; ps < NPS - 1; ps++) tot += pv_sm[ps * (G * 64) + hd * 64 + dim];
                const int hq = hkv * G + hd;
                out[((long)b * HQ + hq) * 64 + dim] = (float)tot * a_s[hq];
            }
        }
        ATT_TS(9);
    }
    tc::fence_proxy_async_smem();               // reads of the staging area, before the next item's (or a projection's) copies overwrite it
    return true;
}

}  // namespace flexllm
