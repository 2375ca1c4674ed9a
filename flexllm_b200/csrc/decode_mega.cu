// One decode step of the whole model as ONE persistent kernel.
//
// At batch <= 64 every kernel of a decode step is latency-bound (a 4 MB projection streams in under
// a microsecond; its launch, prologue, split-K hand-off and tail cost ten times that), and a step
// is a chain of ~150 such kernels. Here one cooperative grid of one CTA per SM walks the same
// operator order (SpinQuant_Llama_32_1B/SpinQuant_Decoding_mem_opt.h:1050-1126) phase by phase
// with a grid-wide barrier (one atomic arrive + one polled load, about a microsecond) between
// phases instead of a kernel boundary:
//
//   per layer   A  x += dequant(down partial sums) [embedding for layer 0], RMSNorm, int8 quant
//               .  fused q|k|v projection          (tcgen05 kind::i8, split-K over the CTAs)
//               .  attention per (sequence, KV head): dequant, RoPE, FHT-64, quant, cache append,
//                  scores, ordered softmax, u8 quant, P.V; the item that completes a sequence's row quantises it
//               .  o projection
//               C  x += dequant(o partial sums), RMSNorm, int8 quant
//               .  fused gate|up projection
//               D  dequant, silu(gate)*up, FHT-8192, int8 quant (four CTAs per row when the grid allows)
//               .  down projection
//   head        E  x += dequant(down partial sums), final RMSNorm, quant;  lm_head;  greedy argmax or
//                  top-k sampling, token feedback, context lengths + 1
//
// Projections leave raw int32 sums (split-K: one slab of partial sums per split, plain coalesced
// stores; the reader adds the slabs -- integers, exact in any order); the row phase that follows
// applies ((float)acc * s_tok) * s_ch itself, so a projection's result crosses HBM/L2 once. One
// thread (warp 4) issues the TMA loads, one (warp 5) the MMAs, warps 0..3 drain TMEM. As soon as the
// TMA thread has issued the last loads of one projection it starts streaming the WEIGHT tiles of
// the next one into the ring -- weights do not depend on the phases in between -- and only the
// small activation tiles wait for the grid barrier. Arithmetic is the same device code the
// stand-alone kernels use (attention_decode.cuh, fht_core.cuh, sampling.cuh; the RMSNorm statements of
// rmsnorm_core.cuh spread over a CTA), hence bit-identical.
//
// Every wait (mbarrier, grid barrier) is bounded; on a timeout the CTA raises the global error
// flag, all CTAs leave through the tear-down and the host sees FLEXLLM_ETIMEDOUT.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <new>
#include <vector>

#include "attention_decode.cuh"
#include "common.cuh"
#include "fht_core.cuh"
#include "rmsnorm_core.cuh"
#include "sampling.cuh"
#include "tc_common.cuh"

namespace flexllm {
using namespace tc;


constexpr int MG_WORKERS = 512;                 // 16 warps; in a projection phase warps 0..3 run the epilogue and one
                                                // thread of warp 5 issues the TMA loads and the MMAs
constexpr int MG_THREADS = MG_WORKERS;
constexpr int MG_MAX_STAGES = 8;
constexpr int MG_BAR_WORK = 1;                  // named barrier of the 512 workers
constexpr int MG_BAR_FHT = 2;                   // named barrier of the 256 FHT threads
constexpr int MG_BAR_HALF0 = 3, MG_BAR_HALF1 = 4;  // named barriers of the two 256-thread halves (attention)
constexpr int MG_MAX_KS = 10;                   // most split-K slabs a projection may use
constexpr int MG_A_TILE = 128 * 128;            // weight tile: 128 channels x 128 bytes of K
// phases of a layer, then of the head
enum { PH_A = 0, PH_QKV, PH_ATT, PH_O, PH_C, PH_GU, PH_D, PH_DOWN, MG_PHASES_PER_LAYER, PH_E = MG_PHASES_PER_LAYER, PH_LM, PH_TOKEN };
constexpr int MG_FHT_SCRATCH = (8192 + 256 + 80) * 4;   // padded row + reduction slots

struct MegaLayer {
    const float *sqkv, *so, *sgu, *sd, *g0, *g1, *a_s;
    KvLayer kv;
};

struct MegaArgs {
    const CUtensorMap* maps;      // [0] activations xq [BN][D], [1] activations hq [BN][F], [2 + 4l + j] layer weights, [2 + 4L] lm_head
    const MegaLayer* layers;
    int n_layers, B, D, HQ, HKV, F, V;
    float eps, fht_scale;
    float* x; int8_t* xq; float* xs; int8_t* hq; float* att; float* logits;
    int32_t *w_qkv, *w_o, *w_gu, *w_d;
    const int8_t* lm_w; const float* lm_s; const float* g_final;
    const float *cos_t, *sin_t;
    const int32_t* page_table; int max_pages;
    int32_t *ctx, *next, *out_tokens, *state;
    int sample_lanes, sample_k; const float* sample_rnd;     // top-k sampling (sample_k == 0: greedy)
    unsigned long long* sync_ctr; int* error_flag;
    float* fht_x;                 // FHT phase split over 4 CTAs per row: the parts' locally transformed values [max_batch][F]
    int* fht_flags;               // [3][max_batch]: parts published, parts' maxima merged, merged |max| as float bits
    int* att_cnt;                 // [max_batch]: attention items of the sequence that have finished (self-resetting)
    unsigned long long* trace;    // optional phase timeline [barrier][arrive, leave][CTA] in globaltimer ns (last launch)
    int stages, cs, scratch_bytes, max_ctx;
    unsigned long long wait_limit_ns;   // bound of the grid-barrier and flag waits
    int test_barrier_extra;             // test aid: arrivals the FIRST grid barrier waits for beyond those the grid delivers
    int attn_bytes;               // per-half attention scratch: score rows (20 bytes per key) + DecAttnSmem
    int ks_qkv, ks_o, ks_d;       // split-K factors (gate|up and lm_head have enough tiles: 1)
    int slab_rows;                // rows (tokens) per split-K slab = max batch
};

// One projection as the producer, the MMA issuer and the epilogue see it.
struct MegaJob {
    const CUtensorMap *tmA, *tmB;
    int N, tilesA, ksplit, num_kb, ldo;
    int32_t* out;                 // int32 sums; nullptr for the lm_head (fp32 logits)
};

__device__ __forceinline__ MegaJob mega_job(const MegaArgs& a, int layer, int kind) {
    MegaJob j;
    const int QKV = (a.HQ + 2 * a.HKV) * 64;
    j.tmB = a.maps + (kind == 3 ? 1 : 0);
    if (kind == 4) {   // lm_head
        j.tmA = a.maps + 2 + 4 * a.n_layers;
        j.N = a.V; j.ksplit = 1; j.num_kb = a.D >> 7; j.out = nullptr; j.ldo = a.V;
    } else {
        j.tmA = a.maps + 2 + 4 * layer + kind;
        if (kind == 0) { j.N = QKV; j.ksplit = a.ks_qkv; j.num_kb = a.D >> 7; j.out = a.w_qkv; }
        else if (kind == 1) { j.N = a.D; j.ksplit = a.ks_o; j.num_kb = a.D >> 7; j.out = a.w_o; }
        else if (kind == 2) { j.N = 2 * a.F; j.ksplit = 1; j.num_kb = a.D >> 7; j.out = a.w_gu; }
        else { j.N = a.D; j.ksplit = a.ks_d; j.num_kb = a.F >> 7; j.out = a.w_d; }
        j.ldo = j.N;
    }
    j.tilesA = (j.N + 127) >> 7;
    return j;
}

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_volatile_s32(const int* p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Polls the grid-barrier counter until it reaches `target`. Bounded: gives up after the wait
// limit, or as soon as this CTA (shared flag) or any CTA (global flag) has given up.
__device__ __noinline__ bool mega_wait_counter(const unsigned long long* ctr, unsigned long long target, volatile int* abort_flag,
                                               int* error_flag, unsigned long long limit_ns) {
    if (ld_acquire_u64(ctr) >= target) return true;
    const unsigned long long t0 = globaltimer_ns();
    for (uint32_t it = 1;; it++) {
        if (ld_acquire_u64(ctr) >= target) return true;
        if ((it & 63u) == 0) {
            if (*abort_flag) return false;
            if (ld_volatile_s32(error_flag) & 1) { *abort_flag = 1; return false; }
            if (globaltimer_ns() - t0 > limit_ns) { *abort_flag = 1; atomicOr(error_flag, 1); return false; }
        }
    }
}

// Polls an int flag until it reaches `target` (bounded like the counter wait).
__device__ __noinline__ bool mega_wait_flag(const int* flag, int target, volatile int* abort_flag, int* error_flag,
                                            unsigned long long limit_ns) {
    const unsigned long long t0 = globaltimer_ns();
    for (uint32_t it = 1;; it++) {
        int v;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v >= target) return true;
        if ((it & 63u) == 0) {
            if (*abort_flag) return false;
            if (ld_volatile_s32(error_flag) & 1) { *abort_flag = 1; return false; }
            if (globaltimer_ns() - t0 > limit_ns) { *abort_flag = 1; atomicOr(error_flag, 1); return false; }
        }
    }
}

// Grid-wide barrier of the worker threads: everything the CTA wrote before it is visible to every
// CTA after it. Returns false when the step is being abandoned.
__device__ __forceinline__ bool mega_grid_sync(unsigned long long* ctr, unsigned long long target, volatile int* abort_flag,
                                               volatile int* go_flag, int* error_flag, unsigned long long* trace,
                                               unsigned long long limit_ns) {
    named_sync<MG_BAR_WORK, MG_WORKERS>();
    if (threadIdx.x == 0) {
        // release at GPU scope: orders this thread's writes and, through the CTA barrier above, every write of
        // the CTA before the arrival; the acquire loads of the wait plus the CTA barrier below do the reverse
        if (trace) trace[blockIdx.x] = globaltimer_ns();
        asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(ctr), "l"(1ull) : "memory");
        mega_wait_counter(ctr, target, abort_flag, error_flag, limit_ns);
        if (trace) trace[gridDim.x + blockIdx.x] = globaltimer_ns();
        *go_flag = (*abort_flag == 0);      // one verdict for the whole CTA, fixed before anyone reads it
    }
    named_sync<MG_BAR_WORK, MG_WORKERS>();
    return *go_flag != 0;
}

// ---- row phases (all 512 threads of the CTA that owns the row; one float4 per thread) -------------
// x[row] (+)= dequantised projection sums (or the embedding row), then RMSNorm in the reference's
// decode summation order (Modules/LayerNorm.h:210-370: 8 chunks of 4 interleaved chains; the same
// statements as rmsnorm_decode_row, with the row spread over the CTA instead of one warp) and the
// per-token quantiser. acc: `ks` slabs [max_batch][D] of split-K partial sums (integer adds: exact in
// any order), nullptr for the embedding. buf: D + 32 floats, red: 65 floats of shared memory.
__device__ __forceinline__ void mega_row_norm(const MegaArgs& a, int row, const int32_t* acc, int ks, const float* s_ch,
                                              const float* gamma, float* buf, float* red, int tid) {
    constexpr int NT = MG_WORKERS, LANES = 8;
    const int D = a.D, nv = D >> 2, C = D / LANES;
    const int lane = tid & 31, c = tid;
    const bool active = c < nv;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f), g = v;
    float4* xr = reinterpret_cast<float4*>(a.x + (long)row * D);
    if (active) {
        g = __ldg(reinterpret_cast<const float4*>(gamma) + c);
        if (acc == nullptr) {
            int id = a.next[row];
            if (id < 0 || id >= a.V) { if (c == 0) atomicOr(a.error_flag, 2); id = id < 0 ? 0 : a.V - 1; }   // never a wild read
            const float s = a.lm_s[id];
            const char4 t = reinterpret_cast<const char4*>(a.lm_w + (long)id * D)[c];
            v = make_float4((float)t.x * s, (float)t.y * s, (float)t.z * s, (float)t.w * s);
        } else {
            const float st = __ldcg(a.xs + row);
            const int4* ar = reinterpret_cast<const int4*>(acc + (long)row * D) + c;
            const long slab4 = (long)a.slab_rows * D / 4;
            int4 part[MG_MAX_KS];
#pragma unroll
            for (int s = 0; s < MG_MAX_KS; s++)
                if (s < ks) part[s] = __ldcg(ar + s * slab4);
            v = __ldcg(xr + c);
            const float4 sc = __ldg(reinterpret_cast<const float4*>(s_ch) + c);
            int4 sum = make_int4(0, 0, 0, 0);
#pragma unroll
            for (int s = 0; s < MG_MAX_KS; s++)
                if (s < ks) { sum.x += part[s].x; sum.y += part[s].y; sum.z += part[s].z; sum.w += part[s].w; }
            float4 r;
            r.x = ((float)sum.x * st) * sc.x; r.y = ((float)sum.y * st) * sc.y;
            r.z = ((float)sum.z * st) * sc.z; r.w = ((float)sum.w * st) * sc.w;
            v.x = v.x + r.x; v.y = v.y + r.y; v.z = v.z + r.z; v.w = v.w + r.w;
        }
        xr[c] = v;
        const int e = c * 4;
        *reinterpret_cast<float4*>(buf + e + 4 * (e / C)) = v;      // element e at e + 4*(e / C)
    }
    named_sync<MG_BAR_WORK, NT>();
    if (tid < 32) {
        const int chunk = lane >> 2, j = lane & 3;
        float ss = 0.0f;
        {
            const float* bc = buf + chunk * (C + 4);
            const int n = C >> 2;
#pragma unroll 8
            for (int k = 0; k < n; k++) { const float t = bc[4 * k + j]; ss += t * t; }
        }
        float tot = 0.0f;
        for (int cc = 0; cc < LANES; cc++) {
            const float p0 = __shfl_sync(0xffffffffu, ss, cc * 4 + 0), p1 = __shfl_sync(0xffffffffu, ss, cc * 4 + 1);
            const float p2 = __shfl_sync(0xffffffffu, ss, cc * 4 + 2), p3 = __shfl_sync(0xffffffffu, ss, cc * 4 + 3);
            tot += (p0 + p1) + (p2 + p3);
        }
        if (lane == 0) red[64] = 1.0f / sqrtf(tot / (float)D + a.eps);
    }
    named_sync<MG_BAR_WORK, NT>();
    const float r = red[64];
    float mx = -1e32f, mn = 1e32f;
    if (active) {
        float4 o;
        o.x = (v.x * r) * g.x; o.y = (v.y * r) * g.y; o.z = (v.z * r) * g.z; o.w = (v.w * r) * g.w;
        v = o;
        mx = fmaxf(fmaxf(o.x, o.y), fmaxf(o.z, o.w));
        mn = fminf(fminf(o.x, o.y), fminf(o.z, o.w));
    }
    group_max_min<MG_BAR_WORK, NT>(mx, mn, red, tid);
    const float sc = sym_scale_from(mx, mn);
    if (tid == 0) a.xs[row] = sc;
    if (active) {
        char4 o;
        o.x = quant_s8(v.x, sc); o.y = quant_s8(v.y, sc); o.z = quant_s8(v.z, sc); o.w = quant_s8(v.w, sc);
        reinterpret_cast<char4*>(a.xq + (long)row * D)[c] = o;
        asm volatile("fence.proxy.async.global;" ::: "memory");   // xq is read by other CTAs' TMA (async proxy)
    }
}

// Attention output row b -> int8 (Modules/quant.h:349-430), by the 256 threads of the half whose item arrived
// last on the sequence's counter. Arrival: acq_rel atomic by one thread after the half's barrier (orders the
// half's stores before it; the last arriver sees every other item's stores after it).
__device__ __forceinline__ void mega_att_row_quant(const MegaArgs& a, int b, DecAttnSmem& sm, int t, int bar) {
    named_sync_id<256>(bar);
    if (t == 0) {
        int old;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(a.att_cnt + b), "r"(1) : "memory");
        sm.last = old == a.HKV - 1;
        if (sm.last) a.att_cnt[b] = 0;          // next use: the next layer's attention phase, grid barriers away
    }
    named_sync_id<256>(bar);
    if (!sm.last) return;
    const int D = a.D, nv = D >> 2;
    const float4* src = reinterpret_cast<const float4*>(a.att + (long)b * D);
    float4 v[2];
    float mx = -1e32f, mn = 1e32f;
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int c = t + i * 256;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < nv) {
            v[i] = __ldcg(src + c);
            mx = fmaxf(mx, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
            mn = fminf(mn, fminf(fminf(v[i].x, v[i].y), fminf(v[i].z, v[i].w)));
        }
    }
    mx = warp_max(mx); mn = warp_min(mn);
    if ((t & 31) == 0) { sm.red[0][t >> 5] = mx; sm.red[1][t >> 5] = mn; }
    named_sync_id<256>(bar);
#pragma unroll
    for (int w = 0; w < 8; w++) { mx = fmaxf(mx, sm.red[0][w]); mn = fminf(mn, sm.red[1][w]); }
    const float sc = sym_scale_from(mx, mn);
    if (t == 0) a.xs[b] = sc;
    char4* qr = reinterpret_cast<char4*>(a.xq + (long)b * D);
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int c = t + i * 256;
        if (c < nv) {
            char4 o;
            o.x = quant_s8(v[i].x, sc); o.y = quant_s8(v[i].y, sc); o.z = quant_s8(v[i].z, sc); o.w = quant_s8(v[i].w, sc);
            qr[c] = o;
        }
    }
    asm volatile("fence.proxy.async.global;" ::: "memory");   // xq is read by other CTAs' TMA (async proxy)
}

// dequant(gate|up sums) -> silu(gate)*up -> FHT-8192 / scale -> int8 quant. All 512 threads fetch and
// activate the row (every load of a thread in flight at once), threads 0..255 run the butterflies.
__device__ __forceinline__ void mega_row_fht(const MegaArgs& a, const MegaLayer& L, int row, float* buf, float* red, int tid) {
    constexpr int N = 8192;
    const float st = __ldcg(a.xs + row);
    const int4* gr = reinterpret_cast<const int4*>(a.w_gu + (long)row * 2 * N);
    const int4* ur = gr + N / 4;
    const float4* sg = reinterpret_cast<const float4*>(L.sgu);
    const float4* su = sg + N / 4;
    {
        int4 ga[4], ua[4];
        float4 s1[4], s2[4];
#pragma unroll
        for (int it = 0; it < 4; it++) {
            const int c = it * MG_WORKERS + tid;
            ga[it] = __ldcg(gr + c); ua[it] = __ldcg(ur + c); s1[it] = __ldg(sg + c); s2[it] = __ldg(su + c);
        }
#pragma unroll 1
        for (int it = 0; it < 4; it++) {
            const int c = it * MG_WORKERS + tid;
            // (rolled loop: pick this iteration's registers without dynamic indexing)
            const int4 g4 = it == 0 ? ga[0] : it == 1 ? ga[1] : it == 2 ? ga[2] : ga[3];
            const int4 u4 = it == 0 ? ua[0] : it == 1 ? ua[1] : it == 2 ? ua[2] : ua[3];
            const float4 a1 = it == 0 ? s1[0] : it == 1 ? s1[1] : it == 2 ? s1[2] : s1[3];
            const float4 a2 = it == 0 ? s2[0] : it == 1 ? s2[1] : it == 2 ? s2[2] : s2[3];
            float4 g, u, v;
            g.x = ((float)g4.x * st) * a1.x; g.y = ((float)g4.y * st) * a1.y; g.z = ((float)g4.z * st) * a1.z; g.w = ((float)g4.w * st) * a1.w;
            u.x = ((float)u4.x * st) * a2.x; u.y = ((float)u4.y * st) * a2.y; u.z = ((float)u4.z * st) * a2.z; u.w = ((float)u4.w * st) * a2.w;
            v.x = silu_f(g.x) * u.x; v.y = silu_f(g.y) * u.y; v.z = silu_f(g.z) * u.z; v.w = silu_f(g.w) * u.w;
            const int p = pad32(c * 4);
            buf[p] = v.x; buf[p + 1] = v.y; buf[p + 2] = v.z; buf[p + 3] = v.w;
        }
    }
    named_sync<MG_BAR_WORK, MG_WORKERS>();
    if (tid >= 256) return;
    float r[32];
    fht8192_passes<MG_BAR_FHT>(buf, tid, r);
    float mx = -1e32f, mn = 1e32f;
    div_rn_array(r, div_by(a.fht_scale));
#pragma unroll
    for (int v = 0; v < 32; v++) {
        mx = fmaxf(mx, r[v]);
        mn = fminf(mn, r[v]);
    }
    group_max_min<MG_BAR_FHT, 256>(mx, mn, red, tid);
    const float sc = sym_scale_from(mx, mn);
    const DivBy dsc = div_by(sc);
    if (tid == 0) a.xs[row] = sc;
#pragma unroll
    for (int hi = 0; hi < 4; hi++) {
        union { int8_t b[8]; int2 v; } o;
#pragma unroll
        for (int c = 0; c < 8; c++) o.b[c] = (int8_t)round_half_away_to_int(div_for_rounding(r[hi * 8 + c], dsc));
        *reinterpret_cast<int2*>(a.hq + (long)row * N + hi * 2048 + tid * 8) = o.v;
    }
    asm volatile("fence.proxy.async.global;" ::: "memory");   // hq is read by other CTAs' TMA (async proxy)
}

// The same phase with the row split over FOUR CTAs (used when 4 * B CTAs exist): part p owns elements
// p*2048 .. p*2048+2047. The 8192-point transform factors as: stages on index bits 1..10 inside each part,
// stages 11 and 12 across the parts (element i of every part), then the stage on bit 0 inside the part
// again -- the reference's stage order, so the same additions in the same order. Two small exchanges
// through global memory, each guarded by a per-row arrival counter: the locally transformed parts, and
// the row's largest magnitude for the quantiser (maximum of non-negative floats = maximum of their bits).
__device__ __forceinline__ void mega_row_fht4(const MegaArgs& a, const MegaLayer& L, int row, int part, float* buf, float* red, int tid,
                                              volatile int* abort_flag) {
    constexpr int N = 8192, NP = 2048;
    int* flag_a = a.fht_flags + row;
    int* flag_b = a.fht_flags + a.slab_rows + row;
    unsigned* amax_bits = reinterpret_cast<unsigned*>(a.fht_flags + 2 * a.slab_rows) + row;
    {   // 1. this part's 2048 values: dequantise gate and up, silu(gate) * up (one float4 per thread)
        const float st = __ldcg(a.xs + row);
        const int c = part * (NP / 4) + tid;
        const int4* gr = reinterpret_cast<const int4*>(a.w_gu + (long)row * 2 * N);
        const int4 g4 = __ldcg(gr + c), u4 = __ldcg(gr + N / 4 + c);
        const float4 a1 = __ldg(reinterpret_cast<const float4*>(L.sgu) + c), a2 = __ldg(reinterpret_cast<const float4*>(L.sgu) + N / 4 + c);
        float4 g, u;
        g.x = ((float)g4.x * st) * a1.x; g.y = ((float)g4.y * st) * a1.y; g.z = ((float)g4.z * st) * a1.z; g.w = ((float)g4.w * st) * a1.w;
        u.x = ((float)u4.x * st) * a2.x; u.y = ((float)u4.y * st) * a2.y; u.z = ((float)u4.z * st) * a2.z; u.w = ((float)u4.w * st) * a2.w;
        const int p = pad32(tid * 4);
        buf[p] = silu_f(g.x) * u.x; buf[p + 1] = silu_f(g.y) * u.y; buf[p + 2] = silu_f(g.z) * u.z; buf[p + 3] = silu_f(g.w) * u.w;
    }
    named_sync<MG_BAR_WORK, MG_WORKERS>();
    if (tid < 256) {   // 2. stages on bits 1..10: four passes over groups of three index bits, 8 values per thread
        float r[8];
        auto pass = [&](const int b0, const int which) {      // group = bits b0..b0+2; which: 0 all three, 1 the lower two, 2 the upper two
            const int base = (tid & ((1 << b0) - 1)) | ((tid >> b0) << (b0 + 3));
#pragma unroll
            for (int v = 0; v < 8; v++) r[v] = buf[pad32(base | (v << b0))];
            if (which != 2) reg_butterfly<0>(r);
            reg_butterfly<1>(r);
            if (which != 1) reg_butterfly<2>(r);
#pragma unroll
            for (int v = 0; v < 8; v++) buf[pad32(base | (v << b0))] = r[v];
            named_sync<MG_BAR_FHT, 256>();
        };
        pass(1, 0); pass(4, 0); pass(7, 1); pass(8, 2);
    }
    named_sync<MG_BAR_WORK, MG_WORKERS>();
    // 3. publish the part, wait for the other three
    float4 own;
    {
        const int p = pad32(tid * 4);
        own = make_float4(buf[p], buf[p + 1], buf[p + 2], buf[p + 3]);
        reinterpret_cast<float4*>(a.fht_x + (long)row * N + part * NP)[tid] = own;
    }
    named_sync<MG_BAR_WORK, MG_WORKERS>();
    if (tid == 0) {
        asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(flag_a), "r"(1) : "memory");
        mega_wait_flag(flag_a, 4, abort_flag, a.error_flag, a.wait_limit_ns);
    }
    named_sync<MG_BAR_WORK, MG_WORKERS>();
    if (*abort_flag) return;
    // 4. stages 11 and 12 across the parts, then bit 0 inside the thread's four consecutive elements
    float x[4];
    {
        float4 w[4];
#pragma unroll
        for (int q = 0; q < 4; q++)
            w[q] = q == part ? own : __ldcg(reinterpret_cast<const float4*>(a.fht_x + (long)row * N + q * NP) + tid);
        auto bf = [](float& lo, float& hi) { const float s = lo + hi, d = lo - hi; lo = s; hi = d; };
        bf(w[0].x, w[1].x); bf(w[0].y, w[1].y); bf(w[0].z, w[1].z); bf(w[0].w, w[1].w);     // bit 11
        bf(w[2].x, w[3].x); bf(w[2].y, w[3].y); bf(w[2].z, w[3].z); bf(w[2].w, w[3].w);
        bf(w[0].x, w[2].x); bf(w[0].y, w[2].y); bf(w[0].z, w[2].z); bf(w[0].w, w[2].w);     // bit 12
        bf(w[1].x, w[3].x); bf(w[1].y, w[3].y); bf(w[1].z, w[3].z); bf(w[1].w, w[3].w);
        const float4 m = part == 0 ? w[0] : part == 1 ? w[1] : part == 2 ? w[2] : w[3];
        x[0] = m.x + m.y; x[1] = m.x - m.y; x[2] = m.z + m.w; x[3] = m.z - m.w;             // bit 0
    }
    div_rn_array(x, div_by(a.fht_scale));
    float mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3])), mn = fminf(fminf(x[0], x[1]), fminf(x[2], x[3]));
    group_max_min<MG_BAR_WORK, MG_WORKERS>(mx, mn, red, tid);
    if (tid == 0) {   // 5. the row's largest magnitude over the four parts
        const float am = fmaxf(fabsf(mx), fabsf(mn));
        atomicMax(amax_bits, __float_as_uint(am));
        asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(flag_b), "r"(1) : "memory");
        mega_wait_flag(flag_b, 4, abort_flag, a.error_flag, a.wait_limit_ns);
    }
    named_sync<MG_BAR_WORK, MG_WORKERS>();
    if (*abort_flag) return;
    float sc = __uint_as_float(__ldcg(amax_bits)) / 127.0f;          // sym_scale_from on the merged maximum
    if (sc == 0.0f) sc = 1.0f;
    const DivBy dsc = div_by(sc);
    if (part == 0 && tid == 0) a.xs[row] = sc;
    char4 o;
    o.x = (int8_t)round_half_away_to_int(div_for_rounding(x[0], dsc)); o.y = (int8_t)round_half_away_to_int(div_for_rounding(x[1], dsc));
    o.z = (int8_t)round_half_away_to_int(div_for_rounding(x[2], dsc)); o.w = (int8_t)round_half_away_to_int(div_for_rounding(x[3], dsc));
    reinterpret_cast<char4*>(a.hq + (long)row * N + part * NP)[tid] = o;
    asm volatile("fence.proxy.async.global;" ::: "memory");   // hq is read by other CTAs' TMA (async proxy)
}

// greedy token of one row by the 512 workers (ties to the lowest index, Logits.h:13-17), then the
// step's bookkeeping for that sequence
__device__ __forceinline__ void mega_row_argmax(const MegaArgs& a, int row, int col, int n_cols, float* sv, int* si) {
    const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
    const float* l = a.logits + (long)row * a.V;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int v = tid; v < a.V; v += MG_WORKERS) {
        const float t = __ldcg(l + v);
        if (t > best || bi == 0x7fffffff) { best = t; bi = v; }
    }
    auto better = [](float x, int xi, float y, int yi) { return x > y || (x == y && xi < yi); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ob, oi, best, bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) { sv[w] = best; si[w] = bi; }
    named_sync<MG_BAR_WORK, MG_WORKERS>();
    if (w == 0) {
        best = lane < MG_WORKERS / 32 ? sv[lane] : -INFINITY;
        bi = lane < MG_WORKERS / 32 ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ob, oi, best, bi)) { best = ob; bi = oi; }
        }
        if (lane == 0) {
            a.next[row] = bi;
            if (col < n_cols) a.out_tokens[(long)row * n_cols + col] = bi;
            a.ctx[row] += 1;
        }
    }
}

// top-k sampling of one row by the 512 workers (sampling.cuh), then the same bookkeeping. Out of line: it runs
// once per step and must not weigh on the register allocation of the phases that run every layer.
__device__ __noinline__ void mega_row_sample(const MegaArgs& a, int row, int col, int n_cols, SampleSmem& sm) {
    const int s = topk_sample_row<MG_WORKERS>(a.logits + (long)row * a.V, a.V, a.sample_lanes, a.sample_k,
                                              a.sample_rnd[(long)col * a.B + row], sm, (int)threadIdx.x, MG_BAR_WORK, nullptr, nullptr);
    if (threadIdx.x == 0) {
        a.next[row] = s;
        if (col < n_cols) a.out_tokens[(long)row * n_cols + col] = s;
        a.ctx[row] += 1;
    }
}

// ---- the kernel -----------------------------------------------------------------------------------
// ATT selects which attention bodies are compiled in. The whole kernel is several hundred KB of instructions and a
// latency-bound step pays for every instruction-cache miss, so the host launches the leanest variant that covers the
// launch (measured: 5 % off the step against the variant that holds every body):
//   0  every body: both item layouts, the staged copies and the per-thread-load body for contexts beyond the staging area
//   1  two items per CTA, staged copies only (more items than CTAs, every context fits half of the operand ring)
//   2  one item per CTA on all 512 threads, staged copies only (no more items than CTAs, every context fits the ring)
// A variant that meets a context it was not built for raises the device-data error bit and skips the item.
template <int BN, int ATT>
__global__ void __launch_bounds__(MG_THREADS, 1) decode_mega_kernel(const __grid_constant__ MegaArgs a) {
    constexpr int STAGE_BYTES = MG_A_TILE + BN * 128;
    constexpr int TMEM_COLS = 2 * BN;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t ring = (raw + 1023u) & ~1023u;
    uint8_t* ring_ptr = smem_raw + (ring - raw);
    const int STAGES = a.stages;
    uint8_t* scratch = ring_ptr + (size_t)STAGES * STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(scratch + a.scratch_bytes);
    const uint32_t bar_full = smem_u32(bars);
    const uint32_t bar_empty = bar_full + 8 * MG_MAX_STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * MG_MAX_STAGES;
    const uint32_t bar_tempty = bar_tfull + 16;
    const uint32_t bar_att = bar_tempty + 16;            // attention staging: (K pages, V pages) of each half of the CTA
    unsigned long long* base_slot = reinterpret_cast<unsigned long long*>(bars + 2 * MG_MAX_STAGES + 8);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_slot + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* go_flag = abort_flag + 1;
    __shared__ float arg_v[MG_WORKERS / 32];
    __shared__ int arg_i[MG_WORKERS / 32];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, G = gridDim.x;
    const int L = a.n_layers;
    const int n_barriers = MG_PHASES_PER_LAYER * L + 2;
    const int col = a.state[0], n_cols = a.state[1];      // read before anyone can reach the last phase

    if (tid == 0) {
        for (int s = 0; s < MG_MAX_STAGES; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int s = 0; s < 2; s++) { mbar_init(bar_tfull + 8 * s, 1); mbar_init(bar_tempty + 8 * s, 4); }
        for (int s = 0; s < 4; s++) mbar_init(bar_att + 8 * s, 1);
        *abort_flag = 0;
        // every launch adds exactly n_barriers * G arrivals, so the launch's base is the counter rounded
        // down to a multiple of that (no CTA can be a whole launch ahead of another)
        const unsigned long long per = (unsigned long long)n_barriers * (unsigned long long)G;
        *base_slot = ld_acquire_u64(a.sync_ctr) / per * per;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const unsigned long long ctr_base = *base_slot;
    auto target_of = [&](int barrier_index) { return ctr_base + (unsigned long long)(barrier_index + 1) * (unsigned long long)G; };

    // ---- per-thread pipeline bookkeeping (each role uses its own part; the rest is carried unused)
    int pstage = 0; uint32_t pphase = 0;         // TMA thread: position in the ring
    int early_n = 0, early_stage0 = 0;           // TMA thread: weight tiles of the NEXT projection already in flight
    int cstage = 0; uint32_t cphase = 0;         // MMA thread: position in the ring
    int item_base = 0;                           // items (tile, split) this CTA has processed so far
    uint32_t att_uses = 0;                       // attention items this half of the CTA has run on the staged path (mbarrier parity)
    const bool is_tma = (warp == 4 && lane == 0), is_mma = (warp == 5 && lane == 0);

    // k blocks of this CTA in a projection, in issue order: items t = cta, cta + G, ...; inside an item kb0..kb1-1
    struct KbIter {
        int t, kb, kb0, kb1, n_items, ksplit, num_kb, G;
        __device__ void range() {
            const int split = t % ksplit;
            kb0 = kb = split * num_kb / ksplit;            // small numbers: 32-bit arithmetic
            kb1 = (split + 1) * num_kb / ksplit;
        }
        __device__ void init(const MegaJob& j, int cta, int G_) {
            n_items = j.tilesA * j.ksplit; ksplit = j.ksplit; num_kb = j.num_kb; G = G_; t = cta; kb = kb0 = kb1 = 0;
            if (t < n_items) range();
        }
        __device__ bool valid() const { return t < n_items; }
        __device__ void next() { if (++kb == kb1) { t += G; if (t < n_items) range(); } }
    };
    // Weight tiles of the first k blocks of projection j, as many as the ring holds: issued before the
    // phases in between have run (weights do not depend on them). The activation half of each stage
    // follows at the start of j's own phase; the stage's barrier expects both. TMA thread only.
    auto prefetch_weights = [&](const MegaJob& j) {
        KbIter it; it.init(j, cta, G);
        tma_prefetch_desc(j.tmA);
        early_n = 0; early_stage0 = pstage;
        while (early_n < STAGES && it.valid()) {
            if (!mbar_wait(bar_empty + 8 * pstage, pphase ^ 1u, abort_flag)) return;
            mbar_expect_tx(bar_full + 8 * pstage, STAGE_BYTES);
            tma_load_2d(ring + pstage * STAGE_BYTES, j.tmA, bar_full + 8 * pstage, it.kb * 128, (it.t / j.ksplit) * 128);
            if (++pstage == STAGES) { pstage = 0; pphase ^= 1u; }
            early_n++;
            it.next();
        }
    };
    // The same tiles asked into L2 only (the ring is in use by the attention phase). TMA thread only.
    auto prefetch_weights_l2 = [&](const MegaJob& j) {
        KbIter it; it.init(j, cta, G);
        tma_prefetch_desc(j.tmA);
        for (int n = 0; n < STAGES && it.valid(); n++, it.next()) tma_prefetch_l2_2d(j.tmA, it.kb * 128, (it.t / j.ksplit) * 128);
    };
    // One projection. Roles: warp 4 lane 0 TMA, warp 5 lane 0 MMA, warps 0..3 epilogue.
    auto gemm_phase = [&](const MegaJob& j, const MegaJob* next_job) {
        const int n_items = j.tilesA * j.ksplit;
        const int n_mine = cta < n_items ? (n_items - cta + G - 1) / G : 0;
        if (is_tma) {
            asm volatile("fence.proxy.async.global;" ::: "memory");
            KbIter it; it.init(j, cta, G);
            // activation halves of the stages whose weights are already on their way
            int s2 = early_stage0;
            for (int i = 0; i < early_n; i++) {
                tma_load_2d(ring + s2 * STAGE_BYTES + MG_A_TILE, j.tmB, bar_full + 8 * s2, it.kb * 128, 0);
                if (++s2 == STAGES) s2 = 0;
                it.next();
            }
            early_n = 0;
            bool pok = true;
            while (it.valid()) {
                if (!mbar_wait(bar_empty + 8 * pstage, pphase ^ 1u, abort_flag)) { pok = false; break; }
                const uint32_t full = bar_full + 8 * pstage;
                mbar_expect_tx(full, STAGE_BYTES);
                tma_load_2d(ring + pstage * STAGE_BYTES, j.tmA, full, it.kb * 128, (it.t / j.ksplit) * 128);
                tma_load_2d(ring + pstage * STAGE_BYTES + MG_A_TILE, j.tmB, full, it.kb * 128, 0);
                if (++pstage == STAGES) { pstage = 0; pphase ^= 1u; }
                it.next();
            }
            if (pok && next_job) prefetch_weights(*next_job);
        } else if (is_mma) {
            constexpr uint32_t idesc = umma_idesc_i8(128, BN, 1, 1);
            KbIter it; it.init(j, cta, G);
            int i = 0;
            while (it.valid()) {
                const int idx = item_base + i, as = idx & 1;
                if (it.kb == it.kb0) {
                    if (!mbar_wait(bar_tempty + 8 * as, (uint32_t)((idx >> 1) & 1) ^ 1u, abort_flag)) break;
                    tc_fence_after();
                }
                if (!mbar_wait(bar_full + 8 * cstage, cphase, abort_flag)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + as * BN;
                const uint32_t sa = ring + cstage * STAGE_BYTES;
                const uint64_t adesc = umma_desc_k_sw128(sa), bdesc = umma_desc_k_sw128(sa + MG_A_TILE);
#pragma unroll
                for (int k = 0; k < 4; k++) umma_i8(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (it.kb > it.kb0 || k > 0) ? 1u : 0u);
                umma_commit(bar_empty + 8 * cstage);
                if (++cstage == STAGES) { cstage = 0; cphase ^= 1u; }
                if (it.kb + 1 == it.kb1) { umma_commit(bar_tfull + 8 * as); i++; }
                it.next();
            }
        } else if (warp < 4) {
            const int q = warp;
            // per-token scales for the lm_head epilogue: lane holds tokens lane and lane + 32
            float xs0 = 0.f, xs1 = 0.f;
            if (j.out == nullptr) {
                if (lane < a.B) xs0 = __ldcg(a.xs + lane);
                if (lane + 32 < a.B) xs1 = __ldcg(a.xs + lane + 32);
            }
            for (int i = 0; i < n_mine; i++) {
                const int t = cta + i * G;
                const int ta = t / j.ksplit, split = t - ta * j.ksplit;
                const int idx = item_base + i, as = idx & 1;
                const int rowA = ta * 128 + q * 32 + lane;
                const bool row_ok = rowA < j.N;
                const float sa = (j.out == nullptr && row_ok) ? a.lm_s[rowA] : 0.0f;
                int32_t* slab = j.out ? j.out + (long)split * a.slab_rows * j.ldo : nullptr;   // this split's partial sums
                int got = (lane == 0) ? (mbar_wait(bar_tfull + 8 * as, (uint32_t)((idx >> 1) & 1), abort_flag) ? 1 : 0) : 1;
                got = __shfl_sync(0xffffffffu, got, 0);
                if (!got) break;
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < BN / 32; c++) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + as * BN + c * 32, v);
                    tmem_ld_wait();
                    if (slab) {
                        // the per-layer path: raw sums, one coalesced store per token (kept apart from the lm_head
                        // path so that the code walked every layer stays short)
                        int32_t* dst = slab + rowA + (long)(c * 32) * j.ldo;
                        const int ntok = a.B - c * 32;
#pragma unroll
                        for (int jj = 0; jj < 32; jj++)
                            if (row_ok && jj < ntok) dst[(long)jj * j.ldo] = (int)v[jj];
                    } else {
#pragma unroll
                        for (int jj = 0; jj < 32; jj++) {
                            const int tok = c * 32 + jj;
                            const float st = __shfl_sync(0xffffffffu, c == 0 ? xs0 : xs1, jj);
                            if (row_ok && tok < a.B) a.logits[(long)tok * j.ldo + rowA] = ((float)(int)v[jj] * st) * sa;
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tempty + 8 * as);
            }
        }
        item_base += n_mine;
    };

    if (is_tma) {
        tma_prefetch_desc(a.maps); tma_prefetch_desc(a.maps + 1);
        prefetch_weights(mega_job(a, 0, 0));
    }
    float* rowbuf = reinterpret_cast<float*>(scratch);
    float* rowred = rowbuf + 8192 + 256;
    // ---- the step: phases 9l + k of layer l (k = 0..8), then the head (k = 9, 10, 11); one call site per
    //      kind of phase keeps the kernel's code small enough to stay in the instruction cache
    const int n_phases = MG_PHASES_PER_LAYER * L + 3;
    for (int p = 0; p < n_phases; p++) {
        int l = p / MG_PHASES_PER_LAYER, k = p - MG_PHASES_PER_LAYER * l;
        if (l >= L) { k = MG_PHASES_PER_LAYER + (p - MG_PHASES_PER_LAYER * L); l = L - 1; }
        const MegaLayer& ly = a.layers[l];
        if (k == PH_A || k == PH_C || k == PH_E) {
            if (cta < a.B) {
                const int32_t* acc; int ks; const float *s_ch, *gamma;
                if (k == PH_C) { acc = a.w_o; ks = a.ks_o; s_ch = ly.so; gamma = ly.g1; }
                else if (k == PH_E) { acc = a.w_d; ks = a.ks_d; s_ch = ly.sd; gamma = a.g_final; }
                else { acc = p == 0 ? nullptr : a.w_d; ks = a.ks_d; s_ch = p == 0 ? nullptr : a.layers[l - 1].sd; gamma = ly.g0; }
                mega_row_norm(a, cta, acc, ks, s_ch, gamma, rowbuf, rowred, tid);
            } else if ((p == 0 || (k == PH_C && l + 1 < L)) && G > a.B) {
                // CTAs without a row ask L2 for the KV pages an attention phase will read (any CTA can do this
                // for any item: L2 is shared): the first layer's at the start of the step, and in every phase C
                // those of the NEXT layer, long before they are needed. (Tried and slower: the same requests from the
                // idle CTAs of the FHT phase, or from all CTAs at its start -- the page-table look-ups are a chain of
                // latencies that then sits on that phase's critical path.)
                const MegaLayer& nx = a.layers[p == 0 ? 0 : l + 1];
                if (ATT == 2 || (ATT == 0 && a.B * a.HKV <= G)) {
                    // few items (at most one per CTA): groups of 128 threads with one dependent load per thread
                    // (measured: 1.5 % off the step at 16 sequences; at 32 sequences the plain form below was 0.7 % faster)
                    const int grp = tid >> 7, stride = G - a.B;
                    for (int idx = cta - a.B + grp * stride; idx < a.B * a.HKV; idx += 4 * stride)
                        dec_attn_prefetch_l2_g128(nx.kv, a.page_table, a.max_pages, a.ctx, a.HKV, idx % a.HKV, idx / a.HKV, tid & 127);
                } else {
                    for (int idx = cta - a.B; idx < a.B * a.HKV; idx += G - a.B)
                        dec_attn_prefetch_l2(nx.kv, a.page_table, a.max_pages, a.ctx, a.HKV, idx % a.HKV, idx / a.HKV, tid, MG_WORKERS);
                }
            }
        } else if (k == PH_ATT) {
            DecAttnIn in;
            in.q = in.k = in.v = nullptr; in.qs = in.ks = in.vs = nullptr; in.qkv_f32 = nullptr;
            in.qkv_acc = a.w_qkv; in.tok_scale = a.xs; in.ch_scale = ly.sqkv;
            in.n_slabs = a.ks_qkv; in.slab_stride = (long)a.slab_rows * (a.HQ + 2 * a.HKV) * 64;
            in.max_pos = a.max_ctx; in.error_flag = a.error_flag;
            // two (sequence, KV head) items at a time, one per half of the CTA: an item is a chain of
            // global-memory round trips, so two chains side by side nearly double the throughput
            const int half = tid >> 8;
            uint8_t* dsm = scratch + (size_t)half * a.attn_bytes;
            DecAttnSmem& sm = *reinterpret_cast<DecAttnSmem*>(dsm + a.attn_bytes - sizeof(DecAttnSmem));
            // the operand ring is idle during this phase (the next projection's weights are only asked into L2): each half
            // of the CTA stages its item's K pages, then V pages, in its half of the ring
            const int half_bytes = ((STAGES * STAGE_BYTES) >> 1) & ~127;
            DecAttnStage stg;
            stg.kv = ring_ptr + (size_t)half * half_bytes;
            stg.bar_k = bar_att + 16 * half; stg.bar_v = stg.bar_k + 8;
            stg.cap_pages = half_bytes / 4096 < 20 ? half_bytes / 4096 : 20;
            stg.abort_flag = abort_flag;
            if (is_tma) prefetch_weights_l2(mega_job(a, l, 1));
            if (ATT != 1 && (ATT == 2 || a.B * a.HKV <= G)) {
                // no more items than CTAs: one item per CTA, worked on by all 512 threads (an item is a chain of dependent
                // stages; twice the threads shorten the stages that scale -- scores, exponentials, quantiser, P.V)
                if (cta < a.B * a.HKV) {
                    const int b = cta / a.HKV;
                    const int pos = dec_guarded_pos(a.ctx, b, a.max_ctx, a.error_flag);
                    uint8_t* dsm1 = scratch;
                    DecAttnSmem& sm1 = *reinterpret_cast<DecAttnSmem*>(dsm1 + a.attn_bytes - sizeof(DecAttnSmem));
                    DecAttnStage st1;
                    st1.kv = ring_ptr; st1.bar_k = bar_att; st1.bar_v = bar_att + 8;
                    const int ring_pages = (STAGES * STAGE_BYTES) / 4096;
                    st1.cap_pages = ring_pages < 40 ? ring_pages : 40;
                    st1.abort_flag = abort_flag;
                    bool ok1 = true;
                    if (pos / PAGE + 1 <= st1.cap_pages) {
                        st1.parity = att_uses & 1u;
                        att_uses++;
                        ok1 = dec_attn_staged_body<512>(in, a.cos_t, a.sin_t, ly.a_s, ly.kv, a.page_table, a.max_pages, a.HQ, a.HKV, a.cs, a.att,
                                                        cta % a.HKV, b, pos, dsm1, sm1, st1, tid, MG_BAR_WORK);
                    } else if (ATT == 0) {
                        dec_attn_fused_body<2, 512>(in, a.cos_t, a.sin_t, ly.a_s, ly.kv, a.page_table, a.max_pages, a.ctx, a.HQ, a.HKV, a.cs,
                                                    a.att, nullptr, cta % a.HKV, b, dsm1, sm1, tid, MG_BAR_WORK);
                    } else if (tid == 0) {
                        atomicOr(a.error_flag, 2);
                    }
                    if (ok1) {
                        named_sync<MG_BAR_WORK, MG_WORKERS>();
                        if (tid < 256) mega_att_row_quant(a, b, sm1, tid, MG_BAR_HALF0);
                    }
                }
            } else if (ATT != 2) {
                // items spread over the CTAs first (item i on CTA i mod G)
                for (int idx = cta + half * G; idx < a.B * a.HKV; idx += 2 * G) {
                    const int b = idx / a.HKV;
                    const int pos = dec_guarded_pos(a.ctx, b, a.max_ctx, a.error_flag);
                    if (pos / PAGE + 1 <= stg.cap_pages) {
                        stg.parity = att_uses & 1u;
                        att_uses++;
                        if (!dec_attn_staged_body<256>(in, a.cos_t, a.sin_t, ly.a_s, ly.kv, a.page_table, a.max_pages, a.HQ, a.HKV, a.cs, a.att,
                                                       idx % a.HKV, b, pos, dsm, sm, stg, tid & 255, MG_BAR_HALF0 + half))
                            break;
                    } else if (ATT == 0) {     // contexts beyond the staging area: per-thread global loads
                        dec_attn_fused_body<2, 256>(in, a.cos_t, a.sin_t, ly.a_s, ly.kv, a.page_table, a.max_pages, a.ctx, a.HQ, a.HKV, a.cs,
                                                    a.att, nullptr, idx % a.HKV, b, dsm, sm, tid & 255, MG_BAR_HALF0 + half);
                    } else if ((tid & 255) == 0) {
                        atomicOr(a.error_flag, 2);
                    }
                    // the item that completes its sequence's attention row (the last of its HKV items to arrive)
                    // quantises the row for the o projection -- no separate phase, no extra grid barrier
                    mega_att_row_quant(a, b, sm, tid & 255, MG_BAR_HALF0 + half);
                }
            }
            // both halves are done with the ring (each thread has fenced its accesses): the o projection's weights may come in
            named_sync<MG_BAR_WORK, MG_WORKERS>();
            if (is_tma && !*abort_flag) prefetch_weights(mega_job(a, l, 1));
        } else if (k == PH_D) {
            // CTAs per row: four when the grid has them (always so for up to 32 sequences: the host refuses smaller grids,
            // and the one-CTA-per-row code is then not even compiled in), else one
            const int parts = (BN <= 32 || 4 * a.B <= G) ? 4 : 1;
            if (cta < parts * a.B) {
                if (BN <= 32 || parts == 4) mega_row_fht4(a, ly, cta >> 2, cta & 3, rowbuf, rowred, tid, abort_flag);
                else mega_row_fht(a, ly, cta, rowbuf, rowred, tid);
            }
        } else if (k == PH_TOKEN) {
            if (cta < a.B) {
                if (a.sample_k > 0) mega_row_sample(a, cta, col, n_cols, *reinterpret_cast<SampleSmem*>(scratch));
                else mega_row_argmax(a, cta, col, n_cols, arg_v, arg_i);
            }
            if (cta == 0 && tid == 0) a.state[0] = col + 1;
        } else {
            const int kind = k == PH_QKV ? 0 : k == PH_O ? 1 : k == PH_GU ? 2 : k == PH_DOWN ? 3 : 4;
            if (kind == 3 && cta == G - 1 && tid < 3 * a.slab_rows) a.fht_flags[tid] = 0;   // idle until the next FHT phase
            const MegaJob j = mega_job(a, l, kind);
            const MegaJob nj = kind < 3 ? mega_job(a, l, kind + 1) : (p + 1 < MG_PHASES_PER_LAYER * L ? mega_job(a, l + 1, 0) : mega_job(a, 0, 4));
            gemm_phase(j, (kind == 4 || kind == 0) ? nullptr : &nj);      // after q|k|v comes the attention phase, which uses the ring itself
        }
        if (p + 1 < n_phases) {
            if (!mega_grid_sync(a.sync_ctr, target_of(p) + (p == 0 ? (unsigned long long)a.test_barrier_extra : 0ull), abort_flag, go_flag,
                                a.error_flag, a.trace ? a.trace + (size_t)p * 2 * G : nullptr, a.wait_limit_ns))
                break;
        }
    }

    // ---------------------------------------------------------------- tear-down
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // a wait ran out: give copies still in flight time to land before shared memory is released
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
        if (tid == 0) atomicOr(a.error_flag, 1);
        __syncthreads();
    }
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

}  // namespace flexllm

// ------------------------------------------------------------------------------------------ host
#include "decode_mega.h"


namespace flexllm {

int* device_error_flag();
int gemm_sm_count();

struct MegaPlan {
    MegaArgs args;
    void* dev_maps = nullptr; void* dev_layers = nullptr; void* dev_work = nullptr; void* dev_ctr = nullptr; void* dev_trace = nullptr;
    void* dev_fht_x = nullptr; void* dev_fht_flags = nullptr; int n_flags = 0;
    size_t trace_bytes = 0;
    size_t work_bytes = 0;
    int grid = 0, bn = 0;
    size_t smem = 0;
    int cap_pair = 0, cap_single = 0;       // pages of KV the staging areas of the two attention item layouts hold
};

void mega_destroy(MegaPlan* p) {
    if (!p) return;
    // FLEXLLM_MEGA_TRACE=<file>: the phase timeline of the last step, raw u64 [barrier][arrive, leave][CTA]
    const char* tf = getenv("FLEXLLM_MEGA_TRACE");
    if (tf && p->dev_trace) {
        std::vector<unsigned long long> h(p->trace_bytes / 8);
        if (cudaMemcpy(h.data(), p->dev_trace, p->trace_bytes, cudaMemcpyDeviceToHost) == cudaSuccess) {
            if (FILE* f = fopen(tf, "wb")) { fwrite(h.data(), 1, p->trace_bytes, f); fclose(f); }
        }
    }
    cudaFree(p->dev_trace);
    cudaFree(p->dev_maps); cudaFree(p->dev_layers); cudaFree(p->dev_work); cudaFree(p->dev_ctr);
    cudaFree(p->dev_fht_x); cudaFree(p->dev_fht_flags);
    delete p;
}

int mega_create(const MegaModelView& v, MegaPlan** out) {
    *out = nullptr;
    const char* env = getenv("FLEXLLM_MEGA");
    if (env && atoi(env) == 0) return FLEXLLM_ENOTSUP;
    const int QKV = (v.HQ + 2 * v.HKV) * 64;
    if (v.D % 128 || v.D > 2048 || v.F != 8192 || v.HQ != 4 * v.HKV || v.HQ * 64 != v.D || v.max_batch > 64) return FLEXLLM_ENOTSUP;
    int dev = 0, coop = 0, optin = 0;
    FLEXLLM_CHECK_CUDA(cudaGetDevice(&dev));
    FLEXLLM_CHECK_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    FLEXLLM_CHECK_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    if (!coop) return FLEXLLM_ENOTSUP;
    const int G = gemm_sm_count();
    if (v.max_batch > G) return FLEXLLM_ENOTSUP;
    const int bn = v.max_batch <= 32 ? 32 : 64;
    if (bn == 32 && G < 4 * 32) return FLEXLLM_ENOTSUP;     // the 32-sequence kernel always splits an FFN row over four CTAs
    const void* kerns[3];
    if (bn == 32) { kerns[0] = (const void*)decode_mega_kernel<32, 0>; kerns[1] = (const void*)decode_mega_kernel<32, 1>; kerns[2] = (const void*)decode_mega_kernel<32, 2>; }
    else { kerns[0] = (const void*)decode_mega_kernel<64, 0>; kerns[1] = (const void*)decode_mega_kernel<64, 1>; kerns[2] = (const void*)decode_mega_kernel<64, 2>; }
    const void* kern = kerns[0];
    cudaFuncAttributes fa;
    FLEXLLM_CHECK_CUDA(cudaFuncGetAttributes(&fa, kern));
    const int stage_bytes = MG_A_TILE + bn * 128;
    const int cs = (v.max_ctx + 1 + 63) / 64 * 64;
    int attn_bytes = (20 * cs < 4096 ? 4096 : 20 * cs) + (int)sizeof(DecAttnSmem);
    attn_bytes = (attn_bytes + 127) / 128 * 128;
    int scratch = MG_FHT_SCRATCH;
    if (2 * attn_bytes > scratch) scratch = 2 * attn_bytes;
    scratch = (scratch + 127) / 128 * 128;
    const long avail = (long)optin - (long)fa.sharedSizeBytes - 1024 - 256 - scratch;
    int stages = (int)(avail / stage_bytes);
    if (stages > MG_MAX_STAGES) stages = MG_MAX_STAGES;
    if (stages < 3) return FLEXLLM_ENOTSUP;      // long contexts: the per-operator kernels take over
    const size_t smem = 1024 + (size_t)stages * stage_bytes + scratch + 256;
    for (int i = 0; i < 3; i++) {
        FLEXLLM_CHECK_CUDA(cudaFuncSetAttribute(kerns[i], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        int per_sm = 0;
        FLEXLLM_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kerns[i], MG_THREADS, smem));
        if (per_sm < 1) return FLEXLLM_ENOTSUP;
    }

    MegaPlan* p = new (std::nothrow) MegaPlan();
    if (!p) return FLEXLLM_ENOMEM;
    p->grid = G; p->bn = bn; p->smem = smem;
    {
        const int ring = stages * stage_bytes, half = (ring >> 1) & ~127;
        p->cap_pair = half / 4096 < 20 ? half / 4096 : 20;
        p->cap_single = ring / 4096 < 40 ? ring / 4096 : 40;
    }
    const int n_maps = 2 + 4 * v.layers + 1;
    std::vector<CUtensorMap> maps(n_maps);
    std::vector<MegaLayer> layers(v.layers);
    int rc = make_tmap_2d_u8(&maps[0], v.xq, (uint64_t)v.max_batch, (uint64_t)v.D, bn);
    if (rc == FLEXLLM_OK) rc = make_tmap_2d_u8(&maps[1], v.hq, (uint64_t)v.max_batch, (uint64_t)v.F, bn);
    for (int l = 0; rc == FLEXLLM_OK && l < v.layers; l++) {
        const MegaLayerView& s = v.L[l];
        rc = make_tmap_2d_u8(&maps[2 + 4 * l + 0], s.wqkv, (uint64_t)QKV, (uint64_t)v.D, 128);
        if (rc == FLEXLLM_OK) rc = make_tmap_2d_u8(&maps[2 + 4 * l + 1], s.wo, (uint64_t)v.D, (uint64_t)v.D, 128);
        if (rc == FLEXLLM_OK) rc = make_tmap_2d_u8(&maps[2 + 4 * l + 2], s.wgu, (uint64_t)2 * v.F, (uint64_t)v.D, 128);
        if (rc == FLEXLLM_OK) rc = make_tmap_2d_u8(&maps[2 + 4 * l + 3], s.wd, (uint64_t)v.D, (uint64_t)v.F, 128);
        MegaLayer& d = layers[l];
        d.sqkv = s.sqkv; d.so = s.so; d.sgu = s.sgu; d.sd = s.sd; d.g0 = s.g0; d.g1 = s.g1; d.a_s = s.a_s;
        d.kv.k = v.cache->k + (size_t)l * v.cache->page_bytes;
        d.kv.v = v.cache->v + (size_t)l * v.cache->page_bytes;
        d.kv.ks = v.cache->ks + (size_t)l * (v.cache->scale_bytes / 4);
        d.kv.vs = v.cache->vs + (size_t)l * (v.cache->scale_bytes / 4);
    }
    if (rc == FLEXLLM_OK) rc = make_tmap_2d_u8(&maps[2 + 4 * v.layers], v.lm_w, (uint64_t)v.V, (uint64_t)v.D, 128);
    if (rc != FLEXLLM_OK) { mega_destroy(p); return rc; }

    auto split = [&](int tiles, int num_kb) { int k = G / tiles; if (k < 1) k = 1; if (k > num_kb) k = num_kb; if (k > MG_MAX_KS) k = MG_MAX_KS; return k; };
    const int ks_qkv = split((QKV + 127) / 128, v.D / 128), ks_o = split(v.D / 128, v.D / 128), ks_d = split(v.D / 128, v.F / 128);
    // split-K partial sums: one slab [max_batch][N] per split, written with plain stores and summed by the reader
    const size_t n_qkv = (size_t)ks_qkv * v.max_batch * QKV, n_o = (size_t)ks_o * v.max_batch * v.D, n_d = (size_t)ks_d * v.max_batch * v.D,
                 n_gu = (size_t)v.max_batch * 2 * v.F;
    p->work_bytes = (n_qkv + n_o + n_d + n_gu) * sizeof(int32_t);
    cudaError_t e = cudaMalloc(&p->dev_maps, n_maps * sizeof(CUtensorMap));
    if (e == cudaSuccess) e = cudaMalloc(&p->dev_layers, v.layers * sizeof(MegaLayer));
    if (e == cudaSuccess) e = cudaMalloc(&p->dev_work, p->work_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&p->dev_ctr, 256);
    if (e == cudaSuccess) e = cudaMemcpy(p->dev_maps, maps.data(), n_maps * sizeof(CUtensorMap), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(p->dev_layers, layers.data(), v.layers * sizeof(MegaLayer), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(p->dev_work, 0, p->work_bytes);
    if (e == cudaSuccess) e = cudaMemset(p->dev_ctr, 0, 256);
    p->n_flags = 4 * v.max_batch;
    if (e == cudaSuccess) e = cudaMalloc(&p->dev_fht_x, (size_t)v.max_batch * v.F * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&p->dev_fht_flags, p->n_flags * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(p->dev_fht_flags, 0, p->n_flags * sizeof(int));
    if (e == cudaSuccess && getenv("FLEXLLM_MEGA_TRACE")) {
        p->trace_bytes = (size_t)(MG_PHASES_PER_LAYER * v.layers + 2) * 2 * G * sizeof(unsigned long long);
        e = cudaMalloc(&p->dev_trace, p->trace_bytes);
        if (e == cudaSuccess) e = cudaMemset(p->dev_trace, 0, p->trace_bytes);
    }
    if (e != cudaSuccess) {
        mega_destroy(p);
        g_last_cuda_error = (int)e;
        return e == cudaErrorMemoryAllocation ? FLEXLLM_ENOMEM : FLEXLLM_ECUDA;
    }
    MegaArgs& a = p->args;
    a.maps = (const CUtensorMap*)p->dev_maps; a.layers = (const MegaLayer*)p->dev_layers;
    a.n_layers = v.layers; a.B = 0; a.D = v.D; a.HQ = v.HQ; a.HKV = v.HKV; a.F = v.F; a.V = v.V;
    a.eps = v.eps; a.fht_scale = v.fht_scale;
    a.x = v.x; a.xq = v.xq; a.xs = v.xs; a.hq = v.hq; a.att = v.att; a.logits = v.logits;
    a.w_qkv = (int32_t*)p->dev_work; a.w_o = a.w_qkv + n_qkv; a.w_d = a.w_o + n_o; a.w_gu = a.w_d + n_d;
    a.lm_w = v.lm_w; a.lm_s = v.lm_s; a.g_final = v.g_final; a.cos_t = v.cos_t; a.sin_t = v.sin_t;
    a.page_table = v.page_table; a.max_pages = v.max_pages;
    a.ctx = v.ctx; a.next = v.next; a.out_tokens = v.out_tokens; a.state = v.state;
    a.sync_ctr = (unsigned long long*)p->dev_ctr; a.error_flag = device_error_flag();
    a.fht_x = (float*)p->dev_fht_x; a.fht_flags = (int*)p->dev_fht_flags; a.att_cnt = a.fht_flags + 3 * v.max_batch;
    a.trace = (unsigned long long*)p->dev_trace;
    a.sample_lanes = 0; a.sample_k = 0; a.sample_rnd = nullptr;
    a.stages = stages; a.cs = cs; a.scratch_bytes = scratch; a.attn_bytes = attn_bytes; a.max_ctx = v.max_ctx;
    a.ks_qkv = ks_qkv; a.ks_o = ks_o; a.ks_d = ks_d; a.slab_rows = v.max_batch;
    if (!a.error_flag) { mega_destroy(p); return FLEXLLM_ECUDA; }
    *out = p;
    return FLEXLLM_OK;
}

void mega_set_sampling(MegaPlan* p, int lanes, int top_k, const float* rnd) {
    p->args.sample_lanes = lanes; p->args.sample_k = top_k; p->args.sample_rnd = rnd;
}

int mega_reset(MegaPlan* p, cudaStream_t st) {
    FLEXLLM_CHECK_CUDA(cudaMemsetAsync(p->dev_ctr, 0, 256, st));
    FLEXLLM_CHECK_CUDA(cudaMemsetAsync(p->dev_fht_flags, 0, p->n_flags * sizeof(int), st));
    return FLEXLLM_OK;
}

// Test aids (flexllm_debug_hook): a shorter bound for the kernel's grid-barrier and flag waits, and a one-shot
// request that the next launch's first grid barrier wait for more arrivals than the grid delivers, so that the
// bounded wait runs out, every CTA leaves through the tear-down and the error word is raised.
static std::atomic<long long> g_hook_wait_limit_ns{0};
static std::atomic<int> g_hook_barrier_extra{0};

// The leanest kernel variant that covers a launch of B sequences whose positions stay <= max_pos.
int mega_variant(const MegaPlan* p, int B, int max_pos) {
    const int pages = max_pos / PAGE + 1;
    if (B * p->args.HKV <= p->grid) return pages <= p->cap_single ? 2 : 0;
    return pages <= p->cap_pair ? 1 : 0;
}

int mega_launch(MegaPlan* p, int B, int variant, cudaStream_t st) {
    if (B < 1 || B > p->bn || variant < 0 || variant > 2) return FLEXLLM_EINVAL;
    if (variant == 2 && B * p->args.HKV > p->grid) return FLEXLLM_EINVAL;
    if (variant == 1 && B * p->args.HKV <= p->grid) return FLEXLLM_EINVAL;
    p->args.B = B;
    const long long lim = g_hook_wait_limit_ns.load();
    p->args.wait_limit_ns = lim > 0 ? (unsigned long long)lim : kWaitLimitNs;
    p->args.test_barrier_extra = g_hook_barrier_extra.exchange(0);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p->grid); cfg.blockDim = dim3(MG_THREADS); cfg.dynamicSmemBytes = p->smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;     // all CTAs co-resident: the grid barrier cannot starve
    at[0].val.cooperative = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    if (p->bn == 32) {
        if (variant == 0) cudaLaunchKernelEx(&cfg, decode_mega_kernel<32, 0>, p->args);
        else if (variant == 1) cudaLaunchKernelEx(&cfg, decode_mega_kernel<32, 1>, p->args);
        else cudaLaunchKernelEx(&cfg, decode_mega_kernel<32, 2>, p->args);
    } else {
        if (variant == 0) cudaLaunchKernelEx(&cfg, decode_mega_kernel<64, 0>, p->args);
        else if (variant == 1) cudaLaunchKernelEx(&cfg, decode_mega_kernel<64, 1>, p->args);
        else cudaLaunchKernelEx(&cfg, decode_mega_kernel<64, 2>, p->args);
    }
    return launch_status();
}

}  // namespace flexllm

#ifdef FLEXLLM_ATT_TRACE
// development builds only: the time stamps of the traced attention item (see attention_decode.cuh)
extern "C" __attribute__((visibility("default"))) int flexllm_att_trace(unsigned long long* out32) {
    return flexllm::cuda_status(cudaMemcpyFromSymbol(out32, flexllm::g_att_ts, 32 * sizeof(unsigned long long)));
}
#endif

// See include/flexllm_b200.h.
extern "C" int flexllm_debug_hook(int which, long long value) {
    switch (which) {
        case 0: flexllm::g_hook_wait_limit_ns.store(value > 0 ? value : 0); return FLEXLLM_OK;
        case 1: flexllm::g_hook_barrier_extra.store(value > 0 ? 1 : 0); return FLEXLLM_OK;
        default: return FLEXLLM_EINVAL;
    }
}
