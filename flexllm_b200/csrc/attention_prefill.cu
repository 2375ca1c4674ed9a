// Prefill GQA attention, int8 x int8, on tcgen05 tensor cores.
//
// Semantics (bit-for-bit the composition the CPU oracle states; reference operators:
// Modules/MHA.h:189-243 Q.K^T, :246-273 mask, Modules/Softmax.h:25-161, Modules/quant.h:252-295
// unsigned static quant of P, Modules/MHA.h:339-389 P.V, Modules/quant.h:297-326 dequant):
//
//   S[q][k]  = sum_d Q[q][d] K[k][d]                       s8 x s8 -> s32   (tensor cores)
//   x[q][k]  = (((float)S * qs[q]) * ks[k]) * 0.125         k <= q only
//   P        = softmax(x): max, e = exp(x - max), four interleaved partial sums over k mod 4 in
//              increasing k, (p0+p1)+(p2+p3), r = 1/total, P = e * r
//   U[q][k]  = min(round((P * vs[k]) / a_s), 255)           u8
//   O[q][d]  = sum_k U[q][k] V[k][d]                        u8 x s8 -> s32   (tensor cores)
//   out      = (float)O * a_s
//
// The reference quantises the FINAL normalised P and accumulates a whole row of P.V in one int32,
// so a rescaling online softmax cannot reproduce it. The kernel therefore sweeps the keys three
// times instead of materialising S x S scores in one pass:
//   sweep 0: Q.K^T tile -> row max
//   sweep 1: Q.K^T tile again -> e = exp(x - max), ordered partial sums; e is parked in a global
//            scratch (128 x 64 fp32 per tile, written and read back by the same thread, L2-resident)
//   sweep 2: e read back -> U (u8, 64-byte-swizzled shared memory) -> O += U.V
// One thread owns one query row (TMEM lane), so every per-row fp32 chain runs in the reference's
// order. One CTA = 128 queries of one (batch, query head) against 64-key tiles; 4 softmax warps +
// TMA warp + MMA warp; TMEM: S (64 columns) + O (64 columns) = 128 columns, so four CTAs share an SM
// and their 16 softmax warps hide each other's latencies.
#include <cstdlib>

#include "attention_decode.cuh"     // layout of the paged KV cache
#include "common.cuh"
#include "tc_common.cuh"

namespace flexllm {
using namespace tc;

// ------------------------------------------------------------------ pre-pass
// Q/K: dequant -> RoPE -> FHT-64/8 -> per-head int8 quant (same arithmetic as qk_prepare_kernel),
// written head-major [B][H][S][64] with scales [B][H][S] so that one head's rows are contiguous.
__global__ void __launch_bounds__(256) attn_qk_prepare_kernel(const int8_t* __restrict__ q, const float* __restrict__ s,
                                                              const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                              int B, int S, int H, int8_t* __restrict__ q_out,
                                                              float* __restrict__ s_out) {
    const long w = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const long total = (long)B * S * H;
    if (w >= total) return;
    const int h = (int)(w % H);
    const long bt = w / H;
    const int t = (int)(bt % S);
    const int b = (int)(bt / S);
    const float sc_in = s[w];
    const float x0 = (float)q[w * 64 + lane] * sc_in;
    const float x1 = (float)q[w * 64 + 32 + lane] * sc_in;
    const float c = cos_t[(long)t * 32 + lane], sn = sin_t[(long)t * 32 + lane];
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
    const long o = ((long)b * H + h) * S + t;
    if (lane == 0) s_out[o] = sc;
    q_out[o * 64 + lane] = quant_s8(a, sc);
    q_out[o * 64 + 32 + lane] = quant_s8(bb, sc);
}

// V [B][S][HKV][64] -> V^T [B][HKV][64][S] (keys contiguous, the K-major operand of P.V) and
// vs [B][S][HKV] -> [B][HKV][S].
__global__ void __launch_bounds__(256) attn_v_transpose_kernel(const int8_t* __restrict__ v, const float* __restrict__ vs,
                                                               int B, int S, int HKV, int8_t* __restrict__ vT,
                                                               float* __restrict__ vsT) {
    __shared__ int8_t tile[64][64 + 4];
    const int s0 = blockIdx.x * 64, h = blockIdx.y, b = blockIdx.z;
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
        const int r = i >> 4, c4 = i & 15;   // r: token in tile, c4: group of 4 dims
        int val = 0;
        if (s0 + r < S) val = *reinterpret_cast<const int*>(v + (((long)b * S + s0 + r) * HKV + h) * 64 + c4 * 4);
        *reinterpret_cast<int*>(&tile[r][c4 * 4]) = val;
    }
    if (threadIdx.x < 64 && s0 + threadIdx.x < S)
        vsT[((long)b * HKV + h) * S + s0 + threadIdx.x] = vs[((long)b * S + s0 + threadIdx.x) * HKV + h];
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        const int d = i >> 6, r = i & 63;
        if (s0 + r < S) vT[(((long)b * HKV + h) * 64 + d) * S + s0 + r] = tile[r][d];
    }
}

// ------------------------------------------------------------------ main kernel
struct AttnArgs {
    int B, HQ, HKV;
    int Sq;             // queries per sequence in this call (positions q_off .. q_off + Sq - 1)
    int q_off;          // position of the first query, a multiple of 128; the keys are positions 0 .. q_off + Sq - 1
    int Sk;             // contiguous K/V: rows per (batch, KV head) of the K, V^T and scale buffers
    const float* qs;    // [B][HQ][Sq]
    const float* ks;    // contiguous: [B][HKV][Sk]; paged: the cache's K scale pool [page][HKV][64]
    const float* vs;    // likewise
    const int32_t* page_table; int max_pages;   // non-null: K / V^T tiles are pages of the KV cache (one 64-key tile = one page)
    const float* a_s;   // [HQ]
    float* out;         // [B][Sq][HQ*64]
    int32_t* oacc;      // optional, same shape
    uint8_t* ecache;    // exp values of sweep 1 kept for sweep 2 (attn_ecache_head_bytes per (batch, head))
    int* error_flag;
};

__device__ __forceinline__ uint64_t umma_desc_k_sw64(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(512 >> 4) << 32;   // 8 rows of 64 bytes
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)4 << 61;            // SWIZZLE_64B
    return d;
}

// Key tile = 64 keys. TMEM per CTA: S (64 columns) + O (64 columns) = 128 columns, so four CTAs share
// an SM (16 softmax warps per SM hide each other's latencies).
constexpr int ATT_KT = 64;                    // keys per tile
constexpr int ATT_SLOTS = 4;                  // K / V^T tile ring
constexpr int ATT_Q_BYTES = 128 * 64;
constexpr int ATT_TILE_BYTES = 64 * 64;       // one K tile [64 keys][64 B] or one V^T tile [64 dims][64 keys]
constexpr int ATT_P_BYTES = 128 * 64;         // U tile [128 queries][64 keys] u8
constexpr int ATT_SMEM = ATT_Q_BYTES + ATT_SLOTS * ATT_TILE_BYTES + 2 * ATT_P_BYTES + 1024 + 256;
constexpr int ATT_TMEM_COLS = 128;

// Bytes of exp-cache one (batch, query head) needs: for every 128-query tile qt = q_off/128 + t (t < n_qt) its
// 2*(qt+1) key tiles of 128 x 64 fp32.
__host__ __device__ inline size_t attn_ecache_head_bytes(int q_off, int Sq) {
    const size_t n_qt = (Sq + 127) / 128, qt0 = q_off / 128;
    return n_qt * (2 * qt0 + n_qt + 1) * (size_t)(128 * ATT_KT * 4);   // sum_{t < n_qt} 2*(qt0+t+1) tiles
}

__global__ void __launch_bounds__(192, 4) attn_prefill_kernel(const __grid_constant__ CUtensorMap tmapQ,
                                                              const __grid_constant__ CUtensorMap tmapK,
                                                              const __grid_constant__ CUtensorMap tmapV,
                                                              const AttnArgs args) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t sQ = base;
    const uint32_t sT = sQ + ATT_Q_BYTES;                         // tile ring
    const uint32_t sP = sT + ATT_SLOTS * ATT_TILE_BYTES;          // two U tiles
    uint8_t* sP_ptr = base_ptr + ATT_Q_BYTES + ATT_SLOTS * ATT_TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP_ptr + 2 * ATT_P_BYTES);
    // barriers: q_full, t_full[4], t_empty[4], s_full, s_empty, p_full[2], p_empty[2], o_full
    const uint32_t bar_qfull = smem_u32(bars);
    const uint32_t bar_tfull = bar_qfull + 8;
    const uint32_t bar_tempty = bar_tfull + 8 * ATT_SLOTS;
    const uint32_t bar_sfull = bar_tempty + 8 * ATT_SLOTS;
    const uint32_t bar_sempty = bar_sfull + 8;
    const uint32_t bar_pfull = bar_sempty + 8;
    const uint32_t bar_pempty = bar_pfull + 16;
    const uint32_t bar_ofull = bar_pempty + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8 + 2 * ATT_SLOTS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = args.q_off + args.Sq;                            // keys (positions 0 .. S-1)
    const int n_qt = (args.Sq + 127) >> 7;
    const int qt_l = n_qt - 1 - (int)(blockIdx.x % n_qt);          // query tile within the call: heavy tiles (late queries) first
    const int qt0 = args.q_off >> 7, qt = qt0 + qt_l;              // ... and within the sequence
    const int hq = (int)((blockIdx.x / n_qt) % args.HQ);
    const int b = (int)(blockIdx.x / ((long)n_qt * args.HQ));
    const int hkv = hq / (args.HQ / args.HKV);
    const int n_kt_all = (S + ATT_KT - 1) / ATT_KT;
    const int n_kt = 2 * (qt + 1) < n_kt_all ? 2 * (qt + 1) : n_kt_all;   // causal: 64-key tiles 0 .. 2*qt+1 (those that hold keys)
    const bool paged = args.page_table != nullptr;
    const int32_t* pt = paged ? args.page_table + (long)b * args.max_pages : nullptr;
    // this CTA's slice of the exp cache: [n_kt][16 float4 chunks][128 rows] float4
    float4* ecache = reinterpret_cast<float4*>(args.ecache + ((size_t)b * args.HQ + hq) * attn_ecache_head_bytes(args.q_off, args.Sq) +
                                               ((size_t)2 * qt_l * qt0 + (size_t)qt_l * (qt_l + 1)) * (size_t)(128 * ATT_KT * 4));

    if (threadIdx.x == 0) {
        mbar_init(bar_qfull, 1);
        for (int i = 0; i < ATT_SLOTS; i++) { mbar_init(bar_tfull + 8 * i, 1); mbar_init(bar_tempty + 8 * i, 1); }
        mbar_init(bar_sfull, 1); mbar_init(bar_sempty, 4);
        for (int i = 0; i < 2; i++) { mbar_init(bar_pfull + 8 * i, 4); mbar_init(bar_pempty + 8 * i, 1); }
        mbar_init(bar_ofull, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 5) { tmem_alloc(smem_u32(tmem_slot), ATT_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 64;

    if (warp == 4) {
        // ------------------------------------------------------------ TMA producer
        // iterations 0 .. 2*n_kt-1: K tiles of sweeps 0 and 1; then n_kt V^T tiles for sweep 2
        if (lane == 0) {
            tma_prefetch_desc(&tmapQ); tma_prefetch_desc(&tmapK); tma_prefetch_desc(&tmapV);
            mbar_expect_tx(bar_qfull, ATT_Q_BYTES);
            tma_load_2d(sQ, &tmapQ, bar_qfull, 0, ((b * args.HQ + hq) * args.Sq) + qt_l * 128);
            int slot = 0; uint32_t phase = 0;
            for (int it = 0; it < 3 * n_kt; it++) {
                const int sweep = it / n_kt, j = it - sweep * n_kt;
                if (!mbar_wait(bar_tempty + 8 * slot, phase ^ 1u, abort_flag)) break;
                const uint32_t full = bar_tfull + 8 * slot;
                const uint32_t dst = sT + slot * ATT_TILE_BYTES;
                mbar_expect_tx(full, ATT_TILE_BYTES);
                if (paged) {        // one tile = one page of the cache: K rows [64 keys][64 B], V^T rows [64 dims][64 keys]
                    const int row = (__ldg(pt + j) * args.HKV + hkv) * 64;
                    tma_load_2d(dst, sweep < 2 ? &tmapK : &tmapV, full, 0, row);
                } else if (sweep < 2) tma_load_2d(dst, &tmapK, full, 0, ((b * args.HKV + hkv) * args.Sk) + j * ATT_KT);
                else tma_load_2d(dst, &tmapV, full, j * ATT_KT, (b * args.HKV + hkv) * 64);
                if (++slot == ATT_SLOTS) { slot = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_i8(128, ATT_KT, 1, 1);
            constexpr uint32_t idesc_pv = umma_idesc_i8(128, 64, 0, 1);   // U unsigned, V signed
            bool ok = mbar_wait(bar_qfull, 0, abort_flag);
            const uint64_t qdesc = umma_desc_k_sw64(sQ);
            int slot = 0; uint32_t tphase = 0;
            for (int it = 0; ok && it < 3 * n_kt; it++) {
                const int sweep = it / n_kt, j = it - sweep * n_kt;
                if (!mbar_wait(bar_tfull + 8 * slot, tphase, abort_flag)) { ok = false; break; }
                const uint32_t sTile = sT + slot * ATT_TILE_BYTES;
                if (sweep < 2) {
                    // S = Q.K^T for this key tile (S is single-buffered: iteration it is its phase)
                    if (!mbar_wait(bar_sempty, (uint32_t)(it & 1) ^ 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t kdesc = umma_desc_k_sw64(sTile);
                    umma_i8(tmem_S, qdesc, kdesc, idesc_qk, 0u);
                    umma_i8(tmem_S, qdesc + 2, kdesc + 2, idesc_qk, 1u);
                    umma_commit(bar_sfull);
                } else {
                    // O += U.V for this key tile once the softmax warps have written U
                    const int pb = j & 1;
                    if (!mbar_wait(bar_pfull + 8 * pb, (uint32_t)((j >> 1) & 1), abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t pdesc = umma_desc_k_sw64(sP + pb * ATT_P_BYTES);
                    const uint64_t vdesc = umma_desc_k_sw64(sTile);
                    umma_i8(tmem_O, pdesc, vdesc, idesc_pv, j > 0 ? 1u : 0u);
                    umma_i8(tmem_O, pdesc + 2, vdesc + 2, idesc_pv, 1u);
                    umma_commit(bar_pempty + 8 * pb);
                }
                umma_commit(bar_tempty + 8 * slot);
                if (++slot == ATT_SLOTS) { slot = 0; tphase ^= 1u; }
            }
            if (ok) umma_commit(bar_ofull);
        }
    } else {
        // ------------------------------------------------------------ softmax warps 0..3
        const int row_in_tile = warp * 32 + lane;
        const int qpos = qt * 128 + row_in_tile;               // position of this thread's query
        const bool q_ok = qpos < S;
        const int qlim = q_ok ? qpos : -1;                     // keys 0..qlim are visible to this row
        const float qscale = q_ok ? args.qs[((long)b * args.HQ + hq) * args.Sq + (qpos - args.q_off)] : 0.0f;
        const float* ksp = args.ks + ((long)b * args.HKV + hkv) * args.Sk;      // contiguous layout
        const float* vsp = args.vs + ((long)b * args.HKV + hkv) * args.Sk;
        const float a_s = args.a_s[hq];
        const DivBy d_as = div_by(a_s);
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        float mx = -1e32f;
        float ps0 = 0.f, ps1 = 0.f, ps2 = 0.f, ps3 = 0.f;
        bool ok = true;
        // ---- sweeps 0 and 1: scores from the tensor core, 16 columns at a time
        for (int it = 0; ok && it < 2 * n_kt; it++) {
            const int sweep = it / n_kt, j = it - sweep * n_kt;
            int got = (lane == 0) ? (mbar_wait(bar_sfull, (uint32_t)(it & 1), abort_flag) ? 1 : 0) : 1;
            got = __shfl_sync(0xffffffffu, got, 0);
            if (!got) { ok = false; break; }
            tc_fence_after();
            const int k0 = j * ATT_KT;
            const float* kst = paged ? args.ks + ((long)__ldg(pt + j) * args.HKV + hkv) * 64 : ksp + k0;   // this tile's key scales
#pragma unroll 1
            for (int c = 0; c < ATT_KT / 16; c++) {
                uint32_t v[16];
                tmem_ld_32x16(tmem_S + lane_addr + c * 16, v);
                const int kc = k0 + c * 16;
                // key scales of these 16 keys (same addresses for the whole warp); keys beyond S are masked
                float ksv[16];
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                    const float4 t = (kc + i < S) ? *reinterpret_cast<const float4*>(kst + c * 16 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                    ksv[i] = t.x; ksv[i + 1] = t.y; ksv[i + 2] = t.z; ksv[i + 3] = t.w;
                }
                tmem_ld_wait();
                if (sweep == 0) {
                    // the row maximum is tracked WITHOUT the factor 0.125 (scaling by a power of two is exact and keeps
                    // the order, so max(x * 0.125) == max(x) * 0.125: applied once after the sweep)
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        float x = ((float)(int)v[i] * qscale) * ksv[i];
                        x = (kc + i <= qlim) ? x : -1e32f;                       // causal mask (MHA.h:262-267)
                        mx = x > mx ? x : mx;
                    }
                } else {
                    float e[16];
#pragma unroll
                    for (int i4 = 0; i4 < 16; i4 += 4) {          // four exponentials at a time (their chains interleave)
                        float xx[4], ee[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const float x = (((float)(int)v[i4 + i] * qscale) * ksv[i4 + i]) * 0.125f;
                            xx[i] = (kc + i4 + i <= qlim) ? x - mx : -1e32f;    // masked: exp(-1e32) is exactly 0
                        }
                        ref_expf_x4<true>(xx, ee);
#pragma unroll
                        for (int i = 0; i < 4; i++) e[i4 + i] = ee[i];
                    }
                    // ordered chains: key mod 4 == i mod 4 because kc is a multiple of 16; adding the
                    // exact zeros of masked keys leaves the sums unchanged, as in the reference
#pragma unroll
                    for (int i = 0; i < 16; i += 4) { ps0 += e[i]; ps1 += e[i + 1]; ps2 += e[i + 2]; ps3 += e[i + 3]; }
                    float4* dst = ecache + ((size_t)(j * 16 + c * 4) * 128 + row_in_tile);
#pragma unroll
                    for (int i = 0; i < 4; i++) dst[(size_t)i * 128] = make_float4(e[4 * i], e[4 * i + 1], e[4 * i + 2], e[4 * i + 3]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sempty);
            if (it == n_kt - 1) mx = mx * 0.125f;             // end of sweep 0: the maximum of the scaled scores
        }
        // ---- sweep 2: U = min(round((e * r * vs) / a_s), 255) from the cached e, into shared memory
        const float rinv = 1.0f / ((ps0 + ps1) + (ps2 + ps3));
        for (int j = 0; ok && j < n_kt; j++) {
            const int pb = j & 1;
            // fetch the first half of this tile's e values before waiting for the buffer
            float4 ev[8];
#pragma unroll
            for (int i = 0; i < 8; i++) ev[i] = ecache[((size_t)(j * 16 + i) * 128 + row_in_tile)];
            int got = (lane == 0) ? (mbar_wait(bar_pempty + 8 * pb, (uint32_t)((j >> 1) & 1) ^ 1u, abort_flag) ? 1 : 0) : 1;
            got = __shfl_sync(0xffffffffu, got, 0);
            if (!got) { ok = false; break; }
            const int k0 = j * ATT_KT;
            const float* vst = paged ? args.vs + ((long)__ldg(pt + j) * args.HKV + hkv) * 64 : vsp + k0;   // this tile's value scales
            uint8_t* prow = sP_ptr + pb * ATT_P_BYTES + row_in_tile * 64;
#pragma unroll
            for (int c = 0; c < 4; c++) {          // 16 keys = one 16-byte chunk of the U row
                if (c == 2) {
#pragma unroll
                    for (int i = 0; i < 8; i++) ev[i] = ecache[((size_t)(j * 16 + 8 + i) * 128 + row_in_tile)];
                }
                uint32_t packed[4];
#pragma unroll
                for (int i4 = 0; i4 < 4; i4++) {
                    const int kk = k0 + c * 16 + i4 * 4;
                    const float4 vs4 = (kk < S) ? *reinterpret_cast<const float4*>(vst + c * 16 + i4 * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                    const float4 e4 = ev[(c & 1) * 4 + i4];
                    const float ee[4] = {e4.x, e4.y, e4.z, e4.w};
                    const float vv[4] = {vs4.x, vs4.y, vs4.z, vs4.w};
                    uint32_t w = 0;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float p = ee[i] * rinv;
                        int r = round_half_away_to_int(div_for_rounding(p * vv[i], d_as));
                        r = r > 255 ? 255 : r;
                        w |= ((uint32_t)r & 0xffu) << (8 * i);
                    }
                    packed[i4] = w;
                }
                // 64-byte rows with 64-byte swizzle: chunk index XOR ((row >> 1) & 3)
                const int chunk = c ^ ((row_in_tile >> 1) & 3);
                *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
            fence_proxy_async_smem();   // make the U tile visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_pfull + 8 * pb);
        }
        // ---- epilogue: O -> out
        if (ok) {
            int got = (lane == 0) ? (mbar_wait(bar_ofull, 0, abort_flag) ? 1 : 0) : 1;
            got = __shfl_sync(0xffffffffu, got, 0);
            if (got) {
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < 4; c++) {
                    uint32_t v[16];
                    tmem_ld_32x16(tmem_O + lane_addr + c * 16, v);
                    tmem_ld_wait();
                    if (q_ok) {
                        const long o = (((long)b * args.Sq + (qpos - args.q_off)) * args.HQ + hq) * 64 + c * 16;
#pragma unroll
                        for (int i = 0; i < 16; i += 4) {
                            float4 r;
                            r.x = (float)(int)v[i] * a_s; r.y = (float)(int)v[i + 1] * a_s;
                            r.z = (float)(int)v[i + 2] * a_s; r.w = (float)(int)v[i + 3] * a_s;
                            *reinterpret_cast<float4*>(args.out + o + i) = r;
                            if (args.oacc)
                                *reinterpret_cast<int4*>(args.oacc + o + i) = make_int4((int)v[i], (int)v[i + 1], (int)v[i + 2], (int)v[i + 3]);
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
        if (threadIdx.x == 0 && args.error_flag) atomicOr(args.error_flag, 1);
        __syncthreads();
    }
    if (warp == 5) { tc_fence_after(); tmem_dealloc(tmem_base, ATT_TMEM_COLS); }
}


// ------------------------------------------------------------------ single-sweep variant (not bit-exact)
// The same attention with a flash-style online softmax: ONE sweep over the key tiles, a running row maximum and
// denominator, fast exponentials (ex2.approx), P quantised per key tile to u8 against that tile's largest value scale,
// P.V on the tensor core per tile, and the running output rescaled in fp32 registers. It does NOT reproduce the
// reference's arithmetic (which quantises the final normalised P against a static scale and accumulates a whole row in
// int32): it exists to measure what that exactness costs, is off by default, and is checked to fp32 tolerance only.
//   per tile j:  x = S * (qs * 0.125 * log2 e) * ks[k];  m' = max(m, max_k x);  alpha = 2^(m - m')
//                c_j = 255 / max_k vs[k];  pc = 2^(x - m') * c_j;  U = rint(pc * vs[k]) (<= 255);  l = l * alpha + sum(pc) / c_j
//                O_j = U . V (tensor core, int32);  o = o * alpha + O_j / c_j
//   out = o / l
// TMEM: S and O double-buffered (4 x 64 columns): the MMA warp runs one key tile ahead of the softmax warps.
constexpr int ATO_TMEM_COLS = 256;
constexpr int ATO_SLOTS = 6;
constexpr int ATO_SMEM = ATT_Q_BYTES + ATO_SLOTS * ATT_TILE_BYTES + 2 * ATT_P_BYTES + 1024 + 256;

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(192, 2) attn_prefill_online_kernel(const __grid_constant__ CUtensorMap tmapQ,
                                                                     const __grid_constant__ CUtensorMap tmapK,
                                                                     const __grid_constant__ CUtensorMap tmapV,
                                                                     const AttnArgs args) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t sQ = base;
    const uint32_t sT = sQ + ATT_Q_BYTES;
    const uint32_t sP = sT + ATO_SLOTS * ATT_TILE_BYTES;
    uint8_t* sP_ptr = base_ptr + ATT_Q_BYTES + ATO_SLOTS * ATT_TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP_ptr + 2 * ATT_P_BYTES);
    // barriers: q_full, t_full[6], t_empty[6], s_full[2], s_empty[2], p_full[2], p_empty[2], o_full[2], o_empty[2]
    const uint32_t bar_qfull = smem_u32(bars);
    const uint32_t bar_tfull = bar_qfull + 8;
    const uint32_t bar_tempty = bar_tfull + 8 * ATO_SLOTS;
    const uint32_t bar_sfull = bar_tempty + 8 * ATO_SLOTS;
    const uint32_t bar_sempty = bar_sfull + 16;
    const uint32_t bar_pfull = bar_sempty + 16;
    const uint32_t bar_pempty = bar_pfull + 16;
    const uint32_t bar_ofull = bar_pempty + 16;
    const uint32_t bar_oempty = bar_ofull + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1 + 2 * ATO_SLOTS + 12);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = args.q_off + args.Sq;
    const int n_qt = (args.Sq + 127) >> 7;
    const int qt_l = n_qt - 1 - (int)(blockIdx.x % n_qt);
    const int qt0 = args.q_off >> 7, qt = qt0 + qt_l;
    const int hq = (int)((blockIdx.x / n_qt) % args.HQ);
    const int b = (int)(blockIdx.x / ((long)n_qt * args.HQ));
    const int hkv = hq / (args.HQ / args.HKV);
    const int n_kt_all = (S + ATT_KT - 1) / ATT_KT;
    const int n_kt = 2 * (qt + 1) < n_kt_all ? 2 * (qt + 1) : n_kt_all;
    const bool paged = args.page_table != nullptr;
    const int32_t* pt = paged ? args.page_table + (long)b * args.max_pages : nullptr;

    if (threadIdx.x == 0) {
        mbar_init(bar_qfull, 1);
        for (int i = 0; i < ATO_SLOTS; i++) { mbar_init(bar_tfull + 8 * i, 1); mbar_init(bar_tempty + 8 * i, 1); }
        for (int i = 0; i < 2; i++) {
            mbar_init(bar_sfull + 8 * i, 1); mbar_init(bar_sempty + 8 * i, 4);
            mbar_init(bar_pfull + 8 * i, 4); mbar_init(bar_pempty + 8 * i, 1);
            mbar_init(bar_ofull + 8 * i, 1); mbar_init(bar_oempty + 8 * i, 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 5) { tmem_alloc(smem_u32(tmem_slot), ATO_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 4) {
        // ------------------------------------------------------------ TMA producer: K_0, then K_{j+1}, V_j for every tile j
        if (lane == 0) {
            tma_prefetch_desc(&tmapQ); tma_prefetch_desc(&tmapK); tma_prefetch_desc(&tmapV);
            mbar_expect_tx(bar_qfull, ATT_Q_BYTES);
            tma_load_2d(sQ, &tmapQ, bar_qfull, 0, ((b * args.HQ + hq) * args.Sq) + qt_l * 128);
            int slot = 0; uint32_t phase = 0;
            auto load = [&](bool is_k, int j) {
                if (!mbar_wait(bar_tempty + 8 * slot, phase ^ 1u, abort_flag)) return false;
                const uint32_t full = bar_tfull + 8 * slot;
                const uint32_t dst = sT + slot * ATT_TILE_BYTES;
                mbar_expect_tx(full, ATT_TILE_BYTES);
                if (paged) tma_load_2d(dst, is_k ? &tmapK : &tmapV, full, 0, (__ldg(pt + j) * args.HKV + hkv) * 64);
                else if (is_k) tma_load_2d(dst, &tmapK, full, 0, ((b * args.HKV + hkv) * args.Sk) + j * ATT_KT);
                else tma_load_2d(dst, &tmapV, full, j * ATT_KT, (b * args.HKV + hkv) * 64);
                if (++slot == ATO_SLOTS) { slot = 0; phase ^= 1u; }
                return true;
            };
            bool ok = load(true, 0);
            for (int j = 0; ok && j < n_kt; j++) {
                if (j + 1 < n_kt) ok = load(true, j + 1);
                if (ok) ok = load(false, j);
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer: Q.K^T one tile ahead of U.V
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_i8(128, ATT_KT, 1, 1);
            constexpr uint32_t idesc_pv = umma_idesc_i8(128, 64, 0, 1);
            bool ok = mbar_wait(bar_qfull, 0, abort_flag);
            const uint64_t qdesc = umma_desc_k_sw64(sQ);
            int slot = 0; uint32_t tphase = 0;
            auto next_tile = [&](uint32_t& sTile) {       // waits for the next ring slot in load order
                if (!mbar_wait(bar_tfull + 8 * slot, tphase, abort_flag)) return false;
                sTile = sT + slot * ATT_TILE_BYTES;
                return true;
            };
            auto release_tile = [&]() {
                umma_commit(bar_tempty + 8 * slot);
                if (++slot == ATO_SLOTS) { slot = 0; tphase ^= 1u; }
            };
            auto issue_qk = [&](int j) {
                uint32_t sTile;
                const int sb = j & 1;
                if (!next_tile(sTile)) return false;
                if (!mbar_wait(bar_sempty + 8 * sb, (uint32_t)((j >> 1) & 1) ^ 1u, abort_flag)) return false;
                tc_fence_after();
                const uint64_t kdesc = umma_desc_k_sw64(sTile);
                umma_i8(tmem_base + sb * 64, qdesc, kdesc, idesc_qk, 0u);
                umma_i8(tmem_base + sb * 64, qdesc + 2, kdesc + 2, idesc_qk, 1u);
                umma_commit(bar_sfull + 8 * sb);
                release_tile();
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; ok && j < n_kt; j++) {
                if (j + 1 < n_kt && !issue_qk(j + 1)) { ok = false; break; }
                const int pb = j & 1;
                uint32_t sTile;
                if (!next_tile(sTile)) { ok = false; break; }
                if (!mbar_wait(bar_pfull + 8 * pb, (uint32_t)((j >> 1) & 1), abort_flag)) { ok = false; break; }
                if (!mbar_wait(bar_oempty + 8 * pb, (uint32_t)((j >> 1) & 1) ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint64_t pdesc = umma_desc_k_sw64(sP + pb * ATT_P_BYTES);
                const uint64_t vdesc = umma_desc_k_sw64(sTile);
                umma_i8(tmem_base + 128 + pb * 64, pdesc, vdesc, idesc_pv, 0u);
                umma_i8(tmem_base + 128 + pb * 64, pdesc + 2, vdesc + 2, idesc_pv, 1u);
                umma_commit(bar_ofull + 8 * pb);
                umma_commit(bar_pempty + 8 * pb);
                release_tile();
            }
        }
    } else {
        // ------------------------------------------------------------ softmax warps 0..3: one query row per thread
        const int row_in_tile = warp * 32 + lane;
        const int qpos = qt * 128 + row_in_tile;
        const bool q_ok = qpos < S;
        const int qlim = q_ok ? qpos : -1;
        const float qsl = q_ok ? args.qs[((long)b * args.HQ + hq) * args.Sq + (qpos - args.q_off)] * (0.125f * 1.4426950408889634f) : 0.0f;
        const float* ksp = args.ks + ((long)b * args.HKV + hkv) * args.Sk;
        const float* vsp = args.vs + ((long)b * args.HKV + hkv) * args.Sk;
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        float m = -1e30f, l = 0.0f;
        float o[64];
#pragma unroll
        for (int i = 0; i < 64; i++) o[i] = 0.0f;
        float alpha_prev = 1.0f, f_prev = 0.0f;
        bool ok = true;
        auto wait_bar = [&](uint32_t bar, uint32_t parity) {
            int got = (lane == 0) ? (mbar_wait(bar, parity, abort_flag) ? 1 : 0) : 1;
            return __shfl_sync(0xffffffffu, got, 0) != 0;
        };
        auto fold_o = [&](int jj) {        // o = o * alpha + O_jj * f, O_jj from its TMEM buffer
            const int ob = jj & 1;
            if (!wait_bar(bar_ofull + 8 * ob, (uint32_t)((jj >> 1) & 1))) return false;
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t v[16];
                tmem_ld_32x16(tmem_base + 128 + ob * 64 + lane_addr + c * 16, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; i++) o[c * 16 + i] = __fmaf_rn(o[c * 16 + i], alpha_prev, (float)(int)v[i] * f_prev);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_oempty + 8 * ob);
            return true;
        };
        for (int j = 0; ok && j < n_kt; j++) {
            const int sb = j & 1;
            const int k0 = j * ATT_KT;
            const float* kst = paged ? args.ks + ((long)__ldg(pt + j) * args.HKV + hkv) * 64 : ksp + k0;
            const float* vst = paged ? args.vs + ((long)__ldg(pt + j) * args.HKV + hkv) * 64 : vsp + k0;
            // this tile's largest value scale (keys beyond the sequence count as 0)
            float vmax = fmaxf(k0 + lane < S ? vst[lane] : 0.0f, k0 + 32 + lane < S ? vst[32 + lane] : 0.0f);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, off));
            vmax = fmaxf(vmax, 1e-30f);
            const float cj = 255.0f / vmax, lcj = lg2_approx(cj), fj = vmax * (1.0f / 255.0f);
            const bool diag = k0 + ATT_KT - 1 > qt * 128;          // tile may hold keys beyond some row's own position
            if (!wait_bar(bar_sfull + 8 * sb, (uint32_t)((j >> 1) & 1))) { ok = false; break; }
            tc_fence_after();
            const uint32_t tS = tmem_base + sb * 64 + lane_addr;
            // pass 1: the tile's row maximum
            float tmax = -1e30f;
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t v[16];
                tmem_ld_32x16(tS + c * 16, v);
                float ksv[16];
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                    const float4 t = (k0 + c * 16 + i < S) ? *reinterpret_cast<const float4*>(kst + c * 16 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                    ksv[i] = t.x; ksv[i + 1] = t.y; ksv[i + 2] = t.z; ksv[i + 3] = t.w;
                }
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    float x = ((float)(int)v[i] * qsl) * ksv[i];
                    if (diag) x = (k0 + c * 16 + i <= qlim) ? x : -1e30f;
                    tmax = fmaxf(tmax, x);
                }
            }
            const float m_new = fmaxf(m, tmax);
            const float alpha = ex2_approx(m - m_new);
            const float mref = m_new - lcj;                        // 2^(x - mref) = 2^(x - m_new) * c_j
            if (!wait_bar(bar_pempty + 8 * sb, (uint32_t)((j >> 1) & 1) ^ 1u)) { ok = false; break; }
            // pass 2: pc, its sum, U into shared memory
            uint8_t* prow = sP_ptr + sb * ATT_P_BYTES + row_in_tile * 64;
            float sum = 0.0f;
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t v[16];
                tmem_ld_32x16(tS + c * 16, v);
                float ksv[16], vsv[16];
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                    const bool in = k0 + c * 16 + i < S;
                    const float4 t = in ? *reinterpret_cast<const float4*>(kst + c * 16 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                    const float4 u = in ? *reinterpret_cast<const float4*>(vst + c * 16 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                    ksv[i] = t.x; ksv[i + 1] = t.y; ksv[i + 2] = t.z; ksv[i + 3] = t.w;
                    vsv[i] = u.x; vsv[i + 1] = u.y; vsv[i + 2] = u.z; vsv[i + 3] = u.w;
                }
                tmem_ld_wait();
                uint32_t packed[4];
#pragma unroll
                for (int i4 = 0; i4 < 4; i4++) {
                    uint32_t w = 0;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int ii = i4 * 4 + i;
                        const float x = ((float)(int)v[ii] * qsl) * ksv[ii];
                        float pc = ex2_approx(x - mref);
                        if (diag) pc = (k0 + c * 16 + ii <= qlim) ? pc : 0.0f;
                        sum += pc;
                        uint32_t r = __float2uint_rn(pc * vsv[ii]);
                        r = r > 255u ? 255u : r;
                        w |= r << (8 * i);
                    }
                    packed[i4] = w;
                }
                const int chunk = c ^ ((row_in_tile >> 1) & 3);
                *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(bar_pfull + 8 * sb); mbar_arrive(bar_sempty + 8 * sb); }
            l = __fmaf_rn(l, alpha, sum * fj);
            m = m_new;
            // the previous tile's U.V has had this tile's softmax to finish: fold it in now
            if (j > 0 && !fold_o(j - 1)) { ok = false; break; }
            alpha_prev = alpha; f_prev = fj;
        }
        if (ok) ok = fold_o(n_kt - 1);
        if (ok && q_ok) {
            const float rl = 1.0f / l;
            const long ob = (((long)b * args.Sq + (qpos - args.q_off)) * args.HQ + hq) * 64;
#pragma unroll
            for (int i = 0; i < 64; i += 4)
                *reinterpret_cast<float4*>(args.out + ob + i) = make_float4(o[i] * rl, o[i + 1] * rl, o[i + 2] * rl, o[i + 3] * rl);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
        if (threadIdx.x == 0 && args.error_flag) atomicOr(args.error_flag, 1);
        __syncthreads();
    }
    if (warp == 5) { tc_fence_after(); tmem_dealloc(tmem_base, ATO_TMEM_COLS); }
}

int* device_error_flag();

// fp32 front end used by the model: qkv [B*Sq][(HQ+2*HKV)*64] fp32 as the fused q/k/v projection writes it, tokens at
// positions q_off .. q_off + Sq - 1. Query heads: RoPE -> FHT-64/8 -> per-head int8, head-major [B][HQ][Sq][64] for the
// attention kernel's Q tiles. Key heads: the same arithmetic, written straight into the KV cache's pages (row = token).
// Value heads: per-head int8 quant (quant.h:527-650), token-major into a scratch that attn_v_to_pages_kernel transposes
// into the cache's V^T pages.
__global__ void __launch_bounds__(256) attn_qkv_prepare_f32_kernel(const float* __restrict__ qkv, const float* __restrict__ cos_t,
                                                                   const float* __restrict__ sin_t, int B, int Sq, int q_off, int HQ, int HKV,
                                                                   int8_t* __restrict__ q2, float* __restrict__ qs2,
                                                                   int8_t* __restrict__ k_pool, float* __restrict__ ks_pool,
                                                                   const int32_t* __restrict__ page_table, int max_pages,
                                                                   int8_t* __restrict__ v2, float* __restrict__ vs2) {
    // one CTA per token, its eight warps share the token's heads: the token's indices, rotation factors and cache row
    // are worked out once, not per head
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = HQ + 2 * HKV;
    const long bt = blockIdx.x;
    const int t = (int)(bt % Sq);
    const int b = (int)(bt / Sq);
    const int pos = q_off + t;
    const float c = cos_t[(long)pos * 32 + lane], sn = sin_t[(long)pos * 32 + lane];
    const long krow = (long)page_table[(long)b * max_pages + pos / 64] * HKV * 64 + (pos & 63);
    for (int h = warp; h < heads; h += 8) {
        const float* src = qkv + bt * (long)heads * 64 + (long)h * 64;
        const float x0 = src[lane], x1 = src[lane + 32];
        float a, bb;
        if (h < HQ + HKV) {
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
        } else {
            a = x0; bb = x1;
        }
        // scale = max(|max|, |min|) / 127 = the largest magnitude / 127; one reciprocal per head, then every value is
        // divided by the short exact sequence and rounded half away from zero (|quotient| <= 127)
        const float amax = warp_max(fmaxf(fabsf(a), fabsf(bb)));
        float sc = amax / 127.0f;
        if (sc == 0.0f) sc = 1.0f;
        const DivBy dsc = div_by(sc);
        auto q8 = [&](float v) {
            const float qt = div_for_rounding(v, dsc);
            const int m = __float2int_rz(__fadd_rd(fabsf(qt), 0.5f));
            return (int8_t)(qt < 0.0f ? -m : m);
        };
        int8_t* dst; float* sdst;
        if (h < HQ) { const long o = ((long)b * HQ + h) * Sq + t; dst = q2 + o * 64; sdst = qs2 + o; }
        else if (h < HQ + HKV) { const long row = krow + (long)(h - HQ) * 64; dst = k_pool + row * 64; sdst = ks_pool + row; }
        else { const long o = bt * HKV + (h - HQ - HKV); dst = v2 + o * 64; sdst = vs2 + o; }
        if (lane == 0) *sdst = sc;
        dst[lane] = q8(a);
        dst[lane + 32] = q8(bb);
    }
}

// V [B][Sq][HKV][64] (token-major scratch) -> the cache's V^T pages [page][HKV][64 dims][64 tokens] and scale pages,
// for the tokens at positions q_off .. q_off + Sq - 1 (q_off a multiple of 64: one 64-token tile = one page).
__global__ void __launch_bounds__(256) attn_v_to_pages_kernel(const int8_t* __restrict__ v, const float* __restrict__ vs, int Sq, int q_off,
                                                              int HKV, const int32_t* __restrict__ page_table, int max_pages,
                                                              int8_t* __restrict__ v_pool, float* __restrict__ vs_pool) {
    __shared__ int8_t tile[64][64 + 4];
    const int s0 = blockIdx.x * 64, h = blockIdx.y, b = blockIdx.z;
    const long prow = ((long)page_table[(long)b * max_pages + (q_off + s0) / 64] * HKV + h) * 64;
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
        const int r = i >> 4, c4 = i & 15;   // r: token in tile, c4: group of 4 dims
        int val = 0;
        if (s0 + r < Sq) val = *reinterpret_cast<const int*>(v + (((long)b * Sq + s0 + r) * HKV + h) * 64 + c4 * 4);
        *reinterpret_cast<int*>(&tile[r][c4 * 4]) = val;
    }
    if (threadIdx.x < 64 && s0 + threadIdx.x < Sq) vs_pool[prow + threadIdx.x] = vs[((long)b * Sq + s0 + threadIdx.x) * HKV + h];
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        const int d = i >> 6, r = i & 63;
        if (s0 + r < Sq) v_pool[(prow + d) * 64 + r] = tile[r][d];
    }
}

static size_t align_up_(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Workspace of the stand-alone operator (contiguous head-major K, V^T).
struct PrefillWs {
    int8_t *q2, *k2, *vT, *v2;
    float *qs2, *ks2, *vsT, *vs2;
    uint8_t* ecache;
    static size_t bytes(int B, int S, int HQ, int HKV) {
        size_t n = 0;
        n += align_up_((size_t)B * HQ * S * 64, 1024);
        n += 3 * align_up_((size_t)B * HKV * S * 64, 1024);
        n += align_up_((size_t)B * HQ * S * 4, 1024);
        n += 3 * align_up_((size_t)B * HKV * S * 4, 1024);
        n += align_up_((size_t)B * HQ * attn_ecache_head_bytes(0, S), 1024);
        return n + 1024;
    }
    PrefillWs(void* ws, int B, int S, int HQ, int HKV) {
        uint8_t* w = (uint8_t*)align_up_((size_t)ws, 1024);
        q2 = (int8_t*)w; w += align_up_((size_t)B * HQ * S * 64, 1024);
        k2 = (int8_t*)w; w += align_up_((size_t)B * HKV * S * 64, 1024);
        vT = (int8_t*)w; w += align_up_((size_t)B * HKV * S * 64, 1024);
        v2 = (int8_t*)w; w += align_up_((size_t)B * HKV * S * 64, 1024);
        qs2 = (float*)w; w += align_up_((size_t)B * HQ * S * 4, 1024);
        ks2 = (float*)w; w += align_up_((size_t)B * HKV * S * 4, 1024);
        vsT = (float*)w; w += align_up_((size_t)B * HKV * S * 4, 1024);
        vs2 = (float*)w; w += align_up_((size_t)B * HKV * S * 4, 1024);
        ecache = w;
    }
};

// Workspace of the model path (K and V live in the KV cache): head-major Q, token-major V scratch, exp cache.
struct PagedWs {
    int8_t *q2, *v2; float *qs2, *vs2; uint8_t* ecache;
    static size_t bytes(int B, int Sq_max, int HQ, int HKV, size_t ecache_head_bytes) {
        return align_up_((size_t)B * HQ * Sq_max * 64, 1024) + align_up_((size_t)B * HKV * Sq_max * 64, 1024) +
               align_up_((size_t)B * HQ * Sq_max * 4, 1024) + align_up_((size_t)B * HKV * Sq_max * 4, 1024) +
               align_up_((size_t)B * HQ * ecache_head_bytes, 1024) + 1024;
    }
    PagedWs(void* ws, int B, int Sq_max, int HQ, int HKV) {
        uint8_t* w = (uint8_t*)align_up_((size_t)ws, 1024);
        q2 = (int8_t*)w; w += align_up_((size_t)B * HQ * Sq_max * 64, 1024);
        v2 = (int8_t*)w; w += align_up_((size_t)B * HKV * Sq_max * 64, 1024);
        qs2 = (float*)w; w += align_up_((size_t)B * HQ * Sq_max * 4, 1024);
        vs2 = (float*)w; w += align_up_((size_t)B * HKV * Sq_max * 4, 1024);
        ecache = w;
    }
};

// a: everything but the error flag filled in. k_rows / v_rows: rows of the [rows][64 B] (K; paged V^T) or
// [rows][v_row_bytes] (contiguous V^T) matrices the tensor maps describe.
static int mha_prefill_core(AttnArgs a, const int8_t* q2, const int8_t* kmat, uint64_t k_rows, const int8_t* vmat, uint64_t v_rows,
                            uint64_t v_row_bytes, cudaStream_t st, bool online = false) {
    CUtensorMap tq, tk, tv;
    int rc = make_tmap_2d_u8_box(&tq, q2, (uint64_t)a.B * a.HQ * a.Sq, 64, 64, 128, 64);
    if (rc != FLEXLLM_OK) return rc;
    rc = make_tmap_2d_u8_box(&tk, kmat, k_rows, 64, 64, ATT_KT, 64);
    if (rc != FLEXLLM_OK) return rc;
    rc = make_tmap_2d_u8_box(&tv, vmat, v_rows, v_row_bytes, ATT_KT, 64, 64);
    if (rc != FLEXLLM_OK) return rc;
    a.error_flag = device_error_flag();
    static std::atomic<bool> attr_set[kMaxDevices];      // the attribute belongs to (function, device)
    const int dev = current_device();
    if (dev < 0) return FLEXLLM_ECUDA;
    if (!attr_set[dev].load(std::memory_order_acquire)) {
        FLEXLLM_CHECK_CUDA(cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM));
        attr_set[dev].store(true, std::memory_order_release);
    }
    const int n_qt = (a.Sq + 127) / 128;
    const long grid = (long)a.B * a.HQ * n_qt;
    if (online) {
        static std::atomic<bool> attr_set_online[kMaxDevices];
        if (!attr_set_online[dev].load(std::memory_order_acquire)) {
            FLEXLLM_CHECK_CUDA(cudaFuncSetAttribute(attn_prefill_online_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATO_SMEM));
            attr_set_online[dev].store(true, std::memory_order_release);
        }
        attn_prefill_online_kernel<<<(unsigned)grid, 192, ATO_SMEM, st>>>(tq, tk, tv, a);
        return launch_status();
    }
    attn_prefill_kernel<<<(unsigned)grid, 192, ATT_SMEM, st>>>(tq, tk, tv, a);
    return launch_status();
}

// Exp-cache bytes per (batch, query head) that a model with these limits can need: prompts are processed in chunks of
// max_prefill tokens starting at multiples of it.
static size_t paged_ecache_head_bytes(int max_prefill, int max_ctx) {
    size_t worst = 0;
    for (long c0 = 0; c0 < max_ctx; c0 += max_prefill) {
        const int sc = (int)(max_ctx - c0 < max_prefill ? max_ctx - c0 : max_prefill);
        const size_t n = attn_ecache_head_bytes((int)c0, sc);
        if (n > worst) worst = n;
    }
    return worst;
}

size_t mha_prefill_ws_bytes(int B, int max_prefill, int max_ctx, int HQ, int HKV) {
    return PagedWs::bytes(B, max_prefill, HQ, HKV, paged_ecache_head_bytes(max_prefill, max_ctx));
}

// Model path: attention of the Sq tokens at positions q_off .. q_off + Sq - 1 of every sequence, from the fp32 output of
// the fused q/k/v projection, over the paged KV cache: the new keys and values are written into the cache first (which
// is the hand-over to decode: nothing is repacked afterwards), then every query attends to cache positions 0 .. its own.
// q_off is a multiple of 128 (0 for a prompt that fits one call). max_prefill: the Sq the workspace was sized for.
int mha_prefill_paged(const float* qkv, const float* cos_t, const float* sin_t, const float* a_s, int B, int Sq, int q_off, int HQ, int HKV,
                      int max_prefill, flexllm_kv_cache* c, int layer, const int32_t* page_table, int max_pages, float* out,
                      void* workspace, cudaStream_t st) {
    if (Sq % 16 != 0 || q_off % 128 != 0 || Sq > max_prefill || c->hkv != HKV) return FLEXLLM_ENOTSUP;
    PagedWs ws(workspace, B, max_prefill, HQ, HKV);
    int8_t* k_pool = c->k + (size_t)layer * c->page_bytes; int8_t* v_pool = c->v + (size_t)layer * c->page_bytes;
    float* ks_pool = c->ks + (size_t)layer * (c->scale_bytes / 4); float* vs_pool = c->vs + (size_t)layer * (c->scale_bytes / 4);
    attn_qkv_prepare_f32_kernel<<<(unsigned)((long)B * Sq), 256, 0, st>>>(qkv, cos_t, sin_t, B, Sq, q_off, HQ, HKV, ws.q2, ws.qs2, k_pool,
                                                                            ks_pool, page_table, max_pages, ws.v2, ws.vs2);
    dim3 g((Sq + 63) / 64, HKV, B);
    attn_v_to_pages_kernel<<<g, 256, 0, st>>>(ws.v2, ws.vs2, Sq, q_off, HKV, page_table, max_pages, v_pool, vs_pool);
    int rc = launch_status(2);
    if (rc != FLEXLLM_OK) return rc;
    AttnArgs a;
    a.B = B; a.HQ = HQ; a.HKV = HKV; a.Sq = Sq; a.q_off = q_off; a.Sk = 0;
    a.qs = ws.qs2; a.ks = ks_pool; a.vs = vs_pool; a.page_table = page_table; a.max_pages = max_pages;
    a.a_s = a_s; a.out = out; a.oacc = nullptr; a.ecache = ws.ecache;
    const uint64_t rows = (uint64_t)c->n_pages * HKV * 64;
    // FLEXLLM_ATTN_ONLINE=1: the single-sweep variant (not bit-exact) in the model's prefill, for measuring what exactness costs
    static const bool online = [] { const char* e = getenv("FLEXLLM_ATTN_ONLINE"); return e && e[0] == '1'; }();
    return mha_prefill_core(a, ws.q2, k_pool, rows, v_pool, rows, 64, st, online);
}

}  // namespace flexllm

using namespace flexllm;

extern "C" size_t flexllm_mha_prefill_workspace(int B, int S, int HQ, int HKV) {
    if (B <= 0 || S <= 0 || HQ <= 0 || HKV <= 0) return 0;
    return PrefillWs::bytes(B, S, HQ, HKV);
}

static int mha_prefill_contiguous(bool online, const int8_t* q, const float* qs, const int8_t* k, const float* ks,
                                         const int8_t* v, const float* vs, const float* cos_t, const float* sin_t,
                                         const float* a_s, int B, int S, int HQ, int HKV, float* out, int32_t* oacc,
                                         void* workspace, size_t workspace_bytes, void* stream) {
    FLEXLLM_REQUIRE(B >= 0 && S > 0 && HQ > 0 && HKV > 0 && HQ % HKV == 0);
    if (B == 0) return FLEXLLM_OK;
    FLEXLLM_REQUIRE(q && qs && k && ks && v && vs && cos_t && sin_t && a_s && out && workspace);
    if (S % 16 != 0) return FLEXLLM_ENOTSUP;
    FLEXLLM_REQUIRE(workspace_bytes >= flexllm_mha_prefill_workspace(B, S, HQ, HKV));
    FLEXLLM_REQUIRE(aligned(out, 16) && (!oacc || aligned(oacc, 16)) && aligned(v, 4));
    cudaStream_t st = (cudaStream_t)stream;
    PrefillWs ws(workspace, B, S, HQ, HKV);
    const long wq = (long)B * S * HQ, wk = (long)B * S * HKV;
    attn_qk_prepare_kernel<<<(unsigned)((wq + 7) / 8), 256, 0, st>>>(q, qs, cos_t, sin_t, B, S, HQ, ws.q2, ws.qs2);
    attn_qk_prepare_kernel<<<(unsigned)((wk + 7) / 8), 256, 0, st>>>(k, ks, cos_t, sin_t, B, S, HKV, ws.k2, ws.ks2);
    dim3 g((S + 63) / 64, HKV, B);
    attn_v_transpose_kernel<<<g, 256, 0, st>>>(v, vs, B, S, HKV, ws.vT, ws.vsT);
    int rc = launch_status(3);
    if (rc != FLEXLLM_OK) return rc;
    AttnArgs a;
    a.B = B; a.HQ = HQ; a.HKV = HKV; a.Sq = S; a.q_off = 0; a.Sk = S;
    a.qs = ws.qs2; a.ks = ws.ks2; a.vs = ws.vsT; a.page_table = nullptr; a.max_pages = 0;
    a.a_s = a_s; a.out = out; a.oacc = oacc; a.ecache = ws.ecache;
    return mha_prefill_core(a, ws.q2, ws.k2, (uint64_t)B * HKV * S, ws.vT, (uint64_t)B * HKV * 64, (uint64_t)S, st, online);
}

extern "C" int flexllm_mha_i8xi8_prefill(const int8_t* q, const float* qs, const int8_t* k, const float* ks,
                                         const int8_t* v, const float* vs, const float* cos_t, const float* sin_t,
                                         const float* a_s, int B, int S, int HQ, int HKV, float* out, int32_t* oacc,
                                         void* workspace, size_t workspace_bytes, void* stream) {
    return mha_prefill_contiguous(false, q, qs, k, ks, v, vs, cos_t, sin_t, a_s, B, S, HQ, HKV, out, oacc, workspace, workspace_bytes, stream);
}

extern "C" int flexllm_mha_i8xi8_prefill_online(const int8_t* q, const float* qs, const int8_t* k, const float* ks,
                                                const int8_t* v, const float* vs, const float* cos_t, const float* sin_t,
                                                int B, int S, int HQ, int HKV, float* out, void* workspace, size_t workspace_bytes,
                                                void* stream) {
    static const float unused_scale[1] = {1.0f};
    return mha_prefill_contiguous(true, q, qs, k, ks, v, vs, cos_t, sin_t, unused_scale, B, S, HQ, HKV, out, nullptr, workspace, workspace_bytes,
                                  stream);
}
