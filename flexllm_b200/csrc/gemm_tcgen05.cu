// int8 x int8 -> int32 linear layer on the 5th-generation tensor cores (tcgen05, kind::i8).
//
//   acc[m][n] = sum_k a[m][k] * w[n][k]                    exact
//   y[m][n]   = ((float)acc * s_tok[m]) * s_ch[n]          fused epilogue
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer: 128-byte-swizzled K-major tiles of both operands, STAGES-deep ring
//   warp 1      MMA issuer (one thread): 4 x (128 x BN x 32) UMMAs per 128-byte K block into one of
//               two TMEM accumulators; also owns TMEM allocation
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (one TMEM lane = one output row per
//               thread), dequantise, store; runs while the MMA warp fills the other accumulator
//
// The "A side" is the UMMA M operand (128 rows per tile), the "B side" the N operand (BN rows).
//   prefill : A = activations [M][K], B = weights [N][K]            out[rowA][rowB]
//   decode  : A = weights [N][K],     B = activations [M<=64][K]     out[rowB][rowA]   (SWAP)
// so that a handful of tokens still fills the 128-row dimension of the tensor core with weight
// rows and the weight matrix is streamed exactly once. With split-K (decode) partial sums are added
// into a zeroed int32 buffer with red.global.add (integer addition is exact and order-free).
//
// Replaces pref_Linear_Layer_i4xi4 / dec_Linear_Layer_i4xi4 + the dequant layers
// (Modules/Linear_Layer.h:293-341, :862-923; Modules/quant.h:115-164, :434-524) at 8-bit precision.
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tc_common.cuh"

namespace flexllm {

using namespace tc;

// ------------------------------------------------------------------ tensor-map encoding (host)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

int make_tmap_2d_u8_box(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_bytes,
                        uint32_t box_rows, int swizzle_bytes) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return FLEXLLM_ECUDA;
    if (!aligned(base, 16) || (row_bytes % 16) != 0 || box_rows == 0 || box_rows > 256) return FLEXLLM_EINVAL;
    if ((swizzle_bytes != 64 && swizzle_bytes != 128) || box_bytes == 0 || box_bytes > (uint32_t)swizzle_bytes || (box_bytes % 16) != 0)
        return FLEXLLM_EINVAL;
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_bytes, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { g_last_cuda_error = (int)r; return FLEXLLM_ECUDA; }
    return FLEXLLM_OK;
}

int make_tmap_3d_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows, uint32_t kch) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return FLEXLLM_ECUDA;
    if (!aligned(base, 16) || (row_bytes % 128) != 0 || box_rows == 0 || box_rows > 256 || kch == 0 || kch > 8) return FLEXLLM_EINVAL;
    cuuint64_t dims[3] = {128, rows, row_bytes / 128};
    cuuint64_t strides[2] = {row_bytes, 128};
    cuuint32_t box[3] = {128, box_rows, kch};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { g_last_cuda_error = (int)r; return FLEXLLM_ECUDA; }
    return FLEXLLM_OK;
}

int make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
    return make_tmap_2d_u8_box(out, base, rows, row_bytes, 128, box_rows, 128);
}

// ------------------------------------------------------------------ kernel
struct GemmArgs {
    int rowsA, rowsB, K;     // A side (128-row tiles), B side (BN-row tiles), reduction length
    int tilesA, tilesB, ksplit;
    int ldo;                 // leading dimension of the outputs
    int32_t* acc;            // optional int32 output (required when ksplit > 1: added atomically)
    float* y;                // optional fp32 output (ignored when ksplit > 1)
    const float* sA;         // per-row scale of the A side
    const float* sB;         // per-row scale of the B side
    int* error_flag;         // set to 1 if a device-side wait ran out
    // fused epilogue extras
    const float* residual;   // optional: y = residual + dequant (same layout as y)
    int32_t* work;           // split-K: zeroed int32 partial-sum buffer [rowsB][ldo]; the last arriver
                             // turns it into the outputs and leaves it zeroed again
    int* counters;           // split-K: zeroed arrival counters, one per (A tile, warp quarter)
};

// KCH = 128-byte K chunks per pipeline stage (1 for prefill; > 1 for the weight-streaming decode
// orientation, where fetching KCH*128 contiguous bytes per weight row keeps HBM pages open).
template <int BN, int KCH = 1> struct GemmCfg {
    static constexpr int A_TILE = 128 * 128;
    static constexpr int B_TILE = BN * 128;
    static constexpr int A_BYTES = KCH * A_TILE;
    static constexpr int B_BYTES = KCH * B_TILE;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES_MAX = (200 * 1024) / STAGE_BYTES;
    static constexpr int STAGES = KCH > 1 ? (STAGES_MAX > 8 ? 8 : STAGES_MAX)
                                          : (BN == 256 ? 4 : BN == 128 ? 6 : BN == 64 ? 8 : BN == 32 ? 8 : 10);
    static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    // prefill orientation: per-warp staging (32 rows x 32 fp32, plus the tile's column scales) that turns the accumulator rows a thread
    // owns into row-contiguous 128-byte global stores
    static constexpr int STG_WARP_FLOATS = 32 * 32 + 256;      // one 32 x 32 chunk + the tile's column scales
    static constexpr int STG_BYTES = BN >= 32 ? 4 * STG_WARP_FLOATS * 4 : 0;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + STG_BYTES;
};

template <int BN, bool SWAP, int KCH = 1>
__global__ void __launch_bounds__(192, 1) gemm_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmapA,
                                                                 const __grid_constant__ CUtensorMap tmapB,
                                                                 const GemmArgs args) {
    using Cfg = GemmCfg<BN, KCH>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte aligned operand ring, then barriers
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t ring = (raw + 1023u) & ~1023u;
    uint8_t* ring_ptr = smem_raw + (ring - raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring_ptr + STAGES * Cfg::STAGE_BYTES);
    // bars: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then tmem base word, abort flag
    const uint32_t bar_full = smem_u32(bars);
    const uint32_t bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES;
    const uint32_t bar_tempty = bar_tfull + 16;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    pdl_sync();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = ((args.K + 127) >> 7) / KCH;      // pipeline steps of KCH chunks (K % (128*KCH) == 0 when KCH > 1)
    const int total_tiles = args.tilesA * args.tilesB * args.ksplit;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int s = 0; s < 2; s++) { mbar_init(bar_tfull + 8 * s, 1); mbar_init(bar_tempty + 8 * s, 4); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_base_slot), Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmapA);
            tma_prefetch_desc(&tmapB);
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
                const int split = t % args.ksplit;
                const int tb = (t / args.ksplit) % args.tilesB;
                const int ta = t / (args.ksplit * args.tilesB);
                const int kb0 = (int)((long)split * num_kb / args.ksplit);
                const int kb1 = (int)((long)(split + 1) * num_kb / args.ksplit);
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t full = bar_full + 8 * stage;
                    mbar_expect_tx(full, Cfg::STAGE_BYTES);
                    const uint32_t dstA = ring + stage * Cfg::STAGE_BYTES;
                    if (KCH == 1) {
                        tma_load_2d(dstA, &tmapA, full, kb * 128, ta * 128);
                        tma_load_2d(dstA + Cfg::A_BYTES, &tmapB, full, kb * 128, tb * BN);
                    } else {
                        tma_load_3d(dstA, &tmapA, full, 0, ta * 128, kb * KCH);
                        tma_load_3d(dstA + Cfg::A_BYTES, &tmapB, full, 0, tb * BN, kb * KCH);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(128, BN, 1, 1);
            int stage = 0; uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, it++) {
                const int split = t % args.ksplit;
                const int kb0 = (int)((long)split * num_kb / args.ksplit);
                const int kb1 = (int)((long)(split + 1) * num_kb / args.ksplit);
                const int as = it & 1;
                const uint32_t aphase = (it >> 1) & 1;
                if (!mbar_wait(bar_tempty + 8 * as, aphase ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + as * BN;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = ring + stage * Cfg::STAGE_BYTES;
#pragma unroll
                    for (int c = 0; c < KCH; c++) {
                        const uint64_t adesc = umma_desc_k_sw128(sa + c * Cfg::A_TILE);
                        const uint64_t bdesc = umma_desc_k_sw128(sa + Cfg::A_BYTES + c * Cfg::B_TILE);
#pragma unroll
                        for (int k = 0; k < 4; k++)   // 32 int8 = 32 bytes = 2 descriptor address units per step
                            umma_i8(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > kb0 || c > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(bar_empty + 8 * stage);   // slot is free once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(bar_tfull + 8 * as);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, it++) {
            const int tb = (t / args.ksplit) % args.tilesB;
            const int ta = t / (args.ksplit * args.tilesB);
            const int as = it & 1;
            const uint32_t aphase = (it >> 1) & 1;
            // everything the epilogue needs besides the accumulator is fetched BEFORE the wait, so its
            // global-memory latency hides behind the main loop
            const int rowA = ta * 128 + q * 32 + lane;
            const bool rowA_ok = rowA < args.rowsA;
            const float sa = (rowA_ok && args.sA) ? args.sA[rowA] : 0.0f;
            float sbv[SWAP ? BN : 1];
            if (SWAP && args.sB) {
#pragma unroll
                for (int j = 0; j < BN; j++) { const int tok = tb * BN + j; sbv[j] = tok < args.rowsB ? args.sB[tok] : 0.0f; }
            }
            float* stg = reinterpret_cast<float*>(ring_ptr + STAGES * Cfg::STAGE_BYTES + 256) + q * Cfg::STG_WARP_FLOATS;
            if (!SWAP && BN >= 32) {
                // column scales of this tile into shared memory, and the residual rows into L2
                float* sbw = stg + 1024;
                if (args.sB)
                    for (int i = lane; i < BN; i += 32) sbw[i] = tb * BN + i < args.rowsB ? args.sB[tb * BN + i] : 0.0f;
                if (args.residual) {
                    for (int i = lane; i < 32 * (BN / 32); i += 32) {
                        const int rr = i / (BN / 32), seg = i - rr * (BN / 32);
                        const int row = ta * 128 + q * 32 + rr, col = tb * BN + seg * 32;
                        if (row < args.rowsA && col < args.rowsB)
                            asm volatile("prefetch.global.L2 [%0];" ::"l"(args.residual + (long)row * args.ldo + col));
                    }
                }
            }
            // lane 0 polls; the verdict is broadcast so that the warp stays converged for the
            // warp-collective TMEM loads below
            int got = (lane == 0) ? (mbar_wait(bar_tfull + 8 * as, aphase, abort_flag) ? 1 : 0) : 1;
            got = __shfl_sync(0xffffffffu, got, 0);
            if (!got) { ok = false; break; }
            tc_fence_after();
            if (!SWAP && BN >= 32) {
                // ---- prefill orientation, staged: lane = token row of the tile. 32 columns at a time are
                // dequantised into this warp's staging buffer (16-byte granules XOR-swizzled by the row), then
                // written out with every warp instruction covering 4 rows x 128 contiguous bytes (the direct
                // form stores 32 rows x 16 bytes per instruction and was bound by the store path).
                const float* sbw = stg + 1024;
                __syncwarp();
                // the TMEM load of chunk c + 1 is in flight while chunk c is processed
                constexpr int NCH = BN / 32;
                const uint32_t tsrc = tmem_base + ((uint32_t)(q * 32) << 16) + as * BN;
                auto process = [&](const uint32_t (&v)[32], const int c) {
                    const int colB0 = tb * BN + c * 32;
                    if (args.acc && rowA_ok) {
                        const long o = (long)rowA * args.ldo + colB0;
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            if (colB0 + j < args.rowsB)
                                *reinterpret_cast<int4*>(args.acc + o + j) = make_int4((int)v[j], (int)v[j + 1], (int)v[j + 2], (int)v[j + 3]);
                    }
                    if (args.y) {
                        float* buf = stg;
                        const int g = lane & 7;
                        // this lane's share of the residual for the write-out below, requested first
                        float4 rs[8];
                        if (args.residual) {
#pragma unroll
                            for (int it = 0; it < 8; it++) {
                                const int rr = it * 4 + (lane >> 3);
                                const int row = ta * 128 + q * 32 + rr, col = colB0 + 4 * g;
                                rs[it] = (row < args.rowsA && col < args.rowsB)
                                             ? *reinterpret_cast<const float4*>(args.residual + (long)row * args.ldo + col)
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        }
#pragma unroll
                        for (int gg = 0; gg < 8; gg++) {
                            const float4 sb = *reinterpret_cast<const float4*>(sbw + c * 32 + 4 * gg);
                            float4 r;
                            r.x = ((float)(int)v[4 * gg] * sa) * sb.x;
                            r.y = ((float)(int)v[4 * gg + 1] * sa) * sb.y;
                            r.z = ((float)(int)v[4 * gg + 2] * sa) * sb.z;
                            r.w = ((float)(int)v[4 * gg + 3] * sa) * sb.w;
                            *reinterpret_cast<float4*>(buf + lane * 32 + ((gg ^ (lane & 7)) << 2)) = r;
                        }
                        __syncwarp();
#pragma unroll
                        for (int it = 0; it < 8; it++) {
                            const int rr = it * 4 + (lane >> 3);
                            const int row = ta * 128 + q * 32 + rr, col = colB0 + 4 * g;
                            if (row < args.rowsA && col < args.rowsB) {
                                float4 r = *reinterpret_cast<const float4*>(buf + rr * 32 + ((g ^ (rr & 7)) << 2));
                                if (args.residual) { r.x = rs[it].x + r.x; r.y = rs[it].y + r.y; r.z = rs[it].z + r.z; r.w = rs[it].w + r.w; }
                                *reinterpret_cast<float4*>(args.y + (long)row * args.ldo + col) = r;
                            }
                        }
                        __syncwarp();      // the staging buffer is reused by the next chunk
                    }
                };
                uint32_t va[32], vb[32];
                tmem_ld_32x32(tsrc, va);
#pragma unroll 1
                for (int c = 0; c < NCH; c += 2) {
                    tmem_ld_wait();
                    if (c + 1 < NCH) tmem_ld_32x32(tsrc + (c + 1) * 32, vb);
                    process(va, c);
                    if (c + 1 < NCH) {
                        tmem_ld_wait();
                        if (c + 2 < NCH) tmem_ld_32x32(tsrc + (c + 2) * 32, va);
                        process(vb, c + 1);
                    }
                }
            } else {
        #pragma unroll (SWAP ? BN / 16 : 1)
            for (int c = 0; c < BN / 16; c++) {
                uint32_t v[16];
                tmem_ld_32x16(tmem_base + ((uint32_t)(q * 32) << 16) + as * BN + c * 16, v);
                tmem_ld_wait();
                const int colB0 = tb * BN + c * 16;
                if (!SWAP) {
                    // out[rowA][colB0 + j]: token = rowA, channel = colB
                    if (rowA_ok) {
                        const long o = (long)rowA * args.ldo + colB0;
#pragma unroll
                        for (int j = 0; j < 16; j += 4) {
                            if (colB0 + j < args.rowsB) {
                                if (args.acc) {
                                    *reinterpret_cast<int4*>(args.acc + o + j) =
                                        make_int4((int)v[j], (int)v[j + 1], (int)v[j + 2], (int)v[j + 3]);
                                }
                                if (args.y) {
                                    const float4 sb = *reinterpret_cast<const float4*>(args.sB + colB0 + j);
                                    float4 r;
                                    r.x = ((float)(int)v[j] * sa) * sb.x;
                                    r.y = ((float)(int)v[j + 1] * sa) * sb.y;
                                    r.z = ((float)(int)v[j + 2] * sa) * sb.z;
                                    r.w = ((float)(int)v[j + 3] * sa) * sb.w;
                                    if (args.residual) {
                                        const float4 rs = *reinterpret_cast<const float4*>(args.residual + o + j);
                                        r.x = rs.x + r.x; r.y = rs.y + r.y; r.z = rs.z + r.z; r.w = rs.w + r.w;
                                    }
                                    *reinterpret_cast<float4*>(args.y + o + j) = r;
                                }
                            }
                        }
                    }
                } else {
                    // out[colB0 + j][rowA]: token = colB, channel = rowA; a warp store covers 32 channels
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int tok = colB0 + j;
                        if (rowA_ok && tok < args.rowsB) {
                            const long o = (long)tok * args.ldo + rowA;
                            if (args.ksplit > 1) {
                                atomicAdd((args.work ? args.work : args.acc) + o, (int)v[j]);
                            } else {
                                if (args.acc) args.acc[o] = (int)v[j];
                                if (args.y) {
                                    float r = ((float)(int)v[j] * sbv[SWAP ? c * 16 + j : 0]) * sa;
                                    if (args.residual) r = args.residual[o] + r;
                                    args.y[o] = r;
                                }
                            }
                        }
                    }
                }
            }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * as);
            if (SWAP && args.ksplit > 1 && args.work) {
                // split-K with fused finalisation: the warp that arrives last on this (tile, quarter)
                // reads the complete integer sums, writes the outputs and re-zeroes the work buffer
                __threadfence();
                int last = 0;
                if (lane == 0) last = (atomicAdd(args.counters + ta * 4 + q, 1) == args.ksplit - 1);
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence();
                    if (rowA_ok) {
                        // batches of 16 tokens: the loads of a batch are independent, so their
                        // L2 latencies overlap
                        for (int t0 = 0; t0 < args.rowsB; t0 += 16) {
                            int vv[16];
#pragma unroll
                            for (int j = 0; j < 16; j++) {
                                const int tok = t0 + j;
                                vv[j] = tok < args.rowsB ? __ldcg(args.work + (long)tok * args.ldo + rowA) : 0;
                            }
                            float rs[16];
                            if (args.residual) {
#pragma unroll
                                for (int j = 0; j < 16; j++) {
                                    const int tok = t0 + j;
                                    rs[j] = tok < args.rowsB ? args.residual[(long)tok * args.ldo + rowA] : 0.0f;
                                }
                            }
#pragma unroll
                            for (int j = 0; j < 16; j++) {
                                const int tok = t0 + j;
                                if (tok < args.rowsB) {
                                    const long o = (long)tok * args.ldo + rowA;
                                    args.work[o] = 0;
                                    if (args.acc) args.acc[o] = vv[j];
                                    if (args.y) {
                                        float r = ((float)vv[j] * args.sB[tok]) * sa;   // L1/L2 hit: fetched before the wait
                                        if (args.residual) r = rs[j] + r;
                                        args.y[o] = r;
                                    }
                                }
                            }
                        }
                    }
                    if (lane == 0) args.counters[ta * 4 + q] = 0;
                }
            }
        }
    }

    // ---------------------------------------------------------------- tear-down
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // a wait ran out: give copies still in flight time to land before shared memory is released
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
        if (threadIdx.x == 0 && args.error_flag) atomicOr(args.error_flag, 1);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// ------------------------------------------------------------------ host launcher
struct TmapKey {
    const void* base; uint64_t rows, row_bytes; uint32_t box_rows, kch;   // kch 0: 2-D map
    bool operator==(const TmapKey& o) const {
        return base == o.base && rows == o.rows && row_bytes == o.row_bytes && box_rows == o.box_rows && kch == o.kch;
    }
};
struct TmapKeyHash {
    size_t operator()(const TmapKey& k) const {
        size_t h = std::hash<const void*>()(k.base);
        h ^= std::hash<uint64_t>()(k.rows * 1000003ull + k.row_bytes * 31ull + k.box_rows + 977ull * k.kch) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        return h;
    }
};
// Encoding a tensor map costs a few microseconds of host time; the same weights and activation
// buffers come back every layer call, so maps are cached by (pointer, shape, box).
static int cached_tmap(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows, uint32_t kch = 0) {
    static std::mutex mu;
    static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
    TmapKey key{base, rows, row_bytes, box_rows, kch};
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return FLEXLLM_OK; }
    int st = kch ? make_tmap_3d_u8(out, base, rows, row_bytes, box_rows, kch) : make_tmap_2d_u8(out, base, rows, row_bytes, box_rows);
    if (st != FLEXLLM_OK) return st;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return FLEXLLM_OK;
}

// One error word per device: bit 0 is raised by any kernel of the library whose bounded device-side wait ran
// out, bit 1 by a kernel that found (and clamped) a token id or context length in device memory out of range. It lives in the library's device image (no allocation needed to reach it); its device address
// is looked up once per device. Process-wide: a time-out raised by a launch from one host thread is
// seen by a status check from any other.
static __device__ int g_error_flag;
struct DevFlag { std::once_flag once; int* p = nullptr; };
static DevFlag g_dev_flag[kMaxDevices];

int* device_error_flag() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    DevFlag& f = g_dev_flag[dev];
    std::call_once(f.once, [&] {
        int* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, g_error_flag) == cudaSuccess) f.p = p;
    });
    return f.p;
}

static int sm_count() {
    static int n[kMaxDevices] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDevices) return 148;
    if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
    return n[dev] > 0 ? n[dev] : 148;
}

template <int BN, bool SWAP, int KCH = 1>
static int launch_gemm(const int8_t* A, int rowsA, const int8_t* B, int rowsB, int K, int ksplit, int ldo,
                       int32_t* acc, float* y, const float* sA, const float* sB, cudaStream_t st,
                       const float* residual = nullptr, int32_t* work = nullptr, int* counters = nullptr) {
    using Cfg = GemmCfg<BN, KCH>;
    CUtensorMap ta, tb;
    int rc = cached_tmap(&ta, A, (uint64_t)rowsA, (uint64_t)K, 128, KCH > 1 ? KCH : 0);
    if (rc != FLEXLLM_OK) return rc;
    rc = cached_tmap(&tb, B, (uint64_t)rowsB, (uint64_t)K, BN, KCH > 1 ? KCH : 0);
    if (rc != FLEXLLM_OK) return rc;
    GemmArgs g;
    g.rowsA = rowsA; g.rowsB = rowsB; g.K = K;
    g.tilesA = (rowsA + 127) / 128; g.tilesB = (rowsB + BN - 1) / BN; g.ksplit = ksplit;
    g.ldo = ldo; g.acc = acc; g.y = y; g.sA = sA; g.sB = sB; g.error_flag = device_error_flag();
    g.residual = residual; g.work = work; g.counters = counters;
    auto kern = gemm_i8_tcgen05_kernel<BN, SWAP, KCH>;
    // the attribute belongs to (function, device): once per device, not once per process
    static std::atomic<bool> attr_set[kMaxDevices];
    const int dev = current_device();
    if (dev < 0) return FLEXLLM_ECUDA;
    if (!attr_set[dev].load(std::memory_order_acquire)) {
        FLEXLLM_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_set[dev].store(true, std::memory_order_release);
    }
    const int total = g.tilesA * g.tilesB * g.ksplit;
    const int grid = total < sm_count() ? total : sm_count();
    launch_k(kern, dim3(grid), dim3(192), (size_t)Cfg::SMEM_BYTES, st, ta, tb, g);
    return launch_status();
}

// Prefill orientation: activations on the 128-row side. residual (optional): y = residual + dequant.
int gemm_i8_prefill(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch, int M, int N, int K,
                    int32_t* acc, float* y, cudaStream_t st, const float* residual) {
    if (N > 128) return launch_gemm<256, false>(a, M, w, N, K, 1, N, acc, y, s_tok, s_ch, st, residual);
    if (N > 64) return launch_gemm<128, false>(a, M, w, N, K, 1, N, acc, y, s_tok, s_ch, st, residual);
    if (N > 32) return launch_gemm<64, false>(a, M, w, N, K, 1, N, acc, y, s_tok, s_ch, st, residual);
    if (N > 16) return launch_gemm<32, false>(a, M, w, N, K, 1, N, acc, y, s_tok, s_ch, st, residual);
    return launch_gemm<16, false>(a, M, w, N, K, 1, N, acc, y, s_tok, s_ch, st, residual);
}

// Decode orientation: weights on the 128-row side, M <= 64 tokens on the N side, optional split-K.
// With ksplit > 1 the partial sums go through `work` (zeroed int32 [M][N]) and `counters` (zeroed,
// 4 per 128-channel tile); the last-arriving warp writes acc / y (+ residual) and re-zeroes both.
int gemm_i8_decode(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch, int M, int N, int K,
                   int ksplit, int32_t* acc, float* y, cudaStream_t st, const float* residual, int32_t* work, int* counters) {
    if (M > 64) return FLEXLLM_ENOTSUP;
    // chunks of K per pipeline stage: KCH*128 contiguous bytes per weight row and TMA request
    int kch = 1;
    if (K % 512 == 0) kch = 4;
    else if (K % 256 == 0) kch = 2;
    const int steps = (K + 127) / 128 / kch;
    if (ksplit > steps) ksplit = steps;
    if (ksplit < 1) ksplit = 1;
    if (ksplit > 1 && !(work && counters)) return FLEXLLM_EINVAL;
#define FLEXLLM_DEC(BN_, KCH_) \
    return launch_gemm<BN_, true, KCH_>(w, N, a, M, K, ksplit, N, acc, y, s_ch, s_tok, st, residual, work, counters)
    if (M > 32) { if (kch == 4) FLEXLLM_DEC(64, 4); if (kch == 2) FLEXLLM_DEC(64, 2); FLEXLLM_DEC(64, 1); }
    if (M > 16) { if (kch == 4) FLEXLLM_DEC(32, 4); if (kch == 2) FLEXLLM_DEC(32, 2); FLEXLLM_DEC(32, 1); }
    if (kch == 4) FLEXLLM_DEC(16, 4);
    if (kch == 2) FLEXLLM_DEC(16, 2);
    FLEXLLM_DEC(16, 1);
#undef FLEXLLM_DEC
}

// Reads and clears the current device's error word (synchronises the device: the copy is ordered
// behind all work queued so far).
int gemm_check_error_flag() {
    int* f = device_error_flag();
    if (!f) return FLEXLLM_ECUDA;
    int h = 0;
    FLEXLLM_CHECK_CUDA(cudaMemcpy(&h, f, sizeof(int), cudaMemcpyDeviceToHost));
    if (h) {
        FLEXLLM_CHECK_CUDA(cudaMemset(f, 0, sizeof(int)));
        return (h & 1) ? FLEXLLM_ETIMEDOUT : FLEXLLM_EDEVDATA;      // bit 0: a wait ran out; bit 1: an index in device memory was clamped
    }
    return FLEXLLM_OK;
}

int gemm_sm_count() { return sm_count(); }

// ------------------------------------------------------------------ allocation-free decode linear
// Built-in scratch for the split-K partial sums of flexllm_linear_decode_i8_noalloc: a fixed array in
// the library's device image, so the entry point never has to ask the driver for memory. Every GPU
// that loads the library carries these 4 MiB until the process exits.
constexpr long kNoAllocMaxElems = 64L * 16384L;   // tokens x output channels, int32 each
static __device__ __align__(256) int32_t g_noalloc_scratch[kNoAllocMaxElems];

struct NoAllocDev { std::once_flag once; int32_t* scratch = nullptr; int* flag = nullptr; int rc = FLEXLLM_ECUDA; };
static NoAllocDev g_noalloc_dev[kMaxDevices];

template <int BN>
static int launch_gemm_noalloc(const int8_t* w, int N, const int8_t* a, int M, int K, int ksplit, int32_t* acc, int* flag,
                               cudaStream_t st) {
    using Cfg = GemmCfg<BN>;
    CUtensorMap ta, tb;   // encoded on the stack: no cache, nothing retained
    int rc = make_tmap_2d_u8(&ta, w, (uint64_t)N, (uint64_t)K, 128);
    if (rc != FLEXLLM_OK) return rc;
    rc = make_tmap_2d_u8(&tb, a, (uint64_t)M, (uint64_t)K, BN);
    if (rc != FLEXLLM_OK) return rc;
    GemmArgs g;
    g.rowsA = N; g.rowsB = M; g.K = K;
    g.tilesA = (N + 127) / 128; g.tilesB = 1; g.ksplit = ksplit;
    g.ldo = N; g.acc = acc; g.y = nullptr; g.sA = nullptr; g.sB = nullptr; g.error_flag = flag;
    g.residual = nullptr; g.work = nullptr; g.counters = nullptr;
    auto kern = gemm_i8_tcgen05_kernel<BN, true>;
    static std::atomic<bool> attr_set[kMaxDevices];
    const int dev = current_device();
    if (dev < 0) return FLEXLLM_ECUDA;
    if (!attr_set[dev].load(std::memory_order_acquire)) {
        FLEXLLM_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_set[dev].store(true, std::memory_order_release);
    }
    const int total = g.tilesA * g.ksplit;
    const int grid = total < sm_count() ? total : sm_count();
    kern<<<grid, 192, Cfg::SMEM_BYTES, st>>>(ta, tb, g);
    return launch_status();
}

}  // namespace flexllm

using namespace flexllm;

// See include/flexllm_b200.h.
extern "C" int flexllm_device_status(void) { return gemm_check_error_flag(); }

// See include/flexllm_b200.h: the prefill GEMM with nothing to store (the epilogue warps still drain TMEM).
extern "C" int flexllm_gemm_i8_mainloop_probe(const int8_t* a, const int8_t* w, int M, int N, int K, void* stream) {
    FLEXLLM_REQUIRE(a && w && M > 0 && N > 128 && K > 0 && (K % 16) == 0 && aligned(a, 16) && aligned(w, 16));
    return launch_gemm<256, false>(a, M, w, N, K, 1, N, nullptr, nullptr, nullptr, nullptr, (cudaStream_t)stream);
}

// See include/flexllm_b200.h. The first call on a device resolves the device addresses of the
// built-in arrays (cudaGetSymbolAddress: the array's name is only a host-side handle, not a device
// pointer); make that first call outside any stream capture.
extern "C" int flexllm_linear_decode_i8_noalloc(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch,
                                                int M, int N, int K, float* y, void* stream) {
    FLEXLLM_REQUIRE(M >= 0 && N > 0 && K > 0 && (K % 16) == 0 && (N % 8) == 0);
    if (M == 0) return FLEXLLM_OK;
    FLEXLLM_REQUIRE(a && s_tok && w && s_ch && y);
    FLEXLLM_REQUIRE(aligned(a, 16) && aligned(w, 16) && aligned(y, 16) && aligned(s_ch, 16));
    if (M > 64) return FLEXLLM_ENOTSUP;
    if ((long)M * N > kNoAllocMaxElems) return FLEXLLM_ETOOBIG;   // larger than the built-in scratch
    const int dev = current_device();
    if (dev < 0) return FLEXLLM_ECUDA;
    NoAllocDev& d = g_noalloc_dev[dev];
    // set-up, once per device, with that device current: the array's name is only a host-side handle,
    // the kernel needs the address cudaGetSymbolAddress returns. The error word is the library's
    // per-device one, so a time-out in this path is reported by flexllm_device_status() like any other.
    std::call_once(d.once, [&] {
        d.rc = cuda_status(cudaGetSymbolAddress((void**)&d.scratch, g_noalloc_scratch));
        if (d.rc == FLEXLLM_OK) { d.flag = device_error_flag(); if (!d.flag) d.rc = FLEXLLM_ECUDA; }
    });
    if (d.rc != FLEXLLM_OK) return d.rc;
    cudaStream_t st = (cudaStream_t)stream;
    // split-K as in the allocating entry point: enough CTAs to pull the weights at full HBM rate
    const int tiles = (N + 127) / 128, num_kb = (K + 127) / 128;
    int ks = sm_count() / tiles;
    if (ks > num_kb / 2) ks = num_kb / 2;
    if (ks < 1) ks = 1;
    // the array keeps whatever the previous call left in it: the partial sums must start from zero
    FLEXLLM_CHECK_CUDA(cudaMemsetAsync(d.scratch, 0, (size_t)M * N * sizeof(int32_t), st));
    int rc;
    if (M > 32) rc = launch_gemm_noalloc<64>(w, N, a, M, K, ks, d.scratch, d.flag, st);
    else if (M > 16) rc = launch_gemm_noalloc<32>(w, N, a, M, K, ks, d.scratch, d.flag, st);
    else rc = launch_gemm_noalloc<16>(w, N, a, M, K, ks, d.scratch, d.flag, st);
    if (rc != FLEXLLM_OK) return rc;
    return flexllm_dequant(d.scratch, s_tok, s_ch, M, N, y, stream);
}
