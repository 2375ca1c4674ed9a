// Walsh-Hadamard transforms of the SpinQuant online rotations.
//
// The reference computes the transform with an Omega network (Modules/FHT.h:31-53). Its fp32
// result is bit-identical to in-place butterflies (lo,hi) <- (lo+hi, lo-hi) applied on index
// bits in the order 1, 2, ..., log2(N)-1, 0; every kernel here keeps exactly that stage order.
//
//  * fht8192_kernel  : R4, the 8192-point transform on the down_proj input. One CTA per token,
//                      the row lives in shared memory, three register passes of 5+5+3 stages.
//                      Optionally fused with silu(gate)*up on the way in and with the per-token
//                      int8 quantiser on the way out.
//  * fht_generic     : any power of two <= 8192, one stage per barrier (API completeness).
//  * qk_prepare      : R3, the 64-point transform on Q/K heads, in registers with warp shuffles,
//                      fused with dequant, RoPE and the per-head int8 quantiser.
#include "common.cuh"
#include "fht_core.cuh"

namespace flexllm {

// FUSED: 0 = y = FHT(x)/scale (fp32 out); 1 = h = silu(g)*u, FHT, /scale, per-token int8 quant;
// 2 = like 1 without the silu, input gathered from `win.g` ranks as x[g][rows][N/g], int8 output only
// for the column window [win.col0, win.col0 + win.cols) written compactly (tensor-parallel down_proj).
struct FhtWindow { int g; long rows; int col0, cols; };
template <int FUSED>
__global__ void __launch_bounds__(256) fht8192_kernel(const float* __restrict__ x, const float* __restrict__ u, long ld_in,
                                                      float scale, float* __restrict__ y, int8_t* __restrict__ q,
                                                      float* __restrict__ s, float* __restrict__ act, FhtWindow win) {
    constexpr int N = 8192;
    __shared__ float buf[N + N / 32];
    __shared__ float red[64];
    pdl_sync();
    const int tid = threadIdx.x;
    const long row = blockIdx.x;
    const float4* xr = reinterpret_cast<const float4*>(x + row * ld_in);   // ld_in: input row stride in floats
    const float4* ur = FUSED ? reinterpret_cast<const float4*>(u + row * ld_in) : nullptr;
    // two batches of four 16-byte vectors per operand: all loads of a batch are issued before the first value is used
    // (SiLU's exponential is long enough to keep the next loads from being hoisted over it otherwise)
#pragma unroll
    for (int half = 0; half < N / 1024; half += 4) {
        float4 vv[4], ww[4];
#pragma unroll
        for (int it = 0; it < 4; it++) {
            const int c = (half + it) * 256 + tid;
            if (FUSED == 2) {
                const int segw = N / win.g, e = c * 4, seg = e / segw;
                vv[it] = *reinterpret_cast<const float4*>(x + ((long)seg * win.rows + row) * segw + (e - seg * segw));
            } else {
                vv[it] = xr[c];
            }
            if (FUSED == 1) ww[it] = ur[c];
        }
#pragma unroll
        for (int it = 0; it < 4; it++) {
            const int c = (half + it) * 256 + tid;
            float4 v = vv[it];
            if (FUSED == 1) {
                const float4 w = ww[it];
                v = silu_mul_x4(v, w);
                if (act) reinterpret_cast<float4*>(act + row * N)[c] = v;
            }
            const int p = pad32(c * 4);
            buf[p] = v.x; buf[p + 1] = v.y; buf[p + 2] = v.z; buf[p + 3] = v.w;
        }
    }
    float r[32];
    fht8192_passes<0>(buf, tid, r);
    div_rn_array(r, div_by(scale));
    // the quantiser's scale is max(|max|, |min|) / 127: the largest magnitude alone carries it
    float mx = 0.0f;
#pragma unroll
    for (int v = 0; v < 32; v++) mx = fmaxf(mx, fabsf(r[v]));
    float mn = -mx;
    if (!FUSED) {
#pragma unroll
        for (int hi = 0; hi < 4; hi++) {
            float4* yo = reinterpret_cast<float4*>(y + row * N + hi * 2048 + tid * 8);
            yo[0] = make_float4(r[hi * 8 + 0], r[hi * 8 + 1], r[hi * 8 + 2], r[hi * 8 + 3]);
            yo[1] = make_float4(r[hi * 8 + 4], r[hi * 8 + 5], r[hi * 8 + 6], r[hi * 8 + 7]);
        }
    } else {
        group_max_min<0, 256>(mx, mn, red, tid);
        const float sc = sym_scale_from(mx, mn);
        const DivBy dsc = div_by(sc);
        if (tid == 0) s[row] = sc;
#pragma unroll
        for (int hi = 0; hi < 4; hi++) {
            union { int8_t b[8]; int2 v; } o;
#pragma unroll
            for (int c = 0; c < 8; c++) o.b[c] = (int8_t)round_half_away_to_int(div_for_rounding(r[hi * 8 + c], dsc));
            const int idx0 = hi * 2048 + tid * 8;
            if (FUSED == 2) {
                if (idx0 >= win.col0 && idx0 < win.col0 + win.cols)
                    *reinterpret_cast<int2*>(q + row * win.cols + (idx0 - win.col0)) = o.v;
            } else {
                *reinterpret_cast<int2*>(q + row * N + idx0) = o.v;
            }
        }
    }
}

__global__ void __launch_bounds__(256) fht_generic_kernel(const float* __restrict__ x, int N, float scale,
                                                          float* __restrict__ y) {
    extern __shared__ float sb[];
    const long row = blockIdx.x;
    for (int i = threadIdx.x; i < N; i += blockDim.x) sb[i] = x[row * N + i];
    __syncthreads();
    auto stage = [&](int h) {
        for (int p = threadIdx.x; p < N / 2; p += blockDim.x) {
            int i = (p / h) * 2 * h + (p % h);
            float a = sb[i], b = sb[i + h];
            sb[i] = a + b;
            sb[i + h] = a - b;
        }
        __syncthreads();
    };
    for (int h = 2; h < N; h <<= 1) stage(h);
    stage(1);
    for (int i = threadIdx.x; i < N; i += blockDim.x) y[row * N + i] = sb[i] / scale;
}

// One warp per (token, head): lane L holds elements L and L+32 of the 64-wide head.
__global__ void __launch_bounds__(256) qk_prepare_kernel(const int8_t* __restrict__ q, const float* __restrict__ s,
                                                         const int32_t* __restrict__ pos, const float* __restrict__ cos_t,
                                                         const float* __restrict__ sin_t, long T, int H,
                                                         int8_t* __restrict__ q_out, float* __restrict__ s_out) {
    const long w = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= T * H) return;
    const long t = w / H;
    const int p = pos[t];
    const float sc_in = s[w];
    const float x0 = (float)q[w * 64 + lane] * sc_in;
    const float x1 = (float)q[w * 64 + 32 + lane] * sc_in;
    const float c = cos_t[(long)p * 32 + lane], sn = sin_t[(long)p * 32 + lane];
    float a = x0 * c - x1 * sn;   // element lane
    float b = x0 * sn + x1 * c;   // element lane + 32
    auto lane_stage = [&](int bit) {
        float pa = __shfl_xor_sync(0xffffffffu, a, 1 << bit);
        float pb = __shfl_xor_sync(0xffffffffu, b, 1 << bit);
        if (lane & (1 << bit)) { a = pa - a; b = pb - b; }
        else { a = a + pa; b = b + pb; }
    };
    lane_stage(1); lane_stage(2); lane_stage(3); lane_stage(4);
    { float lo = a, hi = b; a = lo + hi; b = lo - hi; }   // index bit 5
    lane_stage(0);
    a = a / 8.0f;
    b = b / 8.0f;
    float mx = warp_max(fmaxf(a, b)), mn = warp_min(fminf(a, b));
    const float sc = sym_scale_from(mx, mn);
    if (lane == 0) s_out[w] = sc;
    q_out[w * 64 + lane] = quant_s8(a, sc);
    q_out[w * 64 + 32 + lane] = quant_s8(b, sc);
}

// gate and up halves of one fused projection output: rows of `ld` floats, gate at g, up at u
int swiglu_fht_quant_strided(const float* g, const float* u, long ld, int M, float scale, int8_t* q, float* s, cudaStream_t st) {
    if (M == 0) return FLEXLLM_OK;
    launch_k(fht8192_kernel<1>, dim3(M), dim3(256), 0, st, g, u, ld, scale, (float*)nullptr, q, s, (float*)nullptr, FhtWindow{1, 0, 0, 0});
    return launch_status();
}

// h gathered from g ranks as [g][M][8192/g] -> FHT-8192/scale -> per-token int8 (scale from the whole
// row), this rank's columns [r*8192/g, (r+1)*8192/g) written compactly.
int fht_quant_gathered(const float* h, int M, int g, int r, float scale, int8_t* q, float* s, cudaStream_t st) {
    if (M == 0) return FLEXLLM_OK;
    const int W = 8192 / g;
    launch_k(fht8192_kernel<2>, dim3(M), dim3(256), 0, st, h, (const float*)nullptr, 0L, scale, (float*)nullptr, q, s, (float*)nullptr,
             FhtWindow{g, (long)M, r * W, W});
    return launch_status();
}

// The same input layout, whole rows out: h [g][M][8192/g] -> FHT-8192/scale -> per-token int8 [M][8192].
int fht_quant_gathered_rows(const float* h, int M, int g, float scale, int8_t* q, float* s, cudaStream_t st) {
    if (M == 0) return FLEXLLM_OK;
    launch_k(fht8192_kernel<2>, dim3(M), dim3(256), 0, st, h, (const float*)nullptr, 0L, scale, (float*)nullptr, q, s, (float*)nullptr,
             FhtWindow{g, (long)M, 0, 8192});
    return launch_status();
}

}  // namespace flexllm

using namespace flexllm;

extern "C" int flexllm_fht(const float* x, long rows, int N, float scale, float* y, void* stream) {
    FLEXLLM_REQUIRE(x && y && rows >= 0 && N >= 2 && N <= 8192 && (N & (N - 1)) == 0);
    if (rows == 0) return FLEXLLM_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (N == 8192 && aligned(x, 16) && aligned(y, 16)) {
        fht8192_kernel<0><<<(unsigned)rows, 256, 0, st>>>(x, nullptr, N, scale, y, nullptr, nullptr, nullptr, FhtWindow{1, 0, 0, 0});
    } else {
        int threads = N / 2 < 256 ? (N / 2 < 32 ? 32 : N / 2) : 256;
        fht_generic_kernel<<<(unsigned)rows, threads, N * sizeof(float), st>>>(x, N, scale, y);
    }
    return launch_status();
}

extern "C" int flexllm_swiglu_fht_quant(const float* g, const float* u, int M, int N, float scale, int8_t* q,
                                        float* s, float* act, void* stream) {
    FLEXLLM_REQUIRE(g && u && q && s && M >= 0);
    if (N != 8192) return FLEXLLM_ENOTSUP;
    FLEXLLM_REQUIRE(aligned(g, 16) && aligned(u, 16) && aligned(q, 8) && (!act || aligned(act, 16)));
    if (M == 0) return FLEXLLM_OK;
    fht8192_kernel<1><<<M, 256, 0, (cudaStream_t)stream>>>(g, u, N, scale, nullptr, q, s, act, FhtWindow{1, 0, 0, 0});
    return launch_status();
}

extern "C" int flexllm_qk_prepare(const int8_t* q, const float* s, const int32_t* pos, const float* cos_t,
                                  const float* sin_t, long T, int H, int8_t* q_out, float* s_out, void* stream) {
    FLEXLLM_REQUIRE(q && s && pos && cos_t && sin_t && q_out && s_out && T >= 0 && H > 0);
    if (T == 0) return FLEXLLM_OK;
    const long warps = T * H;
    qk_prepare_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, (cudaStream_t)stream>>>(q, s, pos, cos_t, sin_t, T, H, q_out, s_out);
    return launch_status();
}
