// Decode linear layer for a handful of tokens: int8 GEMV by weight streaming.
//
//   acc[b][n] = sum_k a[b][k] * w[n][k]      (exact, dp4a)        b < BT <= 8
//   y[b][n]   = ((float)acc * s_tok[b]) * s_ch[n]
//
// HBM-bound on the weight matrix (N*K bytes read once). Each warp owns R consecutive output
// channels; its 32 lanes stride over K with 128-bit loads (512 contiguous bytes per warp per row),
// the activations sit in shared memory, partial sums are combined with warp shuffles.
// Replaces dec_Linear_Layer_i4xi4 + dec_dequant_layer_qint_fp32 (Modules/Linear_Layer.h:862-923,
// Modules/quant.h:434-524) at 8-bit precision.
#include "common.cuh"

namespace flexllm {

__device__ __forceinline__ int4 ldg_stream(const int4* p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// KS = 1: each of the CTA's four warps owns R output channels over the whole K. KS = 4 (few channels, long rows): the
// four warps share R channels, a quarter of K each, and combine through shared memory -- four times as many warps for
// the same matrix, so that short launches still keep enough loads in flight.
template <int BT, int R, int KS>
__global__ void __launch_bounds__(128) gemv_i8_kernel(const int8_t* __restrict__ a, const float* __restrict__ s_tok,
                                                      const int8_t* __restrict__ w, const float* __restrict__ s_ch,
                                                      int M, int N, int K, int32_t* __restrict__ acc_out,
                                                      float* y, const float* residual) {
    extern __shared__ int4 a_sm[];   // [BT][K/16], then (KS = 4) the warps' partial sums [4][R][BT]
    const int kv = K >> 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = KS == 1 ? (blockIdx.x * 4 + warp) * R : blockIdx.x * R;
    const int kq = KS == 1 ? kv : kv >> 2;
    const int kbeg = KS == 1 ? 0 : warp * kq, kend = kbeg + kq;
    const bool active = n0 < N;
    const int4* wr[R];
#pragma unroll
    for (int r = 0; r < R; r++) wr[r] = reinterpret_cast<const int4*>(w + (long)min(n0 + r, N - 1) * K);
    // the first weights are asked for before the activations are staged (they do not depend on them)
    int4 nx0[R], nx1[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int c0 = kbeg + lane, c1 = c0 + 32;
        nx0[r] = (active && c0 < kend) ? ldg_stream(wr[r] + c0) : make_int4(0, 0, 0, 0);
        nx1[r] = (active && c1 < kend) ? ldg_stream(wr[r] + c1) : make_int4(0, 0, 0, 0);
    }
    pdl_sync();
    for (int i = threadIdx.x; i < BT * kv; i += blockDim.x) {
        int b = i / kv;
        a_sm[i] = b < M ? reinterpret_cast<const int4*>(a)[(long)b * kv + (i - b * kv)] : make_int4(0, 0, 0, 0);
    }
    __syncthreads();
    int acc[R][BT];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int b = 0; b < BT; b++) acc[r][b] = 0;

    if (active) {
        for (int c0 = kbeg + lane; c0 < kend; c0 += 64) {
            const int c1 = c0 + 32;
            const bool has1 = c1 < kend;
            int4 wv0[R], wv1[R];
#pragma unroll
            for (int r = 0; r < R; r++) { wv0[r] = nx0[r]; wv1[r] = nx1[r]; }
            const int d0 = c0 + 64, d1 = c1 + 64;          // next iteration's weights, one step ahead
#pragma unroll
            for (int r = 0; r < R; r++) {
                nx0[r] = d0 < kend ? ldg_stream(wr[r] + d0) : make_int4(0, 0, 0, 0);
                nx1[r] = d1 < kend ? ldg_stream(wr[r] + d1) : make_int4(0, 0, 0, 0);
            }
#pragma unroll
            for (int b = 0; b < BT; b++) {
                const int4 av0 = a_sm[b * kv + c0];
                const int4 av1 = has1 ? a_sm[b * kv + c1] : make_int4(0, 0, 0, 0);
#pragma unroll
                for (int r = 0; r < R; r++) {
                    int t = acc[r][b];
                    t = __dp4a(wv0[r].x, av0.x, t); t = __dp4a(wv0[r].y, av0.y, t);
                    t = __dp4a(wv0[r].z, av0.z, t); t = __dp4a(wv0[r].w, av0.w, t);
                    t = __dp4a(wv1[r].x, av1.x, t); t = __dp4a(wv1[r].y, av1.y, t);
                    t = __dp4a(wv1[r].z, av1.z, t); t = __dp4a(wv1[r].w, av1.w, t);
                    acc[r][b] = t;
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int b = 0; b < BT; b++) {
            int t = acc[r][b];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            acc[r][b] = t;
        }
    if (KS == 4) {
        int* part = reinterpret_cast<int*>(a_sm + (size_t)BT * kv);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < R; r++)
#pragma unroll
                for (int b = 0; b < BT; b++) part[(warp * R + r) * BT + b] = acc[r][b];
        }
        __syncthreads();
        if (threadIdx.x < R * BT) {
            const int r = threadIdx.x / BT, b = threadIdx.x - r * BT;
            const int n = n0 + r;
            if (n < N && b < M) {
                const int t = part[(0 * R + r) * BT + b] + part[(1 * R + r) * BT + b] + part[(2 * R + r) * BT + b] + part[(3 * R + r) * BT + b];
                if (acc_out) acc_out[(long)b * N + n] = t;
                if (y) {
                    float v = ((float)t * s_tok[b]) * (s_ch ? s_ch[n] : 1.0f);
                    if (residual) v = residual[(long)b * N + n] + v;   // y may alias residual
                    y[(long)b * N + n] = v;
                }
            }
        }
        return;
    }
    if (active && lane == 0) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int n = n0 + r;
            if (n < N) {
                const float sc = s_ch ? s_ch[n] : 1.0f;
#pragma unroll
                for (int b = 0; b < BT; b++)
                    if (b < M) {
                        if (acc_out) acc_out[(long)b * N + n] = acc[r][b];
                        if (y) {
                            float v = ((float)acc[r][b] * s_tok[b]) * sc;
                            if (residual) v = residual[(long)b * N + n] + v;   // y may alias residual
                            y[(long)b * N + n] = v;
                        }
                    }
            }
        }
    }
}

template <int BT, int R, int KS>
static int launch_gemv_as(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch, int M, int N, int K,
                          int32_t* acc, float* y, const float* residual, cudaStream_t st) {
    const size_t smem = (size_t)BT * K + (KS == 4 ? (size_t)4 * R * BT * sizeof(int) : 0);
    auto kern = gemv_i8_kernel<BT, R, KS>;
    if (smem > 48 * 1024) FLEXLLM_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int grid = KS == 1 ? (N + 4 * R - 1) / (4 * R) : (N + R - 1) / R;
    launch_k(kern, dim3(grid), dim3(128), smem, st, a, s_tok, w, s_ch, M, N, K, acc, y, residual);
    return launch_status();
}

template <int BT>
static int launch_gemv(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch, int M, int N, int K,
                       int32_t* acc, float* y, const float* residual, cudaStream_t st) {
    // rows per warp: keep at least ~4 CTAs per SM worth of grid; few channels with long rows: split K over the CTA's warps
    if (N >= 148 * 4 * 4 * 4) return launch_gemv_as<BT, 4, 1>(a, s_tok, w, s_ch, M, N, K, acc, y, residual, st);
    // (every CTA stages all BT activation rows: with many tokens four times as many CTAs cost more than they hide)
    if ((BT <= 2 || (BT == 4 && K >= 4096)) && N / 2 < 148 * 16 && K >= 1024 && (K & 63) == 0)
        return launch_gemv_as<BT, 2, 4>(a, s_tok, w, s_ch, M, N, K, acc, y, residual, st);
    return launch_gemv_as<BT, 2, 1>(a, s_tok, w, s_ch, M, N, K, acc, y, residual, st);
}

// M <= 8 tokens. Returns FLEXLLM_ENOTSUP for larger M (the caller then uses the tensor-core path).
int gemv_i8(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch, int M, int N, int K,
            int32_t* acc, float* y, const float* residual, cudaStream_t st) {
    if (M > 8) return FLEXLLM_ENOTSUP;
    if (M <= 1) return launch_gemv<1>(a, s_tok, w, s_ch, M, N, K, acc, y, residual, st);
    if (M <= 2) return launch_gemv<2>(a, s_tok, w, s_ch, M, N, K, acc, y, residual, st);
    if (M <= 4) return launch_gemv<4>(a, s_tok, w, s_ch, M, N, K, acc, y, residual, st);
    return launch_gemv<8>(a, s_tok, w, s_ch, M, N, K, acc, y, residual, st);
}

}  // namespace flexllm
