// Shared helpers for the sm_100a kernels: status codes, launch checks, warp/block reductions.
// Every translation unit is compiled with -fmad=false: fp32 multiplies and adds are rounded
// separately, exactly as the reference's C simulation does them.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/flexllm_b200.h"

namespace flexllm {

extern thread_local int g_last_cuda_error;
// Number of kernels this library has launched in this process (graph replays count the kernels
// inside the graph). Read through flexllm_launch_count().
extern unsigned long long g_launch_count;
inline void note_launches(int n) { g_launch_count += (unsigned long long)n; }

inline int cuda_status(cudaError_t e) {
    if (e == cudaSuccess) return FLEXLLM_OK;
    g_last_cuda_error = (int)e;
    return FLEXLLM_ECUDA;
}
// status of the `n` launches that have just been issued
inline int launch_status(int n = 1) { note_launches(n); return cuda_status(cudaGetLastError()); }

#define FLEXLLM_CHECK_CUDA(expr)                                   \
    do {                                                           \
        int _st = ::flexllm::cuda_status((expr));                  \
        if (_st != FLEXLLM_OK) return _st;                         \
    } while (0)

#define FLEXLLM_REQUIRE(cond)                 \
    do {                                      \
        if (!(cond)) return FLEXLLM_EINVAL;   \
    } while (0)

inline bool aligned(const void* p, size_t a) { return ((uintptr_t)p % a) == 0; }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide max and min (order-free, hence exact). `red` needs 64 floats of shared memory.
__device__ __forceinline__ void block_max_min(float& mx, float& mn, float* red) {
    mx = warp_max(mx);
    mn = warp_min(mn);
    int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (l == 0) { red[w] = mx; red[32 + w] = mn; }
    __syncthreads();
    float a = (l < nw) ? red[l] : -1e32f;
    float b = (l < nw) ? red[32 + l] : 1e32f;
    mx = warp_max(a);
    mn = warp_min(b);
}

// Symmetric 8-bit scale from a row's max and min (Modules/quant.h:84-96).
__device__ __forceinline__ float sym_scale_from(float mx, float mn) {
    float a = fabsf(mx), b = fabsf(mn);
    float s = (a > b ? a : b) / 127.0f;
    if (s == 0.0f) s = 1.0f;
    return s;
}

__device__ __forceinline__ int8_t quant_s8(float x, float s) { return (int8_t)(int)roundf(x / s); }

// exp() used by SiLU and softmax. The reference calls the C library's expf, whose last-bit
// rounding the C standard leaves open. This build evaluates the CORRECTLY ROUNDED single-precision
// exponential: exp in double precision (error below one double ulp), rounded once to fp32. The
// result is independent of the device math library's fp32 approximation and is reproduced bit for
// bit by (float)exp((double)x) on any host with an accurate double-precision libm.
__device__ __forceinline__ float ref_expf(float x) { return __double2float_rn(exp((double)x)); }

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + ref_expf(-g)); }

}  // namespace flexllm
