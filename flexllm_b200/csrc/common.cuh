// Shared helpers for the sm_100a kernels: status codes, launch checks, warp/block reductions.
// Every translation unit is compiled with -fmad=false: fp32 multiplies and adds are rounded
// separately, exactly as the reference's C simulation does them.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/flexllm_b200.h"

namespace flexllm {

extern thread_local int g_last_cuda_error;
// Number of kernels this library has launched in this process (graph replays count the kernels
// inside the graph). Read through flexllm_launch_count().
extern std::atomic<unsigned long long> g_launch_count;
inline void note_launches(int n) { g_launch_count.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

// Host-side per-device state (function attributes, scratch, error word) is kept in arrays of this size.
constexpr int kMaxDevices = 64;
// Index of the current device, or -1 when it cannot be had or does not fit the per-device arrays.
inline int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    return dev;
}

inline int cuda_status(cudaError_t e) {
    if (e == cudaSuccess) return FLEXLLM_OK;
    g_last_cuda_error = (int)e;
    return FLEXLLM_ECUDA;
}
// status of the `n` launches that have just been issued
inline int launch_status(int n = 1) { note_launches(n); return cuda_status(cudaGetLastError()); }

// Programmatic dependent launch (decode path): when g_pdl is set by the model runner, kernels are
// launched with the stream-serialization attribute relaxed, so the next kernel's launch and CTA
// scheduling overlap the tail of the previous one. Every kernel launched this way calls pdl_sync()
// before it touches memory: it first lets its own dependents start launching, then waits until the
// kernel before it has completed and flushed (so data hazards are exactly those of an ordinary stream).
extern thread_local int g_pdl;
__device__ __forceinline__ void pdl_sync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
template <class... KArgs, class... Args>
inline void launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    if (g_pdl) {
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
    }
    cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

#define FLEXLLM_CHECK_CUDA(expr)                                   \
    do {                                                           \
        int _st = ::flexllm::cuda_status((expr));                  \
        if (_st != FLEXLLM_OK) return _st;                         \
    } while (0)

#define TRY_RC(expr)                          \
    do {                                      \
        int _rc = (expr);                     \
        if (_rc != FLEXLLM_OK) return _rc;    \
    } while (0)

#define FLEXLLM_REQUIRE(cond)                 \
    do {                                      \
        if (!(cond)) return FLEXLLM_EINVAL;   \
    } while (0)

inline bool aligned(const void* p, size_t a) { return ((uintptr_t)p % a) == 0; }

// bar.sync on a named barrier: the NT threads that call it (all of them must) wait for each other.
// BAR = 0 with NT = blockDim synchronises like __syncthreads().
template <int BAR, int NT> __device__ __forceinline__ void named_sync() {
    // the non-aligned form: lanes of a warp may arrive separately (one lane of a warp can be busy
    // issuing TMA or MMA work while the others already wait)
    asm volatile("barrier.sync %0, %1;" ::"n"(BAR), "n"(NT) : "memory");
}

// the barrier number chosen at run time
template <int NT> __device__ __forceinline__ void named_sync_id(int bar) {
    asm volatile("barrier.sync %0, %1;" ::"r"(bar), "n"(NT) : "memory");
}

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

// Same for a group of NT threads (thread index `tid` within the group) that synchronises on named
// barrier BAR, so that other warps of the CTA need not take part.
template <int BAR, int NT> __device__ __forceinline__ void group_max_min(float& mx, float& mn, float* red, int tid) {
    mx = warp_max(mx);
    mn = warp_min(mn);
    const int w = tid >> 5, l = tid & 31;
    constexpr int nw = NT / 32;
    named_sync<BAR, NT>();
    if (l == 0) { red[w] = mx; red[32 + w] = mn; }
    named_sync<BAR, NT>();
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

// round to nearest, halves away from zero (std::round), without a branch: floor(|t| + 0.5) with the sum rounded DOWN is
// exact (an integer is never crossed upwards), the truncating conversion saturates, and the sign is put back
__device__ __forceinline__ int round_half_away_to_int(float t) {
    const int r = __float2int_rz(__fadd_rd(fabsf(t), 0.5f));
    return t < 0.0f ? -r : r;
}

__device__ __forceinline__ int8_t quant_s8(float x, float s) { return (int8_t)round_half_away_to_int(x / s); }

// Correctly rounded x / s for MANY x and ONE s, without the full division each time. With
// y = RN(1/s): q0 = RN(x*y) is within two ulps of x/s; a residual step r = x - q*s (exact in one
// FMA), q' = RN(q + r*y) brings it within one ulp, and by Markstein's theorem a second such step
// from a faithful q with a correctly rounded reciprocal yields RN(x/s) exactly. Valid while no
// intermediate over- or underflows: DivBy::ok says |s| is in [2^-40, 2^40], div_in_range(x) that
// |x| is in [2^-60, 2^60] or zero (zero is returned as x*y: the steps would lose the sign of -0).
// Checked against x / s on the host: all 2^32 x for s = sqrt(8192), and 7e9 random and adversarial
// (x, s) pairs, without a mismatch.
// Callers whose result is only ROUNDED TO AN INTEGER afterwards (quantisers) need no range check on
// x: an x too small for the steps to be exact gives a quotient far below 0.5 either way.
struct DivBy { float s, y; bool ok; };
__device__ __forceinline__ DivBy div_by(float s) {
    DivBy d;
    d.s = s; d.y = 1.0f / s;
    const float as = fabsf(s);
    d.ok = as >= 0x1p-40f && as <= 0x1p40f;
    return d;
}
__device__ __forceinline__ bool div_in_range(float x) {
    const float ax = fabsf(x);
    return ax <= 0x1p60f && (ax >= 0x1p-60f || ax == 0.0f);
}
// branch-free; exact under the conditions above
__device__ __forceinline__ float div_rn_fast(float x, const DivBy& d) {
    const float q0 = __fmul_rn(x, d.y);
    const float r0 = __fmaf_rn(-q0, d.s, x);
    const float q1 = __fmaf_rn(r0, d.y, q0);
    const float r1 = __fmaf_rn(-q1, d.s, x);
    const float q2 = __fmaf_rn(r1, d.y, q1);
    return x == 0.0f ? q0 : q2;
}
__device__ __noinline__ static float div_rn_slow(float x, float s) { return x / s; }
// for quantisers: the quotient is rounded to an integer next (see above); `d.ok` is uniform over the
// row / head, so the branch never diverges and the ordinary division stays out of line
__device__ __forceinline__ float div_for_rounding(float x, const DivBy& d) { return d.ok ? div_rn_fast(x, d) : div_rn_slow(x, d.s); }
// r[i] = RN(r[i] / s) for a register array: one test for the whole array, then the short sequence
template <int N> __device__ __forceinline__ void div_rn_array(float (&r)[N], const DivBy& d) {
    bool fast = d.ok;
#pragma unroll
    for (int i = 0; i < N; i++) fast = fast && div_in_range(r[i]);
    if (fast) {
#pragma unroll
        for (int i = 0; i < N; i++) r[i] = div_rn_fast(r[i], d);
    } else {
#pragma unroll
        for (int i = 0; i < N; i++) r[i] = div_rn_slow(r[i], d.s);
    }
}

// exp() used by SiLU and softmax. The reference calls the C library's expf, whose last-bit
// rounding the C standard leaves open. This build evaluates the CORRECTLY ROUNDED single-precision
// exponential, which (float)exp((double)x) reproduces bit for bit on any host with an accurate
// double-precision libm.
//
// Fast path (|x| < 80), in double precision: x = k*ln2/32 + r with |r| <= ln2/64,
// exp(x) = 2^(k>>5) * 2^((k&31)/32) * exp(r), exp(r) by a degree-5 Taylor polynomial (truncation
// error below 2^-48), the 32-entry table of 2^(j/32) generated with exact integer arithmetic
// (exp_constants.inc). The double result carries a relative error below 2^-45; if it lies within
// that distance of a float rounding boundary (about one input in two million) the accurate library
// exp decides instead, as it does outside the fast range.
#include "exp_constants.inc"
static __device__ double g_exp2_table[32] = FLEXLLM_EXP2_TABLE;

// out of line on purpose: the rare path must not bloat the unrolled loops that call ref_expf
__device__ __noinline__ static float ref_expf_accurate(float x) { return __double2float_rn(exp((double)x)); }

__device__ __forceinline__ float ref_expf(float x) {
    if (x < -104.0f) return 0.0f;                                // exp(x) < 2^-150 rounds to +0
    const double xd = (double)x;
    const double shift = 0x1.8p52;                               // 1.5 * 2^52: adding it rounds to an integer
    const double t = __fma_rn(xd, FLEXLLM_EXP_INV_LN2_32, shift);
    const int k = __double2loint(t);                             // round(x * 32/ln2), |k| < 3700
    const double kd = t - shift;
    double r = __fma_rn(kd, -FLEXLLM_EXP_LN2_32_HI, xd);         // exact: the head has 40 significant bits
    r = __fma_rn(kd, -FLEXLLM_EXP_LN2_32_LO, r);
    double p = __fma_rn(r, 1.0 / 120.0, 1.0 / 24.0);
    p = __fma_rn(p, r, 1.0 / 6.0);
    p = __fma_rn(p, r, 0.5);
    p = __fma_rn(p, r, 1.0);
    p = __fma_rn(p, r, 1.0);
    const double res = __ldg(&g_exp2_table[k & 31]) * p;         // in [0.98, 2.1): exponent field stays in range below
    const int hi = __double2hiint(res) + ((k >> 5) << 20);       // multiply by 2^(k>>5)
    const int lo = __double2loint(res);
    // rounding to float cuts 29 mantissa bits; the boundary pattern is 1 followed by 28 zeros
    const unsigned low29 = (unsigned)lo & 0x1fffffffu;
    const unsigned dist = low29 > 0x10000000u ? low29 - 0x10000000u : 0x10000000u - low29;
    // one rare branch: near a rounding boundary, or outside the fast range (also NaN, overflow,
    // subnormal results)
    if (dist < 256u || !(fabsf(x) < 80.0f)) return ref_expf_accurate(x);
    return __double2float_rn(__hiloint2double(hi, lo));
}

// Four evaluations at once: the same arithmetic per value, written so that the four dependency chains interleave
// (one test and one rare branch for the group instead of one per value).
// EARLY: first test whether all four lie below -104 (masked keys, the tail of a peaked softmax) and return zeros.
template <bool EARLY = false>
__device__ __forceinline__ void ref_expf_x4(const float (&x)[4], float (&e)[4]) {
    if (EARLY && x[0] < -104.0f && x[1] < -104.0f && x[2] < -104.0f && x[3] < -104.0f) {
        e[0] = e[1] = e[2] = e[3] = 0.0f;
        return;
    }
    const double shift = 0x1.8p52;
    unsigned hard = 0u;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const double xd = (double)x[i];
        const double t = __fma_rn(xd, FLEXLLM_EXP_INV_LN2_32, shift);
        const int k = __double2loint(t);
        const double kd = t - shift;
        double r = __fma_rn(kd, -FLEXLLM_EXP_LN2_32_HI, xd);
        r = __fma_rn(kd, -FLEXLLM_EXP_LN2_32_LO, r);
        double p = __fma_rn(r, 1.0 / 120.0, 1.0 / 24.0);
        p = __fma_rn(p, r, 1.0 / 6.0);
        p = __fma_rn(p, r, 0.5);
        p = __fma_rn(p, r, 1.0);
        p = __fma_rn(p, r, 1.0);
        const double res = __ldg(&g_exp2_table[k & 31]) * p;
        const int hi = __double2hiint(res) + ((k >> 5) << 20);
        const int lo = __double2loint(res);
        const unsigned low29 = (unsigned)lo & 0x1fffffffu;
        const unsigned dist = low29 > 0x10000000u ? low29 - 0x10000000u : 0x10000000u - low29;
        const bool zero = x[i] < -104.0f;                               // exp(x) < 2^-150 rounds to +0
        const bool rare = !zero && (dist < 256u || !(fabsf(x[i]) < 80.0f));
        e[i] = zero ? 0.0f : __double2float_rn(__hiloint2double(hi, lo));
        hard |= rare ? (1u << i) : 0u;
    }
    if (hard) {
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (hard & (1u << i)) e[i] = ref_expf_accurate(x[i]);
    }
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + ref_expf(-g)); }
// silu(g) * u on four values (same arithmetic per value)
__device__ __forceinline__ float4 silu_mul_x4(const float4 g, const float4 u) {
    const float x[4] = {-g.x, -g.y, -g.z, -g.w};
    float e[4];
    ref_expf_x4(x, e);
    float4 o;
    o.x = (g.x / (1.0f + e[0])) * u.x; o.y = (g.y / (1.0f + e[1])) * u.y;
    o.z = (g.z / (1.0f + e[2])) * u.z; o.w = (g.w / (1.0f + e[3])) * u.w;
    return o;
}

}  // namespace flexllm
