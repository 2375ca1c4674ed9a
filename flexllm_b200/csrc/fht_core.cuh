// The 8192-point Walsh-Hadamard butterflies shared by the FHT kernel and the persistent decode-step
// kernel: a row of 8192 floats in (padded) shared memory, 256 threads, three register passes of
// 5 + 5 + 3 stages in the reference's stage order (index bits 1, 2, ..., 12, then 0; Modules/FHT.h:31-53).
#pragma once
#include "common.cuh"

namespace flexllm {

__device__ __forceinline__ int pad32(int i) { return i + (i >> 5); }

template <int B, int N>
__device__ __forceinline__ void reg_butterfly(float (&r)[N]) {
#pragma unroll
    for (int v = 0; v < N; v++) {
        if (!(v & (1 << B))) {
            float lo = r[v], hi = r[v | (1 << B)];
            r[v] = lo + hi;
            r[v | (1 << B)] = lo - hi;
        }
    }
}

// `buf` holds the row at pad32(i); on return thread `tid` of the 256 holds the transformed
// (unscaled) elements i = hi*2048 + tid*8 + c in r[hi*8 + c], hi < 4, c < 8. Synchronises the 256
// threads on named barrier BAR (first thing, so the caller's writes to `buf` need no barrier).
template <int BAR>
__device__ __forceinline__ void fht8192_passes(float* buf, const int tid, float (&r)[32]) {
    named_sync<BAR, 256>();
    // pass 1: index bits 1..5 in registers
    {
        const int base = (tid & 1) | ((tid >> 1) << 6);
#pragma unroll
        for (int v = 0; v < 32; v++) r[v] = buf[pad32(base | (v << 1))];
        reg_butterfly<0>(r); reg_butterfly<1>(r); reg_butterfly<2>(r); reg_butterfly<3>(r); reg_butterfly<4>(r);
#pragma unroll
        for (int v = 0; v < 32; v++) buf[pad32(base | (v << 1))] = r[v];
    }
    named_sync<BAR, 256>();
    // pass 2: index bits 6..10
    {
        const int base = (tid & 63) | ((tid >> 6) << 11);
#pragma unroll
        for (int v = 0; v < 32; v++) r[v] = buf[pad32(base | (v << 6))];
        reg_butterfly<0>(r); reg_butterfly<1>(r); reg_butterfly<2>(r); reg_butterfly<3>(r); reg_butterfly<4>(r);
#pragma unroll
        for (int v = 0; v < 32; v++) buf[pad32(base | (v << 6))] = r[v];
    }
    named_sync<BAR, 256>();
    // pass 3: index bits 11, 12, then 0. Register v: bits 0..2 -> index bits 0..2, bits 3,4 -> 11,12
    {
        const int base = tid << 3;
#pragma unroll
        for (int v = 0; v < 32; v++) r[v] = buf[pad32(base | (v & 7) | ((v >> 3) << 11))];
        reg_butterfly<3>(r); reg_butterfly<4>(r); reg_butterfly<0>(r);
    }
}

}  // namespace flexllm
