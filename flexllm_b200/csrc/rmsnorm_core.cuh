// RMSNorm of one row in the reference's DECODE summation order (Modules/LayerNorm.h:210-370 with
// `lanes` chunks of 4 interleaved chains), by one warp that already holds the row in registers:
// lane = chunk*4 + j sums the squares of chunk elements k with k mod 4 == j in increasing k; chunk
// totals (p0+p1)+(p2+p3) are added from 0 in chunk order. Optionally followed by the per-token
// int8 quantiser. Shared by rmsnorm_decode_kernel and the persistent decode-step kernel.
#pragma once
#include "common.cuh"

namespace flexllm {

// v[i] = float4 number (lane + 32 i) of the row (D / 4 of them); g likewise for gamma when KEEP_G,
// else gamma is re-read from memory. buf: D + 4*lanes floats of shared memory owned by this warp.
template <int MAXV, bool KEEP_G>
__device__ __forceinline__ void rmsnorm_decode_row(float4 (&v)[MAXV], float4 (&g)[KEEP_G ? MAXV : 1], const float* __restrict__ gamma,
                                                   const int D, const float eps, const int lanes, float* buf, const int lane,
                                                   float* y_row, int8_t* q_row, float* s_out) {
    const int C = D / lanes;
    const int nv = D >> 2;
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
        const int c = lane + i * 32;
        if (c < nv) { const int e = c * 4; *reinterpret_cast<float4*>(buf + e + 4 * (e / C)) = v[i]; }   // element e at e + 4*(e / C)
    }
    __syncwarp();
    const int chunk = lane >> 2, j = lane & 3;
    float ss = 0.0f;
    if (chunk < lanes) {
        const float* bc = buf + chunk * (C + 4);
        const int n = C >> 2;
#pragma unroll 8
        for (int k = 0; k < n; k++) { const float t = bc[4 * k + j]; ss += t * t; }
    }
    float tot = 0.0f;
    for (int c = 0; c < lanes; c++) {
        const float p0 = __shfl_sync(0xffffffffu, ss, c * 4 + 0), p1 = __shfl_sync(0xffffffffu, ss, c * 4 + 1);
        const float p2 = __shfl_sync(0xffffffffu, ss, c * 4 + 2), p3 = __shfl_sync(0xffffffffu, ss, c * 4 + 3);
        tot += (p0 + p1) + (p2 + p3);
    }
    const float r = 1.0f / sqrtf(tot / (float)D + eps);
    float mx = -1e32f, mn = 1e32f;
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
        const int c = lane + i * 32;
        if (c < nv) {
            const float4 gg = KEEP_G ? g[KEEP_G ? i : 0] : reinterpret_cast<const float4*>(gamma)[c];
            float4 o;
            o.x = (v[i].x * r) * gg.x; o.y = (v[i].y * r) * gg.y; o.z = (v[i].z * r) * gg.z; o.w = (v[i].w * r) * gg.w;
            v[i] = o;
            if (y_row) reinterpret_cast<float4*>(y_row)[c] = o;
            mx = fmaxf(mx, fmaxf(fmaxf(o.x, o.y), fmaxf(o.z, o.w)));
            mn = fminf(mn, fminf(fminf(o.x, o.y), fminf(o.z, o.w)));
        }
    }
    if (q_row) {
        mx = warp_max(mx); mn = warp_min(mn);
        const float sc = sym_scale_from(mx, mn);
    const DivBy dsc = div_by(sc);       // one reciprocal per row: every element is then quantised without a full division
        if (lane == 0) *s_out = sc;
        char4* qr = reinterpret_cast<char4*>(q_row);
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
            const int c = lane + i * 32;
            if (c < nv) {
                char4 o;
                o.x = (int8_t)round_half_away_to_int(div_for_rounding(v[i].x, dsc)); o.y = (int8_t)round_half_away_to_int(div_for_rounding(v[i].y, dsc)); o.z = (int8_t)round_half_away_to_int(div_for_rounding(v[i].z, dsc)); o.w = (int8_t)round_half_away_to_int(div_for_rounding(v[i].w, dsc));
                qr[c] = o;
            }
        }
    }
}

}  // namespace flexllm
