// Row-wise and elementwise operators of the quantized Llama path: per-token quantisation, dequant,
// static quantisation, RMSNorm(+quant), SiLU, gate, residual, RoPE, softmax, greedy argmax.
// All are HBM-bound: one pass over the data with 128-bit accesses where the layout allows.
#include <atomic>

#include "common.cuh"
#include "rmsnorm_core.cuh"

namespace flexllm {

thread_local int g_last_cuda_error = 0;
thread_local int g_pdl = 0;
std::atomic<unsigned long long> g_launch_count{0};

// ---------------------------------------------------------------------------------------------
// Per-token symmetric int8 quantisation (Modules/quant.h:6-112, symmetric branch).
// One CTA per row; the row stays in registers between the max/min pass and the rounding pass.
// ---------------------------------------------------------------------------------------------
template <int VPT>  // float4 vectors per thread
__global__ void __launch_bounds__(256) quant_per_token_kernel(const float* __restrict__ x, int K,
                                                              int8_t* __restrict__ q, float* __restrict__ s) {
    __shared__ float red[64];
    pdl_sync();
    const long row = blockIdx.x;
    const float4* xr = reinterpret_cast<const float4*>(x + row * K);
    const int nv = K >> 2;
    float4 v[VPT];
    float mx = -1e32f, mn = 1e32f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        int c = threadIdx.x + i * 256;
        if (c < nv) {
            v[i] = xr[c];
            mx = fmaxf(mx, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
            mn = fminf(mn, fminf(fminf(v[i].x, v[i].y), fminf(v[i].z, v[i].w)));
        }
    }
    block_max_min(mx, mn, red);
    const float sc = sym_scale_from(mx, mn);
    const DivBy dsc = div_by(sc);       // one reciprocal per row: every element is then quantised without a full division
    if (threadIdx.x == 0) s[row] = sc;
    char4* qr = reinterpret_cast<char4*>(q + row * K);
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        int c = threadIdx.x + i * 256;
        if (c < nv) {
            char4 o;
            o.x = (int8_t)round_half_away_to_int(div_for_rounding(v[i].x, dsc)); o.y = (int8_t)round_half_away_to_int(div_for_rounding(v[i].y, dsc));
            o.z = (int8_t)round_half_away_to_int(div_for_rounding(v[i].z, dsc)); o.w = (int8_t)round_half_away_to_int(div_for_rounding(v[i].w, dsc));
            qr[c] = o;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Asymmetric per-token quantisation (Modules/quant.h:53-81): s = (max - min) / (2^bits - 1) (0 -> 1), zero point
// b = min, q = (unsigned) round((x - b) / s). Same structure as the symmetric kernel above.
// ---------------------------------------------------------------------------------------------
template <int VPT>
__global__ void __launch_bounds__(256) quant_per_token_asym_kernel(const float* __restrict__ x, int K, float base, unsigned mask,
                                                                   uint8_t* __restrict__ q, float* __restrict__ s, float* __restrict__ b) {
    __shared__ float red[64];
    const long row = blockIdx.x;
    const float4* xr = reinterpret_cast<const float4*>(x + row * K);
    const int nv = K >> 2;
    float4 v[VPT];
    float mx = -1e32f, mn = 1e32f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        int c = threadIdx.x + i * 256;
        if (c < nv) {
            v[i] = xr[c];
            mx = fmaxf(mx, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
            mn = fminf(mn, fminf(fminf(v[i].x, v[i].y), fminf(v[i].z, v[i].w)));
        }
    }
    block_max_min(mx, mn, red);
    float sc = (mx - mn) / base;
    if (sc == 0.0f) sc = 1.0f;
    if (threadIdx.x == 0) { s[row] = sc; b[row] = mn; }
    uchar4* qr = reinterpret_cast<uchar4*>(q + row * K);
    auto qz = [&](float t) { return (unsigned char)((unsigned)(long long)roundf((t - mn) / sc) & mask); };
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        int c = threadIdx.x + i * 256;
        if (c < nv) qr[c] = make_uchar4(qz(v[i].x), qz(v[i].y), qz(v[i].z), qz(v[i].w));
    }
}

// y = ((float)acc * s_tok[m]) * s_ch[n] + b_tok[m] * wsum[n]     (Modules/quant.h:146-148; every operation rounded on its own)
__global__ void dequant_asym_kernel(const int32_t* __restrict__ acc, const float* __restrict__ s_tok, const float* __restrict__ b_tok,
                                    const float* __restrict__ s_ch, const float* __restrict__ wsum, int M, int N, float* __restrict__ y) {
    const long nv = (long)M * (N >> 2);
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
        const int m = (int)(i / (N >> 2)), c = (int)(i % (N >> 2));
        const int4 a = reinterpret_cast<const int4*>(acc)[i];
        const float4 w = reinterpret_cast<const float4*>(s_ch)[c];
        const float4 z = reinterpret_cast<const float4*>(wsum)[c];
        const float st = s_tok[m], bt = b_tok[m];
        float4 o;
        o.x = ((float)a.x * st) * w.x + bt * z.x; o.y = ((float)a.y * st) * w.y + bt * z.y;
        o.z = ((float)a.z * st) * w.z + bt * z.z; o.w = ((float)a.w * st) * w.w + bt * z.w;
        reinterpret_cast<float4*>(y)[i] = o;
    }
}

// ---------------------------------------------------------------------------------------------
// Dequant (Modules/quant.h:151): y = ((float)acc * s_tok[m]) * s_ch[n]
// ---------------------------------------------------------------------------------------------
__global__ void dequant_kernel(const int32_t* __restrict__ acc, const float* __restrict__ s_tok,
                               const float* __restrict__ s_ch, int M, int N, float* __restrict__ y) {
    const long nv = (long)M * (N >> 2);
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
        int m = (int)(i / (N >> 2)), c = (int)(i % (N >> 2));
        int4 a = reinterpret_cast<const int4*>(acc)[i];
        float4 w = reinterpret_cast<const float4*>(s_ch)[c];
        float st = s_tok[m];
        float4 o;
        o.x = ((float)a.x * st) * w.x; o.y = ((float)a.y * st) * w.y;
        o.z = ((float)a.z * st) * w.z; o.w = ((float)a.w * st) * w.w;
        reinterpret_cast<float4*>(y)[i] = o;
    }
}

// ---------------------------------------------------------------------------------------------
// Static symmetric quantisation (Modules/quant.h:252-295, :166-211)
// ---------------------------------------------------------------------------------------------
__global__ void static_quant_kernel(const float* __restrict__ x, long rows, int n, const float* __restrict__ s,
                                    int s_stride, float f, int is_signed, uint8_t* __restrict__ q) {
    const long total = rows * n;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        long r = i / n;
        float d = f * s[r * s_stride];
        int v = (int)roundf(x[i] / d);
        if (is_signed) v = v > 127 ? 127 : (v < -128 ? -128 : v);
        else v = v > 255 ? 255 : v;
        q[i] = (uint8_t)v;
    }
}

// ---------------------------------------------------------------------------------------------
// RMSNorm (+ optional per-token int8 quant).
// Sum of squares follows the reference order exactly:
//   prefill (LayerNorm.h:82-114): 4 chains j = k mod 4 over the whole row, (p0+p1)+(p2+p3);
//   decode  (LayerNorm.h:263-300): `lanes` contiguous chunks, 4 chains inside each, chunk totals
//                                  added from 0 in chunk order.
// A chain is a strictly sequential fp32 accumulation, so one thread owns it. To keep all 32 lanes
// busy a warp runs 32 chains at once: in the prefill order the 4 chains of 8 different rows, in the
// decode order the (up to) 32 chains of one row. The rows sit in shared memory (prefill) or in
// registers (decode) between the sum and the output pass: each is read from global memory once.
// ---------------------------------------------------------------------------------------------
constexpr int RMS_WARPS = 4;
constexpr int RMS_PIECE = 128;           // floats per row per staging step
constexpr int RMS_PSTRIDE = RMS_PIECE + 4;   // padded: rows land in different banks

template <int MAXV>  // float4 per lane kept in registers for the output pass (D <= MAXV*128)
__device__ __forceinline__ void rmsnorm_output_row(const float* __restrict__ xr, const float* __restrict__ gamma, int D, float r,
                                                   float* __restrict__ yr, int8_t* __restrict__ qr8, float* __restrict__ srow, int lane) {
    const int nv = D >> 2;
    float4 o[MAXV];
    float mx = -1e32f, mn = 1e32f;
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
        int c = lane + i * 32;
        if (c < nv) {
            float4 v = reinterpret_cast<const float4*>(xr)[c];
            float4 g = reinterpret_cast<const float4*>(gamma)[c];
            o[i].x = (v.x * r) * g.x; o[i].y = (v.y * r) * g.y; o[i].z = (v.z * r) * g.z; o[i].w = (v.w * r) * g.w;
            if (yr) reinterpret_cast<float4*>(yr)[c] = o[i];
            mx = fmaxf(mx, fmaxf(fmaxf(o[i].x, o[i].y), fmaxf(o[i].z, o[i].w)));
            mn = fminf(mn, fminf(fminf(o[i].x, o[i].y), fminf(o[i].z, o[i].w)));
        }
    }
    if (qr8) {
        mx = warp_max(mx); mn = warp_min(mn);
        const float sc = sym_scale_from(mx, mn);
    const DivBy dsc = div_by(sc);       // one reciprocal per row: every element is then quantised without a full division
        if (lane == 0) *srow = sc;
        char4* qr = reinterpret_cast<char4*>(qr8);
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
            int c = lane + i * 32;
            if (c < nv) {
                char4 w;
                w.x = (int8_t)round_half_away_to_int(div_for_rounding(o[i].x, dsc)); w.y = (int8_t)round_half_away_to_int(div_for_rounding(o[i].y, dsc)); w.z = (int8_t)round_half_away_to_int(div_for_rounding(o[i].z, dsc)); w.w = (int8_t)round_half_away_to_int(div_for_rounding(o[i].w, dsc));
                qr[c] = w;
            }
        }
    }
}

// Prefill order: a CTA of 8 warps takes 8 consecutive rows. All threads bring the rows into shared memory (coalesced
// 128-bit loads, all in flight at once); warp 0 then runs the 32 chains (4 per row) over them; afterwards every warp
// normalises and quantises one row straight from shared memory -- each row is read from global memory once. Row stride
// D + 4 floats: the 32 chains' reads (row rr, element 4k + j) fall into 32 different banks. Requires D % 128 == 0.
constexpr int RMSP_ROWS = 8;
__global__ void __launch_bounds__(RMSP_ROWS * 32) rmsnorm_prefill_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                                         int M, int D, float eps, float* __restrict__ y,
                                                                         int8_t* __restrict__ q, float* __restrict__ s) {
    extern __shared__ __align__(16) float rows_sm[];          // [8][D + 4], then rinv[8]
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ld = D + 4, nv = D >> 2;
    const long row0 = (long)blockIdx.x * RMSP_ROWS;
    float* rinv_sm = rows_sm + RMSP_ROWS * ld;
    {   // warp w brings in row w
        const bool in = row0 + w < M;
        const float4* src = reinterpret_cast<const float4*>(x + (row0 + w) * D);
        float4* dst = reinterpret_cast<float4*>(rows_sm + w * ld);
        for (int c = lane; c < nv; c += 32) dst[c] = in ? src[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncthreads();
    if (w == 0) {
        const int rr = lane >> 2, j = lane & 3;      // chain (row rr, residue j)
        const float* src = rows_sm + rr * ld + j;
        float ss = 0.0f;
#pragma unroll 8
        for (int k = 0; k < nv; k++) { const float v = src[4 * k]; ss += v * v; }
        // (p0+p1)+(p2+p3) inside each group of four lanes
        const int base = lane & ~3;
        const float p0 = __shfl_sync(0xffffffffu, ss, base), p1 = __shfl_sync(0xffffffffu, ss, base + 1);
        const float p2 = __shfl_sync(0xffffffffu, ss, base + 2), p3 = __shfl_sync(0xffffffffu, ss, base + 3);
        const float tot = (p0 + p1) + (p2 + p3);
        if (j == 0) rinv_sm[rr] = 1.0f / sqrtf(tot / (float)D + eps);
    }
    __syncthreads();
    const long row = row0 + w;
    if (row >= M) return;
    const float r = rinv_sm[w];
    const float4* xr = reinterpret_cast<const float4*>(rows_sm + w * ld);
    const float4* g4 = reinterpret_cast<const float4*>(gamma);
    float4* yr = y ? reinterpret_cast<float4*>(y + row * D) : nullptr;
    // first pass: the normalised row's largest magnitude (max(|max|, |min|) of the row = max of |.|), fp32 output if asked for;
    // second pass: the same products again (same bits) and the quantiser -- nothing of the row is held in registers
    float amax = 0.0f;
#pragma unroll 4
    for (int c = lane; c < nv; c += 32) {
        const float4 v = xr[c], g = g4[c];
        float4 o;
        o.x = (v.x * r) * g.x; o.y = (v.y * r) * g.y; o.z = (v.z * r) * g.z; o.w = (v.w * r) * g.w;
        if (yr) yr[c] = o;
        amax = fmaxf(fmaxf(amax, fabsf(o.x)), fmaxf(fabsf(o.y), fmaxf(fabsf(o.z), fabsf(o.w))));
    }
    if (q) {
        amax = warp_max(amax);
        float sc = amax / 127.0f;
        if (sc == 0.0f) sc = 1.0f;
        const DivBy dsc = div_by(sc);       // one reciprocal per row: every element is then quantised without a full division
        if (lane == 0) s[row] = sc;
        char4* qr = reinterpret_cast<char4*>(q + row * D);
        auto q8 = [&](float t) {            // round half away from zero of the correctly rounded quotient; |quotient| <= 127
            const float qt = div_for_rounding(t, dsc);
            const int m = __float2int_rz(__fadd_rd(fabsf(qt), 0.5f));
            return (int8_t)(qt < 0.0f ? -m : m);
        };
#pragma unroll 4
        for (int c = lane; c < nv; c += 32) {
            const float4 v = xr[c], g = g4[c];
            char4 v4;
            v4.x = q8((v.x * r) * g.x); v4.y = q8((v.y * r) * g.y); v4.z = q8((v.z * r) * g.z); v4.w = q8((v.w * r) * g.w);
            qr[c] = v4;
        }
    }
}

// Decode order with `lanes` (4 or 8) chunks: one warp per row, lane = chunk*4 + j. The row and gamma
// are fetched with one batch of independent 128-bit loads and stay in registers for the output pass
// (a decode step is latency-bound: one global round trip instead of one per loop iteration).
template <int MAXV>
__global__ void __launch_bounds__(RMS_WARPS * 32) rmsnorm_decode_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                                        int M, int D, float eps, int lanes, float* __restrict__ y,
                                                                        int8_t* __restrict__ q, float* __restrict__ s) {
    extern __shared__ __align__(16) float rowbuf[];          // RMS_WARPS x (D + 4*lanes)
    pdl_sync();
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long row = (long)blockIdx.x * RMS_WARPS + w;
    if (row >= M) return;
    const int nv = D >> 2;
    float* buf = rowbuf + (size_t)w * (D + 4 * lanes);
    const float* xr = x + row * D;
    constexpr bool KEEP_G = MAXV <= 16;                       // gamma in registers too when it fits
    float4 v[MAXV], g[KEEP_G ? MAXV : 1];
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
        const int c = lane + i * 32;
        if (c < nv) { v[i] = reinterpret_cast<const float4*>(xr)[c]; if (KEEP_G) g[i] = reinterpret_cast<const float4*>(gamma)[c]; }
    }
    rmsnorm_decode_row<MAXV, KEEP_G>(v, g, gamma, D, eps, lanes, buf, lane, y ? y + row * D : nullptr, q ? q + row * D : nullptr,
                                     s ? s + row : nullptr);
}

// ---------------------------------------------------------------------------------------------
// SiLU / gate / residual (Swish.h:19, Linear_Layer.h:626, Residual_Layer.h:61)
// ---------------------------------------------------------------------------------------------
template <int OP>  // 0 silu, 1 mul, 2 add
__global__ void eltwise_kernel(const float* __restrict__ a, const float* __restrict__ b, long n, float* __restrict__ y) {
    const long nv = n >> 2;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
        float4 u = reinterpret_cast<const float4*>(a)[i];
        float4 o;
        if (OP == 0) { o.x = silu_f(u.x); o.y = silu_f(u.y); o.z = silu_f(u.z); o.w = silu_f(u.w); }
        else {
            float4 v = reinterpret_cast<const float4*>(b)[i];
            if (OP == 1) { o.x = u.x * v.x; o.y = u.y * v.y; o.z = u.z * v.z; o.w = u.w * v.w; }
            else { o.x = u.x + v.x; o.y = u.y + v.y; o.z = u.z + v.z; o.w = u.w + v.w; }
        }
        reinterpret_cast<float4*>(y)[i] = o;
    }
    // tail
    for (long i = (nv << 2) + blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        if (OP == 0) y[i] = silu_f(a[i]);
        else if (OP == 1) y[i] = a[i] * b[i];
        else y[i] = a[i] + b[i];
    }
}

// ---------------------------------------------------------------------------------------------
// RoPE by table (RoPE.h:61-90): one warp per (token, head); lane k holds x[k] and x[k+32].
// ---------------------------------------------------------------------------------------------
__global__ void rope_kernel(const float* __restrict__ x, const int32_t* __restrict__ pos, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, long T, int H, float* __restrict__ y) {
    const long w = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= T * H) return;
    const long t = w / H;
    const int p = pos[t];
    const float c = cos_t[(long)p * 32 + lane], sn = sin_t[(long)p * 32 + lane];
    const float x0 = x[w * 64 + lane], x1 = x[w * 64 + 32 + lane];
    y[w * 64 + lane] = x0 * c - x1 * sn;
    y[w * 64 + 32 + lane] = x0 * sn + x1 * c;
}

// ---------------------------------------------------------------------------------------------
// Softmax (Softmax.h:25-161 / :474-634): one warp per row. exp values are written to p first,
// then lanes 0..3 run the four sequential chains k = j mod 4, then every lane scales.
// ---------------------------------------------------------------------------------------------
__global__ void softmax_kernel(const float* __restrict__ x, long rows, int len, const int32_t* __restrict__ valid,
                               float* __restrict__ p) {
    const long row = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* xr = x + row * len;
    float* pr = p + row * len;
    const int nvld = valid ? valid[row] : len;
    float mx = -1e32f;
    for (int k = lane; k < len; k += 32) {
        float v = k < nvld ? xr[k] : -1e32f;
        mx = v > mx ? v : mx;
    }
    mx = warp_max(mx);
    for (int k = lane; k < len; k += 32) {
        float v = k < nvld ? xr[k] : -1e32f;
        pr[k] = ref_expf(v - mx);
    }
    __syncwarp();
    float ps = 0.0f;
    if (lane < 4) {
#pragma unroll 8
        for (int k = lane; k < len; k += 4) ps += pr[k];
    }
    float p0 = __shfl_sync(0xffffffffu, ps, 0), p1 = __shfl_sync(0xffffffffu, ps, 1);
    float p2 = __shfl_sync(0xffffffffu, ps, 2), p3 = __shfl_sync(0xffffffffu, ps, 3);
    const float r = 1.0f / ((p0 + p1) + (p2 + p3));
    for (int k = lane; k < len; k += 32) pr[k] = pr[k] * r;
}

// ---------------------------------------------------------------------------------------------
// Greedy argmax, ties to the lowest index (Logits.h:13-17 strict '>'). One CTA per row.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, long V, int32_t* __restrict__ idx) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_sync();
    const float* l = logits + (long)blockIdx.x * V;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (long v = threadIdx.x; v < V; v += blockDim.x) {
        float t = l[v];
        if (t > best || bi == 0x7fffffff) { best = t; bi = (int)v; }   // strided scan visits increasing v
    }
    auto better = [](float a, int ai, float b, int bi2) { return a > b || (a == b && ai < bi2); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ob, oi, best, bi)) { best = ob; bi = oi; }
    }
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[w] = best; si[w] = bi; }
    __syncthreads();
    if (w == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ob = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ob, oi, best, bi)) { best = ob; bi = oi; }
        }
        if (lane == 0) idx[blockIdx.x] = bi;
    }
}

static inline int grid_for(long n, int block, int cap = 148 * 16) {
    long g = (n + block - 1) / block;
    if (g < 1) g = 1;
    return (int)(g > cap ? cap : g);
}

}  // namespace flexllm

using namespace flexllm;

extern "C" int flexllm_version(void) { return 100; }

extern "C" const char* flexllm_status_string(int st) {
    switch (st) {
        case FLEXLLM_OK: return "ok";
        case FLEXLLM_EINVAL: return "invalid argument";
        case FLEXLLM_ECUDA: return "CUDA error";
        case FLEXLLM_ETIMEDOUT: return "device wait timed out";
        case FLEXLLM_ENOTSUP: return "unsupported shape";
        case FLEXLLM_ENOMEM: return "out of memory";
        case FLEXLLM_ETOOBIG: return "problem exceeds a fixed built-in buffer";
        case FLEXLLM_EDEVDATA: return "token id or context length in device memory out of range (clamped)";
        case FLEXLLM_EIO: return "parameter file missing or too short";
        default: return "unknown status";
    }
}

extern "C" int flexllm_last_cuda_error(void) { return g_last_cuda_error; }
extern "C" unsigned long long flexllm_launch_count(void) { return g_launch_count.load(std::memory_order_relaxed); }

extern "C" int flexllm_quant_per_token(const float* x, int M, int K, int8_t* q, float* s, void* stream) {
    FLEXLLM_REQUIRE(M >= 0 && K > 0 && (K % 4) == 0 && K <= 8192);
    if (M == 0) return FLEXLLM_OK;   // empty batch: nothing to do, pointers may be null
    FLEXLLM_REQUIRE(x && q && s);
    FLEXLLM_REQUIRE(aligned(x, 16) && aligned(q, 4));
    cudaStream_t st = (cudaStream_t)stream;
    const int nv = K / 4;
    if (nv <= 256) launch_k(quant_per_token_kernel<1>, dim3(M), dim3(256), 0, st, x, K, q, s);
    else if (nv <= 512) launch_k(quant_per_token_kernel<2>, dim3(M), dim3(256), 0, st, x, K, q, s);
    else if (nv <= 1024) launch_k(quant_per_token_kernel<4>, dim3(M), dim3(256), 0, st, x, K, q, s);
    else launch_k(quant_per_token_kernel<8>, dim3(M), dim3(256), 0, st, x, K, q, s);
    return launch_status();
}

extern "C" int flexllm_quant_per_token_asym(const float* x, int M, int K, int bits, uint8_t* q, float* s, float* b, void* stream) {
    FLEXLLM_REQUIRE(M >= 0 && K > 0 && (K % 4) == 0 && K <= 8192);
    if (bits < 2 || bits > 7) return FLEXLLM_ENOTSUP;
    if (M == 0) return FLEXLLM_OK;
    FLEXLLM_REQUIRE(x && q && s && b && aligned(x, 16) && aligned(q, 4));
    cudaStream_t st = (cudaStream_t)stream;
    const float base = (float)((1 << bits) - 1);
    const unsigned mask = (1u << bits) - 1u;
    const int nv = K / 4;
    if (nv <= 256) quant_per_token_asym_kernel<1><<<M, 256, 0, st>>>(x, K, base, mask, q, s, b);
    else if (nv <= 512) quant_per_token_asym_kernel<2><<<M, 256, 0, st>>>(x, K, base, mask, q, s, b);
    else if (nv <= 1024) quant_per_token_asym_kernel<4><<<M, 256, 0, st>>>(x, K, base, mask, q, s, b);
    else quant_per_token_asym_kernel<8><<<M, 256, 0, st>>>(x, K, base, mask, q, s, b);
    return launch_status();
}

extern "C" int flexllm_dequant_asym(const int32_t* acc, const float* s_tok, const float* b_tok, const float* s_ch, const float* wsum,
                                    int M, int N, float* y, void* stream) {
    FLEXLLM_REQUIRE(acc && s_tok && b_tok && s_ch && wsum && y && M >= 0 && N > 0 && (N % 4) == 0);
    FLEXLLM_REQUIRE(aligned(acc, 16) && aligned(s_ch, 16) && aligned(wsum, 16) && aligned(y, 16));
    if (M == 0) return FLEXLLM_OK;
    dequant_asym_kernel<<<grid_for((long)M * N / 4, 256), 256, 0, (cudaStream_t)stream>>>(acc, s_tok, b_tok, s_ch, wsum, M, N, y);
    return launch_status();
}

// The integer product of the asymmetric layers runs on the int8 GEMMs (activation values of up to 7 bits are non-negative
// int8); the zero point enters in the dequantiser.
extern "C" int flexllm_linear_prefill_asym(const uint8_t* a, const float* s_tok, const float* b_tok, const int8_t* w, const float* s_ch,
                                           const float* wsum, int M, int N, int K, int32_t* acc, float* y, void* stream) {
    FLEXLLM_REQUIRE(acc && y);
    TRY_RC(flexllm_linear_prefill_i8(reinterpret_cast<const int8_t*>(a), nullptr, w, nullptr, M, N, K, acc, nullptr, stream));
    return flexllm_dequant_asym(acc, s_tok, b_tok, s_ch, wsum, M, N, y, stream);
}
extern "C" int flexllm_linear_decode_asym(const uint8_t* a, const float* s_tok, const float* b_tok, const int8_t* w, const float* s_ch,
                                          const float* wsum, int M, int N, int K, int32_t* acc, float* y, void* stream) {
    FLEXLLM_REQUIRE(acc && y);
    TRY_RC(flexllm_linear_decode_i8(reinterpret_cast<const int8_t*>(a), nullptr, w, nullptr, M, N, K, acc, nullptr, stream));
    return flexllm_dequant_asym(acc, s_tok, b_tok, s_ch, wsum, M, N, y, stream);
}

extern "C" int flexllm_dequant(const int32_t* acc, const float* s_tok, const float* s_ch, int M, int N, float* y,
                               void* stream) {
    FLEXLLM_REQUIRE(acc && s_tok && s_ch && y && M >= 0 && N > 0 && (N % 4) == 0);
    FLEXLLM_REQUIRE(aligned(acc, 16) && aligned(s_ch, 16) && aligned(y, 16));
    if (M == 0) return FLEXLLM_OK;
    dequant_kernel<<<grid_for((long)M * N / 4, 256), 256, 0, (cudaStream_t)stream>>>(acc, s_tok, s_ch, M, N, y);
    return launch_status();
}

extern "C" int flexllm_static_quant(const float* x, long rows, int n, const float* s, int s_stride, float f,
                                    int is_signed, uint8_t* q, void* stream) {
    FLEXLLM_REQUIRE(x && s && q && rows >= 0 && n > 0 && (s_stride == 0 || s_stride == 1));
    if (rows == 0) return FLEXLLM_OK;
    static_quant_kernel<<<grid_for(rows * n, 256), 256, 0, (cudaStream_t)stream>>>(x, rows, n, s, s_stride, f, is_signed, q);
    return launch_status();
}

extern "C" int flexllm_rmsnorm_quant(const float* x, const float* gamma, int M, int D, float eps, int order,
                                     float* y, int8_t* q, float* s, void* stream) {
    FLEXLLM_REQUIRE(x && gamma && (y || q) && (!q || s) && M >= 0 && D > 0);
    FLEXLLM_REQUIRE((D % 4) == 0 && D <= 4096 && (order == 0 || order == 4 || order == 8));
    FLEXLLM_REQUIRE(order == 0 || (D % (order * 4)) == 0);
    FLEXLLM_REQUIRE(aligned(x, 16) && aligned(gamma, 16) && (!y || aligned(y, 16)) && (!q || aligned(q, 4)));
    if (M == 0) return FLEXLLM_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (order == 0) {
        if (D % RMS_PIECE != 0) return FLEXLLM_ENOTSUP;
        const int grid = (M + RMSP_ROWS - 1) / RMSP_ROWS;
        const size_t smem = ((size_t)RMSP_ROWS * (D + 4) + RMSP_ROWS) * sizeof(float);
        static std::atomic<int> attr_done[kMaxDevices];
        const int dev = current_device();
        if (dev < 0) return FLEXLLM_ECUDA;
        if (!attr_done[dev].load(std::memory_order_acquire)) {
            FLEXLLM_CHECK_CUDA(cudaFuncSetAttribute(rmsnorm_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    (int)(((size_t)RMSP_ROWS * (4096 + 4) + RMSP_ROWS) * sizeof(float))));
            // three 66 KB CTAs per SM need the largest shared-memory carve-out
            FLEXLLM_CHECK_CUDA(cudaFuncSetAttribute(rmsnorm_prefill_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
            attr_done[dev].store(1, std::memory_order_release);
        }
        rmsnorm_prefill_kernel<<<grid, RMSP_ROWS * 32, smem, st>>>(x, gamma, M, D, eps, y, q, s);
    } else {
        const int grid = (M + RMS_WARPS - 1) / RMS_WARPS;
        const size_t smem = (size_t)RMS_WARPS * (D + 4 * order) * sizeof(float);
        if (D <= 2048) launch_k(rmsnorm_decode_kernel<16>, dim3(grid), dim3(RMS_WARPS * 32), smem, st, x, gamma, M, D, eps, order, y, q, s);
        else {
            FLEXLLM_CHECK_CUDA(cudaFuncSetAttribute(rmsnorm_decode_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            rmsnorm_decode_kernel<32><<<grid, RMS_WARPS * 32, smem, st>>>(x, gamma, M, D, eps, order, y, q, s);
        }
    }
    return launch_status();
}

extern "C" int flexllm_swish(const float* g, long n, float* y, void* stream) {
    FLEXLLM_REQUIRE(g && y && n >= 0 && aligned(g, 16) && aligned(y, 16));
    if (n == 0) return FLEXLLM_OK;
    eltwise_kernel<0><<<grid_for((n + 3) / 4, 256), 256, 0, (cudaStream_t)stream>>>(g, nullptr, n, y);
    return launch_status();
}
extern "C" int flexllm_gate(const float* a, const float* b, long n, float* y, void* stream) {
    FLEXLLM_REQUIRE(a && b && y && n >= 0 && aligned(a, 16) && aligned(b, 16) && aligned(y, 16));
    if (n == 0) return FLEXLLM_OK;
    eltwise_kernel<1><<<grid_for((n + 3) / 4, 256), 256, 0, (cudaStream_t)stream>>>(a, b, n, y);
    return launch_status();
}
extern "C" int flexllm_residual(const float* a, const float* b, long n, float* y, void* stream) {
    FLEXLLM_REQUIRE(a && b && y && n >= 0 && aligned(a, 16) && aligned(b, 16) && aligned(y, 16));
    if (n == 0) return FLEXLLM_OK;
    eltwise_kernel<2><<<grid_for((n + 3) / 4, 256), 256, 0, (cudaStream_t)stream>>>(a, b, n, y);
    return launch_status();
}

extern "C" int flexllm_rope(const float* x, const int32_t* pos, const float* cos_t, const float* sin_t, long T,
                            int H, float* y, void* stream) {
    FLEXLLM_REQUIRE(x && pos && cos_t && sin_t && y && T >= 0 && H > 0);
    if (T == 0) return FLEXLLM_OK;
    const long warps = T * H;
    rope_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, (cudaStream_t)stream>>>(x, pos, cos_t, sin_t, T, H, y);
    return launch_status();
}

extern "C" int flexllm_softmax(const float* x, long rows, int len, const int32_t* valid, float* p, void* stream) {
    FLEXLLM_REQUIRE(x && p && rows >= 0 && len > 0);
    if (rows == 0) return FLEXLLM_OK;
    softmax_kernel<<<(unsigned)((rows + 3) / 4), 128, 0, (cudaStream_t)stream>>>(x, rows, len, valid, p);
    return launch_status();
}

extern "C" int flexllm_logits_argmax(const float* logits, int B, long V, int32_t* idx, void* stream) {
    FLEXLLM_REQUIRE(logits && idx && B >= 0 && V > 0);
    if (B == 0) return FLEXLLM_OK;
    launch_k(argmax_kernel, dim3(B), dim3(1024), 0, (cudaStream_t)stream, logits, V, idx);
    return launch_status();
}
