// Small kernels that exist only for the tensor-parallel partition: they read activations in the
// rank-blocked layout an all-gather produces ([ranks][rows][W], rank r holding columns
// [r*W, (r+1)*W) of each logical row) and write this rank's compact column slice.
#include "common.cuh"
#include "fht_core.cuh"

namespace flexllm {

// Per-token int8 quantisation of logical rows of D = g*W values gathered as x[g][M][W]: the scale
// comes from the whole row (quant.h:84-96), only this rank's W columns are written.
template <int VPT>
__global__ void __launch_bounds__(256) quant_gathered_kernel(const float* __restrict__ x, int M, int W, int g, int r,
                                                             int8_t* __restrict__ q, float* __restrict__ s) {
    __shared__ float red[64];
    pdl_sync();
    const long row = blockIdx.x;
    const int wv = W >> 2, nv = g * wv;
    float4 v[VPT];
    float mx = -1e32f, mn = 1e32f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        const int c = threadIdx.x + i * 256;
        if (c < nv) {
            const int seg = c / wv, o = c - seg * wv;
            v[i] = reinterpret_cast<const float4*>(x + ((long)seg * M + row) * W)[o];
            mx = fmaxf(mx, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
            mn = fminf(mn, fminf(fminf(v[i].x, v[i].y), fminf(v[i].z, v[i].w)));
        }
    }
    block_max_min(mx, mn, red);
    const float sc = sym_scale_from(mx, mn);
    const DivBy dsc = div_by(sc);       // one reciprocal per row: every element is then quantised without a full division
    if (threadIdx.x == 0) s[row] = sc;
    char4* qr = reinterpret_cast<char4*>(q + row * W);
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        const int c = threadIdx.x + i * 256;
        if (c < nv && c / wv == r) {
            char4 o;
            o.x = (int8_t)round_half_away_to_int(div_for_rounding(v[i].x, dsc)); o.y = (int8_t)round_half_away_to_int(div_for_rounding(v[i].y, dsc)); o.z = (int8_t)round_half_away_to_int(div_for_rounding(v[i].z, dsc)); o.w = (int8_t)round_half_away_to_int(div_for_rounding(v[i].w, dsc));
            qr[c - r * wv] = o;
        }
    }
}

// h[m][c] = silu(gate[m][c]) * up[m][c] on this rank's W channels; gu rows are [gate W | up W].
__global__ void swiglu_slice_kernel(const float* __restrict__ gu, long M, int W, float* __restrict__ h) {
    pdl_sync();
    const int wv = W >> 2;
    const long nv = M * wv;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
        const long m = i / wv; const int c = (int)(i - m * wv);
        const float4 g = reinterpret_cast<const float4*>(gu + m * 2 * W)[c];
        const float4 u = reinterpret_cast<const float4*>(gu + m * 2 * W + W)[c];
        float4 o;
        o = silu_mul_x4(g, u);
        reinterpret_cast<float4*>(h)[i] = o;
    }
}

// y = residual + ((float)acc * s_tok[m]) * s_ch[n]   (dequant after the int32 all-reduce, fused with
// the residual add; quant.h:151 + Residual_Layer.h:61). y may alias residual.
__global__ void dequant_residual_kernel(const int32_t* __restrict__ acc, const float* __restrict__ s_tok,
                                        const float* __restrict__ s_ch, long M, int N, const float* residual, float* y) {
    pdl_sync();
    const int nv4 = N >> 2;
    const long nv = M * nv4;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
        const long m = i / nv4; const int c = (int)(i - m * nv4);
        const int4 a = reinterpret_cast<const int4*>(acc)[i];
        const float4 w = reinterpret_cast<const float4*>(s_ch)[c];
        const float st = s_tok[m];
        float4 o;
        o.x = ((float)a.x * st) * w.x; o.y = ((float)a.y * st) * w.y; o.z = ((float)a.z * st) * w.z; o.w = ((float)a.w * st) * w.w;
        if (residual) {
            const float4 rs = reinterpret_cast<const float4*>(residual)[i];
            o.x = rs.x + o.x; o.y = rs.y + o.y; o.z = rs.z + o.z; o.w = rs.w + o.w;
        }
        reinterpret_cast<float4*>(y)[i] = o;
    }
}

// Vocab-parallel greedy token. Each rank's argmax over its slice is gathered as (value, global
// index); the winner is the largest value, ties to the lowest index (Logits.h:13-17).
struct ArgPair { float val; int idx; };
__global__ void __launch_bounds__(1024) argmax_pair_kernel(const float* __restrict__ logits, long V, int offset, ArgPair* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_sync();
    const float* l = logits + (long)blockIdx.x * V;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (long v = threadIdx.x; v < V; v += blockDim.x) {
        const float t = l[v];
        if (t > best || bi == 0x7fffffff) { best = t; bi = (int)v; }
    }
    auto better = [](float a, int ai, float b, int bi2) { return a > b || (a == b && ai < bi2); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
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
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ob, oi, best, bi)) { best = ob; bi = oi; }
        }
        if (lane == 0) { out[blockIdx.x].val = best; out[blockIdx.x].idx = bi + offset; }
    }
}
// pairs [g][B] -> idx [B]
__global__ void argmax_select_kernel(const ArgPair* __restrict__ pairs, int g, int B, int32_t* __restrict__ idx) {
    pdl_sync();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    ArgPair best = pairs[b];
    for (int r = 1; r < g; r++) {
        const ArgPair p = pairs[(long)r * B + b];
        if (p.val > best.val || (p.val == best.val && p.idx < best.idx)) best = p;
    }
    idx[b] = best.idx;
}

// ---------------------------------------------------------------------------------------------
// Token-row partition ("each rank owns a block of rows between the projections"): kernels that let a rank
// quantise ITS column slice of a row with the scale of the WHOLE row, and the regrouping of exchanged blocks.
// ---------------------------------------------------------------------------------------------

// amax[m] = max_k |x[m][k]| over this rank's W columns (the per-token quantiser's max(|max|, |min|),
// Modules/quant.h:84-96, restricted to the slice; the maximum over the ranks follows by all-reduce).
__global__ void __launch_bounds__(256) row_absmax_kernel(const float* __restrict__ x, int W, float* __restrict__ amax) {
    __shared__ float red[64];
    const long row = blockIdx.x;
    const float4* xr = reinterpret_cast<const float4*>(x + row * W);
    float mx = -1e32f, mn = 1e32f;
    for (int c = threadIdx.x; c < (W >> 2); c += 256) {
        const float4 v = xr[c];
        mx = fmaxf(mx, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
        mn = fminf(mn, fminf(fminf(v.x, v.y), fminf(v.z, v.w)));
    }
    block_max_min(mx, mn, red);
    if (threadIdx.x == 0) { const float a = fabsf(mx), b = fabsf(mn); amax[row] = a > b ? a : b; }
}

// q[m][k] = round(x[m][k] / s[m]) with s[m] = amax[m] / 127 (0 -> 1): the per-token quantiser given the row's
// largest magnitude. s_out (optional) receives the scales.
__global__ void __launch_bounds__(256) quant_given_amax_kernel(const float* __restrict__ x, int W, const float* __restrict__ amax,
                                                               int8_t* __restrict__ q, float* __restrict__ s_out) {
    const long row = blockIdx.x;
    float sc = amax[row] / 127.0f;
    if (sc == 0.0f) sc = 1.0f;
    const DivBy dsc = div_by(sc);
    if (threadIdx.x == 0 && s_out) s_out[row] = sc;
    const float4* xr = reinterpret_cast<const float4*>(x + row * W);
    char4* qr = reinterpret_cast<char4*>(q + row * W);
    for (int c = threadIdx.x; c < (W >> 2); c += 256) {
        const float4 v = xr[c];
        char4 o;
        o.x = (int8_t)round_half_away_to_int(div_for_rounding(v.x, dsc)); o.y = (int8_t)round_half_away_to_int(div_for_rounding(v.y, dsc));
        o.z = (int8_t)round_half_away_to_int(div_for_rounding(v.z, dsc)); o.w = (int8_t)round_half_away_to_int(div_for_rounding(v.w, dsc));
        qr[c] = o;
    }
}

// KV-cache hand-over from the head-sharded prefill to the sequence-sharded decode: `stage` holds, for every source
// rank s, the pages of this rank's sequences with s's KV heads, [s][n_pages][hl][elems]; they are interleaved into
// the decode cache's pages [n_pages][g * hl][elems] (head s * hl + h). elems = 4096 bytes (K, V pages) or 64 floats.
__global__ void __launch_bounds__(256) kv_regroup_kernel(const int4* __restrict__ stage, int n_pages, int g, int hl, int elems16,
                                                         int4* __restrict__ dst) {
    const long total = (long)g * n_pages * hl * elems16;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const int e = (int)(i % elems16);
        long t = i / elems16;
        const int h = (int)(t % hl); t /= hl;
        const int pg = (int)(t % n_pages);
        const int s = (int)(t / n_pages);
        dst[(((long)pg * g + s) * hl + h) * elems16 + e] = stage[i];
    }
}

int row_absmax(const float* x, long M, int W, float* amax, cudaStream_t st) {
    if (M == 0) return FLEXLLM_OK;
    row_absmax_kernel<<<(unsigned)M, 256, 0, st>>>(x, W, amax);
    return launch_status();
}
int quant_given_amax(const float* x, long M, int W, const float* amax, int8_t* q, float* s_out, cudaStream_t st) {
    if (M == 0) return FLEXLLM_OK;
    quant_given_amax_kernel<<<(unsigned)M, 256, 0, st>>>(x, W, amax, q, s_out);
    return launch_status();
}
// gu [M][2 * Fl] -> send [g][M][Fl / g]
int kv_regroup(const void* stage, int n_pages, int g, int hl, int elem_bytes, void* dst, cudaStream_t st) {
    const long total = (long)g * n_pages * hl * (elem_bytes / 16);
    if (total == 0) return FLEXLLM_OK;
    long blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    kv_regroup_kernel<<<(unsigned)blocks, 256, 0, st>>>((const int4*)stage, n_pages, g, hl, elem_bytes / 16, (int4*)dst);
    return launch_status();
}

int quant_gathered(const float* x, int M, int W, int g, int r, int8_t* q, float* s, cudaStream_t st) {
    if (M == 0) return FLEXLLM_OK;
    const int nv = g * W / 4;
    if (nv <= 256) launch_k(quant_gathered_kernel<1>, dim3(M), dim3(256), 0, st, x, M, W, g, r, q, s);
    else if (nv <= 512) launch_k(quant_gathered_kernel<2>, dim3(M), dim3(256), 0, st, x, M, W, g, r, q, s);
    else if (nv <= 1024) launch_k(quant_gathered_kernel<4>, dim3(M), dim3(256), 0, st, x, M, W, g, r, q, s);
    else if (nv <= 2048) launch_k(quant_gathered_kernel<8>, dim3(M), dim3(256), 0, st, x, M, W, g, r, q, s);
    else return FLEXLLM_ENOTSUP;
    return launch_status();
}
int swiglu_slice(const float* gu, long M, int W, float* h, cudaStream_t st) {
    if (M == 0) return FLEXLLM_OK;
    long blocks = (M * (W / 4) + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    launch_k(swiglu_slice_kernel, dim3((unsigned)blocks), dim3(256), 0, st, gu, M, W, h);
    return launch_status();
}
int dequant_residual(const int32_t* acc, const float* s_tok, const float* s_ch, long M, int N, const float* residual, float* y,
                     cudaStream_t st) {
    if (M == 0) return FLEXLLM_OK;
    long blocks = (M * (N / 4) + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    launch_k(dequant_residual_kernel, dim3((unsigned)blocks), dim3(256), 0, st, acc, s_tok, s_ch, M, N, residual, y);
    return launch_status();
}
int argmax_pair(const float* logits, int B, long V, int offset, void* pairs, cudaStream_t st) {
    launch_k(argmax_pair_kernel, dim3(B), dim3(1024), 0, st, logits, V, offset, (ArgPair*)pairs);
    return launch_status();
}
int argmax_select(const void* pairs, int g, int B, int32_t* idx, cudaStream_t st) {
    launch_k(argmax_select_kernel, dim3((B + 63) / 64), dim3(64), 0, st, (const ArgPair*)pairs, g, B, idx);
    return launch_status();
}

}  // namespace flexllm
