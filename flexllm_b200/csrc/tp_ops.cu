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
        o.x = silu_f(g.x) * u.x; o.y = silu_f(g.y) * u.y; o.z = silu_f(g.z) * u.z; o.w = silu_f(g.w) * u.w;
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
// quantise ITS column slice of a row with the scale of the WHOLE row, and the two halves of the 8192-point
// Hadamard transform around its one exchange.
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

// First half of the FHT-8192 on a rank that holds Fl = 2^LB consecutive elements of each row (its gate/up
// channels): h = silu(gate) * up, then the butterflies on index bits 1 .. LB-1 (the reference's stage order is
// bits 1, 2, ..., 12, then 0; bits LB .. 12 pair elements of different ranks and bit 0 comes after them). The
// result is written in all-to-all order: out[dest][m][j] = element dest * W + j, W = Fl / g, so that rank `dest`
// receives, from every rank, the same W-wide window of the local index. One CTA of Fl / 8 threads per row.
template <int LB>
__global__ void __launch_bounds__((1 << LB) / 8) swiglu_fht_local_kernel(const float* __restrict__ gu, long M, int g, float* __restrict__ out) {
    constexpr int Fl = 1 << LB, NT = Fl / 8;
    __shared__ float buf[Fl + Fl / 32];
    const int tid = threadIdx.x;
    const long m = blockIdx.x;
    const float4* gr = reinterpret_cast<const float4*>(gu + m * 2 * Fl);
    const float4* ur = gr + Fl / 4;
#pragma unroll
    for (int it = 0; it < 2; it++) {
        const int c = it * NT + tid;
        const float4 a = gr[c], u = ur[c];
        const int p = pad32(c * 4);
        buf[p] = silu_f(a.x) * u.x; buf[p + 1] = silu_f(a.y) * u.y; buf[p + 2] = silu_f(a.z) * u.z; buf[p + 3] = silu_f(a.w) * u.w;
    }
    __syncthreads();
    float r[8];
    // one pass = the group of index bits b0, b0+1, b0+2 held in registers; SKIP low bits of the group were done by the pass before
    auto pass = [&](const int b0, const int skip) {
        const int base = (tid & ((1 << b0) - 1)) | ((tid >> b0) << (b0 + 3));
#pragma unroll
        for (int v = 0; v < 8; v++) r[v] = buf[pad32(base | (v << b0))];
        if (skip < 1) reg_butterfly<0>(r);
        if (skip < 2) reg_butterfly<1>(r);
        reg_butterfly<2>(r);
#pragma unroll
        for (int v = 0; v < 8; v++) buf[pad32(base | (v << b0))] = r[v];
        __syncthreads();
    };
    constexpr int NB = LB - 1;                  // bits 1 .. LB-1
    constexpr int FULL = NB / 3, REM = NB - 3 * FULL;
#pragma unroll
    for (int k = 0; k < FULL; k++) pass(1 + 3 * k, 0);
    if (REM) pass(LB - 3, 3 - REM);
    const int W = Fl / g;
#pragma unroll
    for (int it = 0; it < 2; it++) {
        const int c = it * NT + tid, e = c * 4, p = pad32(e);
        const int dest = e / W, j = e - dest * W;
        *reinterpret_cast<float4*>(out + ((long)dest * M + m) * W + j) = make_float4(buf[p], buf[p + 1], buf[p + 2], buf[p + 3]);
    }
}

// Second half, on the rank that received window W of every rank: in[src][m][j] is element src * Fl + r * W + j of the
// row after the local stages. Butterflies over the rank index (index bits LB, LB+1, ... in that order), then the stage
// on bit 0 (neighbouring j), then / scale. Output hf[m][src * W + j] (this order is the K order of the rank's down_proj
// slice) and the row's largest magnitude, merged over the CTA's threads with an integer max on the float bits
// (non-negative floats order like their bit patterns). amax must be zero on entry. 4 consecutive j per thread.
template <int G>
__global__ void __launch_bounds__(256) fht_cross_kernel(const float* __restrict__ in, long M, int W, float scale, float* __restrict__ hf,
                                                        unsigned* __restrict__ amax_bits) {
    const int tpr = W >> 2;                                   // threads per row
    const long idx = (long)blockIdx.x * 256 + threadIdx.x;
    const long m = idx / tpr;
    const int j4 = (int)(idx - m * tpr);
    if (m >= M) return;
    float4 w[G];
#pragma unroll
    for (int s = 0; s < G; s++) w[s] = reinterpret_cast<const float4*>(in + ((long)s * M + m) * W)[j4];
    auto bf = [](float& lo, float& hi) { const float a = lo + hi, d = lo - hi; lo = a; hi = d; };
#pragma unroll
    for (int bit = 1; bit < G; bit <<= 1)
#pragma unroll
        for (int s = 0; s < G; s++)
            if (!(s & bit)) { bf(w[s].x, w[s | bit].x); bf(w[s].y, w[s | bit].y); bf(w[s].z, w[s | bit].z); bf(w[s].w, w[s | bit].w); }
    const DivBy d = div_by(scale);
    float mx = 0.0f;
#pragma unroll
    for (int s = 0; s < G; s++) {
        float x[4] = {w[s].x + w[s].y, w[s].x - w[s].y, w[s].z + w[s].w, w[s].z - w[s].w};      // bit 0
        div_rn_array(x, d);
        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3]))));
        reinterpret_cast<float4*>(hf + m * (long)(G * W) + (long)s * W)[j4] = make_float4(x[0], x[1], x[2], x[3]);
    }
    // threads of a warp belong to one row (W / 4 is a multiple of 32)
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) atomicMax(amax_bits + m, __float_as_uint(mx));
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
int swiglu_fht_local(const float* gu, long M, int Fl, int g, float* send, cudaStream_t st) {
    if (M == 0) return FLEXLLM_OK;
    if (Fl == 4096) swiglu_fht_local_kernel<12><<<(unsigned)M, 512, 0, st>>>(gu, M, g, send);
    else if (Fl == 2048) swiglu_fht_local_kernel<11><<<(unsigned)M, 256, 0, st>>>(gu, M, g, send);
    else if (Fl == 1024) swiglu_fht_local_kernel<10><<<(unsigned)M, 128, 0, st>>>(gu, M, g, send);
    else return FLEXLLM_ENOTSUP;
    return launch_status();
}
// recv [g][M][W] -> hf [M][g * W], amax [M] (zeroed here)
int fht_cross(const float* recv, long M, int W, int g, float scale, float* hf, float* amax, cudaStream_t st) {
    if (M == 0) return FLEXLLM_OK;
    if (W % 128) return FLEXLLM_ENOTSUP;
    FLEXLLM_CHECK_CUDA(cudaMemsetAsync(amax, 0, (size_t)M * sizeof(float), st));
    const long threads = M * (W / 4);
    const unsigned grid = (unsigned)((threads + 255) / 256);
    if (g == 2) fht_cross_kernel<2><<<grid, 256, 0, st>>>(recv, M, W, scale, hf, (unsigned*)amax);
    else if (g == 4) fht_cross_kernel<4><<<grid, 256, 0, st>>>(recv, M, W, scale, hf, (unsigned*)amax);
    else if (g == 8) fht_cross_kernel<8><<<grid, 256, 0, st>>>(recv, M, W, scale, hf, (unsigned*)amax);
    else return FLEXLLM_ENOTSUP;
    return launch_status();
}
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
