// HMT (hierarchical memory transformer) long-context plug-in on top of the prefill path: the segment recurrence of
// Modules/HMT.h. A long prompt is cut into segments of seg_len tokens; per segment n
//   stage 0 (n > 0): the prefill graph runs on [T, first sum_len tokens of the segment, T] (T = a learned segment-summary
//            embedding); the residual-stream row of the trailing T is the summary S_n (HMT.h:48-121). The memory
//            cross-attention (HMT.h:278-355, fp32): Q = Wq S_n, scores against the cached keys of ALL mem_num slots
//            (empty slots are zero vectors, as in the reference), dec_Softmax with scale sqrt(hidden)
//            (HMT_SpinQuant_Unit.h:97-105), P_n = sum_s A_s M_s;
//   stage 1: the prefill graph runs on [P_n, the rec_len last tokens of the previous segment, the segment, P_n] -- P_n is
//            zero for the first segment, the trailing P_n is left out for the last (HMT.h:125-170); the row of the
//            trailing P_n is the new memory M_n, stored with its key Wk M_n in slot n mod mem_num (HMT.h:175-190,
//            :357-470).
// Every prefill starts at position 0 with an empty KV cache; only the memory slots carry over, so the attention window
// stays at 1 + rec_len + seg_len + 1 tokens whatever the prompt length. After the last segment the model holds that
// segment's KV cache and first token, and decoding continues as after any prefill. One sequence at a time, as in the
// reference. The fp32 linear unit keeps the reference's accumulation order: four interleaved chains over k mod 4,
// combined (p0 + p1) + (p2 + p3) (PE.h:655-756); the softmax its four block-partitioned lanes of four partial sums.
#include <cmath>
#include <new>
#include <vector>

#include "common.cuh"

namespace flexllm {

// y[n] = (p0 + p1) + (p2 + p3), p[c] = sum_{k = c, c+4, ...} a[k] * w[n][k].  Four lanes per output, eight outputs per warp.
__global__ void __launch_bounds__(256) linear_fp32_chain4_kernel(const float* __restrict__ a, const float* __restrict__ w, int N, int K,
                                                                 float* __restrict__ y) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = t >> 2, c = t & 3;
    float p = 0.0f;
    if (n < N) {
        const float* wr = w + (long)n * K;
        for (int k = c; k < K; k += 4) p = p + a[k] * wr[k];        // compiled without fused multiply-add
    }
    const int base = threadIdx.x & 28 & 31;                         // first lane of this output's group of four
    const float p0 = __shfl_sync(0xffffffffu, p, base), p1 = __shfl_sync(0xffffffffu, p, base + 1);
    const float p2 = __shfl_sync(0xffffffffu, p, base + 2), p3 = __shfl_sync(0xffffffffu, p, base + 3);
    if (n < N && c == 0) y[n] = (p0 + p1) + (p2 + p3);
}

// the same with the matrix given transposed: y[n] = chains over s of a[s] * m[s][n]   (P_n = sum_s A_s M_s over the memory rows)
__global__ void __launch_bounds__(256) linear_fp32_chain4_t_kernel(const float* __restrict__ a, const float* __restrict__ m, int N, int K,
                                                                   float* __restrict__ y) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float p[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < K; k++) p[k & 3] = p[k & 3] + a[k] * m[(long)k * N + n];
    y[n] = (p[0] + p[1]) + (p[2] + p[3]);
}

// dec_Softmax with enable_scale and enable_sub_max over `dim` values in `lanes` block-partitioned lanes (Softmax.h:261-363):
// one warp; thread (lane i, chain c) adds the exponentials of its lane block with k mod 4 == c in increasing k.
__global__ void __launch_bounds__(32) softmax_dec_kernel(const float* __restrict__ x, int dim, int lanes, float scale, float* __restrict__ p) {
    __shared__ float e_sm[1024];
    const int t = threadIdx.x;
    float mx = -1e32f;
    for (int i = t; i < dim; i += 32) mx = fmaxf(mx, x[i]);
    mx = warp_max(mx);
    for (int i = t; i < dim; i += 32) e_sm[i] = ref_expf((x[i] - mx) / scale);
    __syncwarp();
    const int per = dim / lanes;
    float s = 0.0f;
    if (t < 4 * lanes) {
        const int i = t >> 2, c = t & 3;
        for (int k = c; k < per; k += 4) s += e_sm[i * per + k];
    }
    float total = 0.0f;
    for (int i = 0; i < lanes; i++) {
        const float s0 = __shfl_sync(0xffffffffu, s, 4 * i), s1 = __shfl_sync(0xffffffffu, s, 4 * i + 1);
        const float s2 = __shfl_sync(0xffffffffu, s, 4 * i + 2), s3 = __shfl_sync(0xffffffffu, s, 4 * i + 3);
        total += (s0 + s1) + (s2 + s3);
    }
    const float r = 1.0f / total;
    for (int i = t; i < dim; i += 32) p[i] = e_sm[i] * r;
}

}  // namespace flexllm

using namespace flexllm;

struct flexllm_hmt {
    flexllm_model* model;
    flexllm_hmt_config cfg;
    int D;
    float *wq = nullptr, *wk = nullptr, *t_embed = nullptr;     // [D][D], [D][D], [D]
    float *mem = nullptr, *kmem = nullptr;                      // [mem_num][D] memory vectors and their keys (ring: slot = segment mod mem_num)
    float *pn = nullptr, *qn = nullptr, *an = nullptr, *pa = nullptr, *kn = nullptr;   // P_n [D], Q_n [D], scores, probabilities [mem_num], K_n [D]
    float* seq = nullptr;                                       // assembled stage input [max rows][D]
    int max_rows = 0;
    std::vector<void*> owned;
};

static int hmt_alloc(flexllm_hmt* h, float** p, size_t n) {
    void* q = nullptr;
    cudaError_t e = cudaMalloc(&q, n * sizeof(float));
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; return e == cudaErrorMemoryAllocation ? FLEXLLM_ENOMEM : FLEXLLM_ECUDA; }
    h->owned.push_back(q);
    *p = (float*)q;
    return FLEXLLM_OK;
}

extern "C" int flexllm_hmt_destroy(flexllm_hmt* h) {
    if (!h) return FLEXLLM_OK;
    for (void* p : h->owned) cudaFree(p);
    delete h;
    return FLEXLLM_OK;
}

extern "C" int flexllm_hmt_create(flexllm_hmt** out, flexllm_model* model, const flexllm_hmt_config* cfg, int hidden, const float* wq,
                                  const float* wk, const float* t_embed) {
    FLEXLLM_REQUIRE(out && model && cfg && wq && wk && t_embed && hidden > 0 && hidden % 4 == 0);
    FLEXLLM_REQUIRE(cfg->seg_len > 0 && cfg->sum_len > 0 && cfg->rec_len >= 0 && cfg->mem_num > 0 && cfg->mem_num <= 1024);
    if (cfg->mem_num % 16 != 0) return FLEXLLM_ENOTSUP;         // four lanes of whole groups of four
    flexllm_hmt* h = new (std::nothrow) flexllm_hmt();
    if (!h) return FLEXLLM_ENOMEM;
    h->model = model; h->cfg = *cfg; h->D = hidden;
    const size_t D = hidden, Mn = cfg->mem_num;
    h->max_rows = (1 + cfg->rec_len + cfg->seg_len + 1 + 15) / 16 * 16;
    int rc, max_prefill = 0;
    // a stage must fit ONE prefill chunk: the summary / memory rows are read from the residual stream by position
    if ((rc = flexllm_model_limits(model, nullptr, &max_prefill, nullptr)) || max_prefill < h->max_rows) {
        delete h;
        return rc ? rc : FLEXLLM_ENOTSUP;
    }
    if ((rc = hmt_alloc(h, &h->wq, D * D)) || (rc = hmt_alloc(h, &h->wk, D * D)) || (rc = hmt_alloc(h, &h->t_embed, D)) ||
        (rc = hmt_alloc(h, &h->mem, Mn * D)) || (rc = hmt_alloc(h, &h->kmem, Mn * D)) || (rc = hmt_alloc(h, &h->pn, D)) ||
        (rc = hmt_alloc(h, &h->qn, D)) || (rc = hmt_alloc(h, &h->an, Mn)) || (rc = hmt_alloc(h, &h->pa, Mn)) || (rc = hmt_alloc(h, &h->kn, D)) ||
        (rc = hmt_alloc(h, &h->seq, (size_t)h->max_rows * D))) {
        flexllm_hmt_destroy(h);
        return rc;
    }
    cudaError_t e = cudaMemcpy(h->wq, wq, D * D * 4, cudaMemcpyDefault);
    if (e == cudaSuccess) e = cudaMemcpy(h->wk, wk, D * D * 4, cudaMemcpyDefault);
    if (e == cudaSuccess) e = cudaMemcpy(h->t_embed, t_embed, D * 4, cudaMemcpyDefault);
    if (e != cudaSuccess) { flexllm_hmt_destroy(h); return cuda_status(e); }
    *out = h;
    return FLEXLLM_OK;
}

static int hmt_linear(const float* a, const float* w, int N, int K, float* y, cudaStream_t st) {
    linear_fp32_chain4_kernel<<<(N * 4 + 255) / 256, 256, 0, st>>>(a, w, N, K, y);
    return launch_status();
}

// embeds [T][D] fp32 (device): the whole prompt. Leaves the model ready to decode (KV cache and first token of the last
// segment's stage 1). trace (optional, device, [segments][4][D]): S_n, P_n, M_n, K_n per segment (rows of segments that do
// not produce one stay untouched).
extern "C" int flexllm_hmt_prefill(flexllm_hmt* h, const float* embeds, int T, int32_t* next_out, float* trace, void* stream) {
    FLEXLLM_REQUIRE(h && embeds && T > 0);
    cudaStream_t st = (cudaStream_t)stream;
    const flexllm_hmt_config& c = h->cfg;
    const size_t D = h->D;
    const int seg_num = (T + c.seg_len - 1) / c.seg_len;
    void* xv = nullptr;
    TRY_RC(flexllm_model_buffer(h->model, 0, &xv));
    const float* x = (const float*)xv;                          // residual stream of the model's last prefill: row = position
    FLEXLLM_CHECK_CUDA(cudaMemsetAsync(h->mem, 0, (size_t)c.mem_num * D * 4, st));
    FLEXLLM_CHECK_CUDA(cudaMemsetAsync(h->kmem, 0, (size_t)c.mem_num * D * 4, st));
    FLEXLLM_CHECK_CUDA(cudaMemsetAsync(h->pn, 0, D * 4, st));
    const float scale = sqrtf((float)h->D);
    auto row_copy = [&](float* dst, const float* src, size_t rows) { return cuda_status(cudaMemcpyAsync(dst, src, rows * D * 4, cudaMemcpyDeviceToDevice, st)); };
    for (int seg = 0; seg < seg_num; seg++) {
        const int cur = seg < seg_num - 1 ? c.seg_len : T - seg * c.seg_len;
        const int sl = cur < c.sum_len ? cur : c.sum_len;
        const size_t off = (size_t)seg * c.seg_len;
        float* tr = trace ? trace + (size_t)seg * 4 * D : nullptr;
        if (seg > 0) {
            // ---- stage 0: [T, first sl tokens, T]
            const int n0 = 1 + sl + 1, s0 = (n0 + 15) / 16 * 16;
            FLEXLLM_CHECK_CUDA(cudaMemsetAsync(h->seq, 0, (size_t)s0 * D * 4, st));
            TRY_RC(row_copy(h->seq, h->t_embed, 1));
            TRY_RC(row_copy(h->seq + D, embeds + off * D, sl));
            TRY_RC(row_copy(h->seq + (size_t)(1 + sl) * D, h->t_embed, 1));
            TRY_RC(flexllm_model_prefill_embeds(h->model, h->seq, 1, s0, n0, nullptr, st));
            const float* Sn = x + (size_t)(1 + sl) * D;
            TRY_RC(hmt_linear(Sn, h->wq, h->D, h->D, h->qn, st));                         // Q_n = Wq S_n
            TRY_RC(hmt_linear(h->qn, h->kmem, c.mem_num, h->D, h->an, st));               // scores against every slot's key
            softmax_dec_kernel<<<1, 32, 0, st>>>(h->an, c.mem_num, 4, scale, h->pa);
            linear_fp32_chain4_t_kernel<<<(h->D + 255) / 256, 256, 0, st>>>(h->pa, h->mem, h->D, c.mem_num, h->pn);   // P_n = sum_s A_s M_s
            TRY_RC(launch_status(2));
            if (tr) { TRY_RC(row_copy(tr, Sn, 1)); TRY_RC(row_copy(tr + D, h->pn, 1)); }
        }
        // ---- stage 1: [P_n, rec_len tail tokens of the previous segment, the segment, P_n (not for the last segment)]
        const bool last = seg == seg_num - 1;
        const int n1 = 1 + c.rec_len + cur + (last ? 0 : 1), s1 = (n1 + 15) / 16 * 16;
        FLEXLLM_CHECK_CUDA(cudaMemsetAsync(h->seq, 0, (size_t)s1 * D * 4, st));
        TRY_RC(row_copy(h->seq, h->pn, 1));
        const long tail0 = (long)off - c.rec_len;                 // first tail token (negative for the first segment: zeros)
        const int skip = tail0 < 0 ? (int)-tail0 : 0;
        if (c.rec_len > skip) TRY_RC(row_copy(h->seq + (size_t)(1 + skip) * D, embeds + (size_t)(tail0 + skip) * D, c.rec_len - skip));
        TRY_RC(row_copy(h->seq + (size_t)(1 + c.rec_len) * D, embeds + off * D, cur));
        if (!last) TRY_RC(row_copy(h->seq + (size_t)(1 + c.rec_len + cur) * D, h->pn, 1));
        TRY_RC(flexllm_model_prefill_embeds(h->model, h->seq, 1, s1, n1, last ? next_out : nullptr, st));
        if (!last) {
            const float* Mn = x + (size_t)(1 + c.rec_len + cur) * D;
            const int slot = seg % c.mem_num;
            TRY_RC(hmt_linear(Mn, h->wk, h->D, h->D, h->kn, st));                         // K_n = Wk M_n
            TRY_RC(row_copy(h->mem + (size_t)slot * D, Mn, 1));
            TRY_RC(row_copy(h->kmem + (size_t)slot * D, h->kn, 1));
            if (tr) { TRY_RC(row_copy(tr + 2 * D, Mn, 1)); TRY_RC(row_copy(tr + 3 * D, h->kn, 1)); }
        }
    }
    return FLEXLLM_OK;
}
