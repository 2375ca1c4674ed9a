// Top-k sampling operator (Modules/Logits.h:145-279); device code in sampling.cuh.
#include "sampling.cuh"

namespace flexllm {

// One CTA per row. rnd: uniform numbers, row b of step `*col` (col == nullptr: step 0) at rnd[step * B + b].
__global__ void __launch_bounds__(512) topk_sample_kernel(const float* __restrict__ logits, long V, int lanes, int top_k,
                                                          const float* __restrict__ rnd, const int32_t* __restrict__ col, int B,
                                                          int32_t* __restrict__ idx, int32_t* __restrict__ top_idx,
                                                          float* __restrict__ top_val) {
    __shared__ SampleSmem sm;
    pdl_sync();
    const int b = blockIdx.x;
    const int step = col ? *col : 0;
    const int s = topk_sample_row<512>(logits + (long)b * V, V, lanes, top_k, rnd[(long)step * B + b], sm, (int)threadIdx.x, 0,
                                       top_idx ? top_idx + (long)b * top_k : nullptr, top_val ? top_val + (long)b * top_k : nullptr);
    if (threadIdx.x == 0) idx[b] = s;
}

int topk_sample(const float* logits, int B, long V, int lanes, int top_k, const float* rnd, const int32_t* col, int32_t* idx,
                int32_t* top_idx, float* top_val, cudaStream_t st) {
    if (B == 0) return FLEXLLM_OK;
    if (!logits || !rnd || !idx || V <= 0) return FLEXLLM_EINVAL;
    if (top_k < 1 || top_k > SAMPLE_KMAX || lanes < 1 || lanes > SAMPLE_LMAX || V % lanes || V / lanes < top_k) return FLEXLLM_ENOTSUP;
    launch_k(topk_sample_kernel, dim3(B), dim3(512), 0, st, logits, V, lanes, top_k, rnd, col, B, idx, top_idx, top_val);
    return launch_status();
}

}  // namespace flexllm

using namespace flexllm;

extern "C" int flexllm_topk_sample(const float* logits, int B, long V, int lanes, int top_k, const float* rnd, int32_t* idx,
                                   int32_t* top_idx, float* top_val, void* stream) {
    return topk_sample(logits, B, V, lanes, top_k, rnd, nullptr, idx, top_idx, top_val, (cudaStream_t)stream);
}
