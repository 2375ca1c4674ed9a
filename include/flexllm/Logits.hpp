// Modules/Logits.h: the greedy path (rank 0 of sort_top_k, ties to the lowest index) and the top-k sampler of
// dec_Sampling_Embedding_Layer (per-lane top-k, merge, softmax over k, inverse-CDF sample from a uniform number).
#pragma once
#include "common.hpp"
namespace flexllm {
inline int dec_Logits_argmax(const float* logits, int32_t* idx, int batch, long logits_num, stream_t st = nullptr) {
    return flexllm_logits_argmax(logits, batch, logits_num, idx, st);
}
// block_parallel_samp = lanes, top_k as in the reference's template arguments; rand_seed: one uniform number per row.
inline int dec_Sampling_Layer(const float* logits, const float* rand_seed, int32_t* sampled_idx, int batch, long logits_num,
                              int block_parallel_samp = 32, int top_k = 5, stream_t st = nullptr) {
    return flexllm_topk_sample(logits, batch, logits_num, block_parallel_samp, top_k, rand_seed, sampled_idx, nullptr, nullptr, st);
}
}  // namespace flexllm
