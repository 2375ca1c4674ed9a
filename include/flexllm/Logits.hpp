// Modules/Logits.h (greedy path: rank 0 of sort_top_k, ties to the lowest index)
#pragma once
#include "common.hpp"
namespace flexllm {
inline int dec_Logits_argmax(const float* logits, int32_t* idx, int batch, long logits_num, stream_t st = nullptr) {
    return flexllm_logits_argmax(logits, batch, logits_num, idx, st);
}
}  // namespace flexllm
