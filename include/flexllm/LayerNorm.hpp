// Modules/LayerNorm.h (RMSNorm; the two functions differ in their summation order, see flexllm_b200.h)
#pragma once
#include "common.hpp"
namespace flexllm {
// pref_Layer_Norm (LayerNorm.h:29), optionally fused with the per-token quantiser that follows it
inline int pref_Layer_Norm(const float* x, const float* gamma, float* y, int8_t* q, float* s, int seq_len, int io_hidden_dim,
                           float eps = 0.00001f, stream_t st = nullptr) {
    return flexllm_rmsnorm_quant(x, gamma, seq_len, io_hidden_dim, eps, FLEXLLM_NORM_PREFILL, y, q, s, st);
}
// dec_Layer_Norm (LayerNorm.h:211) with block_parallel = 8 (config_u280_mem_opt.h:56) or 4
inline int dec_Layer_Norm(const float* x, const float* gamma, float* y, int8_t* q, float* s, int tokens, int io_hidden_dim,
                          float eps = 0.00001f, int block_parallel = 8, stream_t st = nullptr) {
    return flexllm_rmsnorm_quant(x, gamma, tokens, io_hidden_dim, eps, block_parallel, y, q, s, st);
}
}  // namespace flexllm
