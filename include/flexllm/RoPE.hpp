// Modules/RoPE.h
#pragma once
#include "common.hpp"
namespace flexllm {
// pref_RoPE_layer (RoPE.h:9): x [tokens][head_num][64], positions per token, tables [P][32]
inline int pref_RoPE_layer(const float* x, float* y, const float* PE_sin, const float* PE_cos, const int32_t* pos, int head_num,
                           long tokens, stream_t st = nullptr) {
    return flexllm_rope(x, pos, PE_cos, PE_sin, tokens, head_num, y, st);
}
// dec_RoPE_layer (RoPE.h:97)
inline int dec_RoPE_layer(const float* x, float* y, const float* PE_sin, const float* PE_cos, const int32_t* pos, int head_num,
                          long tokens, stream_t st = nullptr) {
    return flexllm_rope(x, pos, PE_cos, PE_sin, tokens, head_num, y, st);
}
}  // namespace flexllm
