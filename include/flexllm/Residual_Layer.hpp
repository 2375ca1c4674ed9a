// Modules/Residual_Layer.h
#pragma once
#include "common.hpp"
namespace flexllm {
inline int pref_Residual_Layer(const float* input, const float* residual, float* y, long n, stream_t st = nullptr) {
    return flexllm_residual(input, residual, n, y, st);
}
inline int dec_Residual_Layer(const float* input, const float* residual, float* y, long n, stream_t st = nullptr) {
    return flexllm_residual(input, residual, n, y, st);
}
}  // namespace flexllm
