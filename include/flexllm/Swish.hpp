// Modules/Swish.h
#pragma once
#include "common.hpp"
namespace flexllm {
inline int pref_Swish(const float* x, float* y, long n, stream_t st = nullptr) { return flexllm_swish(x, n, y, st); }
inline int dec_Swish(const float* x, float* y, long n, stream_t st = nullptr) { return flexllm_swish(x, n, y, st); }
}  // namespace flexllm
