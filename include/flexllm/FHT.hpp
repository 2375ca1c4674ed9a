// Modules/FHT.h
#pragma once
#include "common.hpp"
namespace flexllm {
// pref_FHT (FHT.h:8): rows of io_hidden_dim values, divided by scale_factor
inline int pref_FHT(const float* x, float* y, long rows, int io_hidden_dim, float scale_factor, stream_t st = nullptr) {
    return flexllm_fht(x, rows, io_hidden_dim, scale_factor, y, st);
}
// dec_FHT (FHT.h:70)
inline int dec_FHT(const float* x, float* y, long rows, int io_hidden_dim, float scale_factor, stream_t st = nullptr) {
    return flexllm_fht(x, rows, io_hidden_dim, scale_factor, y, st);
}
// fused silu(gate)*up -> FHT-8192 -> per-token quant (the sequence of SpinQuant_Prefilling.h:1017-1035)
inline int swiglu_FHT_quant(const float* gate, const float* up, int8_t* q, float* s, int rows, float scale_factor = 90.50966799f,
                            stream_t st = nullptr) {
    return flexllm_swiglu_fht_quant(gate, up, rows, 8192, scale_factor, q, s, nullptr, st);
}
}  // namespace flexllm
