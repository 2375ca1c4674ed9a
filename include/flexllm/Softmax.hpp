// Modules/Softmax.h (+ pref_causal_mask_template, Modules/MHA.h:247)
#pragma once
#include "common.hpp"
namespace flexllm {
// pref_Softmax (Softmax.h:7); valid[r] = unmasked prefix length of row r (nullptr: no mask)
inline int pref_Softmax(const float* x, float* p, long rows, int io_hidden_dim, const int32_t* valid = nullptr, stream_t st = nullptr) {
    return flexllm_softmax(x, rows, io_hidden_dim, valid, p, st);
}
// dec_MHA_Softmax (Softmax.h:457): rows of arbitrary length
inline int dec_MHA_Softmax(const float* x, float* p, long rows, int io_hidden_dim, stream_t st = nullptr) {
    return flexllm_softmax(x, rows, io_hidden_dim, nullptr, p, st);
}
}  // namespace flexllm
