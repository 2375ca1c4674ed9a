// Modules/quant.h
#pragma once
#include "common.hpp"
namespace flexllm {
// pref_quant_layer_fp32_qint<8, false, ...> (quant.h:6): x [seq_len][input_dim] -> q, s [seq_len]
inline int pref_quant_layer_fp32_qint(const float* x, int8_t* q, float* s, int seq_len, int input_dim, stream_t st = nullptr) {
    return flexllm_quant_per_token(x, seq_len, input_dim, q, s, st);
}
// dec_quant_layer_fp32_qint (quant.h:333): `tokens` rows of one decode batch
inline int dec_quant_layer_fp32_qint(const float* x, int8_t* q, float* s, int tokens, int input_dim, stream_t st = nullptr) {
    return flexllm_quant_per_token(x, tokens, input_dim, q, s, st);
}
// pref_dequant_layer_qint_fp32 (quant.h:116) / pref_static_sym_dequant_layer_qint_fp32 (quant.h:214)
inline int pref_dequant_layer_qint_fp32(const int32_t* acc, const float* input_s, const float* weight_s, float* y, int seq_len,
                                        int output_dim, stream_t st = nullptr) {
    return flexllm_dequant(acc, input_s, weight_s, seq_len, output_dim, y, st);
}
// pref_quant_layer_fp32_qint<qint_bit, true, ...> (quant.h:53-81): asymmetric, q in [0, 2^bits - 1], scale s and zero point b
inline int pref_quant_layer_fp32_qint_asym(const float* x, uint8_t* q, float* s, float* b, int seq_len, int input_dim, int qint_bit = 4,
                                           stream_t st = nullptr) {
    return flexllm_quant_per_token_asym(x, seq_len, input_dim, qint_bit, q, s, b, st);
}
// pref_dequant_layer_qint_fp32<.., true, ..> (quant.h:146-148): acc * s * ws + b * wsum
inline int pref_dequant_layer_qint_fp32_asym(const int32_t* acc, const float* input_s, const float* input_b, const float* weight_s,
                                             const float* weight_sum, float* y, int seq_len, int output_dim, stream_t st = nullptr) {
    return flexllm_dequant_asym(acc, input_s, input_b, weight_s, weight_sum, seq_len, output_dim, y, st);
}
// pref_static_sym_per_tensor_quant_layer_fp32_qint (quant.h:253): one scale, optional factor
inline int pref_static_sym_per_tensor_quant_layer_fp32_qint(const float* x, const float* input_s, uint8_t* q, long rows, int n,
                                                            bool is_signed, float mha_scale_factor = 1.0f, stream_t st = nullptr) {
    return flexllm_static_quant(x, rows, n, input_s, 0, mha_scale_factor, is_signed ? 1 : 0, q, st);
}
// pref_static_sym_quant_layer_fp32_qint (quant.h:167): one scale per row
inline int pref_static_sym_quant_layer_fp32_qint(const float* x, const float* input_s, uint8_t* q, long rows, int n, bool is_signed,
                                                 stream_t st = nullptr) {
    return flexllm_static_quant(x, rows, n, input_s, 1, 1.0f, is_signed ? 1 : 0, q, st);
}
}  // namespace flexllm
