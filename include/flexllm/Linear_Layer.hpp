// Modules/Linear_Layer.h at 8-bit symmetric precision (+ the dequant layer that always follows it)
#pragma once
#include "common.hpp"
namespace flexllm {
// pref_Linear_Layer_i4xi4 (Linear_Layer.h:294) + pref_dequant_layer_qint_fp32: a [seq_len][K] s8, w [N][K] s8
inline int pref_Linear_Layer_i8xi8(const int8_t* a, const float* input_s, const int8_t* w, const float* weight_s, int32_t* acc,
                                   float* y, int seq_len, int output_dim, int input_dim, stream_t st = nullptr) {
    return flexllm_linear_prefill_i8(a, input_s, w, weight_s, seq_len, output_dim, input_dim, acc, y, st);
}
// dec_Linear_Layer_i4xi4 (Linear_Layer.h:863) + dec_dequant_layer_qint_fp32, up to 64 tokens
inline int dec_Linear_Layer_i8xi8(const int8_t* a, const float* input_s, const int8_t* w, const float* weight_s, int32_t* acc,
                                  float* y, int tokens, int output_dim, int input_dim, stream_t st = nullptr) {
    return flexllm_linear_decode_i8(a, input_s, w, weight_s, tokens, output_dim, input_dim, acc, y, st);
}
// pref_Linear_Layer_i4xi4<.., is_uint_input = true> (Linear_Layer.h:294) / dec_Linear_Layer_i4xi4 (:863) with the asymmetric
// dequantiser: a [tokens][K] unsigned (from the asymmetric quantiser), w [N][K] s8; acc is required (int32 [tokens][N])
inline int pref_Linear_Layer_i4xi4(const uint8_t* a, const float* input_s, const float* input_b, const int8_t* w, const float* weight_s,
                                   const float* weight_sum, int32_t* acc, float* y, int seq_len, int output_dim, int input_dim,
                                   stream_t st = nullptr) {
    return flexllm_linear_prefill_asym(a, input_s, input_b, w, weight_s, weight_sum, seq_len, output_dim, input_dim, acc, y, st);
}
inline int dec_Linear_Layer_i4xi4(const uint8_t* a, const float* input_s, const float* input_b, const int8_t* w, const float* weight_s,
                                  const float* weight_sum, int32_t* acc, float* y, int tokens, int output_dim, int input_dim,
                                  stream_t st = nullptr) {
    return flexllm_linear_decode_asym(a, input_s, input_b, w, weight_s, weight_sum, tokens, output_dim, input_dim, acc, y, st);
}
// pref_Gate_Layer_fp32xfp32 (Linear_Layer.h:613) / dec_Gate_Layer_fp32xfp32 (:1104)
// The FFN passes of the decode graph as one call (dec_Layer_Norm_012, dec_quant_layer_qkvo_FFN, the gate / up / down turns
// of dec_Linear_Layer_i4xi4_qkvo_FFN_half and dec_dequant_layer_qkvo_FFN, dec_Swish_Layer_FFN, dec_Gate_layer_FFN, dec_FHT_R4,
// dec_residual_layer: SpinQuant_Decoding_mem_opt.h:1061-1117). w_gate_up: gate rows, then up rows.
inline size_t dec_MLP_block_workspace(int tokens, int hidden, int ffn) { return flexllm_mlp_block_workspace(tokens, hidden, ffn); }
inline int dec_MLP_block(const float* x, const float* gamma, const int8_t* w_gate_up, const float* s_gate_up, const int8_t* w_down,
                         const float* s_down, int tokens, int hidden, int ffn, float eps, int norm_order, float fht_scale, float* y,
                         void* workspace, size_t workspace_bytes, stream_t st = nullptr) {
    return flexllm_mlp_block_decode(x, gamma, w_gate_up, s_gate_up, w_down, s_down, tokens, hidden, ffn, eps, norm_order, fht_scale, y,
                                    workspace, workspace_bytes, st);
}
inline int pref_Gate_Layer_fp32xfp32(const float* input, const float* gate, float* y, long n, stream_t st = nullptr) {
    return flexllm_gate(input, gate, n, y, st);
}
inline int dec_Gate_Layer_fp32xfp32(const float* input, const float* gate, float* y, long n, stream_t st = nullptr) {
    return flexllm_gate(input, gate, n, y, st);
}
}  // namespace flexllm
