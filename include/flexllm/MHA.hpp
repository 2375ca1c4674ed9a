// Modules/MHA.h and the graphs of SpinQuant_Llama_32_1B/MHA_i8xi8.h
#pragma once
#include "common.hpp"
namespace flexllm {
// Q/K path in front of the int8 attention: dequant -> RoPE -> FHT-64 -> per-head int8 quant
inline int MHA_qk_prepare(const int8_t* q, const float* s, const int32_t* pos, const float* PE_cos, const float* PE_sin, long tokens,
                          int head_num, int8_t* q_out, float* s_out, stream_t st = nullptr) {
    return flexllm_qk_prepare(q, s, pos, PE_cos, PE_sin, tokens, head_num, q_out, s_out, st);
}
// MHA_i8xi8_Prefilling_tb (MHA_i8xi8.h:369-427)
inline size_t MHA_i8xi8_Prefilling_workspace(int B, int S, int HQ, int HKV) { return flexllm_mha_prefill_workspace(B, S, HQ, HKV); }
inline int MHA_i8xi8_Prefilling(const int8_t* q, const float* qs, const int8_t* k, const float* ks, const int8_t* v, const float* vs,
                                const float* PE_cos, const float* PE_sin, const float* a_s, int B, int S, int HQ, int HKV, float* out,
                                int32_t* oacc, void* workspace, size_t workspace_bytes, stream_t st = nullptr) {
    return flexllm_mha_i8xi8_prefill(q, qs, k, ks, v, vs, PE_cos, PE_sin, a_s, B, S, HQ, HKV, out, oacc, workspace, workspace_bytes, st);
}
// the same graph in one sweep with an online softmax: close to, not bit-identical with, the call above (no static P scale)
inline int MHA_i8xi8_Prefilling_online(const int8_t* q, const float* qs, const int8_t* k, const float* ks, const int8_t* v, const float* vs,
                                       const float* PE_cos, const float* PE_sin, int B, int S, int HQ, int HKV, float* out,
                                       void* workspace, size_t workspace_bytes, stream_t st = nullptr) {
    return flexllm_mha_i8xi8_prefill_online(q, qs, k, ks, v, vs, PE_cos, PE_sin, B, S, HQ, HKV, out, workspace, workspace_bytes, st);
}
// dec_K_cache_manager / dec_V_cache_manager (MHA.h:485, :774) as a paged pool
class KVCache {
  public:
    KVCache() = default;
    KVCache(const KVCache&) = delete;
    KVCache& operator=(const KVCache&) = delete;
    ~KVCache() { flexllm_kv_cache_destroy(h_); }
    int create(int layers, int n_pages, int hkv, int page = 64) { return flexllm_kv_cache_create(&h_, layers, n_pages, hkv, page); }
    int reset(stream_t st = nullptr) { return flexllm_kv_cache_reset(h_, st); }
    flexllm_kv_cache* handle() const { return h_; }
  private:
    flexllm_kv_cache* h_ = nullptr;
};
// the managers' append alone (MHA.h:493-513, :782-801): k,v [B][HKV][64] with scales stored at position ctx[b]
inline int dec_KV_cache_append(KVCache& cache, int layer, const int8_t* k, const float* ks, const int8_t* v, const float* vs,
                               const int32_t* page_table, int max_pages, const int32_t* ctx, int max_ctx, int B, stream_t st = nullptr) {
    return flexllm_kv_append(cache.handle(), layer, k, ks, v, vs, page_table, max_pages, ctx, max_ctx, B, st);
}
// MHA_i8xi8_decoding_tb (MHA_i8xi8.h:1027-1114)
inline size_t MHA_i8xi8_Decoding_workspace(int B, int HQ, int max_ctx) { return flexllm_mha_decode_workspace(B, HQ, max_ctx); }
inline int MHA_i8xi8_Decoding(KVCache& cache, int layer, const int8_t* q, const float* qs, const int8_t* k, const float* ks,
                              const int8_t* v, const float* vs, const float* PE_cos, const float* PE_sin, const float* a_s,
                              const int32_t* page_table, int max_pages, const int32_t* ctx, int max_ctx, int B, int HQ, float* out,
                              int32_t* oacc, void* workspace, size_t workspace_bytes, stream_t st = nullptr) {
    return flexllm_mha_i8xi8_decode(cache.handle(), layer, q, qs, k, ks, v, vs, PE_cos, PE_sin, a_s, page_table, max_pages, ctx,
                                    max_ctx, B, HQ, out, oacc, workspace, workspace_bytes, st);
}
}  // namespace flexllm
