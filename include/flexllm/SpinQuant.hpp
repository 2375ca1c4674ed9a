// The two top-level graphs: SpinQuant_Prefilling (SpinQuant_Prefilling.h:807) and SpinQuant_Decoding
// (SpinQuant_Decoding_mem_opt.h:947), as one model object.
#pragma once
#include "common.hpp"
namespace flexllm {
class SpinQuantModel {
  public:
    SpinQuantModel() = default;
    SpinQuantModel(const SpinQuantModel&) = delete;
    SpinQuantModel& operator=(const SpinQuantModel&) = delete;
    ~SpinQuantModel() { flexllm_model_destroy(h_); }
    int create(const flexllm_model_config& cfg) { return flexllm_model_create(&h_, &cfg); }
    int load_layer(int layer, const flexllm_layer_weights& w, stream_t st = nullptr) { return flexllm_model_load_layer(h_, layer, &w, st); }
    int load_head(const int8_t* lm_w, const float* lm_s, const float* gamma_final, const float* PE_cos, const float* PE_sin,
                  int table_len, stream_t st = nullptr) {
        return flexllm_model_load_head(h_, lm_w, lm_s, gamma_final, PE_cos, PE_sin, table_len, st);
    }
    // SpinQuant_Prefilling: tokens [B][S] on the device
    int Prefilling(const int32_t* tokens, int B, int S, int32_t* next = nullptr, stream_t st = nullptr) {
        return flexllm_model_prefill(h_, tokens, B, S, next, st);
    }
    // SpinQuant_Decoding: n_steps greedy tokens per sequence, token feedback on the device
    int Decoding(int n_new, int n_steps, bool use_graph = true, stream_t st = nullptr) {
        int rc = flexllm_model_begin(h_, n_new, st);
        return rc ? rc : flexllm_model_decode(h_, n_steps, use_graph ? 1 : 0, st);
    }
    // the same graph fed with embedding vectors [B][S][hidden] (rows from n_valid on are padding)
    int Prefilling_embeds(const float* embeds, int B, int S, int n_valid, int32_t* next = nullptr, stream_t st = nullptr) {
        return flexllm_model_prefill_embeds(h_, embeds, B, S, n_valid, next, st);
    }
    flexllm_model* handle() const { return h_; }
    // demo flow: host ids in, host ids out
    int generate(const int32_t* tokens_host, int B, int S, int n_new, int32_t* out_host, bool use_graph = true, stream_t st = nullptr) {
        return flexllm_model_generate_host(h_, tokens_host, B, S, n_new, out_host, use_graph ? 1 : 0, st);
    }
  private:
    flexllm_model* h_ = nullptr;
};
}  // namespace flexllm
