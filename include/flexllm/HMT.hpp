// Modules/HMT.h: the hierarchical-memory long-context plug-in on top of the prefill graph
#pragma once
#include "SpinQuant.hpp"
namespace flexllm {
// hmt_segment_loader_sync + the memory cross-attention (HMT.h:8-195, :278-470): reference sizes 990 / 495 / 32 / 64
class HMT {
  public:
    HMT() = default;
    HMT(const HMT&) = delete;
    HMT& operator=(const HMT&) = delete;
    ~HMT() { flexllm_hmt_destroy(h_); }
    int create(SpinQuantModel& model, int hidden, const float* wq, const float* wk, const float* t_embed,
               flexllm_hmt_config cfg = flexllm_hmt_config{990, 495, 32, 64}) {
        return flexllm_hmt_create(&h_, model.handle(), &cfg, hidden, wq, wk, t_embed);
    }
    // embeds [tokens][hidden] on the device; afterwards decode with the model as after any prefill
    int Prefilling(const float* embeds, int tokens, int32_t* next = nullptr, float* trace = nullptr, stream_t st = nullptr) {
        return flexllm_hmt_prefill(h_, embeds, tokens, next, trace, st);
    }
  private:
    flexllm_hmt* h_ = nullptr;
};
}  // namespace flexllm
