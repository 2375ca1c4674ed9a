// Host interface of the persistent decode-step kernel (decode_mega.cu), used by the model runner.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

struct flexllm_kv_cache;

namespace flexllm {

struct MegaLayerView {
    const int8_t *wqkv, *wo, *wgu, *wd;
    const float *sqkv, *so, *sgu, *sd, *g0, *g1, *a_s;
};

// Everything the step touches, as the model runner owns it (single GPU, no tensor parallelism).
struct MegaModelView {
    int layers, D, HQ, HKV, F, V, max_batch, max_ctx;
    float eps, fht_scale;
    const MegaLayerView* L;                 // [layers], host array
    const int8_t* lm_w; const float* lm_s; const float* g_final;
    const float *cos_t, *sin_t;
    flexllm_kv_cache* cache;
    const int32_t* page_table; int max_pages;
    int32_t *ctx, *next, *out_tokens, *state;
    float* x; int8_t* xq; float* xs; int8_t* hq; float* att; float* logits;
};

struct MegaPlan;

// FLEXLLM_ENOTSUP when the shapes, the device or the context length rule the kernel out (the caller
// then keeps the kernel-per-operator path).
int mega_create(const MegaModelView& v, MegaPlan** out);
void mega_destroy(MegaPlan* p);
// Zeroes the grid-barrier counter (start of a generation, or after an error).
int mega_reset(MegaPlan* p, cudaStream_t st);
// Token choice of the following steps: top_k == 0 greedy, else top-k sampling with rnd [n_new][B] (device).
void mega_set_sampling(MegaPlan* p, int lanes, int top_k, const float* rnd);
// The kernel is built in three variants that differ in the attention code they carry; mega_variant names the leanest one
// that covers B sequences at positions <= max_pos (0 = the general one, valid for every launch).
int mega_variant(const MegaPlan* p, int B, int max_pos);
// One decode step for B sequences (one kernel launch) with the given variant.
int mega_launch(MegaPlan* p, int B, int variant, cudaStream_t st);

}  // namespace flexllm
