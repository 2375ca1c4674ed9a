// Llama-3.2-1B W8A8 SpinQuant forward on one GPU: the operator order of the reference's two
// top-level graphs, SpinQuant_Prefilling (SpinQuant_Llama_32_1B/SpinQuant_Prefilling.h:807, graph
// :940-1049) and SpinQuant_Decoding (SpinQuant_Decoding_mem_opt.h:947, graph :1050-1126), driven
// the way the demo's host program drives them (SpinQuant_Prefilling_Decoding_mem_opt_demo.cpp:
// prefill launch, KV hand-off, decode launch).
//
// Per layer: RMSNorm+quant -> fused q|k|v projection -> RoPE, FHT-64, per-head int8 quant, KV-cache
// append, int8 attention -> quant -> o projection -> +residual -> RMSNorm+quant -> fused gate|up
// projection -> silu(gate)*up, FHT-8192, quant -> down projection -> +residual.
// Head: RMSNorm+quant -> lm_head -> greedy argmax; the next embedding row is
// (float)lm_head_q[token] * lm_head_s[token] (tied embeddings).
// Prefill uses the prefill RMSNorm summation order and the tcgen05 GEMM / attention kernels; decode
// uses the decode order, the weight-streaming linear layers and the paged attention, and is replayed
// from a CUDA graph (the token feedback stays on the device, as in the reference's decode graph).
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "attention_decode.cuh"     // layout of the paged KV cache (for the hand-over between partitions)
#include "common.cuh"
#include "decode_mega.h"

struct flexllm_tp;

namespace flexllm {
int gemm_i8_prefill(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch, int M, int N, int K,
                    int32_t* acc, float* y, cudaStream_t st, const float* residual);
int swiglu_fht_quant_strided(const float* g, const float* u, long ld, int M, float scale, int8_t* q, float* s, cudaStream_t st);
size_t mha_prefill_ws_bytes(int B, int max_prefill, int max_ctx, int HQ, int HKV);
int mha_prefill_paged(const float* qkv, const float* cos_t, const float* sin_t, const float* a_s, int B, int Sq, int q_off, int HQ, int HKV,
                      int max_prefill, flexllm_kv_cache* c, int layer, const int32_t* page_table, int max_pages, float* out,
                      void* workspace, cudaStream_t st);
int mha_decode_run(flexllm_kv_cache* c, int layer, const int8_t* q, const float* qs, const int8_t* k, const float* ks,
                   const int8_t* v, const float* vs, const float* qkv_f32, const float* cos_t, const float* sin_t,
                   const float* a_s, const int32_t* page_table, int max_pages, const int32_t* ctx, int max_ctx, int B, int HQ,
                   float* out, int32_t* oacc, void* workspace, cudaStream_t st);
int gemm_check_error_flag();
int* device_error_flag();
int quant_gathered(const float* x, int M, int W, int g, int r, int8_t* q, float* s, cudaStream_t st);
int swiglu_slice(const float* gu, long M, int W, float* h, cudaStream_t st);
int dequant_residual(const int32_t* acc, const float* s_tok, const float* s_ch, long M, int N, const float* residual, float* y,
                     cudaStream_t st);
int argmax_pair(const float* logits, int B, long V, int offset, void* pairs, cudaStream_t st);
int argmax_select(const void* pairs, int g, int B, int32_t* idx, cudaStream_t st);
int fht_quant_gathered(const float* h, int M, int g, int r, float scale, int8_t* q, float* s, cudaStream_t st);
int fht_quant_gathered_rows(const float* h, int M, int g, float scale, int8_t* q, float* s, cudaStream_t st);
int row_absmax(const float* x, long M, int W, float* amax, cudaStream_t st);
int quant_given_amax(const float* x, long M, int W, const float* amax, int8_t* q, float* s_out, cudaStream_t st);
int kv_regroup(const void* stage, int n_pages, int g, int hl, int elem_bytes, void* dst, cudaStream_t st);
int topk_sample(const float* logits, int B, long V, int lanes, int top_k, const float* rnd, const int32_t* col, int32_t* idx,
                int32_t* top_idx, float* top_val, cudaStream_t st);

// x[t][:] = (float)lm_w[tok[t]][:] * lm_s[tok[t]]
// An id outside [0, V) (device data the host has not seen, e.g. fed back by a sampler) is clamped so that
// it cannot become a wild read, and reported through the error word.
// Row t of x is token (t0 + t) of the call: sequence b = (t0 + t) / Sc, position c0 + (t0 + t) % Sc of tok [B][S]
// (a decode step passes S = Sc = 1, c0 = t0 = 0: row t = tok[t]).
__global__ void embed_kernel(const int32_t* __restrict__ tok, const int8_t* __restrict__ lm_w, const float* __restrict__ lm_s,
                             int D, int V, float* __restrict__ x, int* error_flag, int S, int c0, int Sc, long t0) {
    pdl_sync();
    const int t = blockIdx.x;
    const long tg = t0 + t;
    int id = tok[(tg / Sc) * S + c0 + tg % Sc];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0 && error_flag) atomicOr(error_flag, 2);
        id = id < 0 ? 0 : V - 1;
    }
    const float s = lm_s[id];
    const char4* w = reinterpret_cast<const char4*>(lm_w + (long)id * D);
    float4* o = reinterpret_cast<float4*>(x + (long)t * D);
    for (int i = threadIdx.x; i < D / 4; i += blockDim.x) {
        const char4 c = w[i];
        o[i] = make_float4((float)c.x * s, (float)c.y * s, (float)c.z * s, (float)c.w * s);
    }
}

// rows (b*S + n - 1) of x -> y[b]   (n: valid rows per sequence, the rest is padding)
__global__ void gather_last_kernel(const float* __restrict__ x, int S, int n, int D, float* __restrict__ y) {
    const int b = blockIdx.x;
    const float4* src = reinterpret_cast<const float4*>(x + ((long)b * S + n - 1) * D);
    float4* dst = reinterpret_cast<float4*>(y + (long)b * D);
    for (int i = threadIdx.x; i < D / 4; i += blockDim.x) dst[i] = src[i];
}

// Device-side generation state: state[0] = next output column, state[1] = number of columns.
// Records the chosen tokens at column state[0] of out [B][state[1]], then advances the column and
// (after a decode step) the context lengths.
__global__ void step_bookkeeping_kernel(const int32_t* __restrict__ next, int B, int32_t* __restrict__ out,
                                        int32_t* __restrict__ state, int32_t* __restrict__ ctx, int advance_ctx) {
    pdl_sync();
    const int b = threadIdx.x;
    const int col = state[0], n_cols = state[1];
    if (b < B) {
        if (col < n_cols) out[(long)b * n_cols + col] = next[b];
        if (advance_ctx) ctx[b] += 1;
    }
    __syncthreads();
    if (b == 0) state[0] = col + 1;
}
__global__ void set_state_kernel(int32_t* state, int col, int n_cols) { state[0] = col; state[1] = n_cols; }

__global__ void fill_ctx_kernel(int32_t* ctx, int B, int v) { if (threadIdx.x < B) ctx[threadIdx.x] = v; }

}  // namespace flexllm

using namespace flexllm;

struct LayerW {
    int8_t *wqkv, *wo, *wgu, *wd;
    float *sqkv, *so, *sgu, *sd, *g0, *g1, *a_s;
};

struct flexllm_model {
    flexllm_model_config cfg;
    std::vector<LayerW> L;
    int8_t* lm_w = nullptr; float* lm_s = nullptr; float* g_final = nullptr;
    float *cos_t = nullptr, *sin_t = nullptr; int table_len = 0;
    flexllm_kv_cache* cache = nullptr;
    int max_pages = 0;
    int32_t *page_table = nullptr, *ctx = nullptr, *next = nullptr, *state = nullptr, *tokens = nullptr, *out_tokens = nullptr;
    size_t out_capacity = 0;
    // activations (sized for max_batch * max_prefill rows)
    float *x = nullptr, *qkv = nullptr, *att = nullptr, *tmp = nullptr, *gu = nullptr, *xs = nullptr, *logits = nullptr, *xlast = nullptr;
    int8_t *xq = nullptr, *hq = nullptr;
    void *attn_ws = nullptr, *dec_ws = nullptr;
    size_t attn_ws_bytes = 0, dec_ws_bytes = 0;
    // decode state
    int B = 0, S = 0;
    int last_chunk = 0;                         // rows per sequence the residual stream x holds after the last prefill
    int n_new = 0;                              // columns of the token table of the running generation
    int pos = 0;                                // context length of the batch = position the next decode step writes
    cudaGraphExec_t graph = nullptr; int graph_B = 0; int graph_kernels = 0;
    int mega_variant = 0, graph_variant = 0;   // attention variant of the persistent kernel for the current decode call / in the captured step
    std::vector<void*> owned;
    // tensor parallelism: g ranks, this one is r; *l = local (per-rank) sizes
    flexllm_tp* tp = nullptr;
    int g = 1, r = 0, HQl = 0, HKVl = 0, Fl = 0, Dl = 0, Vl = 0;
    float *gath = nullptr, *hloc = nullptr;     // all-gather target / local silu(gate)*up slice
    // token-row partition of the prefill + batch-parallel decode (see flexllm_model_prefill)
    flexllm_model* dm = nullptr;                // single-GPU model of this rank's sequences: full weights, all KV heads
    float *amax = nullptr, *xs2 = nullptr;      // per-token largest magnitudes / scales of the row-parallel inputs
    int8_t* aq = nullptr;                       // quantised attention output, this rank's columns
    uint8_t *kv_stage = nullptr, *kvs_stage = nullptr;   // KV hand-over: pages / scale rows as received
    bool rows_mode = false;                     // the last prefill used the token-row partition
    int32_t* acc32 = nullptr;                   // row-parallel partial sums
    void *pairs_l = nullptr, *pairs_g = nullptr;
    // persistent decode-step kernel: -1 not tried yet, 0 not usable for this model, 1 ready
    flexllm::MegaPlan* mega = nullptr; int mega_state = -1;
    // token choice: greedy (sample_k == 0) or the reference's top-k sampling with uniform numbers rnd [n_new][B]
    int sample_lanes = 0, sample_k = 0; const float* sample_rnd = nullptr;
};

template <class T> static int dmalloc(flexllm_model* m, T** p, size_t n) {
    void* q = nullptr;
    cudaError_t e = cudaMalloc(&q, n * sizeof(T) + 256);
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; return e == cudaErrorMemoryAllocation ? FLEXLLM_ENOMEM : FLEXLLM_ECUDA; }
    m->owned.push_back(q);
    *p = (T*)q;
    return FLEXLLM_OK;
}
#define TRY(expr) do { int _rc = (expr); if (_rc != FLEXLLM_OK) return _rc; } while (0)

extern "C" int flexllm_model_create(flexllm_model** out, const flexllm_model_config* c) {
    return flexllm_model_create_tp(out, c, nullptr);
}

extern "C" int flexllm_model_create_tp(flexllm_model** out, const flexllm_model_config* c, flexllm_tp* tp) {
    FLEXLLM_REQUIRE(out && c);
    FLEXLLM_REQUIRE(c->layers > 0 && c->hidden > 0 && c->heads_q > 0 && c->heads_kv > 0 && c->ffn > 0 && c->vocab > 0);
    FLEXLLM_REQUIRE(c->max_batch > 0 && c->max_batch <= 64 && c->max_prefill > 0 && c->max_ctx >= c->max_prefill);
    if (c->heads_q * 64 != c->hidden || c->heads_q != 4 * c->heads_kv || c->ffn != 8192 || c->hidden > 4096) return FLEXLLM_ENOTSUP;
    flexllm_model* m = new (std::nothrow) flexllm_model();
    if (!m) return FLEXLLM_ENOMEM;
    m->cfg = *c;
    const int D = c->hidden, F = c->ffn, V = c->vocab, NL = c->layers;
    m->tp = tp; m->g = flexllm_tp_size(tp); m->r = flexllm_tp_rank(tp);
    const int g = m->g;
    if (c->heads_kv % g || D % (g * 16) || F % g || V % (g * 8)) { delete m; return FLEXLLM_ENOTSUP; }
    m->HQl = c->heads_q / g; m->HKVl = c->heads_kv / g; m->Fl = F / g; m->Dl = D / g; m->Vl = V / g;
    const int HQ = m->HQl, HKV = m->HKVl;            // everything below is sized per rank
    const int QKV = (HQ + 2 * HKV) * 64;
    const size_t Mmax = (size_t)c->max_batch * c->max_prefill;
    m->L.resize(NL);
    int rc = FLEXLLM_OK;
    auto fail = [&](int r) { flexllm_model_destroy(m); return r; };
    for (int l = 0; l < NL && rc == FLEXLLM_OK; l++) {
        LayerW& w = m->L[l];
        if ((rc = dmalloc(m, &w.wqkv, (size_t)QKV * D))) break;
        if ((rc = dmalloc(m, &w.wo, (size_t)D * m->Dl))) break;
        if ((rc = dmalloc(m, &w.wgu, (size_t)2 * m->Fl * D))) break;
        if ((rc = dmalloc(m, &w.wd, (size_t)D * m->Fl))) break;
        if ((rc = dmalloc(m, &w.sqkv, QKV))) break;
        if ((rc = dmalloc(m, &w.so, D))) break;
        if ((rc = dmalloc(m, &w.sgu, 2 * m->Fl))) break;
        if ((rc = dmalloc(m, &w.sd, D))) break;
        if ((rc = dmalloc(m, &w.g0, D))) break;
        if ((rc = dmalloc(m, &w.g1, D))) break;
        if ((rc = dmalloc(m, &w.a_s, HQ))) break;   // local heads
    }
    if (rc) return fail(rc);
    if ((rc = dmalloc(m, &m->lm_w, (size_t)V * D)) || (rc = dmalloc(m, &m->lm_s, V)) || (rc = dmalloc(m, &m->g_final, D))) return fail(rc);
    m->table_len = c->max_ctx + 1;
    if ((rc = dmalloc(m, &m->cos_t, (size_t)m->table_len * 32)) || (rc = dmalloc(m, &m->sin_t, (size_t)m->table_len * 32))) return fail(rc);
    m->max_pages = (c->max_ctx + 64) / 64;
    const int n_pages = m->max_pages * c->max_batch;
    if ((rc = flexllm_kv_cache_create(&m->cache, NL, n_pages, HKV, 64))) return fail(rc);
    if ((rc = dmalloc(m, &m->page_table, (size_t)c->max_batch * m->max_pages)) || (rc = dmalloc(m, &m->ctx, 64)) ||
        (rc = dmalloc(m, &m->next, 64)) || (rc = dmalloc(m, &m->state, 4)) || (rc = dmalloc(m, &m->tokens, (size_t)c->max_batch * c->max_ctx)))
        return fail(rc);
    m->out_capacity = (size_t)c->max_batch * (c->max_ctx + 1);
    if ((rc = dmalloc(m, &m->out_tokens, m->out_capacity))) return fail(rc);
    {   // identity page table: sequence b owns pages [b*max_pages, (b+1)*max_pages)
        std::vector<int32_t> pt((size_t)c->max_batch * m->max_pages);
        for (size_t i = 0; i < pt.size(); i++) pt[i] = (int32_t)i;
        if (cudaMemcpy(m->page_table, pt.data(), pt.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess) return fail(FLEXLLM_ECUDA);
    }
    if ((rc = dmalloc(m, &m->x, Mmax * D)) || (rc = dmalloc(m, &m->qkv, Mmax * QKV)) || (rc = dmalloc(m, &m->att, Mmax * D)) ||
        (rc = dmalloc(m, &m->tmp, Mmax * D)) || (rc = dmalloc(m, &m->gu, Mmax * 2 * m->Fl)) || (rc = dmalloc(m, &m->xs, Mmax)) ||
        (rc = dmalloc(m, &m->xq, Mmax * D)) || (rc = dmalloc(m, &m->hq, Mmax * m->Fl)) ||
        (rc = dmalloc(m, &m->logits, (size_t)c->max_batch * V)) || (rc = dmalloc(m, &m->xlast, (size_t)c->max_batch * D)))
        return fail(rc);
    if (g > 1) {
        if ((rc = dmalloc(m, &m->gath, Mmax * F)) || (rc = dmalloc(m, &m->hloc, Mmax * m->Fl)) || (rc = dmalloc(m, &m->acc32, Mmax * D)))
            return fail(rc);
        uint8_t *pl = nullptr, *pg = nullptr;
        if ((rc = dmalloc(m, &pl, (size_t)64 * 8)) || (rc = dmalloc(m, &pg, (size_t)64 * 8 * g))) return fail(rc);
        m->pairs_l = pl; m->pairs_g = pg;
        // Token-row partition + batch-parallel decode: needs the batch to split evenly over the ranks.
        // FLEXLLM_TP_MODE=allgather keeps every call on the all-gather partition instead.
        const char* mode = getenv("FLEXLLM_TP_MODE");
        if (c->max_batch % g == 0 && !(mode && !strcmp(mode, "allgather"))) {
            flexllm_model_config dc = *c;
            dc.max_batch = c->max_batch / g;
            dc.max_prefill = 16;                    // the decode model never prefills; its row buffers serve the head
            if ((rc = flexllm_model_create(&m->dm, &dc))) return fail(rc);
            const size_t pages_l = (size_t)dc.max_batch * m->max_pages;
            if ((rc = dmalloc(m, &m->amax, Mmax)) || (rc = dmalloc(m, &m->xs2, Mmax)) || (rc = dmalloc(m, &m->aq, Mmax * m->Dl)) ||
                (rc = dmalloc(m, &m->kv_stage, pages_l * c->heads_kv * 4096)) || (rc = dmalloc(m, &m->kvs_stage, pages_l * c->heads_kv * 256)))
                return fail(rc);
        }
    }
    m->attn_ws_bytes = mha_prefill_ws_bytes(c->max_batch, c->max_prefill, c->max_ctx, HQ, HKV);
    m->dec_ws_bytes = flexllm_mha_decode_workspace(c->max_batch, HQ, c->max_ctx);
    uint8_t *a = nullptr, *d = nullptr;
    if ((rc = dmalloc(m, &a, m->attn_ws_bytes)) || (rc = dmalloc(m, &d, m->dec_ws_bytes))) return fail(rc);
    m->attn_ws = a; m->dec_ws = d;
    *out = m;
    return FLEXLLM_OK;
}

extern "C" int flexllm_model_destroy(flexllm_model* m) {
    if (!m) return FLEXLLM_OK;
    if (m->graph) cudaGraphExecDestroy(m->graph);
    if (m->dm) flexllm_model_destroy(m->dm);
    mega_destroy(m->mega);
    if (m->cache) flexllm_kv_cache_destroy(m->cache);
    for (void* p : m->owned) cudaFree(p);
    delete m;
    return FLEXLLM_OK;
}

static int copy_any(void* dst, const void* src, size_t bytes, cudaStream_t st) {
    return cuda_status(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, st));
}

static int copy_cols(void* dst, const void* src, size_t rows, size_t src_row_bytes, size_t col0_bytes, size_t width_bytes, cudaStream_t st) {
    return cuda_status(cudaMemcpy2DAsync(dst, width_bytes, (const char*)src + col0_bytes, src_row_bytes, width_bytes, rows,
                                         cudaMemcpyDefault, st));
}

// Takes the FULL layer weights; with tensor parallelism each rank keeps its slice: rows of q/k/v and
// gate/up (column-parallel, by heads / FFN channels), columns of o and down (row-parallel).
extern "C" int flexllm_model_load_layer(flexllm_model* m, int layer, const flexllm_layer_weights* w, void* stream) {
    FLEXLLM_REQUIRE(m && w && layer >= 0 && layer < m->cfg.layers);
    FLEXLLM_REQUIRE(w->wq && w->wk && w->wv && w->wo && w->wg && w->wu && w->wd && w->sq && w->sk && w->sv && w->so && w->sg &&
                    w->su && w->sd && w->gamma0 && w->gamma1 && w->a_s);
    cudaStream_t st = (cudaStream_t)stream;
    const int D = m->cfg.hidden, F = m->cfg.ffn, r = m->r;
    const size_t q = (size_t)m->HQl * 64, kv = (size_t)m->HKVl * 64, Fl = m->Fl, Dl = m->Dl;
    LayerW& L = m->L[layer];
    TRY(copy_any(L.wqkv, w->wq + r * q * D, q * D, st));
    TRY(copy_any(L.wqkv + q * D, w->wk + r * kv * D, kv * D, st));
    TRY(copy_any(L.wqkv + (q + kv) * D, w->wv + r * kv * D, kv * D, st));
    TRY(copy_any(L.sqkv, w->sq + r * q, q * 4, st));
    TRY(copy_any(L.sqkv + q, w->sk + r * kv, kv * 4, st));
    TRY(copy_any(L.sqkv + q + kv, w->sv + r * kv, kv * 4, st));
    TRY(copy_cols(L.wo, w->wo, D, D, r * Dl, Dl, st));
    TRY(copy_any(L.so, w->so, (size_t)D * 4, st));
    TRY(copy_any(L.wgu, w->wg + r * Fl * D, Fl * D, st));
    TRY(copy_any(L.wgu + Fl * D, w->wu + r * Fl * D, Fl * D, st));
    TRY(copy_any(L.sgu, w->sg + r * Fl, Fl * 4, st));
    TRY(copy_any(L.sgu + Fl, w->su + r * Fl, Fl * 4, st));
    TRY(copy_cols(L.wd, w->wd, D, F, r * Fl, Fl, st));
    TRY(copy_any(L.sd, w->sd, (size_t)D * 4, st));
    TRY(copy_any(L.g0, w->gamma0, (size_t)D * 4, st));
    TRY(copy_any(L.g1, w->gamma1, (size_t)D * 4, st));
    TRY(copy_any(L.a_s, w->a_s + r * m->HQl, (size_t)m->HQl * 4, st));
    if (m->dm) {      // the decode model keeps the full weights (also used by the token-row prefill's o and down projections)
        TRY(flexllm_model_load_layer(m->dm, layer, w, stream));
    }
    return FLEXLLM_OK;
}

extern "C" int flexllm_model_load_head(flexllm_model* m, const int8_t* lm_w, const float* lm_s, const float* gamma_final,
                                       const float* cos_t, const float* sin_t, int table_len, void* stream) {
    FLEXLLM_REQUIRE(m && lm_w && lm_s && gamma_final && cos_t && sin_t && table_len >= m->table_len);
    cudaStream_t st = (cudaStream_t)stream;
    TRY(copy_any(m->lm_w, lm_w, (size_t)m->cfg.vocab * m->cfg.hidden, st));
    TRY(copy_any(m->lm_s, lm_s, (size_t)m->cfg.vocab * 4, st));
    TRY(copy_any(m->g_final, gamma_final, (size_t)m->cfg.hidden * 4, st));
    TRY(copy_any(m->cos_t, cos_t, (size_t)m->table_len * 32 * 4, st));
    TRY(copy_any(m->sin_t, sin_t, (size_t)m->table_len * 32 * 4, st));
    if (m->dm) TRY(flexllm_model_load_head(m->dm, lm_w, lm_s, gamma_final, cos_t, sin_t, table_len, stream));
    return FLEXLLM_OK;
}

// lm_head on the rows of xin [B][D] -> logits, argmax -> m->next
// col: device pointer to the output column this head call fills (selects the row of sampling numbers), or
// nullptr for column 0 (the prefill's token)
static int run_head(flexllm_model* m, const float* xin, int B, int order, cudaStream_t st, const int32_t* col = nullptr) {
    const int D = m->cfg.hidden, V = m->cfg.vocab;
    TRY(flexllm_rmsnorm_quant(xin, m->g_final, B, D, m->cfg.eps, order, nullptr, m->xq, m->xs, st));
    if (m->g == 1) {
        TRY(flexllm_linear_decode_i8(m->xq, m->xs, m->lm_w, m->lm_s, B, V, D, nullptr, m->logits, st));
        if (m->sample_k > 0) TRY(topk_sample(m->logits, B, V, m->sample_lanes, m->sample_k, m->sample_rnd, col, m->next, nullptr, nullptr, st));
        else TRY(flexllm_logits_argmax(m->logits, B, V, m->next, st));
        return FLEXLLM_OK;
    }
    if (m->sample_k > 0) return FLEXLLM_ENOTSUP;      // sampling needs the whole vocabulary on one GPU
    // vocab-parallel: this rank's rows of the (replicated) lm_head, local argmax, gather, select
    const int Vl = m->Vl, off = m->r * Vl;
    TRY(flexllm_linear_decode_i8(m->xq, m->xs, m->lm_w + (size_t)off * D, m->lm_s + off, B, Vl, D, nullptr, m->logits, st));
    TRY(argmax_pair(m->logits, B, Vl, off, m->pairs_l, st));
    TRY(flexllm_tp_allgather(m->tp, m->pairs_l, m->pairs_g, (size_t)B * 8, st));
    TRY(argmax_select(m->pairs_g, m->g, B, m->next, st));
    return FLEXLLM_OK;
}

// Tensor-parallel prefill in the token-row partition, then hand-over to batch-parallel decode.
//
// Between the projections every rank owns a block of M / g token rows (= B / g whole sequences) of the residual
// stream: RMSNorm and the residual adds run on those rows only. Around them, per layer:
//   all-gather   int8 rows + scales of the normalised input          -> column-parallel q|k|v (local heads), gate|up
//   all-reduce   max over the ranks of the per-token largest magnitude of the attention output, so that each rank
//                quantises ITS columns with the whole row's scale
//   all-to-all   (int8) those columns to the rows' owners, which run the o projection for their rows with the full
//                weight matrix (every rank holds the full weights for decode anyway): the integer sums over the whole
//                K are formed on one rank, the residual add is the GEMM's epilogue
//   all-to-all   (fp32) silu(gate) * up of the rank's FFN channels to the rows' owners, which then hold whole rows:
//                8192-point Hadamard transform, quantiser and down projection are the single-GPU kernels on M / g rows
// Every exchanged quantity is a maximum or moves values unchanged, and every sum is formed on one rank in the
// single-GPU order, so the results equal the single-GPU model's bit for bit. Afterwards the KV cache (sharded by KV head during the prefill) is regrouped by
// sequence, and each rank decodes its B / g sequences with the full (replicated, 1.2 GB) weights on the persistent
// decode kernel: independent batch-parallel decode streams, no collective inside a decode step.
// One chunk of the prompt (tokens at positions c0 .. c0 + Sc - 1 of every sequence) through all layers.
static int prefill_rows_chunk(flexllm_model* m, const int32_t* tokens, int B, int S, int c0, int Sc, cudaStream_t st) {
    const int D = m->cfg.hidden, HQ = m->HQl, HKV = m->HKVl;
    const int QKV = (HQ + 2 * HKV) * 64;
    const int g = m->g, r = m->r, Dl = m->Dl, Fl = m->Fl, F = m->cfg.ffn;
    const long M = (long)B * Sc, Mr = M / g;
    int8_t* xq_mine = m->xq + (size_t)r * Mr * D;
    float* xs_mine = m->xs + (size_t)r * Mr;
    int8_t* a_recv = reinterpret_cast<int8_t*>(m->acc32);           // the o projection's input columns as received
    int8_t* a_rows = a_recv + (size_t)Mr * D;                         // ... and as rows [Mr][D]
    embed_kernel<<<(unsigned)Mr, 256, 0, st>>>(tokens, m->lm_w, m->lm_s, D, m->cfg.vocab, m->x, device_error_flag(), S, c0, Sc, (long)r * Mr);
    note_launches(1);
    auto norm_and_gather = [&](const float* gamma) {
        TRY(flexllm_rmsnorm_quant(m->x, gamma, (int)Mr, D, m->cfg.eps, FLEXLLM_NORM_PREFILL, nullptr, xq_mine, xs_mine, st));
        TRY(flexllm_tp_allgather(m->tp, xq_mine, m->xq, (size_t)Mr * D, st));             // in place: block r is already there
        TRY(flexllm_tp_allgather(m->tp, xs_mine, m->xs, (size_t)Mr * 4, st));
        return FLEXLLM_OK;
    };
    for (int l = 0; l < m->cfg.layers; l++) {
        const LayerW& L = m->L[l];
        const LayerW& DL = m->dm->L[l];             // the decode model's copy: full (unsliced) o and down weights
        TRY(norm_and_gather(L.g0));
        TRY(gemm_i8_prefill(m->xq, m->xs, L.wqkv, L.sqkv, (int)M, QKV, D, nullptr, m->qkv, st, nullptr));
        TRY(mha_prefill_paged(m->qkv, m->cos_t, m->sin_t, L.a_s, B, Sc, c0, HQ, HKV, m->cfg.max_prefill, m->cache, l, m->page_table,
                              m->max_pages, m->att, m->attn_ws, st));
        // o projection: every rank quantises its heads' columns of ALL rows with the rows' common scale (all-reduce of
        // the per-token largest magnitude), the int8 columns go to the rows' owners (all-to-all), and each owner runs the
        // whole projection for its rows with the full weight matrix (held for decode anyway) -- the integer sums over the
        // full K are formed on one rank, the residual add is the GEMM's epilogue
        TRY(row_absmax(m->att, M, Dl, m->amax, st));
        TRY(flexllm_tp_allreduce_max_f32(m->tp, m->amax, (size_t)M, st));
        TRY(quant_given_amax(m->att, M, Dl, m->amax, m->aq, m->xs2, st));
        TRY(flexllm_tp_alltoall(m->tp, m->aq, a_recv, (size_t)Mr * Dl, st));                 // [g][Mr][Dl]
        TRY(kv_regroup(a_recv, (int)Mr, g, 1, Dl, a_rows, st));                              // -> [Mr][D]
        TRY(gemm_i8_prefill(a_rows, m->xs2 + (size_t)r * Mr, DL.wo, DL.so, (int)Mr, D, D, nullptr, m->x, st, m->x));
        // MLP
        TRY(norm_and_gather(L.g1));
        TRY(gemm_i8_prefill(m->xq, m->xs, L.wgu, L.sgu, (int)M, 2 * Fl, D, nullptr, m->gu, st, nullptr));
        // silu(gate) * up of this rank's channels goes to the rows' owners (all-to-all, fp32: the only exchange that is not
        // int8); the owner then has whole rows: the 8192-point transform, the quantiser and the down projection with the
        // full weight matrix are the single-GPU kernels on Mr rows
        TRY(swiglu_slice(m->gu, M, Fl, m->hloc, st));
        TRY(flexllm_tp_alltoall(m->tp, m->hloc, m->gath, (size_t)Mr * Fl * 4, st));          // [g][Mr][Fl]
        TRY(fht_quant_gathered_rows(m->gath, (int)Mr, g, m->cfg.fht_scale, m->hq, m->xs2, st));
        TRY(gemm_i8_prefill(m->hq, m->xs2, DL.wd, DL.sd, (int)Mr, D, F, nullptr, m->x, st, m->x));
    }
    return FLEXLLM_OK;
}

static int prefill_rows(flexllm_model* m, const int32_t* tokens, int B, int S, int32_t* next_out, cudaStream_t st) {
    const int D = m->cfg.hidden, HKV = m->HKVl;
    const int g = m->g;
    const int Bl = B / g;
    flexllm_model* dm = m->dm;
    int Sc = S;
    for (int c0 = 0; c0 < S; c0 += m->cfg.max_prefill) {
        Sc = S - c0 < m->cfg.max_prefill ? S - c0 : m->cfg.max_prefill;
        TRY(prefill_rows_chunk(m, tokens, B, S, c0, Sc, st));
    }
    // ---- hand-over: this rank's sequences [r * Bl, (r + 1) * Bl) with all KV heads go to its decode model
    {
        flexllm_kv_cache* src = m->cache; flexllm_kv_cache* dst = dm->cache;
        const int n_pg = Bl * m->max_pages;                       // pages of one rank's sequences (identity page tables on both sides)
        const size_t pg_bytes = (size_t)n_pg * HKV * 4096, sc_bytes = (size_t)n_pg * HKV * 256;
        for (int l = 0; l < m->cfg.layers; l++) {
            const size_t so = (size_t)l * src->page_bytes, ss = (size_t)l * (src->scale_bytes / 4);
            const size_t d_o = (size_t)l * dst->page_bytes, ds = (size_t)l * (dst->scale_bytes / 4);
            TRY(flexllm_tp_alltoall(m->tp, src->k + so, m->kv_stage, pg_bytes, st));
            TRY(kv_regroup(m->kv_stage, n_pg, g, HKV, 4096, dst->k + d_o, st));
            TRY(flexllm_tp_alltoall(m->tp, src->v + so, m->kv_stage, pg_bytes, st));
            TRY(kv_regroup(m->kv_stage, n_pg, g, HKV, 4096, dst->v + d_o, st));
            TRY(flexllm_tp_alltoall(m->tp, src->ks + ss, m->kvs_stage, sc_bytes, st));
            TRY(kv_regroup(m->kvs_stage, n_pg, g, HKV, 256, dst->ks + ds, st));
            TRY(flexllm_tp_alltoall(m->tp, src->vs + ss, m->kvs_stage, sc_bytes, st));
            TRY(kv_regroup(m->kvs_stage, n_pg, g, HKV, 256, dst->vs + ds, st));
        }
    }
    gather_last_kernel<<<Bl, 256, 0, st>>>(m->x, Sc, Sc, D, dm->xlast);      // the last chunk's rows are in x
    note_launches(1);
    TRY(run_head(dm, dm->xlast, Bl, FLEXLLM_NORM_PREFILL, st));
    fill_ctx_kernel<<<1, 64, 0, st>>>(dm->ctx, Bl, S);
    TRY(launch_status());
    dm->B = Bl; dm->S = S; dm->pos = S;
    TRY(flexllm_tp_allgather(m->tp, dm->next, m->next, (size_t)Bl * 4, st));
    if (next_out) TRY(copy_any(next_out, m->next, (size_t)B * 4, st));
    m->B = B; m->S = S; m->pos = S; m->rows_mode = true; m->last_chunk = Sc;
    return FLEXLLM_OK;
}

// One chunk of the prompt (positions c0 .. c0 + Sc - 1 of every sequence) through all layers: single GPU, or the
// all-gather partition of the tensor-parallel model.
static int prefill_chunk(flexllm_model* m, const int32_t* tokens, const float* embeds, int B, int S, int c0, int Sc, cudaStream_t st) {
    const int D = m->cfg.hidden, HQ = m->HQl, HKV = m->HKVl, F = m->cfg.ffn;
    const int QKV = (HQ + 2 * HKV) * 64;
    const int M = B * Sc;
    const int g = m->g, r = m->r, Dl = m->Dl, Fl = m->Fl;
    if (embeds) {       // rows given as vectors (not token ids): sequence b's chunk is contiguous in embeds [B][S][D]
        for (int b = 0; b < B; b++)
            TRY(copy_any(m->x + (size_t)b * Sc * D, embeds + ((size_t)b * S + c0) * D, (size_t)Sc * D * 4, st));
    } else {
        embed_kernel<<<M, 256, 0, st>>>(tokens, m->lm_w, m->lm_s, D, m->cfg.vocab, m->x, device_error_flag(), S, c0, Sc, 0L);
        note_launches(1);
    }
    for (int l = 0; l < m->cfg.layers; l++) {
        const LayerW& L = m->L[l];
        TRY(flexllm_rmsnorm_quant(m->x, L.g0, M, D, m->cfg.eps, FLEXLLM_NORM_PREFILL, nullptr, m->xq, m->xs, st));
        TRY(gemm_i8_prefill(m->xq, m->xs, L.wqkv, L.sqkv, M, QKV, D, nullptr, m->qkv, st, nullptr));
        // the new keys / values go straight into the paged cache, and the chunk's queries attend to the cache
        TRY(mha_prefill_paged(m->qkv, m->cos_t, m->sin_t, L.a_s, B, Sc, c0, HQ, HKV, m->cfg.max_prefill, m->cache, l, m->page_table,
                              m->max_pages, m->att, m->attn_ws, st));
        if (g == 1) {
            TRY(flexllm_quant_per_token(m->att, M, D, m->xq, m->xs, st));
            TRY(gemm_i8_prefill(m->xq, m->xs, L.wo, L.so, M, D, D, nullptr, m->x, st, m->x));       // x += o_proj
            TRY(flexllm_rmsnorm_quant(m->x, L.g1, M, D, m->cfg.eps, FLEXLLM_NORM_PREFILL, nullptr, m->xq, m->xs, st));
            TRY(gemm_i8_prefill(m->xq, m->xs, L.wgu, L.sgu, M, 2 * F, D, nullptr, m->gu, st, nullptr));
            TRY(swiglu_fht_quant_strided(m->gu, m->gu + F, 2L * F, M, m->cfg.fht_scale, m->hq, m->xs, st));
            TRY(gemm_i8_prefill(m->hq, m->xs, L.wd, L.sd, M, D, F, nullptr, m->x, st, m->x));       // x += down_proj
        } else {
            // heads are local: gather the attention output, quantise whole rows, keep this rank's columns
            TRY(flexllm_tp_allgather(m->tp, m->att, m->gath, (size_t)M * Dl * 4, st));
            TRY(quant_gathered(m->gath, M, Dl, g, r, m->xq, m->xs, st));
            TRY(gemm_i8_prefill(m->xq, nullptr, L.wo, nullptr, M, D, Dl, m->acc32, nullptr, st, nullptr));   // partial o_proj
            TRY(flexllm_tp_allreduce_s32(m->tp, m->acc32, (size_t)M * D, st));
            TRY(dequant_residual(m->acc32, m->xs, L.so, M, D, m->x, m->x, st));
            TRY(flexllm_rmsnorm_quant(m->x, L.g1, M, D, m->cfg.eps, FLEXLLM_NORM_PREFILL, nullptr, m->xq, m->xs, st));
            TRY(gemm_i8_prefill(m->xq, m->xs, L.wgu, L.sgu, M, 2 * Fl, D, nullptr, m->gu, st, nullptr));
            TRY(swiglu_slice(m->gu, M, Fl, m->hloc, st));
            TRY(flexllm_tp_allgather(m->tp, m->hloc, m->gath, (size_t)M * Fl * 4, st));
            TRY(fht_quant_gathered(m->gath, M, g, r, m->cfg.fht_scale, m->hq, m->xs, st));
            TRY(gemm_i8_prefill(m->hq, nullptr, L.wd, nullptr, M, D, Fl, m->acc32, nullptr, st, nullptr));   // partial down_proj
            TRY(flexllm_tp_allreduce_s32(m->tp, m->acc32, (size_t)M * D, st));
            TRY(dequant_residual(m->acc32, m->xs, L.sd, M, D, m->x, m->x, st));
        }
    }
    return FLEXLLM_OK;
}

// Prompts longer than max_prefill are processed in chunks of max_prefill tokens (the activation buffers are sized for
// one chunk): chunk after chunk through all layers, each chunk's attention reading the keys and values of the chunks
// before it from the paged KV cache. The reference's host program has one fixed prefill length and repacks the cache
// between its two launches (SpinQuant_Prefilling_Decoding_mem_opt_demo.cpp:947-970); here prefill and decode share one
// paged cache, so there is nothing to repack and no limit but max_ctx.
static int prefill_any(flexllm_model* m, const int32_t* tokens, const float* embeds, int B, int S, int n_valid, int32_t* next_out,
                       cudaStream_t st) {
    m->rows_mode = false;
    const int D = m->cfg.hidden;
    int Sc = S, c_last = 0;
    for (int c0 = 0; c0 < S; c0 += m->cfg.max_prefill) {
        Sc = S - c0 < m->cfg.max_prefill ? S - c0 : m->cfg.max_prefill;
        c_last = c0;
        TRY(prefill_chunk(m, tokens, embeds, B, S, c0, Sc, st));
    }
    // the last chunk's rows are in x; the token comes from the last VALID position (rows after it are padding)
    gather_last_kernel<<<B, 256, 0, st>>>(m->x, Sc, n_valid - c_last, D, m->xlast);
    note_launches(1);
    TRY(run_head(m, m->xlast, B, FLEXLLM_NORM_PREFILL, st));
    fill_ctx_kernel<<<1, 64, 0, st>>>(m->ctx, B, n_valid);
    TRY(launch_status());
    if (next_out) TRY(copy_any(next_out, m->next, (size_t)B * 4, st));
    m->B = B; m->S = n_valid; m->pos = n_valid; m->last_chunk = Sc;
    return FLEXLLM_OK;
}

extern "C" int flexllm_model_prefill(flexllm_model* m, const int32_t* tokens, int B, int S, int32_t* next_out, void* stream) {
    FLEXLLM_REQUIRE(m && tokens && B > 0 && B <= m->cfg.max_batch && S > 0 && S <= m->cfg.max_ctx);
    if (S % 16 != 0) return FLEXLLM_ENOTSUP;
    if (S > m->cfg.max_prefill && m->cfg.max_prefill % 128 != 0) return FLEXLLM_ENOTSUP;     // chunks start at multiples of 128
    cudaStream_t st = (cudaStream_t)stream;
    if (m->dm && B % m->g == 0) return prefill_rows(m, tokens, B, S, next_out, st);
    return prefill_any(m, tokens, nullptr, B, S, S, next_out, st);
}

// Prefill from EMBEDDING VECTORS embeds [B][S][hidden] fp32 (device) instead of token ids -- what the HMT plug-in feeds the
// prefill graph (summary / memory vectors are not rows of the embedding table, Modules/HMT.h:48-170). Rows n_valid .. S-1
// of every sequence are padding up to a multiple of 16 (causal attention: they change nothing before them); the first
// token is chosen at position n_valid - 1 and decoding continues from context length n_valid. Single GPU.
extern "C" int flexllm_model_prefill_embeds(flexllm_model* m, const float* embeds, int B, int S, int n_valid, int32_t* next_out,
                                            void* stream) {
    FLEXLLM_REQUIRE(m && embeds && B > 0 && B <= m->cfg.max_batch && S > 0 && S <= m->cfg.max_ctx && n_valid > 0 && n_valid <= S);
    if (m->g != 1 || S % 16 != 0) return FLEXLLM_ENOTSUP;
    if (S > m->cfg.max_prefill && m->cfg.max_prefill % 128 != 0) return FLEXLLM_ENOTSUP;
    FLEXLLM_REQUIRE(S - n_valid < (S > m->cfg.max_prefill ? S - (S - 1) / m->cfg.max_prefill * m->cfg.max_prefill : S));   // the last valid row lies in the last chunk
    return prefill_any(m, nullptr, embeds, B, S, n_valid, next_out, (cudaStream_t)stream);
}

// Embedding rows of n token ids (tied embeddings: row t = (float)lm_head_q[t] * lm_head_s[t]): tokens [n] -> out [n][hidden].
extern "C" int flexllm_model_embed_tokens(flexllm_model* m, const int32_t* tokens, int n, float* out, void* stream) {
    FLEXLLM_REQUIRE(m && tokens && out && n >= 0);
    if (n == 0) return FLEXLLM_OK;
    embed_kernel<<<n, 256, 0, (cudaStream_t)stream>>>(tokens, m->lm_w, m->lm_s, m->cfg.hidden, m->cfg.vocab, out, device_error_flag(), 1, 0, 1, 0L);
    return launch_status();
}

// One decode step for the B sequences of the last prefill: consumes m->next, leaves the new
// greedy tokens in m->next (and in the output table), appends to the KV cache and advances ctx.
// Builds the persistent decode-step kernel's plan on first use (single GPU only). Shapes or devices
// it does not cover leave the kernel-per-operator path in charge.
static int mega_prepare(flexllm_model* m) {
    if (m->mega_state >= 0) return FLEXLLM_OK;
    m->mega_state = 0;
    if (m->g != 1) return FLEXLLM_OK;
    std::vector<MegaLayerView> lv(m->cfg.layers);
    for (int l = 0; l < m->cfg.layers; l++) {
        const LayerW& w = m->L[l];
        lv[l] = MegaLayerView{w.wqkv, w.wo, w.wgu, w.wd, w.sqkv, w.so, w.sgu, w.sd, w.g0, w.g1, w.a_s};
    }
    MegaModelView v;
    v.layers = m->cfg.layers; v.D = m->cfg.hidden; v.HQ = m->cfg.heads_q; v.HKV = m->cfg.heads_kv; v.F = m->cfg.ffn; v.V = m->cfg.vocab;
    v.max_batch = m->cfg.max_batch; v.max_ctx = m->cfg.max_ctx; v.eps = m->cfg.eps; v.fht_scale = m->cfg.fht_scale;
    v.L = lv.data(); v.lm_w = m->lm_w; v.lm_s = m->lm_s; v.g_final = m->g_final; v.cos_t = m->cos_t; v.sin_t = m->sin_t;
    v.cache = m->cache; v.page_table = m->page_table; v.max_pages = m->max_pages;
    v.ctx = m->ctx; v.next = m->next; v.out_tokens = m->out_tokens; v.state = m->state;
    v.x = m->x; v.xq = m->xq; v.xs = m->xs; v.hq = m->hq; v.att = m->att; v.logits = m->logits;
    const int rc = mega_create(v, &m->mega);
    if (rc == FLEXLLM_OK) { m->mega_state = 1; mega_set_sampling(m->mega, m->sample_lanes, m->sample_k, m->sample_rnd); }
    else if (rc != FLEXLLM_ENOTSUP) return rc;
    return FLEXLLM_OK;
}

static int decode_step_body(flexllm_model* m, cudaStream_t st);
static int decode_step(flexllm_model* m, cudaStream_t st) {
    TRY(mega_prepare(m));
    if (m->mega_state == 1) return mega_launch(m->mega, m->B, m->mega_variant, st);
    static int use_pdl = -1;
    if (use_pdl < 0) { const char* e = getenv("FLEXLLM_PDL"); use_pdl = e ? atoi(e) : 1; }
    g_pdl = use_pdl;
    const int rc = decode_step_body(m, st);
    g_pdl = 0;
    return rc;
}
static int decode_step_body(flexllm_model* m, cudaStream_t st) {
    const int D = m->cfg.hidden, HQ = m->HQl, HKV = m->HKVl, F = m->cfg.ffn;
    const int QKV = (HQ + 2 * HKV) * 64;
    const int B = m->B;
    const int g = m->g, r = m->r, Dl = m->Dl, Fl = m->Fl;
    launch_k(embed_kernel, dim3(B), dim3(256), 0, st, (const int32_t*)m->next, (const int8_t*)m->lm_w, (const float*)m->lm_s, D, m->cfg.vocab, m->x,
             device_error_flag(), 1, 0, 1, 0L);
    note_launches(1);
    for (int l = 0; l < m->cfg.layers; l++) {
        const LayerW& L = m->L[l];
        TRY(flexllm_rmsnorm_quant(m->x, L.g0, B, D, m->cfg.eps, FLEXLLM_NORM_DECODE8, nullptr, m->xq, m->xs, st));
        TRY(flexllm_linear_decode_i8(m->xq, m->xs, L.wqkv, L.sqkv, B, QKV, D, nullptr, m->qkv, st));
        TRY(mha_decode_run(m->cache, l, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, m->qkv, m->cos_t, m->sin_t, L.a_s,
                           m->page_table, m->max_pages, m->ctx, m->cfg.max_ctx, B, HQ, m->att, nullptr, m->dec_ws, st));
        if (g == 1) {
            TRY(flexllm_quant_per_token(m->att, B, D, m->xq, m->xs, st));
            TRY(flexllm_linear_decode_i8_residual(m->xq, m->xs, L.wo, L.so, B, D, D, m->x, m->x, st));
            TRY(flexllm_rmsnorm_quant(m->x, L.g1, B, D, m->cfg.eps, FLEXLLM_NORM_DECODE8, nullptr, m->xq, m->xs, st));
            TRY(flexllm_linear_decode_i8(m->xq, m->xs, L.wgu, L.sgu, B, 2 * F, D, nullptr, m->gu, st));
            TRY(swiglu_fht_quant_strided(m->gu, m->gu + F, 2L * F, B, m->cfg.fht_scale, m->hq, m->xs, st));
            TRY(flexllm_linear_decode_i8_residual(m->hq, m->xs, L.wd, L.sd, B, D, F, m->x, m->x, st));
        } else {
            TRY(flexllm_tp_allgather(m->tp, m->att, m->gath, (size_t)B * Dl * 4, st));
            TRY(quant_gathered(m->gath, B, Dl, g, r, m->xq, m->xs, st));
            TRY(flexllm_linear_decode_i8(m->xq, nullptr, L.wo, nullptr, B, D, Dl, m->acc32, nullptr, st));
            TRY(flexllm_tp_allreduce_s32(m->tp, m->acc32, (size_t)B * D, st));
            TRY(dequant_residual(m->acc32, m->xs, L.so, B, D, m->x, m->x, st));
            TRY(flexllm_rmsnorm_quant(m->x, L.g1, B, D, m->cfg.eps, FLEXLLM_NORM_DECODE8, nullptr, m->xq, m->xs, st));
            TRY(flexllm_linear_decode_i8(m->xq, m->xs, L.wgu, L.sgu, B, 2 * Fl, D, nullptr, m->gu, st));
            TRY(swiglu_slice(m->gu, B, Fl, m->hloc, st));
            TRY(flexllm_tp_allgather(m->tp, m->hloc, m->gath, (size_t)B * Fl * 4, st));
            TRY(fht_quant_gathered(m->gath, B, g, r, m->cfg.fht_scale, m->hq, m->xs, st));
            TRY(flexllm_linear_decode_i8(m->hq, nullptr, L.wd, nullptr, B, D, Fl, m->acc32, nullptr, st));
            TRY(flexllm_tp_allreduce_s32(m->tp, m->acc32, (size_t)B * D, st));
            TRY(dequant_residual(m->acc32, m->xs, L.sd, B, D, m->x, m->x, st));
        }
    }
    TRY(run_head(m, m->x, B, FLEXLLM_NORM_DECODE8, st, m->state));
    launch_k(step_bookkeeping_kernel, dim3(1), dim3(64), 0, st, (const int32_t*)m->next, B, m->out_tokens, m->state, m->ctx, 1);
    return launch_status();
}

// Captures one decode step into a CUDA graph (the launch sequence is identical for every step: the
// context lengths, the token feedback and the output column all live in device memory).
static int build_graph(flexllm_model* m) {
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    cudaStream_t cap;
    FLEXLLM_CHECK_CUDA(cudaStreamCreateWithFlags(&cap, cudaStreamNonBlocking));
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamBeginCapture(cap, cudaStreamCaptureModeThreadLocal);
    int rc = FLEXLLM_OK;
    if (e == cudaSuccess) {
        const unsigned long long before = g_launch_count.load();
        rc = decode_step(m, cap);
        const unsigned long long recorded = g_launch_count.load() - before;   // kernels recorded, not executed
        m->graph_kernels = (int)recorded;
        g_launch_count.fetch_sub(recorded);
        cudaError_t e2 = cudaStreamEndCapture(cap, &g);
        if (e == cudaSuccess) e = e2;
    }
    if (e == cudaSuccess && rc == FLEXLLM_OK) e = cudaGraphInstantiate(&m->graph, g, 0);
    if (g) cudaGraphDestroy(g);
    cudaStreamDestroy(cap);
    if (rc != FLEXLLM_OK) return rc;
    FLEXLLM_CHECK_CUDA(e);
    m->graph_B = m->B; m->graph_variant = m->mega_variant;
    return FLEXLLM_OK;
}

extern "C" int flexllm_model_decode(flexllm_model* m, int n_steps, int use_graph, void* stream) {
    FLEXLLM_REQUIRE(m && m->B > 0 && n_steps >= 0);
    if (m->rows_mode) return flexllm_model_decode(m->dm, n_steps, use_graph, stream);   // this rank's sequences, no collective
    // step i appends at position pos + i, and the page-table rows, the RoPE tables and the attention
    // score rows end at max_ctx: refuse, before anything is launched, steps that would run past it
    FLEXLLM_REQUIRE(n_steps == 0 || (long)m->pos + n_steps - 1 <= (long)m->cfg.max_ctx);
    m->pos += n_steps;
    cudaStream_t st = (cudaStream_t)stream;
    if (flexllm_tp_is_local(m->tp)) use_graph = 0;      // ranks sharing a device: the collectives need their host-side rendezvous
    int done = 0;
    TRY(mega_prepare(m));
    m->mega_variant = m->mega_state == 1 ? mega_variant(m->mega, m->B, m->pos) : 0;      // every position of this call is < m->pos
    if (use_graph && n_steps > 0 && (!m->graph || m->graph_B != m->B || m->graph_variant != m->mega_variant)) {
        // the first step runs eagerly so that every lazily created resource (function attributes,
        // tensor maps, split-K scratch) exists before capture
        TRY(decode_step(m, st));
        done = 1;
        FLEXLLM_CHECK_CUDA(cudaStreamSynchronize(st));
        TRY(build_graph(m));
    }
    for (int i = done; i < n_steps; i++) {
        if (use_graph) { FLEXLLM_CHECK_CUDA(cudaGraphLaunch(m->graph, st)); note_launches(m->graph_kernels); }
        else TRY(decode_step(m, st));
    }
    return FLEXLLM_OK;
}

extern "C" int flexllm_model_begin(flexllm_model* m, int n_new, void* stream) {
    FLEXLLM_REQUIRE(m && m->B > 0 && n_new >= 1 && (size_t)m->B * n_new <= m->out_capacity);
    FLEXLLM_REQUIRE(m->S + n_new - 1 <= m->cfg.max_ctx);
    m->n_new = n_new;
    if (m->rows_mode) return flexllm_model_begin(m->dm, n_new, stream);
    cudaStream_t st = (cudaStream_t)stream;
    set_state_kernel<<<1, 1, 0, st>>>(m->state, 0, n_new);
    step_bookkeeping_kernel<<<1, 64, 0, st>>>(m->next, m->B, m->out_tokens, m->state, m->ctx, 0);
    TRY(mega_prepare(m));
    if (m->mega_state == 1) TRY(mega_reset(m->mega, st));
    return launch_status(2);
}

// Whole request through host buffers: tokens_host [B][S] -> out_host [B][n_new] (greedy; column 0
// is the token chosen by the prefill).
extern "C" int flexllm_model_generate_host(flexllm_model* m, const int32_t* tokens_host, int B, int S, int n_new,
                                           int32_t* out_host, int use_graph, void* stream) {
    FLEXLLM_REQUIRE(m && tokens_host && out_host && n_new >= 1);
    FLEXLLM_REQUIRE(B > 0 && B <= m->cfg.max_batch && S > 0 && S + n_new - 1 <= m->cfg.max_ctx);
    for (size_t i = 0; i < (size_t)B * S; i++) FLEXLLM_REQUIRE(tokens_host[i] >= 0 && tokens_host[i] < m->cfg.vocab);
    cudaStream_t st = (cudaStream_t)stream;
    FLEXLLM_CHECK_CUDA(cudaMemcpyAsync(m->tokens, tokens_host, (size_t)B * S * 4, cudaMemcpyHostToDevice, st));
    TRY(flexllm_model_prefill(m, m->tokens, B, S, nullptr, st));
    TRY(flexllm_model_begin(m, n_new, st));
    TRY(flexllm_model_decode(m, n_new - 1, use_graph, st));
    if (m->rows_mode)      // every rank returns all B sequences: rank blocks of [B / g][n_new] in rank order = sequence order
        TRY(flexllm_tp_allgather(m->tp, m->dm->out_tokens, m->out_tokens, (size_t)(B / m->g) * n_new * 4, st));
    FLEXLLM_CHECK_CUDA(cudaMemcpyAsync(out_host, m->out_tokens, (size_t)B * n_new * 4, cudaMemcpyDeviceToHost, st));
    FLEXLLM_CHECK_CUDA(cudaStreamSynchronize(st));
    return gemm_check_error_flag();
}

// Token choice for the following prefill / decode calls: top_k == 0 -> greedy argmax (the default); otherwise the
// reference's top-k sampling (Logits.h:145-279) with `lanes` lanes and the uniform numbers rnd [n_new][B] in device
// memory (row = output column, i.e. the reference's rand_seeds_mmap per decode step; B = the batch of the
// following prefill). The pointer must stay valid while it is in use.
extern "C" int flexllm_model_set_sampling(flexllm_model* m, int lanes, int top_k, const float* rnd) {
    FLEXLLM_REQUIRE(m && top_k >= 0);
    if (top_k > 0) {
        FLEXLLM_REQUIRE(rnd && lanes > 0);
        if (top_k > 8 || lanes > 64 || m->cfg.vocab % lanes || m->cfg.vocab / lanes < top_k || m->g != 1) return FLEXLLM_ENOTSUP;
    }
    m->sample_lanes = top_k > 0 ? lanes : 0; m->sample_k = top_k; m->sample_rnd = top_k > 0 ? rnd : nullptr;
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }      // the captured step holds the old choice
    if (m->mega) mega_set_sampling(m->mega, m->sample_lanes, m->sample_k, m->sample_rnd);
    return FLEXLLM_OK;
}

extern "C" int flexllm_model_limits(const flexllm_model* m, int* max_batch, int* max_prefill, int* max_ctx) {
    FLEXLLM_REQUIRE(m);
    if (max_batch) *max_batch = m->cfg.max_batch;
    if (max_prefill) *max_prefill = m->cfg.max_prefill;
    if (max_ctx) *max_ctx = m->cfg.max_ctx;
    return FLEXLLM_OK;
}

// Device pointers of internal buffers, for tests: 0 = residual stream x, 1 = logits of the last head
// call, 2 = generated tokens table, 3 = context lengths.
extern "C" int flexllm_model_buffer(flexllm_model* m, int which, void** ptr) {
    FLEXLLM_REQUIRE(m && ptr);
    if (m->rows_mode) {
        // token-row partition: the residual stream is spread over the ranks by rows, logits / tokens / lengths belong to
        // the rank's own sequences. which == 0 gathers the rows (a COLLECTIVE: call it on every rank).
        switch (which) {
            case 0: {
                const size_t n = (size_t)m->B * m->last_chunk / m->g * m->cfg.hidden;      // rows of the last chunk
                TRY(flexllm_tp_allgather(m->tp, m->x, m->gath, n * 4, nullptr));
                FLEXLLM_CHECK_CUDA(cudaStreamSynchronize(nullptr));
                *ptr = m->gath; return FLEXLLM_OK;
            }
            case 1: *ptr = m->dm->logits; return FLEXLLM_OK;
            case 2: *ptr = m->dm->out_tokens; return FLEXLLM_OK;
            case 3: *ptr = m->dm->ctx; return FLEXLLM_OK;
            default: return FLEXLLM_EINVAL;
        }
    }
    switch (which) {
        case 0: *ptr = m->x; break;
        case 1: *ptr = m->logits; break;
        case 2: *ptr = m->out_tokens; break;
        case 3: *ptr = m->ctx; break;
        default: return FLEXLLM_EINVAL;
    }
    return FLEXLLM_OK;
}
