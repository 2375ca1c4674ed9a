/* flexllm_b200 -- C ABI of the B200 (sm_100a) implementation of FlexLLM's quantized
 * Llama-3.2-1B operator path.
 *
 * FlexLLM's operators are C++ function templates over TAPA streams (Modules/ *.h); a host
 * program reaches them through tapa::invoke(top_fn, bitstream, mmaps..., scalars...)
 * (SpinQuant_Llama_32_1B/Linear_Layer_Prefilling_tb.cpp:106-113). There is no FFI in the
 * reference, so each entry point below names the operator template(s) it replaces. The C++ host
 * API in include/flexllm/ keeps the Modules/ names and calls these functions.
 *
 * Conventions
 *  - every pointer is a DEVICE pointer unless the parameter name ends in _host;
 *  - tensors are row-major and dense; weights are [N][K] with K contiguous (the layout of the
 *    reference's parameter files, Linear_Layer_Prefilling_tb.cpp:318-351);
 *  - `stream` is a cudaStream_t passed as void* (NULL = default stream); calls are asynchronous;
 *  - return value: FLEXLLM_OK or a negative FLEXLLM_E* code; nothing aborts or throws;
 *  - the caller owns all buffers; the library owns only the opaque handles it creates;
 *  - there is no CPU fallback: without a CUDA device every compute call returns FLEXLLM_ECUDA.
 */
#ifndef FLEXLLM_B200_H
#define FLEXLLM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FLEXLLM_API __attribute__((visibility("default")))
#else
#define FLEXLLM_API
#endif

#define FLEXLLM_OK 0
#define FLEXLLM_EINVAL (-1)    /* bad dimension, alignment or null pointer */
#define FLEXLLM_ECUDA (-2)     /* CUDA runtime error (see flexllm_last_cuda_error) */
#define FLEXLLM_ETIMEDOUT (-3) /* a bounded device-side wait gave up */
#define FLEXLLM_ENOTSUP (-4)   /* shape outside what the kernels were built for */
#define FLEXLLM_ENOMEM (-5)
#define FLEXLLM_ETOOBIG (-6)   /* problem larger than a fixed built-in buffer */
#define FLEXLLM_EDEVDATA (-7)  /* a token id or context length in DEVICE memory was out of range (clamped) */
#define FLEXLLM_EIO (-8)       /* a parameter file could not be opened, or holds fewer values than asked for */

/* RMSNorm summation orders (Modules/LayerNorm.h:82-130 prefill, :263-321 decode). */
#define FLEXLLM_NORM_PREFILL 0 /* 4 interleaved partial sums over the whole row          */
#define FLEXLLM_NORM_DECODE8 8 /* 8 contiguous chunks, 4 interleaved partial sums in each */
#define FLEXLLM_NORM_DECODE4 4

FLEXLLM_API int flexllm_version(void);
FLEXLLM_API const char* flexllm_status_string(int status);
/* cudaError_t of the most recent failing CUDA call on this thread (0 if none). */
FLEXLLM_API int flexllm_last_cuda_error(void);
/* Kernels launched by this library in this process so far (a graph replay counts its kernel nodes). */
FLEXLLM_API unsigned long long flexllm_launch_count(void);
/* Device-side waits (TMA / MMA pipeline barriers, the grid barrier of the persistent decode kernel) are
 * bounded: a wait that runs out makes the kernel leave through its tear-down, possibly with partial
 * results, and raise one error word per device. Calls are asynchronous, so they cannot report that
 * themselves; this call synchronises the current device, returns FLEXLLM_ETIMEDOUT if any kernel of
 * the library has raised the word since the last check (from any host thread) and clears it, else
 * FLEXLLM_OK. The same word reports FLEXLLM_EDEVDATA: a kernel met a token id outside [0, vocab) or a
 * context length outside [0, max_ctx] in device memory (values the host never sees, e.g. ids fed back by
 * a sampler); such a value is clamped so that it can never become an out-of-bounds access. flexllm_model_generate_host performs this check itself. The reference has no
 * counterpart: a mis-sized stream there simply deadlocks the simulation. */
FLEXLLM_API int flexllm_device_status(void);

/* ---------------------------------------------------------------------------------------------
 * Linear layers.   acc[m][n] = sum_k a[m][k]*w[n][k]  (exact int32);
 *                  y[m][n]   = ((float)acc * s_tok[m]) * s_ch[n]
 * Replaces pref_Linear_Layer_i4xi4 (Modules/Linear_Layer.h:293-341) + pref_dequant_layer_qint_fp32
 * (Modules/quant.h:115-164) at 8-bit symmetric precision, and dec_Linear_Layer_i4xi4
 * (Linear_Layer.h:862-923) + dec_dequant_layer_qint_fp32 (quant.h:434-524) for decode.
 * acc and y may each be NULL (not both). K % 16 == 0.
 * prefill: tcgen05 tensor-core GEMM, any M >= 1, N % 8 == 0.
 * decode : M <= 64 tokens; weight-streaming GEMV (M <= 8) or tensor-core skinny GEMM.
 * ------------------------------------------------------------------------------------------- */
FLEXLLM_API int flexllm_linear_prefill_i8(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch,
                              int M, int N, int K, int32_t* acc, float* y, void* stream);
FLEXLLM_API int flexllm_linear_decode_i8(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch,
                             int M, int N, int K, int32_t* acc, float* y, void* stream);
/* Library-owned state of the decode layer (9..64 tokens): its split-K partial sums go through ONE scratch
 * buffer per device (32 MiB, allocated by the first such call on the device and kept until the process
 * exits -- make that call outside any stream capture). Calls on one stream share it safely; calls that can
 * overlap on the GPU (different streams of one device) would mix their partial sums: serialise them. */

/* The same two layers fused with the residual add that follows them in the model
 * (pref_Residual_Layer / dec_Residual_Layer, Residual_Layer.h:46-87): y = residual + dequant(acc).
 * residual and y have the layout of y above and may alias. */
FLEXLLM_API int flexllm_linear_prefill_i8_residual(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch,
                                       int M, int N, int K, const float* residual, float* y, void* stream);
FLEXLLM_API int flexllm_linear_decode_i8_residual(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch,
                                      int M, int N, int K, const float* residual, float* y, void* stream);

/* Decode linear layer that never allocates (no counterpart in the reference, whose operators own no
 * run-time memory at all). For hosts that must not, or cannot, call cudaMalloc around a decode step:
 * serving loops that have handed the whole device to their own memory pool, and latency-critical
 * loops where an allocation would stall every stream of the device. Same result as
 * flexllm_linear_decode_i8 (y only), always on the tensor-core split-K path; the int32 partial sums
 * live in a 4 MiB array built into the library image (each GPU that loads the library holds it until
 * exit) instead of a cudaMalloc'd scratch buffer. Limits and rules:
 *  - M <= 64 and M*N <= 64*16384 (e.g. 64 tokens x the fused gate|up projection); larger problems
 *    return FLEXLLM_ETOOBIG and leave y untouched;
 *  - the first call on each device looks up the array's device address; make it before any CUDA
 *    stream capture begins;
 *  - all calls share the one array (it is cleared at the start of every call): two calls that can
 *    run concurrently on the GPU, e.g. on different streams, race -- serialise them;
 *  - a device-side wait that runs out is reported by flexllm_device_status(), as for every other
 *    entry point. */
FLEXLLM_API int flexllm_linear_decode_i8_noalloc(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch,
                                     int M, int N, int K, float* y, void* stream);

/* Dynamic per-token symmetric int8 quantisation: s = max|x|/127 (0 -> 1), q = round(x/s).
 * Replaces pref_quant_layer_fp32_qint / dec_quant_layer_fp32_qint (quant.h:6-112, :332-431). */
FLEXLLM_API int flexllm_quant_per_token(const float* x, int M, int K, int8_t* q, float* s, void* stream);

/* y = ((float)acc * s_tok[m]) * s_ch[n].  Replaces pref_dequant_layer_qint_fp32 (quant.h:115-164)
 * and pref_static_sym_dequant_layer_qint_fp32 (quant.h:214-249). */
FLEXLLM_API int flexllm_dequant(const int32_t* acc, const float* s_tok, const float* s_ch, int M, int N, float* y,
                    void* stream);

/* Static symmetric quantisation q = clamp(round(x / (f * s[row]))): signed -> [-128,127],
 * unsigned -> upper clamp 255 only. s_stride 0 = one scale for all rows, 1 = one per row.
 * Replaces pref_static_sym_per_tensor_quant_layer_fp32_qint (quant.h:252-295) and
 * pref_static_sym_quant_layer_fp32_qint (quant.h:166-211). */
FLEXLLM_API int flexllm_static_quant(const float* x, long rows, int n, const float* s, int s_stride, float f,
                         int is_signed, uint8_t* q, void* stream);

/* Walsh-Hadamard transform of each row, natural order, divided by `scale`; bit-identical to
 * pref_FHT / dec_FHT (Modules/FHT.h:7-129). N a power of two, 2 <= N <= 8192. */
FLEXLLM_API int flexllm_fht(const float* x, long rows, int N, float scale, float* y, void* stream);

/* Half-split rotary embedding by table, head_dim 64. x,y [T][H][64]; pos [T]; tables [P][32].
 * Replaces pref_RoPE_layer / dec_RoPE_layer (Modules/RoPE.h:8-173). */
FLEXLLM_API int flexllm_rope(const float* x, const int32_t* pos, const float* cos_t, const float* sin_t, long T,
                 int H, float* y, void* stream);

/* Row softmax with the reference's summation order; valid (NULL or [rows]) = number of leading
 * unmasked entries (the rest are set to -1e32 first). Replaces pref_causal_mask_template
 * (Modules/MHA.h:246-273) + pref_Softmax / dec_MHA_Softmax (Modules/Softmax.h:6-163, :456-635). */
FLEXLLM_API int flexllm_softmax(const float* x, long rows, int len, const int32_t* valid, float* p, void* stream);

/* RMSNorm y = (x * r) * gamma with the summation order of `order` (FLEXLLM_NORM_*), optionally
 * fused with the per-token int8 quantiser that follows it in the model (q, s non-NULL).
 * y may be NULL when q is given. Replaces pref_Layer_Norm / dec_Layer_Norm
 * (Modules/LayerNorm.h:28-183, :210-370) [+ quant.h:6-112]. */
FLEXLLM_API int flexllm_rmsnorm_quant(const float* x, const float* gamma, int M, int D, float eps, int order,
                          float* y, int8_t* q, float* s, void* stream);

/* y = g / (1 + exp(-g))                      pref_Swish / dec_Swish (Modules/Swish.h) */
FLEXLLM_API int flexllm_swish(const float* g, long n, float* y, void* stream);
/* y = a * b                                  pref_Gate_Layer_fp32xfp32 (Linear_Layer.h:612-630) */
FLEXLLM_API int flexllm_gate(const float* a, const float* b, long n, float* y, void* stream);
/* y = a + b                                  pref_Residual_Layer (Residual_Layer.h:46-87) */
FLEXLLM_API int flexllm_residual(const float* a, const float* b, long n, float* y, void* stream);

/* Fused  silu(g)*u -> FHT-N / scale -> per-token int8 quant   (Swish.h + Linear_Layer.h:612-630 +
 * FHT.h + quant.h:6-112, in the order of SpinQuant_Prefilling.h:1017-1035). g,u [M][N] fp32 ->
 * q [M][N] s8, s [M]. act (optional) receives silu(g)*u. N == 8192. */
FLEXLLM_API int flexllm_swiglu_fht_quant(const float* g, const float* u, int M, int N, float scale, int8_t* q,
                             float* s, float* act, void* stream);

/* Greedy token: argmax with ties to the lowest index = rank 0 of sort_top_k (Logits.h:5-31). */
FLEXLLM_API int flexllm_logits_argmax(const float* logits, int B, long V, int32_t* idx, void* stream);

/* Top-k sampling = dec_Sampling_Embedding_Layer without the embedding gather (Logits.h:145-279, instantiated as in
 * SpinQuant_Decoding_mem_opt.h:934: inner_block_parallel 1, enable_sub_max): `lanes` lanes each keep a sorted top-k of
 * their contiguous V/lanes slice (strict '>' insertion in index order), the lists are merged rank by rank, softmax over the
 * k winners, and the token is the first k whose cumulative probability exceeds rnd[b] (a uniform number in [0,1) from the
 * host, the reference's rand_seeds_mmap), else the last. logits [B][V] fp32, rnd [B] -> idx [B]; top_idx / top_val
 * (optional) [B][top_k] receive the merged list. V % lanes == 0, top_k <= 8, lanes <= 64 (the reference: 16..32 lanes, k = 5). */
FLEXLLM_API int flexllm_topk_sample(const float* logits, int B, long V, int lanes, int top_k, const float* rnd, int32_t* idx,
                                    int32_t* top_idx, float* top_val, void* stream);

/* Q/K preparation: x = (float)q*s -> RoPE(pos) -> FHT-64/8 -> per-head dynamic int8 quant.
 * q [T][H][64] s8, s [T][H] -> q_out, s_out same shapes (quant.h:242, RoPE.h:61-90, FHT.h at
 * N=64, quant.h:527-650). */
FLEXLLM_API int flexllm_qk_prepare(const int8_t* q, const float* s, const int32_t* pos, const float* cos_t,
                       const float* sin_t, long T, int H, int8_t* q_out, float* s_out, void* stream);

/* The decode MLP block as one call: the FFN passes of the reference's decode graph (SpinQuant_Decoding_mem_opt.h: the
 * shared dec_Layer_Norm_012 :1061, dec_quant_layer_qkvo_FFN :1066, dec_Linear_Layer_i4xi4_qkvo_FFN_half :1078-1079 and
 * dec_dequant_layer_qkvo_FFN :1082 on their gate / up / down turns, dec_Swish_Layer_FFN, dec_Gate_layer_FFN and dec_FHT_R4
 * :1115-1117, dec_residual_layer :1111): RMSNorm + quantiser -> gate and up linear layers + dequantisers -> Swish and
 * gate -> FHT-8192 -> quantiser -> down linear layer + dequantiser -> residual, for M <= 64 tokens.
 * x, y [M][D] fp32 (y may alias x); gamma [D]; w_gu [2F][D] int8 = gate rows then up rows, s_gu [2F]; w_d [D][F],
 * s_d [D]; order = FLEXLLM_NORM_*; F must be 8192. Results are bit-identical to calling the five operators one by one.
 * workspace: flexllm_mlp_block_workspace(M, D, F) bytes. */
FLEXLLM_API size_t flexllm_mlp_block_workspace(int M, int D, int F);
FLEXLLM_API int flexllm_mlp_block_decode(const float* x, const float* gamma, const int8_t* w_gu, const float* s_gu,
                              const int8_t* w_d, const float* s_d, int M, int D, int F, float eps, int order, float fht_scale,
                              float* y, void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Prefill GQA attention, int8 x int8 (replaces the graph MHA_i8xi8_Prefilling_tb,
 * SpinQuant_Llama_32_1B/MHA_i8xi8.h:369-427, with per-head-per-token scales).
 * q [B][S][HQ][64] s8, qs [B][S][HQ]; k,v [B][S][HKV][64] s8, ks,vs [B][S][HKV]; a_s [HQ];
 * out fp32 [B][S][HQ*64]. Steps: qk_prepare on q and k (positions 0..S-1) -> S = q.k^T (s32) ->
 * score = ((float)S*qs)*ks*0.125 -> causal softmax -> P~ = P*vs[key] -> u8 = min(round(P~/a_s),255)
 * -> O = u8 x v (s32) -> out = (float)O * a_s.  oacc (optional) receives the int32 O.
 * workspace: flexllm_mha_prefill_workspace(B,S,HQ,HKV) bytes.
 * ------------------------------------------------------------------------------------------- */
FLEXLLM_API size_t flexllm_mha_prefill_workspace(int B, int S, int HQ, int HKV);
FLEXLLM_API int flexllm_mha_i8xi8_prefill(const int8_t* q, const float* qs, const int8_t* k, const float* ks,
                              const int8_t* v, const float* vs, const float* cos_t, const float* sin_t,
                              const float* a_s, int B, int S, int HQ, int HKV, float* out, int32_t* oacc,
                              void* workspace, size_t workspace_bytes, void* stream);
/* The same attention in ONE sweep over the keys with a flash-style online softmax (running maximum and denominator,
 * fast exponentials, P quantised per 64-key tile against the tile's largest value scale, output rescaled in fp32).
 * NOT bit-exact with the reference arithmetic above and not used unless asked for: it exists so that the cost of the
 * exact three-sweep kernel is a measured number. Agreement with flexllm_mha_i8xi8_prefill: a few times 1e-3 of the
 * output's largest magnitude. No a_s (P's scale is chosen per tile), no oacc. Same workspace. */
FLEXLLM_API int flexllm_mha_i8xi8_prefill_online(const int8_t* q, const float* qs, const int8_t* k, const float* ks,
                              const int8_t* v, const float* vs, const float* cos_t, const float* sin_t,
                              int B, int S, int HQ, int HKV, float* out, void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Paged int8 KV cache (replaces dec_K_cache_manager / dec_V_cache_manager and their scale caches,
 * Modules/MHA.h:393-559, :713-851). One pool per layer set: pages of `page` tokens;
 * K,V pages [n_pages][HKV][page][64] s8, scale pages [n_pages][HKV][page] fp32, per layer.
 * ------------------------------------------------------------------------------------------- */
typedef struct flexllm_kv_cache flexllm_kv_cache;
FLEXLLM_API int flexllm_kv_cache_create(flexllm_kv_cache** out, int layers, int n_pages, int hkv, int page);
FLEXLLM_API int flexllm_kv_cache_destroy(flexllm_kv_cache* c);
FLEXLLM_API int flexllm_kv_cache_reset(flexllm_kv_cache* c, void* stream);
/* raw device pointers of one layer's pools (for tests and zero-copy hand-off) */
FLEXLLM_API int flexllm_kv_cache_pools(flexllm_kv_cache* c, int layer, int8_t** k, float** ks, int8_t** v, float** vs);

/* Append alone: the new token's int8 K and V heads k,v [B][HKV][64] with scales ks,vs [B][HKV] are stored at
 * position ctx[b] of each sequence (replaces dec_K_cache_manager_template / dec_V_cache_manager_template,
 * Modules/MHA.h:484-513, :773-801, without the read-back). No RoPE, no quantisation: bytes are stored as given. */
FLEXLLM_API int flexllm_kv_append(flexllm_kv_cache* c, int layer, const int8_t* k, const float* ks, const int8_t* v,
                                  const float* vs, const int32_t* page_table, int max_pages, const int32_t* ctx,
                                  int max_ctx, int B, void* stream);

/* One decode step of attention for B sequences on one layer (replaces the graph
 * MHA_i8xi8_decoding_tb, MHA_i8xi8.h:1027-1114): qk_prepare of the new q,k at position ctx[b];
 * append k,v to the cache; attention over ctx[b]+1 keys; out fp32 [B][HQ*64].
 * q [B][HQ][64], qs [B][HQ]; k,v [B][HKV][64], ks,vs [B][HKV]; page_table [B][max_pages] s32;
 * ctx [B] s32 (tokens already cached). */
FLEXLLM_API size_t flexllm_mha_decode_workspace(int B, int HQ, int max_ctx);
FLEXLLM_API int flexllm_mha_i8xi8_decode(flexllm_kv_cache* c, int layer, const int8_t* q, const float* qs,
                             const int8_t* k, const float* ks, const int8_t* v, const float* vs,
                             const float* cos_t, const float* sin_t, const float* a_s,
                             const int32_t* page_table, int max_pages, const int32_t* ctx, int max_ctx,
                             int B, int HQ, float* out, int32_t* oacc, void* workspace,
                             size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Tensor parallelism over the GPUs of one node (no counterpart in the reference, a single-FPGA
 * design): one process per GPU; q/k/v and gate/up column-parallel (by heads / FFN channels), o and
 * down row-parallel with an all-reduce of the exact int32 partial sums, lm_head vocab-parallel.
 * Results are bit-identical to the single-GPU model. Collectives run on NCCL, loaded at run time
 * (nccl_lib_path: fallback path of libnccl.so.2 when the process has not loaded it yet).
 * ------------------------------------------------------------------------------------------- */
typedef struct flexllm_tp flexllm_tp;
FLEXLLM_API int flexllm_tp_unique_id(unsigned char* id128, const char* nccl_lib_path);   /* rank 0; share the 128 bytes */
FLEXLLM_API int flexllm_tp_init(flexllm_tp** out, int rank, int size, const unsigned char* id128, const char* nccl_lib_path);
/* `size` (<= 8) communicators whose ranks SHARE the current device: each is driven by its own host thread of this
 * process, all ranks issue their work to one stream, and a collective is a rendezvous of those threads around device
 * copies in that stream (no NCCL). It runs the partitioned model of any rank count on a single GPU, for checking the
 * partition's arithmetic where fewer GPUs than ranks are at hand; it is not a way to go faster. Its collectives cannot
 * be captured into a CUDA graph (FLEXLLM_ENOTSUP); the model runner ignores use_graph on such a group. out[size]. */
FLEXLLM_API int flexllm_tp_init_local(flexllm_tp** out, int size);
FLEXLLM_API int flexllm_tp_is_local(const flexllm_tp* t);      /* 1 for a communicator made by flexllm_tp_init_local */
FLEXLLM_API int flexllm_tp_destroy(flexllm_tp* t);
FLEXLLM_API int flexllm_tp_rank(const flexllm_tp* t);
FLEXLLM_API int flexllm_tp_size(const flexllm_tp* t);
FLEXLLM_API int flexllm_tp_allreduce_s32(flexllm_tp* t, int32_t* buf, size_t count, void* stream);
FLEXLLM_API int flexllm_tp_allgather(flexllm_tp* t, const void* send, void* recv, size_t bytes_per_rank, void* stream);
/* sum of the ranks' int32 buffers [size][count_per_rank]; rank r receives block r */
FLEXLLM_API int flexllm_tp_reduce_scatter_s32(flexllm_tp* t, const int32_t* send, int32_t* recv, size_t count_per_rank, void* stream);
FLEXLLM_API int flexllm_tp_allreduce_max_f32(flexllm_tp* t, float* buf, size_t count, void* stream);
/* block p of `send` goes to rank p; block p of `recv` comes from rank p */
FLEXLLM_API int flexllm_tp_alltoall(flexllm_tp* t, const void* send, void* recv, size_t bytes_per_pair, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Whole-model runner: the two top-level graphs of the reference, SpinQuant_Prefilling
 * (SpinQuant_Llama_32_1B/SpinQuant_Prefilling.h:807) and SpinQuant_Decoding
 * (SpinQuant_Decoding_mem_opt.h:947), and the host flow of its demo
 * (SpinQuant_Prefilling_Decoding_mem_opt_demo.cpp: prefill, KV hand-off, decode loop).
 * Greedy decoding; tied embeddings (embedding row t = (float)lm_head_q[t] * lm_head_s[t]).
 * The model copies the weights it is given (fusing q|k|v and gate|up) and owns its KV cache,
 * activations and CUDA graph.
 * ------------------------------------------------------------------------------------------- */
typedef struct flexllm_model flexllm_model;
typedef struct {
    int layers, hidden, heads_q, heads_kv, ffn, vocab;
    float eps, fht_scale;              /* 1e-5, sqrt(ffn) = 90.50966799 */
    int max_batch, max_prefill, max_ctx; /* max_ctx = longest prompt + generated tokens */
} flexllm_model_config;
typedef struct {                       /* device or host pointers, row-major [N][K] weights */
    const int8_t *wq, *wk, *wv, *wo, *wg, *wu, *wd;
    const float *sq, *sk, *sv, *so, *sg, *su, *sd; /* per-output-channel scales */
    const float *gamma0, *gamma1;      /* RMSNorm weights before attention / before the MLP */
    const float *a_s;                  /* [heads_q] static scale of the u8 attention probabilities */
} flexllm_layer_weights;
FLEXLLM_API int flexllm_model_create(flexllm_model** out, const flexllm_model_config* cfg);
/* The same model partitioned over the ranks of `tp` (NULL = single GPU). Every rank passes the FULL
 * weights to flexllm_model_load_layer / _load_head and keeps its own slice. */
FLEXLLM_API int flexllm_model_create_tp(flexllm_model** out, const flexllm_model_config* cfg, flexllm_tp* tp);
FLEXLLM_API int flexllm_model_destroy(flexllm_model* m);
FLEXLLM_API int flexllm_model_load_layer(flexllm_model* m, int layer, const flexllm_layer_weights* w, void* stream);
FLEXLLM_API int flexllm_model_load_head(flexllm_model* m, const int8_t* lm_w, const float* lm_s, const float* gamma_final,
                            const float* cos_t, const float* sin_t, int table_len, void* stream);
/* tokens [B][S] (device) -> KV cache filled, first greedy token per sequence in next_out [B] (device, optional). */
FLEXLLM_API int flexllm_model_prefill(flexllm_model* m, const int32_t* tokens, int B, int S, int32_t* next_out, void* stream);
/* Start a generation of n_new tokens per sequence after a prefill (records the prefill's token). */
FLEXLLM_API int flexllm_model_begin(flexllm_model* m, int n_new, void* stream);
/* n_steps further greedy steps; use_graph != 0 replays one captured CUDA graph per step. */
FLEXLLM_API int flexllm_model_decode(flexllm_model* m, int n_steps, int use_graph, void* stream);
/* Whole request through HOST buffers: tokens_host [B][S] -> out_host [B][n_new]; synchronises. */
FLEXLLM_API int flexllm_model_generate_host(flexllm_model* m, const int32_t* tokens_host, int B, int S, int n_new,
                                int32_t* out_host, int use_graph, void* stream);
/* Prefill from embedding vectors embeds [B][S][hidden] fp32 (device) instead of token ids: rows n_valid .. S-1 of every
 * sequence are padding up to a multiple of 16; the first token is chosen at position n_valid - 1 and decoding continues
 * from context length n_valid (what the HMT plug-in needs: its summary and memory vectors are not rows of the embedding
 * table, Modules/HMT.h:48-170). Single GPU. */
FLEXLLM_API int flexllm_model_prefill_embeds(flexllm_model* m, const float* embeds, int B, int S, int n_valid, int32_t* next_out,
                                             void* stream);
/* Embedding rows (tied embeddings) of n token ids: tokens [n] (device) -> out [n][hidden] fp32 (device). */
FLEXLLM_API int flexllm_model_embed_tokens(flexllm_model* m, const int32_t* tokens, int n, float* out, void* stream);

/* ---------------------------------------------------------------------------------------------
 * HMT long-context plug-in (Modules/HMT.h; HMT_SpinQuant_Llama_32_1B/): the prompt is processed in segments of seg_len
 * tokens through the same prefill path; per segment a summary pass over [T, first sum_len tokens, T] queries a ring of
 * mem_num memory vectors by fp32 cross-attention (Q = Wq S, keys Wk M, dec_Softmax with scale sqrt(hidden)) for the
 * prompt vector P, and the main pass over [P, rec_len tokens of the previous segment, the segment, P] yields the new
 * memory vector (hmt_segment_loader_sync_template HMT.h:8-195, cross-attention :278-355, memory caches :357-470).
 * The reference's sizes: seg_len 990, sum_len 495, rec_len 32, mem_num 64. The model must have
 * max_prefill >= 1 + rec_len + seg_len + 1 rounded up to 16, max_batch >= 1. One sequence per call.
 * wq, wk [hidden][hidden] fp32 and t_embed [hidden] (host or device) are copied. After flexllm_hmt_prefill the model
 * holds the last segment's KV cache and first token: continue with flexllm_model_begin / flexllm_model_decode.
 * ------------------------------------------------------------------------------------------- */
typedef struct { int seg_len, sum_len, rec_len, mem_num; } flexllm_hmt_config;
typedef struct flexllm_hmt flexllm_hmt;
FLEXLLM_API int flexllm_hmt_create(flexllm_hmt** out, flexllm_model* model, const flexllm_hmt_config* cfg, int hidden,
                                   const float* wq, const float* wk, const float* t_embed);
FLEXLLM_API int flexllm_hmt_destroy(flexllm_hmt* h);
/* embeds [T][hidden] fp32 (device); next_out [1] (device, optional); trace (device, optional) [segments][4][hidden]
 * receives S_n, P_n, M_n, K_n of each segment that produces them. */
FLEXLLM_API int flexllm_hmt_prefill(flexllm_hmt* h, const float* embeds, int T, int32_t* next_out, float* trace, void* stream);

/* Token choice of the following prefill / decode calls. top_k == 0: greedy argmax (default). Otherwise the reference's
 * top-k sampling (flexllm_topk_sample) with `lanes` lanes and uniform numbers rnd [n_new][B] in DEVICE memory, row c for
 * output column c -- the reference's rand_seeds_mmap, one number per decode step (SpinQuant_Decoding_mem_opt.h:934-937).
 * The token feedback stays on the device in both decode paths. Single GPU only. */
FLEXLLM_API int flexllm_model_set_sampling(flexllm_model* m, int lanes, int top_k, const float* rnd);

/* Measurement aid: the prefill GEMM's TMA -> shared memory -> tcgen05.mma kind::i8 -> TMEM pipeline on
 * a [M][K] x [N][K] problem with an epilogue that reads the accumulators and stores nothing. Its rate is
 * the int8 tensor-core ceiling this library's main loop reaches on the device (N > 128). */
FLEXLLM_API int flexllm_gemm_i8_mainloop_probe(const int8_t* a, const int8_t* w, int M, int N, int K, void* stream);

/* ---------------------------------------------------------------------------------------------
 * The reference's on-disk model (its demo's parameters/ directory; host code, HOST buffers):
 *   <proj>_L%02d.bin int8 [out][in]; w_<proj>_s_sum.h with w_<proj>_s / w_<proj>_sum [layers][out]; w_rmsnorm.h with
 *   RMSNorm_weight[2*layers+1][hidden]; A_s.h; RoPE_sin_cos.h (PE_cos, PE_sin [pos][32]); lm_head_L00.bin,
 *   w_lm_head_lm_head.h; model_embed_tokens_fp32.bin  (readers of the demo:
 *   SpinQuant_Llama_32_1B_Ins/SpinQuant_Prefilling_Decoding_mem_opt_demo.cpp:21-74, :132-175, :437-490).
 * NULL members / arguments are skipped. The buffers a layer fills are exactly what flexllm_model_load_layer takes
 * (host pointers are accepted there), so a checkpoint directory can be loaded layer by layer.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
    int8_t *wq, *wk, *wv, *wo, *wg, *wu, *wd;             /* [out][in] */
    float *sq, *sk, *sv, *so, *sg, *su, *sd;              /* per-channel scales  w_<proj>_s[layer]   */
    float *sumq, *sumk, *sumv, *sumo, *sumg, *sumu, *sumd; /* row sums            w_<proj>_sum[layer] */
    float *gamma0, *gamma1, *a_s;
} flexllm_ckpt_layer_buffers;
FLEXLLM_API int flexllm_ckpt_read_bin(const char* path, size_t offset_bytes, size_t bytes, void* out_host);
/* `count` numbers of the C array `name` defined in the header file `path`, starting at flat index `skip` */
FLEXLLM_API int flexllm_ckpt_read_c_array_f32(const char* path, const char* name, long skip, long count, float* out_host);
FLEXLLM_API int flexllm_ckpt_load_layer(const char* dir, int layer, int hidden, int kv_hidden, int ffn, int heads_q,
                                        const flexllm_ckpt_layer_buffers* buffers);
FLEXLLM_API int flexllm_ckpt_load_head(const char* dir, int layers, int hidden, int vocab, int table_len, int8_t* lm_w,
                                       float* lm_s, float* lm_sum, float* gamma_final, float* cos_t, float* sin_t,
                                       float* embed);

/* ---------------------------------------------------------------------------------------------
 * The reference's shipped precision for the linear layers: asymmetric activations of `bits` bits per token
 * (pref_quant_layer_fp32_qint<4, true, ...>, Modules/quant.h:53-81) against symmetric per-channel weights, with the
 * zero point folded into the dequantiser (quant.h:146-148):
 *     s = (max - min) / (2^bits - 1) (0 -> 1),  b = min,  q = round((x - b) / s)  in [0, 2^bits - 1]
 *     y[m][n] = ((float)acc * s[m]) * s_ch[n] + b[m] * wsum[n],   wsum[n] = sum_k w[n][k] * s_ch[n]
 * q is stored one value per byte; the integer product runs on the same int8 tensor-core GEMM (values of up to 7 bits
 * are non-negative int8), so 2 <= bits <= 7. The linear entries need `acc` (int32 [M][N], also an output).
 * ------------------------------------------------------------------------------------------- */
FLEXLLM_API int flexllm_quant_per_token_asym(const float* x, int M, int K, int bits, uint8_t* q, float* s, float* b, void* stream);
FLEXLLM_API int flexllm_dequant_asym(const int32_t* acc, const float* s_tok, const float* b_tok, const float* s_ch,
                                     const float* wsum, int M, int N, float* y, void* stream);
FLEXLLM_API int flexllm_linear_prefill_asym(const uint8_t* a, const float* s_tok, const float* b_tok, const int8_t* w,
                                            const float* s_ch, const float* wsum, int M, int N, int K, int32_t* acc, float* y,
                                            void* stream);
FLEXLLM_API int flexllm_linear_decode_asym(const uint8_t* a, const float* s_tok, const float* b_tok, const int8_t* w,
                                           const float* s_ch, const float* wsum, int M, int N, int K, int32_t* acc, float* y,
                                           void* stream);

/* Test aids for the failure path of the persistent decode-step kernel (no counterpart in the reference).
 * which = 0: bound, in nanoseconds, of that kernel's grid-barrier and flag waits (0 restores the default
 * of 2 s). which = 1, value != 0: the NEXT decode step's first grid barrier waits for one arrival more than
 * the grid delivers, so the wait runs out, the kernel returns through its tear-down, and
 * flexllm_device_status() reports FLEXLLM_ETIMEDOUT (one-shot). A generation that timed out is void: start
 * again from flexllm_model_prefill / flexllm_model_begin, which also re-arm the barrier counter. */
FLEXLLM_API int flexllm_debug_hook(int which, long long value);

/* The sizes the model was created with. */
FLEXLLM_API int flexllm_model_limits(const flexllm_model* m, int* max_batch, int* max_prefill, int* max_ctx);

/* Device pointers of internal buffers (tests): 0 residual stream, 1 logits, 2 token table, 3 ctx. */
FLEXLLM_API int flexllm_model_buffer(flexllm_model* m, int which, void** ptr);

#ifdef __cplusplus
}
#endif
#endif /* FLEXLLM_B200_H */
