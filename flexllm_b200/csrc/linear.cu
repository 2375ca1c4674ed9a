// C-ABI entry points of the W8A8 linear layers: shape checks, choice between the weight-streaming
// GEMV and the tcgen05 GEMM, split-K bookkeeping for decode.
#include <mutex>

#include "common.cuh"

namespace flexllm {
int gemv_i8(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch, int M, int N, int K,
            int32_t* acc, float* y, const float* residual, cudaStream_t st);
int gemm_i8_prefill(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch, int M, int N, int K,
                    int32_t* acc, float* y, cudaStream_t st, const float* residual);
int gemm_i8_decode(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch, int M, int N, int K,
                   int ksplit, int32_t* acc, float* y, cudaStream_t st, const float* residual, int32_t* work, int* counters);
int gemm_sm_count();

// Library-owned split-K scratch, one per device: int32 partial sums followed by the arrival counters.
// It is allocated ONCE per device, at its full size (64 tokens x 131072 output channels), on the
// first decode linear layer that needs it, and never freed, grown or moved afterwards: CUDA graphs
// that captured a launch hold it by address. That first call must therefore come outside any stream
// capture (an allocation is illegal inside one); a capturing call that finds no scratch yet is
// refused. Invariant: all zero between launches (the kernel's last arriver restores it), so launches
// on ONE stream share it without a memset. Launches that can overlap on the GPU (different streams)
// would mix their partial sums: the caller serialises them (stated at the entry point's declaration).
struct Scratch { std::mutex mu; void* p = nullptr; };
static Scratch g_scratch[kMaxDevices];
constexpr size_t kCounterBytes = 16384;                                  // 4 counters per 128-channel tile, up to 131072 channels
constexpr size_t kScratchBytes = (size_t)64 * 131072 * sizeof(int32_t);  // largest M x N the decode path accepts

int scratch_get(size_t bytes, int32_t** work, int** counters, cudaStream_t st) {
    const int dev = current_device();
    if (dev < 0) return FLEXLLM_ECUDA;
    if (bytes > kScratchBytes) return FLEXLLM_ENOTSUP;
    Scratch& s = g_scratch[dev];
    std::lock_guard<std::mutex> lk(s.mu);
    if (!s.p) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        FLEXLLM_CHECK_CUDA(cudaStreamIsCapturing(st, &cap));
        if (cap != cudaStreamCaptureStatusNone) return FLEXLLM_EINVAL;   // make the first call outside the capture
        void* p = nullptr;
        cudaError_t e = cudaMalloc(&p, kScratchBytes + kCounterBytes);
        if (e != cudaSuccess) { g_last_cuda_error = (int)e; return e == cudaErrorMemoryAllocation ? FLEXLLM_ENOMEM : FLEXLLM_ECUDA; }
        e = cudaMemset(p, 0, kScratchBytes + kCounterBytes);
        if (e != cudaSuccess) { cudaFree(p); return cuda_status(e); }
        s.p = p;
    }
    *work = (int32_t*)s.p;
    *counters = (int*)((char*)s.p + kScratchBytes);
    return FLEXLLM_OK;
}


int decode_ksplit(int N, int K) {
    const int tiles = (N + 127) / 128;
    const int num_kb = (K + 127) / 128;
    int ks = gemm_sm_count() / tiles;
    if (ks > num_kb / 2) ks = num_kb / 2;
    if (ks < 1) ks = 1;
    return ks;
}
}  // namespace flexllm

using namespace flexllm;

static int check_linear(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch, int M, int N, int K,
                        int32_t* acc, float* y) {
    FLEXLLM_REQUIRE(a && w && (acc || y) && M >= 0 && N > 0 && K > 0);
    FLEXLLM_REQUIRE(!y || (s_tok && s_ch));
    FLEXLLM_REQUIRE((K % 16) == 0 && (N % 8) == 0);
    FLEXLLM_REQUIRE(aligned(a, 16) && aligned(w, 16) && (!acc || aligned(acc, 16)) && (!y || aligned(y, 16)) &&
                    (!s_ch || aligned(s_ch, 16)));
    return FLEXLLM_OK;
}

static int linear_prefill(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch, int M, int N, int K,
                          int32_t* acc, float* y, const float* residual, void* stream) {
    int rc = check_linear(a, s_tok, w, s_ch, M, N, K, acc, y);
    if (rc != FLEXLLM_OK) return rc;
    FLEXLLM_REQUIRE(!residual || (y && aligned(residual, 16)));
    if (M == 0) return FLEXLLM_OK;
    return gemm_i8_prefill(a, s_tok, w, s_ch, M, N, K, acc, y, (cudaStream_t)stream, residual);
}

static int linear_decode(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch, int M, int N, int K,
                         int32_t* acc, float* y, const float* residual, void* stream) {
    int rc = check_linear(a, s_tok, w, s_ch, M, N, K, acc, y);
    if (rc != FLEXLLM_OK) return rc;
    FLEXLLM_REQUIRE(!residual || y);
    if (M == 0) return FLEXLLM_OK;
    if (M > 64) return FLEXLLM_ENOTSUP;
    cudaStream_t st = (cudaStream_t)stream;
    if (M <= 8) return gemv_i8(a, s_tok, w, s_ch, M, N, K, acc, y, residual, st);
    const int ks = decode_ksplit(N, K);
    if (ks == 1) return gemm_i8_decode(a, s_tok, w, s_ch, M, N, K, 1, acc, y, st, residual, nullptr, nullptr);
    if ((size_t)((N + 127) / 128) * 16 > kCounterBytes) return FLEXLLM_ENOTSUP;
    int32_t* work = nullptr; int* counters = nullptr;
    rc = scratch_get((size_t)M * N * sizeof(int32_t), &work, &counters, st);
    if (rc != FLEXLLM_OK) return rc;
    return gemm_i8_decode(a, s_tok, w, s_ch, M, N, K, ks, acc, y, st, residual, work, counters);
}

extern "C" int flexllm_linear_prefill_i8(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch,
                                         int M, int N, int K, int32_t* acc, float* y, void* stream) {
    return linear_prefill(a, s_tok, w, s_ch, M, N, K, acc, y, nullptr, stream);
}
extern "C" int flexllm_linear_prefill_i8_residual(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch,
                                                  int M, int N, int K, const float* residual, float* y, void* stream) {
    FLEXLLM_REQUIRE(residual);
    return linear_prefill(a, s_tok, w, s_ch, M, N, K, nullptr, y, residual, stream);
}
extern "C" int flexllm_linear_decode_i8(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch,
                                        int M, int N, int K, int32_t* acc, float* y, void* stream) {
    return linear_decode(a, s_tok, w, s_ch, M, N, K, acc, y, nullptr, stream);
}
extern "C" int flexllm_linear_decode_i8_residual(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch,
                                                 int M, int N, int K, const float* residual, float* y, void* stream) {
    FLEXLLM_REQUIRE(residual);
    return linear_decode(a, s_tok, w, s_ch, M, N, K, nullptr, y, residual, stream);
}

// ---- decode MLP block as one call -----------------------------------------------------------------------------------
namespace flexllm {
int swiglu_fht_quant_strided(const float* g, const float* u, long ld, int M, float scale, int8_t* q, float* s, cudaStream_t st);
static size_t up256(size_t n) { return (n + 255) & ~(size_t)255; }
}  // namespace flexllm
extern "C" int flexllm_rmsnorm_quant(const float* x, const float* gamma, int M, int D, float eps, int order, float* y, int8_t* q,
                                     float* s, void* stream);

extern "C" size_t flexllm_mlp_block_workspace(int M, int D, int F) {
    if (M <= 0 || D <= 0 || F <= 0) return 0;
    return up256((size_t)M * D) + 2 * up256((size_t)M * 4) + up256((size_t)M * 2 * F * 4) + up256((size_t)M * F) + 256;
}

// RMSNorm + quant -> fused gate|up projection -> SiLU(gate) * up, FHT-8192, quant -> down projection + residual: the four
// launches follow one another with programmatic dependent launch, so each kernel's launch and (for the weight-streaming
// GEMV) first weight loads overlap the tail of the one before.
extern "C" int flexllm_mlp_block_decode(const float* x, const float* gamma, const int8_t* w_gu, const float* s_gu, const int8_t* w_d,
                                        const float* s_d, int M, int D, int F, float eps, int order, float fht_scale, float* y,
                                        void* workspace, size_t workspace_bytes, void* stream) {
    FLEXLLM_REQUIRE(x && gamma && w_gu && s_gu && w_d && s_d && y && M >= 0 && D > 0);
    if (F != 8192) return FLEXLLM_ENOTSUP;
    if (M == 0) return FLEXLLM_OK;
    if (M > 64) return FLEXLLM_ENOTSUP;
    FLEXLLM_REQUIRE(workspace && workspace_bytes >= flexllm_mlp_block_workspace(M, D, F));
    uint8_t* w = (uint8_t*)(((uintptr_t)workspace + 255) & ~(uintptr_t)255);
    int8_t* xq = (int8_t*)w; w += up256((size_t)M * D);
    float* xs = (float*)w; w += up256((size_t)M * 4);
    float* hs = (float*)w; w += up256((size_t)M * 4);
    float* gu = (float*)w; w += up256((size_t)M * 2 * F * 4);
    int8_t* hq = (int8_t*)w;
    cudaStream_t st = (cudaStream_t)stream;
    struct PdlScope { int before; PdlScope() : before(g_pdl) { g_pdl = 1; } ~PdlScope() { g_pdl = before; } } pdl;
    TRY_RC(flexllm_rmsnorm_quant(x, gamma, M, D, eps, order, nullptr, xq, xs, st));
    TRY_RC(linear_decode(xq, xs, w_gu, s_gu, M, 2 * F, D, nullptr, gu, nullptr, st));
    TRY_RC(swiglu_fht_quant_strided(gu, gu + F, 2L * F, M, fht_scale, hq, hs, st));
    return linear_decode(hq, hs, w_d, s_d, M, D, F, nullptr, y, x, st);
}
