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
