// Tensor-parallel plumbing: one process per GPU, NCCL over NVLink/NVSwitch for the exchanges the
// model partition needs (the reference is a single-FPGA design and has no counterpart):
//   all-reduce (sum, int32)  partial accumulators of the row-parallel o_proj / down_proj --
//                            integer addition is exact and order-free, so every rank ends up
//                            with the bits a single GPU would have computed
//   reduce-scatter (sum, int32)  the same partial sums when every rank keeps only its block of token rows
//   all-reduce (max, fp32)   per-token largest magnitudes, so that each rank can quantise its own column
//                            slice of a row with the scale of the whole row
//   all-gather (bytes)       int8 rows + scales of the token-row blocks, fp32 activations of the
//                            column-parallel stages in the all-gather partition, and the (value, index)
//                            pairs of the vocab-parallel argmax
//   all-to-all (bytes)       the exchange between the local and the cross-rank stages of the 8192-point
//                            Hadamard transform, and the hand-over of the KV cache from the head-sharded
//                            prefill to the sequence-sharded decode
// NCCL is loaded at run time from the library the process already uses (torch's bundled
// libnccl.so.2), so libflexllm_b200.so itself carries no link-time dependency on it.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <new>

#include "common.cuh"

namespace flexllm {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};
static NcclApi g_nccl;

static int nccl_load(const char* libpath) {
    if (g_nccl.handle) return FLEXLLM_OK;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h && libpath && *libpath) h = dlopen(libpath, RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return FLEXLLM_ENOTSUP;
    NcclApi a;
    a.handle = h;
    a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(h, "ncclGetUniqueId");
    a.CommInitRank = (decltype(a.CommInitRank))dlsym(h, "ncclCommInitRank");
    a.CommDestroy = (decltype(a.CommDestroy))dlsym(h, "ncclCommDestroy");
    a.AllReduce = (decltype(a.AllReduce))dlsym(h, "ncclAllReduce");
    a.AllGather = (decltype(a.AllGather))dlsym(h, "ncclAllGather");
    a.GetErrorString = (decltype(a.GetErrorString))dlsym(h, "ncclGetErrorString");
    a.ReduceScatter = (decltype(a.ReduceScatter))dlsym(h, "ncclReduceScatter");
    a.Send = (decltype(a.Send))dlsym(h, "ncclSend");
    a.Recv = (decltype(a.Recv))dlsym(h, "ncclRecv");
    a.GroupStart = (decltype(a.GroupStart))dlsym(h, "ncclGroupStart");
    a.GroupEnd = (decltype(a.GroupEnd))dlsym(h, "ncclGroupEnd");
    if (!a.GetUniqueId || !a.CommInitRank || !a.CommDestroy || !a.AllReduce || !a.AllGather || !a.ReduceScatter || !a.Send || !a.Recv ||
        !a.GroupStart || !a.GroupEnd)
        return FLEXLLM_ENOTSUP;
    g_nccl = a;
    return FLEXLLM_OK;
}

static int nccl_status(ncclResult_t r) {
    if (r == ncclSuccess) return FLEXLLM_OK;
    g_last_cuda_error = 100000 + (int)r;   // NCCL codes are reported above the CUDA range
    return FLEXLLM_ECUDA;
}

}  // namespace flexllm

struct flexllm_tp {
    int rank, size;
    ncclComm_t comm;
};

using namespace flexllm;

extern "C" int flexllm_tp_unique_id(unsigned char* id128, const char* nccl_lib_path) {
    FLEXLLM_REQUIRE(id128);
    int rc = nccl_load(nccl_lib_path);
    if (rc != FLEXLLM_OK) return rc;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is expected to be 128 bytes");
    ncclUniqueId id;
    rc = nccl_status(g_nccl.GetUniqueId(&id));
    if (rc != FLEXLLM_OK) return rc;
    std::memcpy(id128, &id, 128);
    return FLEXLLM_OK;
}

extern "C" int flexllm_tp_init(flexllm_tp** out, int rank, int size, const unsigned char* id128, const char* nccl_lib_path) {
    FLEXLLM_REQUIRE(out && id128 && size >= 1 && rank >= 0 && rank < size);
    int rc = nccl_load(nccl_lib_path);
    if (rc != FLEXLLM_OK) return rc;
    ncclUniqueId id;
    std::memcpy(&id, id128, 128);
    flexllm_tp* t = new (std::nothrow) flexllm_tp();
    if (!t) return FLEXLLM_ENOMEM;
    t->rank = rank; t->size = size; t->comm = nullptr;
    rc = nccl_status(g_nccl.CommInitRank(&t->comm, size, id, rank));
    if (rc != FLEXLLM_OK) { delete t; return rc; }
    *out = t;
    return FLEXLLM_OK;
}

extern "C" int flexllm_tp_destroy(flexllm_tp* t) {
    if (!t) return FLEXLLM_OK;
    if (t->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(t->comm);
    delete t;
    return FLEXLLM_OK;
}

extern "C" int flexllm_tp_rank(const flexllm_tp* t) { return t ? t->rank : 0; }
extern "C" int flexllm_tp_size(const flexllm_tp* t) { return t ? t->size : 1; }

extern "C" int flexllm_tp_allreduce_s32(flexllm_tp* t, int32_t* buf, size_t count, void* stream) {
    FLEXLLM_REQUIRE(buf || count == 0);
    if (!t || t->size == 1 || count == 0) return FLEXLLM_OK;
    return nccl_status(g_nccl.AllReduce(buf, buf, count, ncclInt32, ncclSum, t->comm, (cudaStream_t)stream));
}

extern "C" int flexllm_tp_allgather(flexllm_tp* t, const void* send, void* recv, size_t bytes_per_rank, void* stream) {
    FLEXLLM_REQUIRE((send && recv) || bytes_per_rank == 0);
    if (bytes_per_rank == 0) return FLEXLLM_OK;
    if (!t || t->size == 1) {
        if (send != recv) FLEXLLM_CHECK_CUDA(cudaMemcpyAsync(recv, send, bytes_per_rank, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
        return FLEXLLM_OK;
    }
    return nccl_status(g_nccl.AllGather(send, recv, bytes_per_rank, ncclInt8, t->comm, (cudaStream_t)stream));
}

extern "C" int flexllm_tp_reduce_scatter_s32(flexllm_tp* t, const int32_t* send, int32_t* recv, size_t count_per_rank, void* stream) {
    FLEXLLM_REQUIRE((send && recv) || count_per_rank == 0);
    if (count_per_rank == 0) return FLEXLLM_OK;
    if (!t || t->size == 1) {
        if (send != recv) FLEXLLM_CHECK_CUDA(cudaMemcpyAsync(recv, send, count_per_rank * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
        return FLEXLLM_OK;
    }
    return nccl_status(g_nccl.ReduceScatter(send, recv, count_per_rank, ncclInt32, ncclSum, t->comm, (cudaStream_t)stream));
}

extern "C" int flexllm_tp_allreduce_max_f32(flexllm_tp* t, float* buf, size_t count, void* stream) {
    FLEXLLM_REQUIRE(buf || count == 0);
    if (!t || t->size == 1 || count == 0) return FLEXLLM_OK;
    return nccl_status(g_nccl.AllReduce(buf, buf, count, ncclFloat32, ncclMax, t->comm, (cudaStream_t)stream));
}

// Rank r sends bytes [p * bytes_per_pair, (p + 1) * bytes_per_pair) of `send` to rank p and receives rank p's block
// for r at the same offset of `recv`.
extern "C" int flexllm_tp_alltoall(flexllm_tp* t, const void* send, void* recv, size_t bytes_per_pair, void* stream) {
    FLEXLLM_REQUIRE((send && recv) || bytes_per_pair == 0);
    if (bytes_per_pair == 0) return FLEXLLM_OK;
    if (!t || t->size == 1) {
        if (send != recv) FLEXLLM_CHECK_CUDA(cudaMemcpyAsync(recv, send, bytes_per_pair, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
        return FLEXLLM_OK;
    }
    cudaStream_t st = (cudaStream_t)stream;
    int rc = nccl_status(g_nccl.GroupStart());
    if (rc != FLEXLLM_OK) return rc;
    for (int p = 0; p < t->size && rc == FLEXLLM_OK; p++) {
        rc = nccl_status(g_nccl.Send((const char*)send + (size_t)p * bytes_per_pair, bytes_per_pair, ncclInt8, p, t->comm, st));
        if (rc == FLEXLLM_OK) rc = nccl_status(g_nccl.Recv((char*)recv + (size_t)p * bytes_per_pair, bytes_per_pair, ncclInt8, p, t->comm, st));
    }
    const int rc2 = nccl_status(g_nccl.GroupEnd());
    return rc != FLEXLLM_OK ? rc : rc2;
}
