// Tensor-parallel plumbing: one process per GPU, NCCL over NVLink/NVSwitch for the exchanges the
// model partition needs (the reference is a single-FPGA design and has no counterpart):
//   all-reduce (sum, int32)  partial accumulators of the row-parallel o_proj / down_proj --
//                            integer addition is exact and order-free, so every rank ends up
//                            with the bits a single GPU would have computed
//   all-gather (bytes)       fp32 activations of the column-parallel stages (attention output,
//                            silu(gate)*up) before the per-token quantisers that need whole rows,
//                            and the (value, index) pairs of the vocab-parallel argmax
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
    if (!a.GetUniqueId || !a.CommInitRank || !a.CommDestroy || !a.AllReduce || !a.AllGather) return FLEXLLM_ENOTSUP;
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
