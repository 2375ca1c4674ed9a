// Tensor-parallel plumbing: one process per GPU, NCCL over NVLink/NVSwitch for the exchanges the
// model partition needs (the reference is a single-FPGA design and has no counterpart):
//   all-reduce (sum, int32)  partial accumulators of the row-parallel o_proj / down_proj --
//                            integer addition is exact and order-free, so every rank ends up
//                            with the bits a single GPU would have computed
//   reduce-scatter (sum, int32)  the same partial sums when a caller keeps only one block of rows per rank (offered;
//                            the model runner's token-row partition needs no sum across ranks)
//   all-reduce (max, fp32)   per-token largest magnitudes, so that each rank can quantise its own column
//                            slice of a row with the scale of the whole row
//   all-gather (bytes)       int8 rows + scales of the token-row blocks, fp32 activations of the
//                            column-parallel stages in the all-gather partition, and the (value, index)
//                            pairs of the vocab-parallel argmax
//   all-to-all (bytes)       column slices of all rows to the rows' owners (int8 attention output, fp32 gated
//                            activations), and the hand-over of the KV cache from the head-sharded prefill to the
//                            sequence-sharded decode
// NCCL is loaded at run time from the library the process already uses (torch's bundled
// libnccl.so.2), so libflexllm_b200.so itself carries no link-time dependency on it.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <condition_variable>
#include <cstring>
#include <mutex>
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

// ---- ranks that share ONE device (flexllm_tp_init_local) ---------------------------------------------------------
// A group of communicators whose ranks are host threads of one process working on one GPU through ONE stream: the
// whole partitioned dataflow (any number of ranks up to 8) can then be run and checked on a single GPU. A collective is
// two host-side rendezvous of the ranks' threads around plain device copies / reductions in that stream: the first
// guarantees that every rank's earlier work is already in the stream, the second that every rank's copies are in it
// before any rank's later work. No kernel waits for another one; nothing here uses NCCL.
constexpr int kMaxLocalRanks = 8;

struct LocalGroup {
    int size = 0, refs = 0;
    std::mutex mu;
    std::condition_variable cv;
    int arrived = 0;
    unsigned long long gen = 0;
    bool failed = false;
    const void* send[kMaxLocalRanks] = {};
    void* recv[kMaxLocalRanks] = {};
    void* tmp = nullptr;            // all-reduce staging, grown on demand
    size_t tmp_bytes = 0;
};

struct LocalPtrs { const void* p[kMaxLocalRanks]; };

template <typename T, bool MAX>
__global__ void local_reduce_kernel(LocalPtrs src, int g, size_t offset, size_t n, T* __restrict__ dst) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        T acc = static_cast<const T*>(src.p[0])[offset + i];
        for (int p = 1; p < g; p++) {
            const T v = static_cast<const T*>(src.p[p])[offset + i];
            acc = MAX ? (v > acc ? v : acc) : acc + v;
        }
        dst[i] = acc;
    }
}

// Rendezvous of the group's threads; false after a time-out or once any rank has reported a failure.
static bool local_rendezvous(LocalGroup* g) {
    std::unique_lock<std::mutex> lk(g->mu);
    if (g->failed) return false;
    const unsigned long long my = g->gen;
    if (++g->arrived == g->size) {
        g->arrived = 0; g->gen++;
        g->cv.notify_all();
        return true;
    }
    const bool ok = g->cv.wait_for(lk, std::chrono::seconds(120), [&] { return g->gen != my || g->failed; });
    if (!ok || g->failed) { g->failed = true; g->cv.notify_all(); return false; }
    return true;
}

static void local_fail(LocalGroup* g) {
    std::lock_guard<std::mutex> lk(g->mu);
    g->failed = true;
    g->cv.notify_all();
}

}  // namespace flexllm

struct flexllm_tp {
    int rank, size;
    ncclComm_t comm;
    flexllm::LocalGroup* local;
};

namespace flexllm {

enum LocalOp { LOCAL_ALLGATHER, LOCAL_ALLTOALL, LOCAL_REDUCE_SCATTER, LOCAL_ALLREDUCE_SUM, LOCAL_ALLREDUCE_MAX };

// One collective of a device-sharing group; `n` is the per-rank byte count (gather, all-to-all), the per-rank element
// count (reduce-scatter) or the total element count (all-reduce).
static int local_collective(flexllm_tp* t, LocalOp op, const void* send, void* recv, size_t n, cudaStream_t st) {
    LocalGroup* g = t->local;
    const int r = t->rank, G = g->size;
    // a captured collective would replay without its rendezvous: refuse (the model runner decodes eagerly on such a group)
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) { local_fail(g); return FLEXLLM_ENOTSUP; }
    {
        std::lock_guard<std::mutex> lk(g->mu);
        g->send[r] = send; g->recv[r] = recv;
        if ((op == LOCAL_ALLREDUCE_SUM || op == LOCAL_ALLREDUCE_MAX) && r == 0 && g->tmp_bytes < n * 4) {
            // rank 0 alone grows the staging buffer, before the first rendezvous (cudaFree waits for the device)
            if (g->tmp) cudaFree(g->tmp);
            g->tmp = nullptr; g->tmp_bytes = 0;
            if (cudaMalloc(&g->tmp, n * 4) == cudaSuccess) g->tmp_bytes = n * 4;
        }
    }
    if (!local_rendezvous(g)) return FLEXLLM_ETIMEDOUT;
    cudaError_t e = cudaSuccess;
    LocalPtrs src;
    for (int p = 0; p < kMaxLocalRanks; p++) src.p[p] = p < G ? g->send[p] : nullptr;
    const int threads = 256;
    auto blocks = [&](size_t cnt) { size_t b = (cnt + threads - 1) / threads; return (unsigned)(b < 1 ? 1 : b > 4096 ? 4096 : b); };
    if (op == LOCAL_ALLGATHER) {
        for (int p = 0; p < G && e == cudaSuccess; p++) {
            char* dst = (char*)recv + (size_t)p * n;
            if (dst != g->send[p]) e = cudaMemcpyAsync(dst, g->send[p], n, cudaMemcpyDeviceToDevice, st);
        }
    } else if (op == LOCAL_ALLTOALL) {
        for (int p = 0; p < G && e == cudaSuccess; p++)
            e = cudaMemcpyAsync((char*)recv + (size_t)p * n, (const char*)g->send[p] + (size_t)r * n, n, cudaMemcpyDeviceToDevice, st);
    } else if (op == LOCAL_REDUCE_SCATTER) {
        local_reduce_kernel<int32_t, false><<<blocks(n), threads, 0, st>>>(src, G, (size_t)r * n, n, (int32_t*)recv);
        e = cudaGetLastError();
    } else {
        // all-reduce in place: every rank reduces one slice of all ranks' buffers into the staging buffer, and after a
        // rendezvous (all slices' reads are in the stream) copies the whole result over its own buffer
        if (!g->tmp || g->tmp_bytes < n * 4) e = cudaErrorMemoryAllocation;
        const size_t per = (n + G - 1) / G, lo = (size_t)r * per < n ? (size_t)r * per : n, cnt = lo + per <= n ? per : n - lo;
        if (e == cudaSuccess && cnt) {
            if (op == LOCAL_ALLREDUCE_SUM)
                local_reduce_kernel<int32_t, false><<<blocks(cnt), threads, 0, st>>>(src, G, lo, cnt, (int32_t*)g->tmp + lo);
            else
                local_reduce_kernel<float, true><<<blocks(cnt), threads, 0, st>>>(src, G, lo, cnt, (float*)g->tmp + lo);
            e = cudaGetLastError();
        }
        if (e != cudaSuccess) local_fail(g);
        if (!local_rendezvous(g)) return e != cudaSuccess ? FLEXLLM_ECUDA : FLEXLLM_ETIMEDOUT;
        e = cudaMemcpyAsync(recv, g->tmp, n * 4, cudaMemcpyDeviceToDevice, st);
    }
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; local_fail(g); }
    if (!local_rendezvous(g)) return e != cudaSuccess ? FLEXLLM_ECUDA : FLEXLLM_ETIMEDOUT;
    return FLEXLLM_OK;
}

}  // namespace flexllm

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
    t->rank = rank; t->size = size; t->comm = nullptr; t->local = nullptr;
    rc = nccl_status(g_nccl.CommInitRank(&t->comm, size, id, rank));
    if (rc != FLEXLLM_OK) { delete t; return rc; }
    *out = t;
    return FLEXLLM_OK;
}

extern "C" int flexllm_tp_init_local(flexllm_tp** out, int size) {
    FLEXLLM_REQUIRE(out && size >= 1 && size <= kMaxLocalRanks);
    LocalGroup* g = new (std::nothrow) LocalGroup();
    if (!g) return FLEXLLM_ENOMEM;
    g->size = size; g->refs = size;
    for (int r = 0; r < size; r++) {
        flexllm_tp* t = new (std::nothrow) flexllm_tp();
        if (!t) { for (int q = 0; q < r; q++) delete out[q]; delete g; return FLEXLLM_ENOMEM; }
        t->rank = r; t->size = size; t->comm = nullptr; t->local = g;
        out[r] = t;
    }
    return FLEXLLM_OK;
}

extern "C" int flexllm_tp_destroy(flexllm_tp* t) {
    if (!t) return FLEXLLM_OK;
    if (t->local) {
        LocalGroup* g = t->local;
        bool last;
        { std::lock_guard<std::mutex> lk(g->mu); last = --g->refs == 0; }
        if (last) { if (g->tmp) cudaFree(g->tmp); delete g; }
        delete t;
        return FLEXLLM_OK;
    }
    if (t->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(t->comm);
    delete t;
    return FLEXLLM_OK;
}

extern "C" int flexllm_tp_is_local(const flexllm_tp* t) { return t && t->local ? 1 : 0; }
extern "C" int flexllm_tp_rank(const flexllm_tp* t) { return t ? t->rank : 0; }
extern "C" int flexllm_tp_size(const flexllm_tp* t) { return t ? t->size : 1; }

extern "C" int flexllm_tp_allreduce_s32(flexllm_tp* t, int32_t* buf, size_t count, void* stream) {
    FLEXLLM_REQUIRE(buf || count == 0);
    if (!t || t->size == 1 || count == 0) return FLEXLLM_OK;
    if (t->local) return local_collective(t, LOCAL_ALLREDUCE_SUM, buf, buf, count, (cudaStream_t)stream);
    return nccl_status(g_nccl.AllReduce(buf, buf, count, ncclInt32, ncclSum, t->comm, (cudaStream_t)stream));
}

extern "C" int flexllm_tp_allgather(flexllm_tp* t, const void* send, void* recv, size_t bytes_per_rank, void* stream) {
    FLEXLLM_REQUIRE((send && recv) || bytes_per_rank == 0);
    if (bytes_per_rank == 0) return FLEXLLM_OK;
    if (!t || t->size == 1) {
        if (send != recv) FLEXLLM_CHECK_CUDA(cudaMemcpyAsync(recv, send, bytes_per_rank, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
        return FLEXLLM_OK;
    }
    if (t->local) return local_collective(t, LOCAL_ALLGATHER, send, recv, bytes_per_rank, (cudaStream_t)stream);
    return nccl_status(g_nccl.AllGather(send, recv, bytes_per_rank, ncclInt8, t->comm, (cudaStream_t)stream));
}

extern "C" int flexllm_tp_reduce_scatter_s32(flexllm_tp* t, const int32_t* send, int32_t* recv, size_t count_per_rank, void* stream) {
    FLEXLLM_REQUIRE((send && recv) || count_per_rank == 0);
    if (count_per_rank == 0) return FLEXLLM_OK;
    if (!t || t->size == 1) {
        if (send != recv) FLEXLLM_CHECK_CUDA(cudaMemcpyAsync(recv, send, count_per_rank * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
        return FLEXLLM_OK;
    }
    if (t->local) return local_collective(t, LOCAL_REDUCE_SCATTER, send, recv, count_per_rank, (cudaStream_t)stream);
    return nccl_status(g_nccl.ReduceScatter(send, recv, count_per_rank, ncclInt32, ncclSum, t->comm, (cudaStream_t)stream));
}

extern "C" int flexllm_tp_allreduce_max_f32(flexllm_tp* t, float* buf, size_t count, void* stream) {
    FLEXLLM_REQUIRE(buf || count == 0);
    if (!t || t->size == 1 || count == 0) return FLEXLLM_OK;
    if (t->local) return local_collective(t, LOCAL_ALLREDUCE_MAX, buf, buf, count, (cudaStream_t)stream);
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
    if (t->local) return local_collective(t, LOCAL_ALLTOALL, send, recv, bytes_per_pair, st);
    int rc = nccl_status(g_nccl.GroupStart());
    if (rc != FLEXLLM_OK) return rc;
    for (int p = 0; p < t->size && rc == FLEXLLM_OK; p++) {
        rc = nccl_status(g_nccl.Send((const char*)send + (size_t)p * bytes_per_pair, bytes_per_pair, ncclInt8, p, t->comm, st));
        if (rc == FLEXLLM_OK) rc = nccl_status(g_nccl.Recv((char*)recv + (size_t)p * bytes_per_pair, bytes_per_pair, ncclInt8, p, t->comm, st));
    }
    const int rc2 = nccl_status(g_nccl.GroupEnd());
    return rc != FLEXLLM_OK ? rc : rc2;
}
