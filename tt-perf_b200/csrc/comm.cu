// Rank-to-rank plumbing of the sharded matmul behind the C ABI: a thin layer over NCCL so that a C++ host (one process
// per GPU) can run the fused GEMM + all-gather / reduce-scatter kernels without any other communication library:
//   * a stream-ordered rank barrier (peer stores of the fused kernels are complete for a peer only after it),
//   * an exchange of small host blobs between the ranks (the CUDA IPC handles of the peer buffers),
//   * all-reduce / all-gather of device buffers for what is not fused (data-parallel gradient averaging).
// The matrix data of the sharded matmul never goes through here: it travels in the GEMM epilogue's peer stores.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, the copy a host framework has already loaded if there is one), so
// the library loads and every single-GPU entry point works on a machine without NCCL; only b200_comm_* then fail with
// B200_ERR_COMM. The reference's counterpart is the fabric set-up and `ttnn::all_gather` of its mesh programs
// (bench/metal/matmul_tensor_parallel.cpp:155-166, 91-93).
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <vector>

#include "common.cuh"

struct b200_comm {
    b200_ctx* ctx = nullptr;
    ncclComm_t nccl = nullptr;
    int n_ranks = 1, rank = 0;
    float* d_flag = nullptr;     // operand of the barrier's one-element all-reduce
    void* d_stage = nullptr;     // staging of b200_comm_exchange_host
    size_t stage_bytes = 0;
};

namespace b200 {

b200_ctx* comm_ctx(b200_comm* comm) { return comm->ctx; }

namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    const char* (*GetLastError)(ncclComm_t) = nullptr;
    bool ok = false;
};

std::mutex g_nccl_mu;
NcclApi g_nccl;

int nccl_api(const NcclApi** out) {
    std::lock_guard<std::mutex> lock(g_nccl_mu);
    if (!g_nccl.ok) {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return fail(B200_ERR_COMM, "NCCL is not available: %s", dlerror());
        NcclApi api;
        api.handle = h;
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(h, "ncclAllReduce"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(h, "ncclAllGather"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
        api.GetLastError = reinterpret_cast<decltype(api.GetLastError)>(dlsym(h, "ncclGetLastError"));
        if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllReduce || !api.AllGather || !api.GetErrorString)
            return fail(B200_ERR_COMM, "libnccl.so.2 lacks an expected symbol");
        api.ok = true;
        g_nccl = api;
    }
    *out = &g_nccl;
    return B200_OK;
}

#define B200_NCCL_TRY(api, expr)                                                                      \
    do {                                                                                              \
        ncclResult_t _r = (expr);                                                                     \
        if (_r != ncclSuccess)                                                                        \
            return ::b200::fail(B200_ERR_COMM, "%s failed: %s (%s:%d)", #expr, (api)->GetErrorString(_r), \
                                __FILE__, __LINE__);                                                  \
    } while (0)

bool to_nccl_type(int dtype, ncclDataType_t* out) {
    switch (dtype) {
        case B200_BF16: *out = ncclBfloat16; return true;
        case B200_F32: *out = ncclFloat32; return true;
        case B200_U32: *out = ncclUint32; return true;
        default: return false;
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_comm_unique_id(void* out_id128) {
    B200_REQUIRE(out_id128 != nullptr, "b200_comm_unique_id: NULL buffer");
    static_assert(sizeof(ncclUniqueId) == 128, "NCCL unique id size");
    const NcclApi* api = nullptr;
    int rc = nccl_api(&api);
    if (rc != B200_OK) return rc;
    ncclUniqueId id;
    B200_NCCL_TRY(api, api->GetUniqueId(&id));
    memcpy(out_id128, &id, sizeof(id));
    return B200_OK;
}

int b200_comm_create(b200_ctx* ctx, const void* id128, int n_ranks, int rank, b200_comm** out_comm) {
    B200_REQUIRE(ctx && id128 && out_comm, "b200_comm_create: NULL argument");
    B200_REQUIRE(n_ranks >= 1 && rank >= 0 && rank < n_ranks, "b200_comm_create: rank %d of %d", rank, n_ranks);
    *out_comm = nullptr;
    const NcclApi* api = nullptr;
    int rc = nccl_api(&api);
    if (rc != B200_OK) return rc;
    DeviceScope scope(ctx->device);
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    b200_comm* c = new b200_comm();
    c->ctx = ctx;
    c->n_ranks = n_ranks;
    c->rank = rank;
    ncclResult_t r = api->CommInitRank(&c->nccl, n_ranks, id, rank);
    if (r != ncclSuccess) {
        delete c;
        return fail(B200_ERR_COMM, "ncclCommInitRank(rank %d of %d) failed: %s", rank, n_ranks, api->GetErrorString(r));
    }
    cudaError_t e = cudaMalloc(&c->d_flag, 256);
    if (e == cudaSuccess) e = cudaMemset(c->d_flag, 0, 256);
    if (e != cudaSuccess) {
        api->CommDestroy(c->nccl);
        delete c;
        return fail(B200_ERR_CUDA, "b200_comm_create: %s", cudaGetErrorString(e));
    }
    *out_comm = c;
    return B200_OK;
}

int b200_comm_destroy(b200_comm* comm) {
    if (!comm) return B200_OK;
    const NcclApi* api = nullptr;
    int rc = nccl_api(&api);
    DeviceScope scope(comm->ctx->device);
    cudaDeviceSynchronize();
    if (rc == B200_OK && comm->nccl) api->CommDestroy(comm->nccl);
    if (comm->d_flag) cudaFree(comm->d_flag);
    if (comm->d_stage) cudaFree(comm->d_stage);
    delete comm;
    return B200_OK;
}

int b200_comm_size(const b200_comm* comm, int* out_n_ranks, int* out_rank) {
    B200_REQUIRE(comm != nullptr, "b200_comm_size: comm is NULL");
    if (out_n_ranks) *out_n_ranks = comm->n_ranks;
    if (out_rank) *out_rank = comm->rank;
    return B200_OK;
}

int b200_comm_barrier(b200_comm* comm, void* stream) {
    B200_REQUIRE(comm != nullptr, "b200_comm_barrier: comm is NULL");
    const NcclApi* api = nullptr;
    int rc = nccl_api(&api);
    if (rc != B200_OK) return rc;
    DeviceScope scope(comm->ctx->device);
    B200_NCCL_TRY(api, api->AllReduce(comm->d_flag, comm->d_flag, 1, ncclFloat32, ncclSum, comm->nccl, comm->ctx->pick(stream)));
    return B200_OK;
}

int b200_comm_allreduce(b200_comm* comm, void* d_buf, int64_t count, int dtype, int op, void* stream) {
    B200_REQUIRE(comm != nullptr, "b200_comm_allreduce: comm is NULL");
    B200_REQUIRE(count >= 0, "b200_comm_allreduce: negative count");
    if (count == 0) return B200_OK;
    B200_REQUIRE(d_buf != nullptr, "b200_comm_allreduce: NULL buffer");
    ncclDataType_t t;
    B200_REQUIRE(to_nccl_type(dtype, &t), "b200_comm_allreduce: dtype must be BF16, F32 or U32");
    ncclRedOp_t o;
    switch (op) {
        case B200_COMM_SUM: o = ncclSum; break;
        case B200_COMM_AVG: o = ncclAvg; break;
        case B200_COMM_MAX: o = ncclMax; break;
        default: return fail(B200_ERR_INVALID_ARG, "b200_comm_allreduce: unknown op %d", op);
    }
    const NcclApi* api = nullptr;
    int rc = nccl_api(&api);
    if (rc != B200_OK) return rc;
    DeviceScope scope(comm->ctx->device);
    B200_NCCL_TRY(api, api->AllReduce(d_buf, d_buf, static_cast<size_t>(count), t, o, comm->nccl, comm->ctx->pick(stream)));
    return B200_OK;
}

int b200_comm_allgather(b200_comm* comm, const void* d_send, void* d_recv, size_t bytes_per_rank, void* stream) {
    B200_REQUIRE(comm != nullptr, "b200_comm_allgather: comm is NULL");
    if (bytes_per_rank == 0) return B200_OK;
    B200_REQUIRE(d_send && d_recv, "b200_comm_allgather: NULL buffer");
    const NcclApi* api = nullptr;
    int rc = nccl_api(&api);
    if (rc != B200_OK) return rc;
    DeviceScope scope(comm->ctx->device);
    B200_NCCL_TRY(api, api->AllGather(d_send, d_recv, bytes_per_rank, ncclUint8, comm->nccl, comm->ctx->pick(stream)));
    return B200_OK;
}

int b200_comm_exchange_host(b200_comm* comm, const void* h_send, void* h_recv, size_t bytes_per_rank) {
    B200_REQUIRE(comm != nullptr, "b200_comm_exchange_host: comm is NULL");
    if (bytes_per_rank == 0) return B200_OK;
    B200_REQUIRE(h_send && h_recv, "b200_comm_exchange_host: NULL buffer");
    B200_REQUIRE(bytes_per_rank <= (size_t(1) << 20), "b200_comm_exchange_host: meant for small blobs (<= 1 MiB per rank)");
    const NcclApi* api = nullptr;
    int rc = nccl_api(&api);
    if (rc != B200_OK) return rc;
    DeviceScope scope(comm->ctx->device);
    const size_t need = bytes_per_rank * (static_cast<size_t>(comm->n_ranks) + 1);
    if (need > comm->stage_bytes) {
        if (comm->d_stage) B200_CUDA_TRY(cudaFree(comm->d_stage));
        comm->d_stage = nullptr;
        comm->stage_bytes = 0;
        B200_CUDA_TRY(cudaMalloc(&comm->d_stage, need));
        comm->stage_bytes = need;
    }
    cudaStream_t st = comm->ctx->stream;
    char* d_send = static_cast<char*>(comm->d_stage);
    char* d_recv = d_send + bytes_per_rank;
    B200_CUDA_TRY(cudaMemcpyAsync(d_send, h_send, bytes_per_rank, cudaMemcpyHostToDevice, st));
    B200_NCCL_TRY(api, api->AllGather(d_send, d_recv, bytes_per_rank, ncclUint8, comm->nccl, st));
    B200_CUDA_TRY(cudaMemcpyAsync(h_recv, d_recv, bytes_per_rank * comm->n_ranks, cudaMemcpyDeviceToHost, st));
    B200_CUDA_TRY(cudaStreamSynchronize(st));
    return B200_OK;
}

}  // extern "C"
