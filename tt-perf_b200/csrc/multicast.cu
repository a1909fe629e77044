// NVLink multicast buffers for the fused all-gather: one allocation per rank, all bound to one NVSwitch multicast
// object, mapped twice on every rank — at a unicast address (the rank's own memory) and at a multicast address, where a
// single `multimem.st` of the GEMM epilogue lands in every rank's copy. The switch replicates the store, so a rank
// sends each output tile over its links once instead of once per peer (the reference's all-gather moves the shard to
// every device in turn: ttnn::all_gather, bench/metal/matmul_tensor_parallel.cpp:91-93).
//
// One process per GPU: rank 0 creates the multicast object and hands its POSIX file descriptor to the other ranks over
// a Unix-domain socket (SCM_RIGHTS), whose name travels through the ranks' communicator. Everything here is collective
// over the communicator and blocks the host; it belongs to set-up, not to the step.
//
// Lifetime rule: a rank must unbind (b200_mc_free) before it exits while its peers still use the object. b200_mc_free is
// collective for that reason: it synchronises the device, meets the other ranks at a barrier, and only then unbinds.
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "ptx.cuh"

struct b200_mc {
    b200_comm* comm = nullptr;
    b200_ctx* ctx = nullptr;
    size_t bytes = 0;            // rounded up to the multicast granularity
    CUmemGenericAllocationHandle mc_handle = 0;
    CUmemGenericAllocationHandle mem_handle = 0;
    CUdeviceptr uc_ptr = 0, mc_ptr = 0;
    bool bound = false, uc_mapped = false, mc_mapped = false;
};

namespace b200 {
namespace {

struct DriverApi {
    CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
    CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
    CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t,
                                 unsigned long long) = nullptr;
    CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
    CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
    CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
    CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
                                           unsigned long long) = nullptr;
    CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
    CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
    CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
    CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
    bool ok = false;
};

std::mutex g_drv_mu;
DriverApi g_drv;

template <typename Fn>
bool load_entry(const char* name, Fn* out) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr) {
        cudaGetLastError();
        return false;
    }
    *out = reinterpret_cast<Fn>(fn);
    return true;
}

int driver_api(const DriverApi** out) {
    std::lock_guard<std::mutex> lock(g_drv_mu);
    if (!g_drv.ok) {
        DriverApi d;
        bool all = load_entry("cuMulticastCreate", &d.MulticastCreate) && load_entry("cuMulticastAddDevice", &d.MulticastAddDevice) &&
                   load_entry("cuMulticastBindMem", &d.MulticastBindMem) && load_entry("cuMulticastUnbind", &d.MulticastUnbind) &&
                   load_entry("cuMulticastGetGranularity", &d.MulticastGetGranularity) && load_entry("cuMemCreate", &d.MemCreate) &&
                   load_entry("cuMemRelease", &d.MemRelease) && load_entry("cuMemAddressReserve", &d.MemAddressReserve) &&
                   load_entry("cuMemAddressFree", &d.MemAddressFree) && load_entry("cuMemMap", &d.MemMap) &&
                   load_entry("cuMemUnmap", &d.MemUnmap) && load_entry("cuMemSetAccess", &d.MemSetAccess) &&
                   load_entry("cuMemExportToShareableHandle", &d.MemExportToShareableHandle) &&
                   load_entry("cuMemImportFromShareableHandle", &d.MemImportFromShareableHandle) &&
                   load_entry("cuDeviceGet", &d.DeviceGet) && load_entry("cuDeviceGetAttribute", &d.DeviceGetAttribute) &&
                   load_entry("cuGetErrorString", &d.GetErrorString);
        if (!all) return fail(B200_ERR_UNSUPPORTED, "this driver lacks the multicast / virtual-memory entry points");
        d.ok = true;
        g_drv = d;
    }
    *out = &g_drv;
    return B200_OK;
}

#define B200_CU_TRY(api, expr)                                                                       \
    do {                                                                                             \
        CUresult _r = (expr);                                                                        \
        if (_r != CUDA_SUCCESS) {                                                                    \
            const char* _s = nullptr;                                                                \
            (api)->GetErrorString(_r, &_s);                                                          \
            return ::b200::fail(B200_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, _s ? _s : "?", __FILE__, __LINE__); \
        }                                                                                            \
    } while (0)

// Rank 0 -> every other rank: one open file descriptor, over an abstract Unix-domain socket.
int send_fd_to_peers(const char* name, size_t name_len, int fd, int peers) {
    int srv = socket(AF_UNIX, SOCK_STREAM, 0);
    if (srv < 0) return fail(B200_ERR_COMM, "socket() failed");
    sockaddr_un addr{};
    addr.sun_family = AF_UNIX;
    memcpy(addr.sun_path, name, name_len);   // leading NUL: abstract namespace, nothing to unlink
    const socklen_t alen = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + name_len);
    if (bind(srv, reinterpret_cast<sockaddr*>(&addr), alen) != 0 || listen(srv, peers) != 0) {
        close(srv);
        return fail(B200_ERR_COMM, "bind/listen on the descriptor socket failed");
    }
    timeval tv{60, 0};
    setsockopt(srv, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    int rc = B200_OK;
    for (int i = 0; i < peers && rc == B200_OK; ++i) {
        int c = accept(srv, nullptr, nullptr);
        if (c < 0) {
            rc = fail(B200_ERR_COMM, "a rank did not come for the multicast descriptor within 60 s");
            break;
        }
        char byte = 1;
        iovec iov{&byte, 1};
        alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {};
        msghdr msg{};
        msg.msg_iov = &iov;
        msg.msg_iovlen = 1;
        msg.msg_control = ctrl;
        msg.msg_controllen = sizeof(ctrl);
        cmsghdr* cm = CMSG_FIRSTHDR(&msg);
        cm->cmsg_level = SOL_SOCKET;
        cm->cmsg_type = SCM_RIGHTS;
        cm->cmsg_len = CMSG_LEN(sizeof(int));
        memcpy(CMSG_DATA(cm), &fd, sizeof(int));
        if (sendmsg(c, &msg, 0) != 1) rc = fail(B200_ERR_COMM, "sendmsg(SCM_RIGHTS) failed");
        close(c);
    }
    close(srv);
    return rc;
}

int recv_fd_from_rank0(const char* name, size_t name_len, int* out_fd) {
    sockaddr_un addr{};
    addr.sun_family = AF_UNIX;
    memcpy(addr.sun_path, name, name_len);
    const socklen_t alen = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + name_len);
    int c = -1;
    for (int attempt = 0; attempt < 600; ++attempt) {   // rank 0 may not be listening yet: up to 60 s
        c = socket(AF_UNIX, SOCK_STREAM, 0);
        if (c < 0) return fail(B200_ERR_COMM, "socket() failed");
        if (connect(c, reinterpret_cast<sockaddr*>(&addr), alen) == 0) break;
        close(c);
        c = -1;
        usleep(100000);
    }
    if (c < 0) return fail(B200_ERR_COMM, "could not reach rank 0's descriptor socket");
    char byte = 0;
    iovec iov{&byte, 1};
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {};
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    timeval tv{60, 0};
    setsockopt(c, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    const ssize_t n = recvmsg(c, &msg, 0);
    close(c);
    cmsghdr* cm = CMSG_FIRSTHDR(&msg);
    if (n != 1 || cm == nullptr || cm->cmsg_type != SCM_RIGHTS) return fail(B200_ERR_COMM, "no descriptor received from rank 0");
    memcpy(out_fd, CMSG_DATA(cm), sizeof(int));
    return B200_OK;
}

// Releases whatever of `m` exists, in reverse order of creation. No collective calls in here.
void mc_release_local(const DriverApi* api, b200_mc* m) {
    CUdevice dev = 0;
    api->DeviceGet(&dev, m->ctx->device);
    if (m->mc_mapped) api->MemUnmap(m->mc_ptr, m->bytes);
    if (m->mc_ptr) api->MemAddressFree(m->mc_ptr, m->bytes);
    if (m->bound) api->MulticastUnbind(m->mc_handle, dev, 0, m->bytes);
    if (m->uc_mapped) api->MemUnmap(m->uc_ptr, m->bytes);
    if (m->uc_ptr) api->MemAddressFree(m->uc_ptr, m->bytes);
    if (m->mem_handle) api->MemRelease(m->mem_handle);
    if (m->mc_handle) api->MemRelease(m->mc_handle);
    m->mc_mapped = m->uc_mapped = m->bound = false;
    m->mc_ptr = m->uc_ptr = 0;
    m->mem_handle = m->mc_handle = 0;
}

}  // namespace
}  // namespace b200

namespace b200 {
b200_ctx* comm_ctx(b200_comm* comm);   // comm.cu

namespace {
// 16 bytes per thread and step from this GPU's memory to a multicast address: every bound GPU receives the block.
__global__ void mc_broadcast_kernel(const uint4* __restrict__ src, uint4* mc_dst, size_t chunks) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < chunks; i += stride)
        ptx::multimem_st_v4(mc_dst + i, src[i]);
}
}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_mc_supported(b200_ctx* ctx, int* out_supported) {
    B200_REQUIRE(ctx && out_supported, "b200_mc_supported: NULL argument");
    *out_supported = 0;
    const DriverApi* api = nullptr;
    if (driver_api(&api) != B200_OK) return B200_OK;   // no entry points: not supported, not an error
    CUdevice dev;
    B200_CU_TRY(api, api->DeviceGet(&dev, ctx->device));
    int v = 0;
    B200_CU_TRY(api, api->DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev));
    *out_supported = v;
    return B200_OK;
}

int b200_mc_alloc(b200_comm* comm, size_t bytes, b200_mc** out_mc, void** out_local_ptr, void** out_multicast_ptr) {
    B200_REQUIRE(comm && out_mc && out_local_ptr && out_multicast_ptr, "b200_mc_alloc: NULL argument");
    B200_REQUIRE(bytes > 0, "b200_mc_alloc: empty buffer");
    *out_mc = nullptr;
    *out_local_ptr = *out_multicast_ptr = nullptr;
    int n_ranks = 1, rank = 0;
    b200_comm_size(comm, &n_ranks, &rank);
    b200_ctx* ctx = comm_ctx(comm);
    const DriverApi* api = nullptr;
    int rc = driver_api(&api);
    if (rc != B200_OK) return rc;
    DeviceScope scope(ctx->device);
    B200_CUDA_TRY(cudaFree(nullptr));   // the primary context exists before driver calls are made
    CUdevice dev;
    B200_CU_TRY(api, api->DeviceGet(&dev, ctx->device));
    int supported = 0;
    B200_CU_TRY(api, api->DeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev));
    // every rank must take the same path: agree on support before anything collective happens
    std::vector<int> all(static_cast<size_t>(n_ranks), 0);
    rc = b200_comm_exchange_host(comm, &supported, all.data(), sizeof(int));
    if (rc != B200_OK) return rc;
    for (int v : all)
        if (!v) return fail(B200_ERR_UNSUPPORTED, "NVLink multicast is not available on every rank's GPU");

    CUmulticastObjectProp mprop{};
    mprop.numDevices = static_cast<unsigned>(n_ranks);
    mprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mprop.flags = 0;
    mprop.size = bytes;
    size_t gran = 0;
    B200_CU_TRY(api, api->MulticastGetGranularity(&gran, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED));
    const size_t size = (bytes + gran - 1) / gran * gran;
    mprop.size = size;

    b200_mc* m = new b200_mc();
    m->comm = comm;
    m->ctx = ctx;
    m->bytes = size;
    auto bail = [&](int code) {
        mc_release_local(api, m);
        delete m;
        return code;
    };
#define B200_MC_STEP(expr)                                                                            \
    do {                                                                                              \
        CUresult _r = (expr);                                                                         \
        if (_r != CUDA_SUCCESS) {                                                                     \
            const char* _s = nullptr;                                                                 \
            api->GetErrorString(_r, &_s);                                                             \
            return bail(fail(B200_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, _s ? _s : "?", __FILE__, __LINE__)); \
        }                                                                                             \
    } while (0)

    // 1. the multicast object: created by rank 0, imported by the others through its file descriptor
    static int counter = 0;
    char name[64] = {};
    size_t name_len = 0;
    if (rank == 0) {
        name_len = 1 + static_cast<size_t>(snprintf(name + 1, sizeof(name) - 1, "b200mc-%d-%d", static_cast<int>(getpid()), counter++));
    }
    std::vector<char> gathered(static_cast<size_t>(n_ranks) * 64);
    rc = b200_comm_exchange_host(comm, name, gathered.data(), 64);
    if (rc != B200_OK) return bail(rc);
    memcpy(name, gathered.data(), 64);   // rank 0's socket name
    name_len = 1 + strlen(name + 1);
    if (rank == 0) {
        B200_MC_STEP(api->MulticastCreate(&m->mc_handle, &mprop));
        int fd = -1;
        B200_MC_STEP(api->MemExportToShareableHandle(&fd, m->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
        rc = send_fd_to_peers(name, name_len, fd, n_ranks - 1);
        close(fd);
        if (rc != B200_OK) return bail(rc);
    } else {
        int fd = -1;
        rc = recv_fd_from_rank0(name, name_len, &fd);
        if (rc != B200_OK) return bail(rc);
        CUresult r = api->MemImportFromShareableHandle(&m->mc_handle, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                                       CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
        close(fd);
        B200_MC_STEP(r);
    }
    // 2. every device joins; binding is only legal once all have joined
    B200_MC_STEP(api->MulticastAddDevice(m->mc_handle, dev));
    int one = 1;
    rc = b200_comm_exchange_host(comm, &one, all.data(), sizeof(int));   // a host-side barrier
    if (rc != B200_OK) return bail(rc);
    // 3. this rank's physical memory, mapped at a unicast address
    CUmemAllocationProp aprop{};
    aprop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    aprop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    aprop.location.id = ctx->device;
    aprop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    B200_MC_STEP(api->MemCreate(&m->mem_handle, size, &aprop, 0));
    B200_MC_STEP(api->MemAddressReserve(&m->uc_ptr, size, gran, 0, 0));
    B200_MC_STEP(api->MemMap(m->uc_ptr, size, 0, m->mem_handle, 0));
    m->uc_mapped = true;
    CUmemAccessDesc access{};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = ctx->device;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    B200_MC_STEP(api->MemSetAccess(m->uc_ptr, size, &access, 1));
    // 4. bind it to the multicast object and map the object at the multicast address
    B200_MC_STEP(api->MulticastBindMem(m->mc_handle, 0, m->mem_handle, 0, size, 0));
    m->bound = true;
    B200_MC_STEP(api->MemAddressReserve(&m->mc_ptr, size, gran, 0, 0));
    B200_MC_STEP(api->MemMap(m->mc_ptr, size, 0, m->mc_handle, 0));
    m->mc_mapped = true;
    B200_MC_STEP(api->MemSetAccess(m->mc_ptr, size, &access, 1));
#undef B200_MC_STEP
    rc = b200_comm_exchange_host(comm, &one, all.data(), sizeof(int));   // everyone is bound before anyone stores
    if (rc != B200_OK) return bail(rc);
    *out_mc = m;
    *out_local_ptr = reinterpret_cast<void*>(m->uc_ptr);
    *out_multicast_ptr = reinterpret_cast<void*>(m->mc_ptr);
    return B200_OK;
}

int b200_mc_broadcast(b200_ctx* ctx, void* mc_dst, const void* d_src, size_t bytes, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_mc_broadcast: ctx is NULL");
    if (bytes == 0) return B200_OK;
    B200_REQUIRE(mc_dst && d_src, "b200_mc_broadcast: NULL buffer");
    B200_REQUIRE(((reinterpret_cast<uintptr_t>(mc_dst) | reinterpret_cast<uintptr_t>(d_src) | bytes) & 15u) == 0,
                 "b200_mc_broadcast: addresses and size must be multiples of 16 bytes");
    DeviceScope scope(ctx->device);
    const size_t chunks = bytes / 16;
    const int blocks = static_cast<int>(std::min<size_t>((chunks + 255) / 256, static_cast<size_t>(ctx->sm_count) * 8));
    mc_broadcast_kernel<<<blocks, 256, 0, ctx->pick(stream)>>>(static_cast<const uint4*>(d_src), static_cast<uint4*>(mc_dst), chunks);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_mc_free(b200_mc* mc) {
    if (!mc) return B200_OK;
    const DriverApi* api = nullptr;
    int rc = driver_api(&api);
    if (rc != B200_OK) return rc;
    DeviceScope scope(mc->ctx->device);
    // Nobody may still be storing through the object when a rank unbinds: drain this device, then meet the others.
    cudaDeviceSynchronize();
    int one = 1, n_ranks = 1;
    b200_comm_size(mc->comm, &n_ranks, nullptr);
    std::vector<int> all(static_cast<size_t>(n_ranks), 0);
    rc = b200_comm_exchange_host(mc->comm, &one, all.data(), sizeof(int));
    mc_release_local(api, mc);
    delete mc;
    return rc;
}

}  // extern "C"
