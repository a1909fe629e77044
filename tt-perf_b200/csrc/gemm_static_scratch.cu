// b200_gemm_static_scratch: the split-K matmul for callers that must not allocate device memory.
//
// Who needs it. b200_gemm's split-K path keeps its fp32 partial sums in context scratch that it grows
// with cudaMalloc on demand. Some hosts cannot tolerate that: an executor that has handed all of HBM to
// its own arena (a foreign cudaMalloc then fails or fragments the arena), a serving loop with a latency
// bound (cudaMalloc and cudaFree synchronise the whole device), or a process whose device memory is
// capped below what a growing scratch block would need. This entry point gives them the same kernels with the
// partial sums in a fixed array that is part of the library image, so a call performs no cudaMalloc,
// no cudaFree and no other allocating routine — it only encodes two tensor maps on the host and
// launches the GEMM and the reduce kernel.
//
// Cost and limits. The array is B200_STATIC_SCRATCH_BYTES (32 MiB) of global memory on every GPU that
// loads the library, held until the process exits. A product whose partial sums
// (k_slices x batch x M x N x 4 bytes) do not fit is refused with B200_ERR_INVALID_ARG. All calls on a
// device share the one array: nothing in it has to start at zero (every element the reduce kernel reads
// is written by the GEMM kernel of the same call first), but two calls whose kernels overlap on the GPU
// — different streams, or different host threads — race on it. Issue them on one stream.
//
// Set-up. The first call on each device looks up the device addresses of the array and of the status
// word (cudaGetSymbolAddress, with that device current). The first call that uses a given kernel variant
// (tile width x operand layouts) on a device also raises that kernel's shared-memory limit
// (cudaFuncSetAttribute). Make one call of every shape class you will use before a stream capture begins.
//
// Errors. A bounded wait that runs out inside these kernels sets a status word next to the array;
// b200_static_scratch_status reads and clears it (b200_synchronize knows nothing about it).
#include <mutex>

#include "gemm_common.cuh"

#define B200_STATIC_SCRATCH_BYTES (size_t(32) << 20)

namespace b200 {
namespace {

// In host code these names are host-side stand-ins, not device addresses: kernels must be given the
// pointers cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) float g_static_scratch[B200_STATIC_SCRATCH_BYTES / sizeof(float)];
static __device__ __align__(256) int g_static_status[64];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
b200_ctx* g_static_ctx[kMaxDevices] = {};  // host-side parameter holders, one per device, never freed

// Looks up (once per device, with that device current) where the static arrays live on `device`.
int static_ctx_for(int device, b200_ctx** out) {
    B200_REQUIRE(device >= 0 && device < kMaxDevices, "b200_gemm_static_scratch: device %d out of range", device);
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (g_static_ctx[device] == nullptr) {
        DeviceScope scope(device);
        cudaDeviceProp prop;
        B200_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
        if (prop.major != 10)
            return fail(B200_ERR_UNSUPPORTED, "b200_gemm_static_scratch: device %d is sm_%d%d, kernels are sm_100a only",
                        device, prop.major, prop.minor);
        void* scratch_ptr = nullptr;
        void* status_ptr = nullptr;
        B200_CUDA_TRY(cudaGetSymbolAddress(&scratch_ptr, g_static_scratch));
        B200_CUDA_TRY(cudaGetSymbolAddress(&status_ptr, g_static_status));
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) {
            cudaGetLastError();
            return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        }
        b200_ctx* c = new b200_ctx();
        c->device = device;
        c->sm_count = prop.multiProcessorCount;
        c->cc_major = prop.major;
        c->cc_minor = prop.minor;
        c->stream = nullptr;
        c->order_streams = false;  // the caller keeps overlapping calls apart (documented); no event is created here
        c->d_status = static_cast<int*>(status_ptr);
        c->d_scratch = scratch_ptr;                    // fixed: ensure_scratch() never grows it because every
        c->scratch_bytes = B200_STATIC_SCRATCH_BYTES;  // request is checked against this size first
        c->encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
        g_static_ctx[device] = c;
    }
    *out = g_static_ctx[device];
    return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_gemm_static_scratch(int device, const b200_gemm_desc* d, void* stream_v) {
    int rc = gemm_validate_desc(d);  // the same descriptor checks as b200_gemm
    if (rc != B200_OK) return rc;
    B200_REQUIRE(stream_v != nullptr, "b200_gemm_static_scratch: pass the stream to run on (there is no context stream)");
    B200_REQUIRE(d->M > 0 && d->N > 0 && d->K > 0, "b200_gemm_static_scratch: M, N and K must be positive");
    B200_REQUIRE(d->algo != B200_GEMM_SIMT, "b200_gemm_static_scratch: there is no SIMT path here");
    const char* why = nullptr;
    if (!gemm_tcgen05_eligible(*d, &why))
        return fail(B200_ERR_INVALID_ARG, "b200_gemm_static_scratch: %s (this entry point has no SIMT path)", why);

    b200_ctx* sctx = nullptr;
    rc = static_ctx_for(device, &sctx);
    if (rc != B200_OK) return rc;

    // Same slice count b200_gemm would pick; when the caller left the choice open, lower it until the
    // partial sums fit the fixed array.
    int splits = gemm_choose_split_k(sctx, *d);
    const size_t per_slice = static_cast<size_t>(d->batch) * d->M * d->N * sizeof(float);
    if (d->split_k == 0) {
        while (splits > 1 && per_slice * splits > B200_STATIC_SCRATCH_BYTES) {
            b200_gemm_desc t = *d;
            t.split_k = splits - 1;
            splits = gemm_choose_split_k(sctx, t);
        }
    }
    if (splits > 1 && per_slice * splits > B200_STATIC_SCRATCH_BYTES)
        return fail(B200_ERR_INVALID_ARG,
                    "b200_gemm_static_scratch: %d K slices of batch %lld x %lld x %lld fp32 partial sums need %zu bytes, "
                    "the static scratch holds %zu; lower split_k or use b200_gemm",
                    splits, (long long)d->batch, (long long)d->M, (long long)d->N, per_slice * splits,
                    (size_t)B200_STATIC_SCRATCH_BYTES);
    DeviceScope scope(device);
    return launch_gemm_tcgen05(sctx, *d, splits, static_cast<cudaStream_t>(stream_v));
}

// Reads and clears the status word of the static-scratch kernels on `device`: *out_status is non-zero when one of
// their bounded waits ran out since the last call (the output of that launch is then invalid). Waits for the work
// queued on `stream` first, so it is the counterpart of b200_synchronize for this entry point. Allocates nothing.
extern "C" int b200_static_scratch_status(int device, void* stream_v, int* out_status) {
    B200_REQUIRE(out_status != nullptr, "b200_static_scratch_status: out_status is NULL");
    B200_REQUIRE(stream_v != nullptr, "b200_static_scratch_status: pass the stream the products ran on");
    *out_status = 0;
    b200_ctx* sctx = nullptr;
    int rc = static_ctx_for(device, &sctx);
    if (rc != B200_OK) return rc;
    DeviceScope scope(device);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    B200_CUDA_TRY(cudaStreamSynchronize(stream));
    int status = 0;
    B200_CUDA_TRY(cudaMemcpyAsync(&status, sctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    B200_CUDA_TRY(cudaStreamSynchronize(stream));
    if (status != 0) {
        B200_CUDA_TRY(cudaMemsetAsync(sctx->d_status, 0, sizeof(g_static_status), stream));
        B200_CUDA_TRY(cudaStreamSynchronize(stream));
        *out_status = status;
        return fail(B200_ERR_DEVICE_TIMEOUT, "a static-scratch kernel gave up a bounded wait (status word %d); its output is invalid",
                    status);
    }
    return B200_OK;
}
