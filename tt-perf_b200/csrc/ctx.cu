// Context, error text and raw device-memory entry points of the C ABI.
#include <stdarg.h>

#include "common.cuh"
#include "ptx.cuh"

namespace b200 {

static thread_local std::string g_last_error;

void set_error(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
}

int fail(int code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

int order_shared_state(b200_ctx* ctx, cudaStream_t stream) {
    if (!ctx->order_streams || pool_is_recording(ctx)) return B200_OK;
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (ctx->shared_used && ctx->shared_last_stream != stream) {
        DeviceScope scope(ctx->device);
        if (ctx->shared_event == nullptr) B200_CUDA_TRY(cudaEventCreateWithFlags(&ctx->shared_event, cudaEventDisableTiming));
        B200_CUDA_TRY(cudaEventRecord(ctx->shared_event, ctx->shared_last_stream));
        B200_CUDA_TRY(cudaStreamWaitEvent(stream, ctx->shared_event, 0));
    }
    ctx->shared_used = true;
    ctx->shared_last_stream = stream;
    return B200_OK;
}

void release_retired_scratch(b200_ctx* ctx) {
    if (ctx->retired_scratch.empty()) return;
    DeviceScope scope(ctx->device);
    cudaDeviceSynchronize();
    for (void* p : ctx->retired_scratch) cudaFree(p);
    ctx->retired_scratch.clear();
}

int ensure_scratch(b200_ctx* ctx, size_t bytes, cudaStream_t stream) {
    if (bytes > ctx->scratch_bytes) {
        if (pool_is_recording(ctx))
            return fail(B200_ERR_UNSUPPORTED, "an op needs %zu bytes of scratch while a trace is being recorded; run the step "
                        "once untraced first so the scratch exists", bytes);
        DeviceScope scope(ctx->device);
        // Round up so that a sweep over growing shapes reallocates rarely.
        size_t want = (bytes + (size_t(64) << 20) - 1) & ~((size_t(64) << 20) - 1);
        if (ctx->d_scratch) {
            if (pool_has_traces(ctx)) {
                // a recorded trace replays on the address it saw: the old block stays mapped until the traces are gone
                ctx->retired_scratch.push_back(ctx->d_scratch);
            } else {
                B200_CUDA_TRY(cudaDeviceSynchronize());
                B200_CUDA_TRY(cudaFree(ctx->d_scratch));
            }
            ctx->d_scratch = nullptr;
            ctx->scratch_bytes = 0;
        }
        cudaError_t e = cudaMalloc(&ctx->d_scratch, want);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(B200_ERR_NOMEM, "scratch allocation of %zu bytes failed: %s", want, cudaGetErrorString(e));
        }
        ctx->scratch_bytes = want;
    }
    return order_shared_state(ctx, stream);
}

}  // namespace b200

namespace b200 {
// One CTA waits on an mbarrier that nothing ever arrives at, with the same bounded wait the GEMM and attention kernels
// use but a short limit, and then does what they do when a wait runs out: it raises the context's status word and
// returns. Nothing faults and nothing hangs; it exists so that the error path (status word -> b200_synchronize ->
// B200_ERR_DEVICE_TIMEOUT -> a clean context) can be exercised on demand.
__global__ void wait_timeout_selftest_kernel(int* status, unsigned long long limit_ns) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        ptx::mbar_init(&bar, 1);
        ptx::mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!ptx::mbar_wait(&bar, 0, &abort_flag, limit_ns)) atomicExch(status, 1);
    }
}
}  // namespace b200

using namespace b200;

extern "C" {

int b200_selftest_wait_timeout(b200_ctx* ctx, uint64_t limit_ns, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_selftest_wait_timeout: ctx is NULL");
    B200_REQUIRE(limit_ns >= 1000 && limit_ns <= 100000000ull, "b200_selftest_wait_timeout: limit must be 1 us .. 100 ms");
    DeviceScope scope(ctx->device);
    wait_timeout_selftest_kernel<<<1, 32, 0, ctx->pick(stream)>>>(ctx->d_status, limit_ns);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

const char* b200_last_error(void) { return g_last_error.c_str(); }

int b200_abi_version(void) { return B200_TTPERF_ABI_VERSION; }

int b200_ctx_create(int device_ordinal, b200_ctx** out_ctx) {
    B200_REQUIRE(out_ctx != nullptr, "b200_ctx_create: out_ctx is NULL");
    *out_ctx = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(B200_ERR_CUDA, "b200_ctx_create: no CUDA device (%s); this library has no CPU path",
                    e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    }
    B200_REQUIRE(device_ordinal >= 0 && device_ordinal < count, "b200_ctx_create: device %d out of range [0,%d)",
                 device_ordinal, count);
    cudaDeviceProp prop;
    B200_CUDA_TRY(cudaGetDeviceProperties(&prop, device_ordinal));
    if (prop.major != 10) {
        return fail(B200_ERR_UNSUPPORTED, "b200_ctx_create: device %d is sm_%d%d; the kernels are built for sm_100a only",
                    device_ordinal, prop.major, prop.minor);
    }
    DeviceScope scope(device_ordinal);
    b200_ctx* ctx = new b200_ctx();
    ctx->device = device_ordinal;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->cc_major = prop.major;
    ctx->cc_minor = prop.minor;
    e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete ctx;
        return fail(B200_ERR_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(e));
    }
    e = cudaMalloc(&ctx->d_status, b200::kStatusBytes);
    if (e == cudaSuccess) e = cudaMemset(ctx->d_status, 0, b200::kStatusBytes);
    if (e != cudaSuccess) {
        cudaStreamDestroy(ctx->stream);
        delete ctx;
        return fail(B200_ERR_CUDA, "status word allocation failed: %s", cudaGetErrorString(e));
    }
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) {
        cudaGetLastError();
        cudaFree(ctx->d_status);
        cudaStreamDestroy(ctx->stream);
        delete ctx;
        return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    }
    ctx->encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    *out_ctx = ctx;
    return B200_OK;
}

int b200_ctx_destroy(b200_ctx* ctx) {
    if (!ctx) return B200_OK;
    DeviceScope scope(ctx->device);
    cudaDeviceSynchronize();
    pool_destroy(ctx);
    for (int i = 0; i < 3; ++i)
        if (ctx->d_stage[i]) cudaFree(ctx->d_stage[i]);
    if (ctx->copy_in) cudaStreamDestroy(ctx->copy_in);
    if (ctx->copy_out) cudaStreamDestroy(ctx->copy_out);
    if (ctx->d_scratch) cudaFree(ctx->d_scratch);
    for (void* p : ctx->retired_scratch) cudaFree(p);
    if (ctx->shared_event) cudaEventDestroy(ctx->shared_event);
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return B200_OK;
}

int b200_ctx_device(const b200_ctx* ctx, int* out) {
    B200_REQUIRE(ctx && out, "b200_ctx_device: NULL argument");
    *out = ctx->device;
    return B200_OK;
}

int b200_ctx_sm_count(const b200_ctx* ctx, int* out) {
    B200_REQUIRE(ctx && out, "b200_ctx_sm_count: NULL argument");
    *out = ctx->sm_count;
    return B200_OK;
}

int b200_ctx_stream(const b200_ctx* ctx, void** out) {
    B200_REQUIRE(ctx && out, "b200_ctx_stream: NULL argument");
    *out = ctx->stream;
    return B200_OK;
}

int b200_synchronize(b200_ctx* ctx, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_synchronize: ctx is NULL");
    if (pool_is_recording(ctx) && ctx->pick(stream) == ctx->stream)
        return fail(B200_ERR_UNSUPPORTED, "b200_synchronize: the context stream is recording a trace");
    DeviceScope scope(ctx->device);
    B200_CUDA_TRY(cudaStreamSynchronize(ctx->pick(stream)));
    int status = 0;
    B200_CUDA_TRY(cudaMemcpy(&status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (status != 0) {
        // A CTA that gave up may have left ticket counters and LayerNorm staging rows non-zero; later kernels rely on
        // finding them at zero, so the whole block is cleared, not only the status word.
        cudaDeviceSynchronize();
        cudaMemset(ctx->d_status, 0, b200::kStatusBytes);
        return fail(B200_ERR_DEVICE_TIMEOUT, "a kernel gave up a bounded wait (status word %d); its output is invalid",
                    status);
    }
    return B200_OK;
}

// Device-side stopwatch: two events on the stream, elapsed time read after the second has completed.
int b200_timer_start(b200_ctx* ctx, void* stream, void** out_timer) {
    B200_REQUIRE(ctx && out_timer, "b200_timer_start: NULL argument");
    DeviceScope scope(ctx->device);
    cudaEvent_t* ev = new cudaEvent_t[2];
    cudaError_t e = cudaEventCreate(&ev[0]);
    if (e == cudaSuccess) e = cudaEventCreate(&ev[1]);
    if (e == cudaSuccess) e = cudaEventRecord(ev[0], ctx->pick(stream));
    if (e != cudaSuccess) {
        delete[] ev;
        return fail(B200_ERR_CUDA, "b200_timer_start: %s", cudaGetErrorString(e));
    }
    *out_timer = ev;
    return B200_OK;
}

int b200_timer_stop(b200_ctx* ctx, void* stream, void* timer, float* out_ms) {
    B200_REQUIRE(ctx && timer && out_ms, "b200_timer_stop: NULL argument");
    DeviceScope scope(ctx->device);
    cudaEvent_t* ev = static_cast<cudaEvent_t*>(timer);
    cudaError_t e = cudaEventRecord(ev[1], ctx->pick(stream));
    if (e == cudaSuccess) e = cudaEventSynchronize(ev[1]);
    if (e == cudaSuccess) e = cudaEventElapsedTime(out_ms, ev[0], ev[1]);
    cudaEventDestroy(ev[0]);
    cudaEventDestroy(ev[1]);
    delete[] ev;
    if (e != cudaSuccess) return fail(B200_ERR_CUDA, "b200_timer_stop: %s", cudaGetErrorString(e));
    return B200_OK;
}

int b200_malloc(b200_ctx* ctx, size_t bytes, void** out_dptr) {
    B200_REQUIRE(ctx && out_dptr, "b200_malloc: NULL argument");
    *out_dptr = nullptr;
    if (bytes == 0) return B200_OK;
    DeviceScope scope(ctx->device);
    cudaError_t e = cudaMalloc(out_dptr, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(B200_ERR_NOMEM, "b200_malloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    }
    return B200_OK;
}

int b200_free(b200_ctx* ctx, void* dptr) {
    B200_REQUIRE(ctx != nullptr, "b200_free: ctx is NULL");
    if (!dptr) return B200_OK;
    DeviceScope scope(ctx->device);
    B200_CUDA_TRY(cudaFree(dptr));
    return B200_OK;
}

int b200_memcpy_h2d(b200_ctx* ctx, void* d_dst, const void* h_src, size_t bytes, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_memcpy_h2d: ctx is NULL");
    if (bytes == 0) return B200_OK;
    B200_REQUIRE(d_dst && h_src, "b200_memcpy_h2d: NULL buffer");
    DeviceScope scope(ctx->device);
    B200_CUDA_TRY(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->pick(stream)));
    return B200_OK;
}

int b200_memcpy_d2h(b200_ctx* ctx, void* h_dst, const void* d_src, size_t bytes, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_memcpy_d2h: ctx is NULL");
    if (bytes == 0) return B200_OK;
    B200_REQUIRE(h_dst && d_src, "b200_memcpy_d2h: NULL buffer");
    if (pool_is_recording(ctx) && ctx->pick(stream) == ctx->stream)
        return fail(B200_ERR_UNSUPPORTED, "b200_memcpy_d2h: the context stream is recording a trace (reading a tensor back "
                    "synchronises)");
    DeviceScope scope(ctx->device);
    B200_CUDA_TRY(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->pick(stream)));
    B200_CUDA_TRY(cudaStreamSynchronize(ctx->pick(stream)));
    return B200_OK;
}

int b200_memcpy_d2d(b200_ctx* ctx, void* d_dst, const void* d_src, size_t bytes, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_memcpy_d2d: ctx is NULL");
    if (bytes == 0) return B200_OK;
    B200_REQUIRE(d_dst && d_src, "b200_memcpy_d2d: NULL buffer");
    DeviceScope scope(ctx->device);
    B200_CUDA_TRY(cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDefault, ctx->pick(stream)));
    return B200_OK;
}

int b200_memset(b200_ctx* ctx, void* d_dst, int byte_value, size_t bytes, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_memset: ctx is NULL");
    if (bytes == 0) return B200_OK;
    B200_REQUIRE(d_dst != nullptr, "b200_memset: NULL buffer");
    DeviceScope scope(ctx->device);
    B200_CUDA_TRY(cudaMemsetAsync(d_dst, byte_value, bytes, ctx->pick(stream)));
    return B200_OK;
}

}  // extern "C"
