// Shared host-side plumbing of the library: the context object, error reporting and
// small device helpers used by several kernels.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>
#include <string>

#include "../../include/b200_ttperf.h"

namespace b200 {

// Thread-local text of the last failure, returned by b200_last_error().
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

#define B200_CUDA_TRY(expr)                                                                          \
    do {                                                                                             \
        cudaError_t _e = (expr);                                                                     \
        if (_e != cudaSuccess) {                                                                     \
            return ::b200::fail(B200_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                                __FILE__, __LINE__);                                                 \
        }                                                                                            \
    } while (0)

#define B200_REQUIRE(cond, ...)                                         \
    do {                                                                \
        if (!(cond)) return ::b200::fail(B200_ERR_INVALID_ARG, __VA_ARGS__); \
    } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// RAII switch of the calling thread's current device.
struct DeviceScope {
    int prev = -1;
    bool changed = false;
    explicit DeviceScope(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) {
            cudaSetDevice(dev);
            changed = true;
        }
    }
    ~DeviceScope() {
        if (changed) cudaSetDevice(prev);
    }
};

}  // namespace b200

// The opaque context of the C ABI.
struct b200_ctx {
    int device = 0;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    cudaStream_t stream = nullptr;     // the context's own stream (used when a call passes NULL)
    int* d_status = nullptr;           // device word: non-zero once a kernel's bounded wait ran out
    void* d_scratch = nullptr;         // split-K partial sums and other per-call scratch
    size_t scratch_bytes = 0;
    b200::EncodeTiledFn encode_tiled = nullptr;
    // b200_matmul_host: device staging for host operands and the two copy streams of its pipeline
    void* d_stage[3] = {nullptr, nullptr, nullptr};
    size_t stage_bytes[3] = {0, 0, 0};
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    std::mutex mu;

    cudaStream_t pick(void* s) const { return s ? static_cast<cudaStream_t>(s) : stream; }
};

namespace b200 {
// Layout of the small device block behind b200_ctx::d_status: the status word, then (from byte 256) ticket counters for
// kernels whose last-arriving CTA finishes a reduction. The counters start at zero and every kernel leaves them at zero.
// The last ticket is reserved for the LayerNorm backward kernel, whose parameter-gradient staging follows the tickets:
// kLnCopies replicas of [dgamma | dbeta | column sums of dx] with up to kLnMaxCols columns each, zero between kernels
// as well.
constexpr int kTicketCount = 4096;
constexpr int kLnCopies = 8;
constexpr int kLnMaxCols = 1024;
constexpr int kLnRows = 3;
constexpr size_t kLnStageBytes = sizeof(float) * kLnCopies * kLnRows * kLnMaxCols;
constexpr size_t kStatusBytes = 256 + sizeof(unsigned) * kTicketCount + kLnStageBytes;
inline unsigned* ctx_tickets(const b200_ctx* ctx) { return reinterpret_cast<unsigned*>(reinterpret_cast<char*>(ctx->d_status) + 256); }
inline float* ctx_ln_stage(const b200_ctx* ctx) {
    return reinterpret_cast<float*>(reinterpret_cast<char*>(ctx->d_status) + 256 + sizeof(unsigned) * kTicketCount);
}
// Grows the context scratch to at least `bytes` (never shrinks). Not allowed during stream capture.
int ensure_scratch(b200_ctx* ctx, size_t bytes);
// Pool / trace state attached to a context (pool.cu).
void pool_destroy(b200_ctx* ctx);
bool pool_is_recording(b200_ctx* ctx);
}  // namespace b200
