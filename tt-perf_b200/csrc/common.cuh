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
#include <vector>

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
    // Scratch blocks that were outgrown while a recorded trace may still hold their address: kept mapped until the last
    // trace is released (or the context destroyed), because a replay writes to the address it recorded.
    std::vector<void*> retired_scratch;
    // The scratch, the ticket counters and the LayerNorm staging rows are one set per context. Calls that use them on
    // different streams are put in order with this event (see order_shared_state); order_streams = false (the
    // allocation-free entry point's parameter holder) leaves the ordering to the caller.
    cudaStream_t shared_last_stream = nullptr;
    bool shared_used = false;
    cudaEvent_t shared_event = nullptr;
    bool order_streams = true;
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
// Grows the context scratch to at least `bytes` (never shrinks; not allowed while a trace is being recorded) and puts
// `stream` in order behind the last stream that used the context's shared state (order_shared_state).
int ensure_scratch(b200_ctx* ctx, size_t bytes, cudaStream_t stream);
// A kernel about to use the context's scratch, ticket counters or LayerNorm staging on `stream` must not overlap the
// previous user on another stream: when the stream changes, an event recorded on the previous stream is waited for
// by the new one. Skipped while a trace is being recorded (record on the context stream only).
int order_shared_state(b200_ctx* ctx, cudaStream_t stream);
// Frees the retired scratch blocks; called when no trace is left that could refer to them.
void release_retired_scratch(b200_ctx* ctx);
// Pool / trace state attached to a context (pool.cu).
void pool_destroy(b200_ctx* ctx);
bool pool_is_recording(b200_ctx* ctx);
bool pool_has_traces(b200_ctx* ctx);
}  // namespace b200
