// Device-memory pool and trace (CUDA graph) record / replay — the runtime pieces behind the reference's
// `Tensor` allocation and `TraceContext` (autograd/traced/trace.hpp:21-88).
//
// Pool. Executors written in the reference's style allocate a fresh tensor for every op result
// (`out = ttnn::add(a, b)`), tens of allocations per training step. Blocks are therefore cached by size and
// never returned to the driver while the context lives: allocation is a host-side list operation, and memory
// a recorded trace refers to stays mapped.
//
// Trace. begin/end wrap cudaStreamBeginCapture / EndCapture on the context stream; execute launches the
// instantiated graph. A replay re-runs the recorded kernels on the recorded addresses, so blocks allocated
// while recording belong to the trace: when freed they go to the trace's own free list (reusable by later
// allocations of the same recording, which keeps the recorded address sequence self-consistent) and return to
// the shared pool only when the trace is released. This matches the reference, where tensors assigned during
// capture must stay alive for replays.
#include <map>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace b200 {

struct PoolBlock {
    size_t size;
    uint32_t trace;  // 0 = shared pool, otherwise the trace that owns the block
};

struct Trace {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaStream_t stream = nullptr;
    bool recording = false;
    std::multimap<size_t, void*> free_blocks;
};

struct PoolState {
    std::multimap<size_t, void*> free_blocks;          // shared cache: size -> block
    std::unordered_map<void*, PoolBlock> blocks;       // every block ever handed out by cudaMalloc
    std::map<uint32_t, Trace> traces;
    uint32_t next_trace = 1;
    uint32_t recording = 0;                            // id of the trace being recorded, 0 if none
    size_t reserved = 0, in_use = 0;
};

static std::mutex g_pools_mu;
static std::unordered_map<const b200_ctx*, PoolState*> g_pools;

static PoolState* pool_of(b200_ctx* ctx) {
    std::lock_guard<std::mutex> lock(g_pools_mu);
    auto it = g_pools.find(ctx);
    if (it != g_pools.end()) return it->second;
    PoolState* p = new PoolState();
    g_pools[ctx] = p;
    return p;
}

static size_t round_size(size_t bytes) {
    if (bytes < 512) return 512;
    if (bytes <= (size_t(1) << 20)) return (bytes + 511) & ~size_t(511);
    return (bytes + (size_t(2) << 20) - 1) & ~((size_t(2) << 20) - 1);
}

static void* take(std::multimap<size_t, void*>& list, size_t size) {
    auto it = list.find(size);
    if (it == list.end()) return nullptr;
    void* p = it->second;
    list.erase(it);
    return p;
}

// Called by b200_ctx_destroy.
void pool_destroy(b200_ctx* ctx) {
    PoolState* p = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_pools_mu);
        auto it = g_pools.find(ctx);
        if (it == g_pools.end()) return;
        p = it->second;
        g_pools.erase(it);
    }
    for (auto& kv : p->traces) {
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
        if (kv.second.graph) cudaGraphDestroy(kv.second.graph);
    }
    for (auto& kv : p->blocks) cudaFree(kv.first);
    delete p;
}

bool pool_is_recording(b200_ctx* ctx) { return pool_of(ctx)->recording != 0; }
bool pool_has_traces(b200_ctx* ctx) { return !pool_of(ctx)->traces.empty(); }

}  // namespace b200

using namespace b200;

extern "C" {

int b200_pool_alloc(b200_ctx* ctx, size_t bytes, void** out) {
    B200_REQUIRE(ctx && out, "b200_pool_alloc: NULL argument");
    *out = nullptr;
    if (bytes == 0) return B200_OK;
    PoolState* p = pool_of(ctx);
    std::lock_guard<std::mutex> lock(ctx->mu);
    const size_t size = round_size(bytes);
    void* ptr = nullptr;
    if (p->recording) ptr = take(p->traces[p->recording].free_blocks, size);
    if (!ptr) ptr = take(p->free_blocks, size);
    if (!ptr) {
        DeviceScope scope(ctx->device);
        cudaError_t e = cudaMalloc(&ptr, size);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(B200_ERR_NOMEM, "b200_pool_alloc(%zu) failed: %s (pool holds %zu bytes, %zu in use)", bytes,
                        cudaGetErrorString(e), p->reserved, p->in_use);
        }
        p->blocks[ptr] = PoolBlock{size, 0};
        p->reserved += size;
    }
    p->blocks[ptr].trace = p->recording;  // a block handed out while recording belongs to that trace
    p->in_use += size;
    *out = ptr;
    return B200_OK;
}

int b200_pool_free(b200_ctx* ctx, void* ptr) {
    B200_REQUIRE(ctx != nullptr, "b200_pool_free: ctx is NULL");
    if (!ptr) return B200_OK;
    PoolState* p = pool_of(ctx);
    std::lock_guard<std::mutex> lock(ctx->mu);
    auto it = p->blocks.find(ptr);
    B200_REQUIRE(it != p->blocks.end(), "b200_pool_free: %p was not allocated by this context's pool", ptr);
    p->in_use -= it->second.size;
    const uint32_t owner = it->second.trace;
    auto tr = owner ? p->traces.find(owner) : p->traces.end();
    if (tr != p->traces.end())
        tr->second.free_blocks.emplace(it->second.size, ptr);
    else
        p->free_blocks.emplace(it->second.size, ptr);
    return B200_OK;
}

int b200_pool_stats(b200_ctx* ctx, size_t* reserved_bytes, size_t* in_use_bytes) {
    B200_REQUIRE(ctx != nullptr, "b200_pool_stats: ctx is NULL");
    PoolState* p = pool_of(ctx);
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (reserved_bytes) *reserved_bytes = p->reserved;
    if (in_use_bytes) *in_use_bytes = p->in_use;
    return B200_OK;
}

int b200_trace_begin(b200_ctx* ctx, uint32_t* out_trace_id) {
    B200_REQUIRE(ctx && out_trace_id, "b200_trace_begin: NULL argument");
    PoolState* p = pool_of(ctx);
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_REQUIRE(p->recording == 0, "b200_trace_begin: trace %u is still being recorded", p->recording);
    DeviceScope scope(ctx->device);
    B200_CUDA_TRY(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
    const uint32_t id = p->next_trace++;
    Trace& t = p->traces[id];
    t.stream = ctx->stream;
    t.recording = true;
    p->recording = id;
    *out_trace_id = id;
    return B200_OK;
}

int b200_trace_end(b200_ctx* ctx, uint32_t trace_id) {
    B200_REQUIRE(ctx != nullptr, "b200_trace_end: ctx is NULL");
    PoolState* p = pool_of(ctx);
    std::lock_guard<std::mutex> lock(ctx->mu);
    auto it = p->traces.find(trace_id);
    B200_REQUIRE(it != p->traces.end() && it->second.recording && p->recording == trace_id,
                 "b200_trace_end: trace %u is not being recorded", trace_id);
    DeviceScope scope(ctx->device);
    Trace& t = it->second;
    t.recording = false;
    p->recording = 0;
    cudaError_t e = cudaStreamEndCapture(t.stream, &t.graph);
    if (e != cudaSuccess || t.graph == nullptr) {
        cudaGetLastError();
        return fail(B200_ERR_CUDA, "b200_trace_end: capture failed: %s (an op synchronised or allocated scratch while "
                    "recording? run the step once untraced first)", cudaGetErrorString(e));
    }
    e = cudaGraphInstantiate(&t.exec, t.graph, 0);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(B200_ERR_CUDA, "b200_trace_end: cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
    }
    return B200_OK;
}

int b200_trace_execute(b200_ctx* ctx, uint32_t trace_id, int blocking) {
    B200_REQUIRE(ctx != nullptr, "b200_trace_execute: ctx is NULL");
    PoolState* p = pool_of(ctx);
    cudaGraphExec_t exec = nullptr;
    cudaStream_t stream = nullptr;
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        auto it = p->traces.find(trace_id);
        B200_REQUIRE(it != p->traces.end() && it->second.exec != nullptr, "b200_trace_execute: unknown or unfinished trace %u",
                     trace_id);
        exec = it->second.exec;
        stream = it->second.stream;
    }
    DeviceScope scope(ctx->device);
    B200_CUDA_TRY(cudaGraphLaunch(exec, stream));
    if (blocking) B200_CUDA_TRY(cudaStreamSynchronize(stream));
    return B200_OK;
}

int b200_trace_execute_on(b200_ctx* ctx, uint32_t trace_id, void* stream_v) {
    B200_REQUIRE(ctx != nullptr, "b200_trace_execute_on: ctx is NULL");
    B200_REQUIRE(stream_v != nullptr, "b200_trace_execute_on: a stream is required (b200_trace_execute uses the context's own)");
    PoolState* p = pool_of(ctx);
    cudaGraphExec_t exec = nullptr;
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        auto it = p->traces.find(trace_id);
        B200_REQUIRE(it != p->traces.end() && it->second.exec != nullptr,
                     "b200_trace_execute_on: unknown or unfinished trace %u", trace_id);
        exec = it->second.exec;
    }
    DeviceScope scope(ctx->device);
    B200_CUDA_TRY(cudaGraphLaunch(exec, static_cast<cudaStream_t>(stream_v)));
    return B200_OK;
}

int b200_trace_release(b200_ctx* ctx, uint32_t trace_id) {
    B200_REQUIRE(ctx != nullptr, "b200_trace_release: ctx is NULL");
    PoolState* p = pool_of(ctx);
    std::lock_guard<std::mutex> lock(ctx->mu);
    auto it = p->traces.find(trace_id);
    B200_REQUIRE(it != p->traces.end(), "b200_trace_release: unknown trace %u", trace_id);
    DeviceScope scope(ctx->device);
    Trace& t = it->second;
    if (t.recording) {
        cudaGraph_t g = nullptr;
        cudaStreamEndCapture(t.stream, &g);
        if (g) cudaGraphDestroy(g);
        cudaGetLastError();
        p->recording = 0;
    }
    cudaStreamSynchronize(t.stream);  // no replay may still be in flight when its blocks become reusable
    if (t.exec) cudaGraphExecDestroy(t.exec);
    if (t.graph) cudaGraphDestroy(t.graph);
    for (auto& kv : t.free_blocks) p->free_blocks.emplace(kv.first, kv.second);
    for (auto& kv : p->blocks)
        if (kv.second.trace == trace_id) kv.second.trace = 0;
    p->traces.erase(it);
    if (p->traces.empty()) release_retired_scratch(ctx);  // nothing recorded can refer to an outgrown scratch block now
    return B200_OK;
}

}  // extern "C"
