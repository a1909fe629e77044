// Sharded matmul across the GPUs of one NVSwitch node, one process per GPU.
//
// The collective is fused into the GEMM: the epilogue's TMA stores write each finished output tile straight into
// its final position in peer GPUs' memory over NVLink (plain peer stores; no TMA multicast, no loads from peers),
// so the transfer overlaps the tensor-core work tile by tile and no separate gather / scatter pass exists.
//
//   N-split + all-gather (bench/metal/matmul_tensor_parallel.cpp:70-92; scripts/matmul_2dev_distributed.py:49-76):
//     rank r holds B[:, r*N/g:(r+1)*N/g]; its tiles of C[:, slice r] are stored into the full C of every rank.
//   K-split + reduce-scatter (not in the reference; defined by the distributed-matmul configuration):
//     rank r holds A[:, K_r], B[K_r, :]; its fp32 partial tiles of row block j are stored into slot r of rank j's
//     staging buffer; after a barrier every rank sums its g slots and rounds to bf16 once.
//
// Peer buffers are shared between the processes with CUDA IPC handles (exchanged by the host program, for example
// through torch.distributed). Completion: the kernel's stores are visible to a peer only after this rank's stream
// work has finished AND the ranks have synchronised (a barrier / tiny all-reduce issued by the host program).
#include <cstring>

#include "gemm_common.cuh"
#include "ptx.cuh"

using namespace b200;

extern "C" {

int b200_ipc_get_handle(b200_ctx* ctx, void* dptr, void* out_handle64) {
    B200_REQUIRE(ctx && dptr && out_handle64, "b200_ipc_get_handle: NULL argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    DeviceScope scope(ctx->device);
    cudaIpcMemHandle_t h;
    B200_CUDA_TRY(cudaIpcGetMemHandle(&h, dptr));
    memcpy(out_handle64, &h, sizeof(h));
    return B200_OK;
}

int b200_ipc_open_handle(b200_ctx* ctx, const void* handle64, void** out_dptr) {
    B200_REQUIRE(ctx && handle64 && out_dptr, "b200_ipc_open_handle: NULL argument");
    DeviceScope scope(ctx->device);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    B200_CUDA_TRY(cudaIpcOpenMemHandle(out_dptr, h, cudaIpcMemLazyEnablePeerAccess));
    return B200_OK;
}

int b200_ipc_close_handle(b200_ctx* ctx, void* dptr) {
    B200_REQUIRE(ctx != nullptr, "b200_ipc_close_handle: ctx is NULL");
    if (!dptr) return B200_OK;
    DeviceScope scope(ctx->device);
    B200_CUDA_TRY(cudaIpcCloseMemHandle(dptr));
    return B200_OK;
}

// ---- several GPUs driven by ONE process (the reference's MeshDevice model) ------------------------------------------
int b200_enable_peer_access(b200_ctx* a, b200_ctx* b) {
    B200_REQUIRE(a && b, "b200_enable_peer_access: NULL context");
    if (a->device == b->device) return B200_OK;
    for (int dir = 0; dir < 2; ++dir) {
        b200_ctx* from = dir ? b : a;
        b200_ctx* to = dir ? a : b;
        int can = 0;
        B200_CUDA_TRY(cudaDeviceCanAccessPeer(&can, from->device, to->device));
        if (!can) return fail(B200_ERR_UNSUPPORTED, "GPU %d cannot access GPU %d directly", from->device, to->device);
        DeviceScope scope(from->device);
        cudaError_t e = cudaDeviceEnablePeerAccess(to->device, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) {
            cudaGetLastError();
        } else if (e != cudaSuccess) {
            return fail(B200_ERR_CUDA, "cudaDeviceEnablePeerAccess(%d -> %d) failed: %s", from->device, to->device,
                        cudaGetErrorString(e));
        }
    }
    return B200_OK;
}

int b200_peer_copy_2d(b200_ctx* dst_ctx, void* dst, size_t dst_pitch, b200_ctx* src_ctx, const void* src, size_t src_pitch,
                      size_t width_bytes, size_t rows) {
    B200_REQUIRE(dst_ctx && src_ctx, "b200_peer_copy_2d: NULL context");
    if (width_bytes == 0 || rows == 0) return B200_OK;
    B200_REQUIRE(dst && src, "b200_peer_copy_2d: NULL buffer");
    B200_REQUIRE(dst_pitch >= width_bytes && src_pitch >= width_bytes, "b200_peer_copy_2d: pitch smaller than the row width");
    // order after the producer's queued work, then copy on the consumer's stream (copy engine over NVLink)
    cudaEvent_t ev;
    {
        DeviceScope scope(src_ctx->device);
        B200_CUDA_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        B200_CUDA_TRY(cudaEventRecord(ev, src_ctx->stream));
    }
    DeviceScope scope(dst_ctx->device);
    B200_CUDA_TRY(cudaStreamWaitEvent(dst_ctx->stream, ev, 0));
    B200_CUDA_TRY(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDefault, dst_ctx->stream));
    B200_CUDA_TRY(cudaEventDestroy(ev));
    return B200_OK;
}

int b200_ctx_wait_ctx(b200_ctx* waiter, b200_ctx* producer) {
    B200_REQUIRE(waiter && producer, "b200_ctx_wait_ctx: NULL context");
    if (waiter == producer) return B200_OK;
    cudaEvent_t ev;
    {
        DeviceScope scope(producer->device);
        B200_CUDA_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        B200_CUDA_TRY(cudaEventRecord(ev, producer->stream));
    }
    DeviceScope scope(waiter->device);
    B200_CUDA_TRY(cudaStreamWaitEvent(waiter->stream, ev, 0));
    B200_CUDA_TRY(cudaEventDestroy(ev));
    return B200_OK;
}

namespace {
struct PeerFlagArrays {
    unsigned* p[8];
};

// One CTA, one thread per rank. Thread 0 advances the epoch; thread r publishes it to rank r and then waits for rank r's
// word in the local array. The fence before the stores orders them behind everything this GPU wrote earlier.
__global__ void peer_barrier_kernel(PeerFlagArrays flags, int n_ranks, int my_rank, unsigned* local_epoch, int* status) {
    __shared__ unsigned epoch;
    if (threadIdx.x == 0) epoch = ++(*local_epoch);
    __syncthreads();
    const int r = threadIdx.x;
    if (r >= n_ranks) return;
    const unsigned e = epoch;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.p[r] + my_rank), "r"(e) : "memory");
    const unsigned* mine = flags.p[my_rank] + r;
    const uint64_t t0 = ptx::globaltimer_ns();
    unsigned spins = 0;
    for (;;) {
        unsigned seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if (static_cast<int>(seen - e) >= 0) break;
        if ((++spins & 0xffu) == 0 && ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) {
            atomicExch(status, 1);
            break;
        }
    }
}
}  // namespace

int b200_peer_barrier(b200_ctx* ctx, void* const* peer_flags, int n_ranks, int my_rank, void* local_epoch, void* stream_v) {
    B200_REQUIRE(ctx && peer_flags && local_epoch, "b200_peer_barrier: NULL argument");
    B200_REQUIRE(n_ranks >= 1 && n_ranks <= 8, "b200_peer_barrier: n_ranks must be in [1, 8] (got %d)", n_ranks);
    B200_REQUIRE(my_rank >= 0 && my_rank < n_ranks, "b200_peer_barrier: my_rank %d out of range", my_rank);
    PeerFlagArrays f{};
    for (int i = 0; i < n_ranks; ++i) {
        B200_REQUIRE(peer_flags[i] != nullptr && (reinterpret_cast<uintptr_t>(peer_flags[i]) & 3u) == 0,
                     "b200_peer_barrier: flag array %d is NULL or not 4-byte aligned", i);
        f.p[i] = static_cast<unsigned*>(peer_flags[i]);
    }
    DeviceScope scope(ctx->device);
    peer_barrier_kernel<<<1, 32, 0, ctx->pick(stream_v)>>>(f, n_ranks, my_rank, static_cast<unsigned*>(local_epoch), ctx->d_status);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

static int check_dist_desc(const char* who, const b200_gemm_desc* d, int n_ranks, int my_rank) {
    B200_REQUIRE(d != nullptr, "%s: desc is NULL", who);
    B200_REQUIRE(n_ranks >= 1 && n_ranks <= 8, "%s: n_ranks must be in [1, 8] (got %d)", who, n_ranks);
    B200_REQUIRE(my_rank >= 0 && my_rank < n_ranks, "%s: my_rank %d out of range", who, my_rank);
    B200_REQUIRE(d->M > 0 && d->N > 0 && d->K > 0 && d->batch == 1, "%s: needs M, N, K > 0 and batch 1", who);
    B200_REQUIRE(d->A && d->B, "%s: A or B is NULL", who);
    B200_REQUIRE(d->lda >= (d->transpose_a ? d->M : d->K) && d->ldb >= (d->transpose_b ? d->K : d->N),
                 "%s: lda or ldb shorter than a row", who);
    const char* why = nullptr;
    if (!gemm_tcgen05_eligible(*d, &why)) return fail(B200_ERR_INVALID_ARG, "%s: %s", who, why);
    return B200_OK;
}

int b200_gemm_allgather(b200_ctx* ctx, const b200_gemm_desc* d, void* const* peer_c, int n_ranks, int my_rank, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_gemm_allgather: ctx is NULL");
    int rc = check_dist_desc("b200_gemm_allgather", d, n_ranks, my_rank);
    if (rc != B200_OK) return rc;
    B200_REQUIRE(peer_c != nullptr, "b200_gemm_allgather: peer_c is NULL");
    B200_REQUIRE(d->ldc >= d->N * n_ranks, "b200_gemm_allgather: ldc (%lld) must cover the gathered width %lld",
                 (long long)d->ldc, (long long)(d->N * n_ranks));
    const size_t es = d->c_dtype == B200_F32 ? 4 : 2;
    B200_REQUIRE((d->N * es) % 16 == 0, "b200_gemm_allgather: the shard width must be a multiple of 16 bytes");
    GemmRoute route;
    route.n_dst = n_ranks;
    route.rotate = my_rank;  // own copy first, then rank+1, rank+2, ...: at any moment the ranks write to different peers
    for (int p = 0; p < n_ranks; ++p) {
        B200_REQUIRE(peer_c[p] != nullptr, "b200_gemm_allgather: peer_c[%d] is NULL", p);
        route.dst[p] = static_cast<char*>(peer_c[p]) + static_cast<size_t>(my_rank) * d->N * es;
        route.rows[p] = d->M;
    }
    b200_gemm_desc local = *d;
    local.C = route.dst[my_rank];
    local.split_k = 1;
    DeviceScope scope(ctx->device);
    if (gemm_pair_eligible(ctx, local, &route)) return launch_gemm_tcgen05_pair(ctx, local, ctx->pick(stream), &route);
    return launch_gemm_tcgen05(ctx, local, 1, ctx->pick(stream), &route);
}

int b200_gemm_allgather_mc(b200_ctx* ctx, const b200_gemm_desc* d, void* mc_c, int n_ranks, int my_rank, int use_multimem,
                           void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_gemm_allgather_mc: ctx is NULL");
    int rc = check_dist_desc("b200_gemm_allgather_mc", d, n_ranks, my_rank);
    if (rc != B200_OK) return rc;
    B200_REQUIRE(mc_c != nullptr, "b200_gemm_allgather_mc: mc_c is NULL");
    B200_REQUIRE(d->ldc >= d->N * n_ranks, "b200_gemm_allgather_mc: ldc (%lld) must cover the gathered width %lld",
                 (long long)d->ldc, (long long)(d->N * n_ranks));
    const size_t es = d->c_dtype == B200_F32 ? 4 : 2;
    B200_REQUIRE((d->N * es) % 16 == 0 && (d->ldc * es) % 16 == 0,
                 "b200_gemm_allgather_mc: shard width and leading dimension must be multiples of 16 bytes");
    GemmRoute route;
    route.mc_dst = static_cast<char*>(mc_c) + static_cast<size_t>(my_rank) * d->N * es;
    route.mc_multimem = use_multimem ? 1 : 0;
    b200_gemm_desc local = *d;
    local.C = route.mc_dst;
    local.split_k = 1;
    DeviceScope scope(ctx->device);
    if (!gemm_pair_supported(local, nullptr))
        return fail(B200_ERR_UNSUPPORTED, "b200_gemm_allgather_mc: this product cannot run on the CTA-pair kernel (M and the shard "
                    "width must be at least 256); use b200_gemm_allgather");
    return launch_gemm_tcgen05_pair(ctx, local, ctx->pick(stream), &route);
}

int b200_gemm_dist_plan_query(b200_ctx* ctx, const b200_gemm_desc* d, int n_ranks, int reduce_scatter, b200_gemm_plan* out_plan) {
    B200_REQUIRE(ctx && out_plan, "b200_gemm_dist_plan_query: NULL argument");
    int rc = check_dist_desc("b200_gemm_dist_plan_query", d, n_ranks, 0);
    if (rc != B200_OK) return rc;
    GemmRoute route;
    route.n_dst = n_ranks;
    b200_gemm_desc local = *d;
    local.split_k = 1;
    if (reduce_scatter) {
        B200_REQUIRE(d->M % n_ranks == 0, "b200_gemm_dist_plan_query: M must divide by the rank count");
        route.scatter_rows = static_cast<int>(d->M / n_ranks);
        local.c_dtype = B200_F32;
        local.ldc = d->N;
    }
    local.C = reinterpret_cast<void*>(uintptr_t(256));  // destinations are checked at launch; the plan only needs an aligned one
    *out_plan = b200_gemm_plan{};
    out_plan->k_slices = 1;
    if (gemm_pair_eligible(ctx, local, &route)) {
        out_plan->kernel = B200_GEMM_KERNEL_TCGEN05_PAIR;
        out_plan->block_n = 256;
    } else {
        out_plan->kernel = B200_GEMM_KERNEL_TCGEN05;
        out_plan->block_n = gemm_plan(ctx, local, false).bn;
    }
    return B200_OK;
}

int b200_gemm_reduce_scatter_partials(b200_ctx* ctx, const b200_gemm_desc* d, void* const* peer_slots, int n_ranks,
                                      int my_rank, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_gemm_reduce_scatter_partials: ctx is NULL");
    int rc = check_dist_desc("b200_gemm_reduce_scatter_partials", d, n_ranks, my_rank);
    if (rc != B200_OK) return rc;
    B200_REQUIRE(peer_slots != nullptr, "b200_gemm_reduce_scatter_partials: peer_slots is NULL");
    B200_REQUIRE(d->M % n_ranks == 0 && (d->M / n_ranks) % 128 == 0,
                 "b200_gemm_reduce_scatter_partials: M / n_ranks must be a multiple of the 128-row tile (M = %lld)",
                 (long long)d->M);
    B200_REQUIRE(d->c_dtype == B200_F32 || d->c_dtype == B200_BF16, "b200_gemm_reduce_scatter_partials: partial tiles are F32 or BF16");
    const size_t pes = d->c_dtype == B200_F32 ? 4 : 2;   // bytes per partial element
    B200_REQUIRE((d->N * pes) % 16 == 0, "b200_gemm_reduce_scatter_partials: a row of partial sums must be a multiple of 16 bytes");
    const long long rows = d->M / n_ranks;
    GemmRoute route;
    route.n_dst = n_ranks;
    route.scatter_rows = static_cast<int>(rows);
    // Every rank walks the row blocks in the same cyclic order but starts one block after its own: at any moment the
    // ranks store into different owners (all starting at block 0 would aim g - 1 senders at one receiver's links) and
    // the local block, which needs no link, comes last, when the other ranks' traffic is tailing off.
    route.m_rotate_rows = static_cast<long long>((my_rank + 1) % n_ranks) * rows;
    for (int p = 0; p < n_ranks; ++p) {
        B200_REQUIRE(peer_slots[p] != nullptr, "b200_gemm_reduce_scatter_partials: peer_slots[%d] is NULL", p);
        // rank p's staging buffer is [n_ranks][rows][N] partial sums; this rank writes slot `my_rank`
        route.dst[p] = static_cast<char*>(peer_slots[p]) + static_cast<size_t>(my_rank) * rows * d->N * pes;
        route.rows[p] = rows;
    }
    b200_gemm_desc local = *d;
    local.C = route.dst[my_rank];
    local.ldc = d->N;
    local.bias = nullptr;
    local.activation = B200_ACT_NONE;
    local.alpha = 1.0f;
    local.causal_mask = 0;
    local.split_k = 1;
    DeviceScope scope(ctx->device);
    if (gemm_pair_eligible(ctx, local, &route)) return launch_gemm_tcgen05_pair(ctx, local, ctx->pick(stream), &route);
    return launch_gemm_tcgen05(ctx, local, 1, ctx->pick(stream), &route);
}

int b200_reduce_slices(b200_ctx* ctx, const float* slices, int n_slices, const b200_gemm_desc* d, void* stream) {
    return b200_reduce_slices_typed(ctx, slices, B200_F32, n_slices, d, stream);
}

int b200_reduce_slices_typed(b200_ctx* ctx, const void* slices, int slices_dtype, int n_slices, const b200_gemm_desc* d,
                             void* stream) {
    B200_REQUIRE(ctx && d, "b200_reduce_slices: NULL argument");
    B200_REQUIRE(slices_dtype == B200_F32 || slices_dtype == B200_BF16, "b200_reduce_slices: slices are F32 or BF16");
    B200_REQUIRE(n_slices >= 1 && d->M >= 0 && d->N >= 0 && d->batch >= 1, "b200_reduce_slices: bad sizes");
    if (d->M == 0 || d->N == 0) return B200_OK;
    B200_REQUIRE(slices && d->C, "b200_reduce_slices: NULL buffer");
    B200_REQUIRE(d->ldc >= d->N, "b200_reduce_slices: ldc < N");
    DeviceScope scope(ctx->device);
    return launch_splitk_reduce(ctx, *d, slices, n_slices, ctx->pick(stream), slices_dtype == B200_BF16);
}

}  // extern "C"
