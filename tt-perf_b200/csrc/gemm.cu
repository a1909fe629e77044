// b200_gemm: argument validation and the choice between the tcgen05 and the SIMT kernel.
#include "gemm_common.cuh"

#include <algorithm>
#include <cstdlib>

namespace b200 {
namespace {

// K == 0: the product is empty, so C = act(mask(bias)).
__global__ void gemm_k0_kernel(int M, int N, int batch, void* C, long long ldc, long long stride_c, int c_f32,
                               EpiParams epi) {
    const long long total = static_cast<long long>(batch) * M * N;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int n = static_cast<int>(i % N);
        const long long r = i / N;
        const int m = static_cast<int>(r % M);
        const int b = static_cast<int>(r / M);
        const float v = epi_apply(epi, 0.0f, m, n);
        const size_t off = static_cast<size_t>(b) * stride_c + static_cast<size_t>(m) * ldc + n;
        if (c_f32)
            static_cast<float*>(C)[off] = v;
        else
            static_cast<__nv_bfloat16*>(C)[off] = __float2bfloat16_rn(v);
    }
}

int validate(const b200_gemm_desc* d) {
    B200_REQUIRE(d != nullptr, "b200_gemm: desc is NULL");
    B200_REQUIRE(d->M >= 0 && d->N >= 0 && d->K >= 0, "b200_gemm: negative dimension (M=%lld N=%lld K=%lld)",
                 (long long)d->M, (long long)d->N, (long long)d->K);
    B200_REQUIRE(d->batch >= 1, "b200_gemm: batch must be >= 1 (got %lld)", (long long)d->batch);
    B200_REQUIRE(d->c_dtype == B200_BF16 || d->c_dtype == B200_F32, "b200_gemm: c_dtype must be BF16 or F32");
    B200_REQUIRE(d->bias_dtype == B200_BF16 || d->bias_dtype == B200_F32, "b200_gemm: bias_dtype must be BF16 or F32");
    B200_REQUIRE(d->activation >= B200_ACT_NONE && d->activation <= B200_ACT_GELU, "b200_gemm: unknown activation %d",
                 d->activation);
    B200_REQUIRE(d->fidelity >= B200_LOFI && d->fidelity <= B200_HIFI4, "b200_gemm: unknown fidelity %d", d->fidelity);
    B200_REQUIRE(d->algo >= B200_GEMM_AUTO && d->algo <= B200_GEMM_SIMT, "b200_gemm: unknown algo %d", d->algo);
    B200_REQUIRE(d->split_k >= 0, "b200_gemm: split_k must be >= 0");
    B200_REQUIRE(d->ab_dtype == B200_BF16 || d->ab_dtype == B200_FP8_E4M3, "b200_gemm: ab_dtype must be BF16 or FP8_E4M3");
    if (d->M == 0 || d->N == 0) return B200_OK;
    B200_REQUIRE(d->C != nullptr, "b200_gemm: C is NULL");
    B200_REQUIRE(d->ldc >= d->N, "b200_gemm: ldc (%lld) < N (%lld)", (long long)d->ldc, (long long)d->N);
    B200_REQUIRE(d->stride_a >= 0 && d->stride_b >= 0 && d->stride_c >= 0, "b200_gemm: negative batch stride");
    B200_REQUIRE(d->batch == 1 || d->stride_c >= d->M * d->ldc || d->stride_c == 0,
                 "b200_gemm: stride_c (%lld) overlaps consecutive outputs", (long long)d->stride_c);
    B200_REQUIRE(d->batch == 1 || d->stride_c != 0, "b200_gemm: stride_c must be non-zero for a batched product");
    if (d->K > 0) {
        B200_REQUIRE(d->A != nullptr && d->B != nullptr, "b200_gemm: A or B is NULL");
        const long long a_cols = d->transpose_a ? d->M : d->K;
        const long long b_cols = d->transpose_b ? d->K : d->N;
        B200_REQUIRE(d->lda >= a_cols, "b200_gemm: lda (%lld) < row length of A (%lld)", (long long)d->lda, a_cols);
        B200_REQUIRE(d->ldb >= b_cols, "b200_gemm: ldb (%lld) < row length of B (%lld)", (long long)d->ldb, b_cols);
    }
    return B200_OK;
}

// The CTA-pair kernel serves large products; B200_GEMM_2CTA=0 keeps everything on the single-CTA kernel.
bool pair_kernel_enabled() {
    static const bool value = [] {
        const char* e = getenv("B200_GEMM_2CTA");
        return e == nullptr || atoi(e) != 0;
    }();
    return value;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

void b200_gemm_desc_init(b200_gemm_desc* d) {
    if (!d) return;
    *d = b200_gemm_desc{};
    d->batch = 1;
    d->alpha = 1.0f;
    d->c_dtype = B200_BF16;
    d->bias_dtype = B200_BF16;
    d->activation = B200_ACT_NONE;
    d->mask_value = -1e9f;
    d->fidelity = B200_HIFI4;
    d->algo = B200_GEMM_AUTO;
    d->split_k = 0;
    d->ab_dtype = B200_BF16;
}

#ifdef B200_GEMM_PROFILE
// Development builds (-DB200_GEMM_PROFILE): the tcgen05 kernels write clock64() stamps for the first 8 tiles of every
// CTA into the context scratch, 8 entries per tile: 0 / 1 first and last MMA issue of the tile, 2 epilogue begin (warp
// 2), 3..6 epilogue end in warps 2..5; entry 7 of a CTA's first tile is the CTA's clock right after the start-up
// barrier. prepare sizes and clears the area (call it before the launch to be examined, and use split_k = 1: K slices
// use the same scratch); the second call copies `count` entries to the host after synchronising.
int b200_debug_gemm_stamps_prepare(b200_ctx* ctx) {
    B200_REQUIRE(ctx != nullptr, "b200_debug_gemm_stamps_prepare: ctx is NULL");
    DeviceScope scope(ctx->device);
    const size_t bytes = static_cast<size_t>(ctx->sm_count) * 64 * sizeof(long long);
    int rc = ensure_scratch(ctx, bytes);
    if (rc != B200_OK) return rc;
    B200_CUDA_TRY(cudaMemsetAsync(ctx->d_scratch, 0, bytes, ctx->stream));
    B200_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return B200_OK;
}
int b200_debug_gemm_stamps(b200_ctx* ctx, long long* host_out, size_t count) {
    B200_REQUIRE(ctx && host_out, "b200_debug_gemm_stamps: NULL argument");
    B200_REQUIRE(count * sizeof(long long) <= ctx->scratch_bytes, "b200_debug_gemm_stamps: more entries than prepared");
    DeviceScope scope(ctx->device);
    B200_CUDA_TRY(cudaDeviceSynchronize());
    B200_CUDA_TRY(cudaMemcpy(host_out, ctx->d_scratch, count * sizeof(long long), cudaMemcpyDeviceToHost));
    return B200_OK;
}
#endif

int b200_gemm_scratch_bytes(b200_ctx* ctx, const b200_gemm_desc* d, size_t* out_bytes) {
    B200_REQUIRE(ctx && out_bytes, "b200_gemm_scratch_bytes: NULL argument");
    int rc = validate(d);
    if (rc != B200_OK) return rc;
    *out_bytes = 0;
    if (d->M == 0 || d->N == 0 || d->K == 0) return B200_OK;
    if (d->algo == B200_GEMM_SIMT) return B200_OK;
    if (!gemm_tcgen05_eligible(*d, nullptr)) return B200_OK;
    const GemmPlan plan = gemm_plan(ctx, *d, pair_kernel_enabled() && gemm_tuned_block_n() == 0);
    if (plan.splits > 1) {
        if (plan.pair)  // whole 256 x 256 tiles
            *out_bytes = static_cast<size_t>(plan.splits) * d->batch * ((d->M + 255) / 256) * ((d->N + 255) / 256) * 256 * 256 * sizeof(float);
        else
            *out_bytes = static_cast<size_t>(plan.splits) * d->batch * d->M * d->N * sizeof(float);
    }
    return B200_OK;
}

int b200_gemm(b200_ctx* ctx, const b200_gemm_desc* d, void* stream_v) {
    B200_REQUIRE(ctx != nullptr, "b200_gemm: ctx is NULL");
    int rc = validate(d);
    if (rc != B200_OK) return rc;
    if (d->M == 0 || d->N == 0) return B200_OK;
    DeviceScope scope(ctx->device);
    cudaStream_t stream = ctx->pick(stream_v);
    if (d->K == 0) {
        EpiParams epi{};
        epi.alpha = d->alpha;
        epi.bias = d->bias;
        epi.bias_f32 = d->bias_dtype == B200_F32;
        epi.act = d->activation;
        epi.gelu_tanh = d->fidelity == B200_LOFI;
        epi.causal = d->causal_mask;
        epi.mask_value = d->mask_value;
        const long long total = d->batch * d->M * d->N;
        const int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, ctx->sm_count * 8ll));
        gemm_k0_kernel<<<blocks, 256, 0, stream>>>((int)d->M, (int)d->N, (int)d->batch, d->C, d->ldc, d->stride_c,
                                                   d->c_dtype == B200_F32, epi);
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    }
    const char* why = nullptr;
    const bool eligible = gemm_tcgen05_eligible(*d, &why);
    if (d->algo == B200_GEMM_TCGEN05 && !eligible)
        return fail(B200_ERR_INVALID_ARG, "b200_gemm: tcgen05 path requested but %s", why);
    if (d->ab_dtype == B200_FP8_E4M3) {  // tensor cores only: there is no scalar kernel for 8-bit operands
        B200_REQUIRE(d->algo != B200_GEMM_SIMT, "b200_gemm: 8-bit operands run on the tcgen05 path only");
        if (!eligible) return fail(B200_ERR_INVALID_ARG, "b200_gemm: 8-bit operands: %s", why);
    }
    if (d->algo == B200_GEMM_SIMT || !eligible) return launch_gemm_simt(ctx, *d, stream);
    GemmPlan plan = gemm_plan(ctx, *d, pair_kernel_enabled() && gemm_tuned_block_n() == 0);
    {
        // tuning sweeps (B200_GEMM_TUNE=1): B200_GEMM_KERNEL=pair pins the CTA-pair kernel with the descriptor's split_k
        static const bool tune = [] { const char* e = getenv("B200_GEMM_TUNE"); return e && atoi(e) != 0; }();
        const char* k = tune ? getenv("B200_GEMM_KERNEL") : nullptr;
        if (k && strcmp(k, "pair") == 0 && gemm_pair_supported(*d, nullptr)) {
            plan.pair = true;
            plan.splits = d->split_k > 1 ? static_cast<int>(d->split_k) : 1;
        }
    }
    if (plan.pair) return launch_gemm_tcgen05_pair(ctx, *d, stream, nullptr, plan.splits);
    return launch_gemm_tcgen05(ctx, *d, plan.splits, stream);
}

}  // extern "C"
