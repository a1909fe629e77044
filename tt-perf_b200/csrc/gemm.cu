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

}  // namespace

int gemm_validate_desc(const b200_gemm_desc* d) {
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

namespace {

// The plan b200_gemm follows for a validated, non-empty product.
b200_gemm_plan resolve_plan(const b200_ctx* ctx, const b200_gemm_desc& d) {
    b200_gemm_plan out{};
    if (d.algo == B200_GEMM_SIMT || !gemm_tcgen05_eligible(d, nullptr)) {
        out.kernel = B200_GEMM_KERNEL_SIMT;
        out.block_n = 64;
        out.k_slices = 1;
        return out;
    }
    const GemmPlan plan = gemm_plan(ctx, d, true);
    out.kernel = plan.pair ? B200_GEMM_KERNEL_TCGEN05_PAIR : B200_GEMM_KERNEL_TCGEN05;
    out.block_n = plan.pair ? 256 : plan.bn;
    out.k_slices = plan.splits;
    out.group_m = 0;
    return out;
}

size_t plan_scratch_bytes(const b200_gemm_desc& d, const b200_gemm_plan& plan) {
    if (plan.k_slices <= 1 || plan.kernel == B200_GEMM_KERNEL_SIMT) return 0;
    if (plan.kernel == B200_GEMM_KERNEL_TCGEN05_PAIR)  // whole 256 x 256 tiles
        return static_cast<size_t>(plan.k_slices) * d.batch * ((d.M + 255) / 256) * ((d.N + 255) / 256) * 256 * 256 * sizeof(float);
    return static_cast<size_t>(plan.k_slices) * d.batch * d.M * d.N * sizeof(float);
}

int run_plan(b200_ctx* ctx, const b200_gemm_desc& d, const b200_gemm_plan& plan, cudaStream_t stream) {
    switch (plan.kernel) {
        case B200_GEMM_KERNEL_SIMT:
            B200_REQUIRE(d.ab_dtype == B200_BF16, "b200_gemm: 8-bit operands run on the tcgen05 path only");
            return launch_gemm_simt(ctx, d, stream);
        case B200_GEMM_KERNEL_TCGEN05:
            return launch_gemm_tcgen05(ctx, d, std::max(1, plan.k_slices), stream, nullptr, plan.block_n, plan.group_m);
        case B200_GEMM_KERNEL_TCGEN05_PAIR:
            B200_REQUIRE(gemm_pair_supported(d, nullptr), "b200_gemm: the CTA-pair kernel needs 16-byte aligned rows of C");
            return launch_gemm_tcgen05_pair(ctx, d, stream, nullptr, std::max(1, plan.k_slices), plan.group_m);
        default:
            return fail(B200_ERR_INVALID_ARG, "b200_gemm: unknown kernel %d in the plan", plan.kernel);
    }
}

// K == 0: nothing to multiply, C = act(mask(bias)).
int run_k0(b200_ctx* ctx, const b200_gemm_desc* d, cudaStream_t stream) {
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

// Checks that apply to b200_gemm and b200_gemm_planned alike once the descriptor is valid and the product non-empty.
int check_route(const b200_gemm_desc* d) {
    const char* why = nullptr;
    const bool eligible = gemm_tcgen05_eligible(*d, &why);
    if (d->algo == B200_GEMM_TCGEN05 && !eligible)
        return fail(B200_ERR_INVALID_ARG, "b200_gemm: tcgen05 path requested but %s", why);
    if (d->ab_dtype == B200_FP8_E4M3) {  // tensor cores only: there is no scalar kernel for 8-bit operands
        B200_REQUIRE(d->algo != B200_GEMM_SIMT, "b200_gemm: 8-bit operands run on the tcgen05 path only");
        if (!eligible) return fail(B200_ERR_INVALID_ARG, "b200_gemm: 8-bit operands: %s", why);
    }
    return B200_OK;
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


int b200_gemm_scratch_bytes(b200_ctx* ctx, const b200_gemm_desc* d, size_t* out_bytes) {
    B200_REQUIRE(ctx && out_bytes, "b200_gemm_scratch_bytes: NULL argument");
    int rc = gemm_validate_desc(d);
    if (rc != B200_OK) return rc;
    *out_bytes = 0;
    if (d->M == 0 || d->N == 0 || d->K == 0) return B200_OK;
    *out_bytes = plan_scratch_bytes(*d, resolve_plan(ctx, *d));
    return B200_OK;
}

int b200_gemm_plan_query(b200_ctx* ctx, const b200_gemm_desc* d, b200_gemm_plan* out_plan) {
    B200_REQUIRE(ctx && out_plan, "b200_gemm_plan_query: NULL argument");
    int rc = gemm_validate_desc(d);
    if (rc != B200_OK) return rc;
    *out_plan = b200_gemm_plan{};
    if (d->M == 0 || d->N == 0 || d->K == 0) {
        out_plan->kernel = B200_GEMM_KERNEL_SIMT;
        out_plan->k_slices = 1;
        return B200_OK;
    }
    rc = check_route(d);
    if (rc != B200_OK) return rc;
    *out_plan = resolve_plan(ctx, *d);
    return B200_OK;
}

int b200_gemm_plan_describe(const b200_gemm_desc* d, const b200_gemm_plan* plan, char* buf, size_t buf_bytes) {
    B200_REQUIRE(d && plan && buf && buf_bytes > 0, "b200_gemm_plan_describe: NULL argument");
    const char* a_major = d->transpose_a ? "MN-major A" : "K-major A";
    const char* b_major = d->transpose_b ? "K-major B" : "MN-major B";
    const char* ab = d->ab_dtype == B200_FP8_E4M3 ? "e4m3" : "bf16";
    const int bk = gemm_bk_elems(*d);
    switch (plan->kernel) {
        case B200_GEMM_KERNEL_SIMT:
            snprintf(buf, buf_bytes, "gemm_simt_kernel (CUDA cores, 64x64x16 tiles)");
            break;
        case B200_GEMM_KERNEL_TCGEN05:
            snprintf(buf, buf_bytes, "gemm_tcgen05_kernel<%d, %s, %s, %s> (128x%dx%d tiles, %d K slice%s%s)", plan->block_n,
                     a_major, b_major, ab, plan->block_n, bk, plan->k_slices, plan->k_slices == 1 ? "" : "s",
                     plan->k_slices > 1 ? " + splitk_reduce_kernel" : "");
            break;
        case B200_GEMM_KERNEL_TCGEN05_PAIR:
            snprintf(buf, buf_bytes, "gemm_tcgen05_2cta_kernel<%s, %s, %s> (cta_group::2, 256x256x%d tiles, %d K slice%s)", a_major,
                     b_major, ab, bk, plan->k_slices, plan->k_slices == 1 ? "" : "s");
            break;
        default:
            return fail(B200_ERR_INVALID_ARG, "b200_gemm_plan_describe: unknown kernel %d", plan->kernel);
    }
    return B200_OK;
}

int b200_gemm(b200_ctx* ctx, const b200_gemm_desc* d, void* stream_v) {
    B200_REQUIRE(ctx != nullptr, "b200_gemm: ctx is NULL");
    int rc = gemm_validate_desc(d);
    if (rc != B200_OK) return rc;
    if (d->M == 0 || d->N == 0) return B200_OK;
    DeviceScope scope(ctx->device);
    cudaStream_t stream = ctx->pick(stream_v);
    if (d->K == 0) return run_k0(ctx, d, stream);
    rc = check_route(d);
    if (rc != B200_OK) return rc;
    return run_plan(ctx, *d, resolve_plan(ctx, *d), stream);
}

int b200_gemm_planned(b200_ctx* ctx, const b200_gemm_desc* d, const b200_gemm_plan* plan, void* stream_v) {
    B200_REQUIRE(ctx && plan, "b200_gemm_planned: NULL argument");
    int rc = gemm_validate_desc(d);
    if (rc != B200_OK) return rc;
    if (d->M == 0 || d->N == 0) return B200_OK;
    DeviceScope scope(ctx->device);
    cudaStream_t stream = ctx->pick(stream_v);
    if (d->K == 0) return run_k0(ctx, d, stream);
    rc = check_route(d);
    if (rc != B200_OK) return rc;
    B200_REQUIRE(plan->k_slices >= 0 && plan->group_m >= 0 && plan->group_m <= 64, "b200_gemm_planned: bad k_slices or group_m");
    if (plan->kernel != B200_GEMM_KERNEL_SIMT) {
        const char* why = nullptr;
        if (!gemm_tcgen05_eligible(*d, &why)) return fail(B200_ERR_INVALID_ARG, "b200_gemm_planned: tcgen05 kernel requested but %s", why);
    }
    return run_plan(ctx, *d, *plan, stream);
}

}  // extern "C"
