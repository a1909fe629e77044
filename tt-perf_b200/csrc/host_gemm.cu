// b200_matmul_host: the matmul as the reference's programs see it end to end — operands in HOST memory, result back
// in host memory (Tensor::from_vector -> to_device -> ttnn::matmul -> .cpu(), bench/metal/matmul_tensor_parallel.cpp:
// 56-93) — as one pipelined call: B is uploaded once, A is uploaded in row panels, each panel's GEMM starts as soon as
// its rows have landed, and each finished panel of C is downloaded while the next one computes. Upload, compute and
// download run on three streams (PCIe is full duplex), so the call costs about max(upload, download) + one panel
// instead of upload + compute + download.
#include <algorithm>

#include "gemm_common.cuh"

namespace b200 {
namespace {

int ensure_stage(b200_ctx* ctx, int which, size_t bytes) {
    if (bytes <= ctx->stage_bytes[which]) return B200_OK;
    if (ctx->d_stage[which]) {
        B200_CUDA_TRY(cudaDeviceSynchronize());
        B200_CUDA_TRY(cudaFree(ctx->d_stage[which]));
        ctx->d_stage[which] = nullptr;
        ctx->stage_bytes[which] = 0;
    }
    cudaError_t e = cudaMalloc(&ctx->d_stage[which], bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(B200_ERR_NOMEM, "b200_matmul_host: staging allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    }
    ctx->stage_bytes[which] = bytes;
    return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_matmul_host(b200_ctx* ctx, const b200_gemm_desc* d, int panels) {
    B200_REQUIRE(ctx && d, "b200_matmul_host: NULL argument");
    B200_REQUIRE(d->M > 0 && d->N > 0 && d->K > 0 && d->batch == 1, "b200_matmul_host: needs M, N, K > 0 and batch 1");
    B200_REQUIRE(d->A && d->B && d->C, "b200_matmul_host: A, B or C is NULL");
    B200_REQUIRE(d->c_dtype == B200_BF16 || d->c_dtype == B200_F32, "b200_matmul_host: bad c_dtype");
    B200_REQUIRE(d->ab_dtype == B200_BF16, "b200_matmul_host: host operands are bf16");
    const int64_t a_rows = d->transpose_a ? d->K : d->M, a_cols = d->transpose_a ? d->M : d->K;
    const int64_t b_rows = d->transpose_b ? d->N : d->K, b_cols = d->transpose_b ? d->K : d->N;
    B200_REQUIRE(d->lda >= a_cols && d->ldb >= b_cols && d->ldc >= d->N, "b200_matmul_host: leading dimension too small");
    DeviceScope scope(ctx->device);
    if (!ctx->copy_in) B200_CUDA_TRY(cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking));
    if (!ctx->copy_out) B200_CUDA_TRY(cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking));
    const size_t ces = d->c_dtype == B200_F32 ? 4 : 2;
    // device copies are dense: ld = row length rounded up to 8 elements so that the TMA path applies
    const int64_t dlda = (a_cols + 7) / 8 * 8, dldb = (b_cols + 7) / 8 * 8, dldc = (d->N + 7) / 8 * 8;
    int rc = ensure_stage(ctx, 0, static_cast<size_t>(a_rows) * dlda * 2);
    if (rc == B200_OK) rc = ensure_stage(ctx, 1, static_cast<size_t>(b_rows) * dldb * 2);
    if (rc == B200_OK) rc = ensure_stage(ctx, 2, static_cast<size_t>(d->M) * dldc * ces);
    if (rc != B200_OK) return rc;
    char* dA = static_cast<char*>(ctx->d_stage[0]);
    char* dB = static_cast<char*>(ctx->d_stage[1]);
    char* dC = static_cast<char*>(ctx->d_stage[2]);

    // panels of 256-row multiples; at least ~32 MFLOP-rows each so the per-panel launch cost stays negligible
    int np = panels > 0 ? panels : 8;
    np = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(np, d->M / 256)));
    const int64_t rows_per = ((d->M + np - 1) / np + 255) / 256 * 256;
    np = static_cast<int>((d->M + rows_per - 1) / rows_per);

    cudaStream_t compute = ctx->stream;
    cudaEvent_t ev_b, ev_in[64], ev_done[64];
    B200_REQUIRE(np <= 64, "b200_matmul_host: too many panels");
    B200_CUDA_TRY(cudaEventCreateWithFlags(&ev_b, cudaEventDisableTiming));
    for (int i = 0; i < np; ++i) {
        B200_CUDA_TRY(cudaEventCreateWithFlags(&ev_in[i], cudaEventDisableTiming));
        B200_CUDA_TRY(cudaEventCreateWithFlags(&ev_done[i], cudaEventDisableTiming));
    }
    auto cleanup = [&]() {
        cudaEventDestroy(ev_b);
        for (int i = 0; i < np; ++i) {
            cudaEventDestroy(ev_in[i]);
            cudaEventDestroy(ev_done[i]);
        }
    };
    // B first (every panel needs all of it), then the A panels, all on the upload stream
    cudaError_t e = cudaMemcpy2DAsync(dB, dldb * 2, d->B, d->ldb * 2, b_cols * 2, b_rows, cudaMemcpyHostToDevice, ctx->copy_in);
    if (e == cudaSuccess) e = cudaEventRecord(ev_b, ctx->copy_in);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(compute, ev_b, 0);
    int status = B200_OK;
    for (int i = 0; i < np && e == cudaSuccess && status == B200_OK; ++i) {
        const int64_t m0 = i * rows_per, m = std::min<int64_t>(rows_per, d->M - m0);
        if (!d->transpose_a) {  // A stored [M, K]: the panel is m contiguous rows
            e = cudaMemcpy2DAsync(dA + m0 * dlda * 2, dlda * 2, static_cast<const char*>(d->A) + m0 * d->lda * 2, d->lda * 2,
                                  d->K * 2, m, cudaMemcpyHostToDevice, ctx->copy_in);
        } else {                // A stored [K, M]: the panel is a column block
            e = cudaMemcpy2DAsync(dA + m0 * 2, dlda * 2, static_cast<const char*>(d->A) + m0 * 2, d->lda * 2, m * 2, d->K,
                                  cudaMemcpyHostToDevice, ctx->copy_in);
        }
        if (e != cudaSuccess) break;
        e = cudaEventRecord(ev_in[i], ctx->copy_in);
        if (e != cudaSuccess) break;
        e = cudaStreamWaitEvent(compute, ev_in[i], 0);
        if (e != cudaSuccess) break;
        b200_gemm_desc p = *d;
        p.M = m;
        p.A = d->transpose_a ? static_cast<const void*>(dA + m0 * 2) : static_cast<const void*>(dA + m0 * dlda * 2);
        p.lda = dlda;
        p.B = dB;
        p.ldb = dldb;
        p.C = dC + m0 * dldc * ces;
        p.ldc = dldc;
        p.split_k = 1;
        status = b200_gemm(ctx, &p, nullptr);
        if (status != B200_OK) break;
        e = cudaEventRecord(ev_done[i], compute);
        if (e != cudaSuccess) break;
        e = cudaStreamWaitEvent(ctx->copy_out, ev_done[i], 0);
        if (e != cudaSuccess) break;
        e = cudaMemcpy2DAsync(static_cast<char*>(d->C) + m0 * d->ldc * ces, d->ldc * ces, dC + m0 * dldc * ces, dldc * ces,
                              d->N * ces, m, cudaMemcpyDeviceToHost, ctx->copy_out);
    }
    cudaError_t e2 = cudaStreamSynchronize(ctx->copy_out);
    cudaError_t e3 = cudaStreamSynchronize(compute);
    cudaStreamSynchronize(ctx->copy_in);
    cleanup();
    if (status != B200_OK) return status;
    if (e != cudaSuccess) return fail(B200_ERR_CUDA, "b200_matmul_host: %s", cudaGetErrorString(e));
    if (e2 != cudaSuccess || e3 != cudaSuccess)
        return fail(B200_ERR_CUDA, "b200_matmul_host: %s", cudaGetErrorString(e2 != cudaSuccess ? e2 : e3));
    return B200_OK;
}
