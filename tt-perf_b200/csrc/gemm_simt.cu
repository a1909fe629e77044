// CUDA-core GEMM for the shapes the TMA path cannot take: leading dimensions or base addresses that are
// not multiples of 16 bytes (for instance the [*,10] logits of the 784-128-10 MLP). Same math and the
// same fused epilogue as the tcgen05 kernel: bf16 inputs, fp32 accumulation. 64x64 tile per CTA,
// 4x4 outputs per thread, arbitrary strides so NN / NT / TN need no copy.
#include "gemm_common.cuh"

namespace b200 {

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

struct SimtParams {
    int M, N, K, batch;
    const uint16_t* A;
    long long a_sm, a_sk, a_sb;  // element strides of op(A)[m][k] and per batch
    const uint16_t* B;
    long long b_sk, b_sn, b_sb;  // element strides of op(B)[k][n] and per batch
    void* C;
    long long ldc, stride_c;
    int c_f32;
    EpiParams epi;
};

__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtParams p) {
    __shared__ float sA[TK][TM + 4];
    __shared__ float sB[TK][TN + 4];
    const int b = blockIdx.z;
    const int m0 = blockIdx.y * TM;
    const int n0 = blockIdx.x * TN;
    const int tx = threadIdx.x & 15;  // column group
    const int ty = threadIdx.x >> 4;  // row group
    const uint16_t* A = p.A + static_cast<size_t>(b) * p.a_sb;
    const uint16_t* B = p.B + static_cast<size_t>(b) * p.b_sb;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < p.K; k0 += TK) {
        // 64 x 16 elements of each operand, 4 per thread
        for (int i = threadIdx.x; i < TM * TK; i += 256) {
            // Walk the contiguous index fastest to keep the loads coalesced in either storage order.
            int mm, kk;
            if (p.a_sk == 1) {
                kk = i % TK;
                mm = i / TK;
            } else {
                mm = i % TM;
                kk = i / TM;
            }
            const int m = m0 + mm, k = k0 + kk;
            sA[kk][mm] = (m < p.M && k < p.K) ? bf16_bits_to_float(A[m * p.a_sm + k * p.a_sk]) : 0.0f;
        }
        for (int i = threadIdx.x; i < TN * TK; i += 256) {
            int nn, kk;
            if (p.b_sk == 1) {
                kk = i % TK;
                nn = i / TK;
            } else {
                nn = i % TN;
                kk = i / TN;
            }
            const int n = n0 + nn, k = k0 + kk;
            sB[kk][nn] = (n < p.N && k < p.K) ? bf16_bits_to_float(B[k * p.b_sk + n * p.b_sn]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], bb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sA[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bb[j] = sB[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= p.N) continue;
            const float v = epi_apply(p.epi, acc[i][j], m, n);
            const size_t off = static_cast<size_t>(b) * p.stride_c + static_cast<size_t>(m) * p.ldc + n;
            if (p.c_f32)
                static_cast<float*>(p.C)[off] = v;
            else
                static_cast<__nv_bfloat16*>(p.C)[off] = __float2bfloat16_rn(v);
        }
    }
}

}  // namespace

int launch_gemm_simt(b200_ctx* ctx, const b200_gemm_desc& d, cudaStream_t stream) {
    (void)ctx;
    SimtParams p{};
    p.M = static_cast<int>(d.M);
    p.N = static_cast<int>(d.N);
    p.K = static_cast<int>(d.K);
    p.batch = static_cast<int>(d.batch);
    p.A = static_cast<const uint16_t*>(d.A);
    p.B = static_cast<const uint16_t*>(d.B);
    if (d.transpose_a) {  // stored [K, M]
        p.a_sm = 1;
        p.a_sk = d.lda;
    } else {
        p.a_sm = d.lda;
        p.a_sk = 1;
    }
    if (d.transpose_b) {  // stored [N, K]
        p.b_sk = 1;
        p.b_sn = d.ldb;
    } else {
        p.b_sk = d.ldb;
        p.b_sn = 1;
    }
    p.a_sb = d.stride_a;
    p.b_sb = d.stride_b;
    p.C = d.C;
    p.ldc = d.ldc;
    p.stride_c = d.stride_c;
    p.c_f32 = d.c_dtype == B200_F32;
    p.epi.alpha = d.alpha;
    p.epi.bias = d.bias;
    p.epi.bias_f32 = d.bias_dtype == B200_F32;
    p.epi.act = d.activation;
    p.epi.gelu_tanh = d.fidelity == B200_LOFI;
    p.epi.causal = d.causal_mask;
    p.epi.mask_value = d.mask_value;
    const long long gx = (d.N + TN - 1) / TN, gy = (d.M + TM - 1) / TM;
    B200_REQUIRE(gy <= 65535 && d.batch <= 65535, "b200_gemm (SIMT path): M or batch too large for this kernel");
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(d.batch));
    gemm_simt_kernel<<<grid, 256, 0, stream>>>(p);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // namespace b200
