// Pieces shared by the GEMM kernels: the fused epilogue and the parameter blocks.
#pragma once
#include "common.cuh"

namespace b200 {

// alpha-scale, bias add, causal mask and activation applied to one fp32 accumulator value.
struct EpiParams {
    float alpha;
    const void* bias;  // [N] or nullptr
    int bias_f32;
    int act;        // b200_activation
    int gelu_tanh;  // LoFi: tanh approximation instead of erf
    int causal;     // replace entries with col > row by mask_value
    float mask_value;
};

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }

__device__ __forceinline__ float gelu_exact(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_tanh_approx(float x) {
    const float k = 0.7978845608028654f;  // sqrt(2/pi)
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x * x * x)));
}

__device__ __forceinline__ float epi_bias(const EpiParams& e, int n) {
    if (e.bias == nullptr) return 0.0f;
    return e.bias_f32 ? static_cast<const float*>(e.bias)[n]
                      : bf16_bits_to_float(static_cast<const uint16_t*>(e.bias)[n]);
}

__device__ __forceinline__ float epi_apply(const EpiParams& e, float acc, int m, int n) {
    float v = acc * e.alpha + epi_bias(e, n);
    if (e.causal && n > m) v = e.mask_value;
    if (e.act == B200_ACT_RELU) {
        v = fmaxf(v, 0.0f);
    } else if (e.act == B200_ACT_GELU) {
        v = e.gelu_tanh ? gelu_tanh_approx(v) : gelu_exact(v);
    }
    return v;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Parameter block of the tcgen05 kernel (one launch covers all batches, tiles and K slices).
struct GemmParams {
    int M, N, K, batch;
    int num_m_tiles, num_n_tiles;
    int num_kb;        // K blocks of 64
    int k_splits;      // >= 1
    int kb_per_split;
    int total_work;    // k_splits * batch * num_m_tiles * num_n_tiles
    int a_batched, b_batched;
    void* C;
    long long ldc, stride_c;
    int c_f32;
    int c_vec_ok;      // rows of C start 16-byte aligned, so 16-byte stores are legal
    float* partial;    // k_splits > 1: fp32 partial sums [split][batch][M][N]
    int partial_round_bf16;  // HiFi2 / LoFi: round partial sums to bf16 precision
    EpiParams epi;
    int* status;
};

// Host-side launchers implemented in the kernel translation units.
int launch_gemm_tcgen05(b200_ctx* ctx, const b200_gemm_desc& d, int k_splits, cudaStream_t stream);
int launch_gemm_simt(b200_ctx* ctx, const b200_gemm_desc& d, cudaStream_t stream);
bool gemm_tcgen05_eligible(const b200_gemm_desc& d, const char** why);
// Chooses the K-slice count for the tcgen05 path (1 = no split).
int gemm_choose_split_k(const b200_ctx* ctx, const b200_gemm_desc& d);
// N-tile width (64, 128 or 256) the tcgen05 path uses for this problem.
int gemm_choose_block_n(const b200_ctx* ctx, const b200_gemm_desc& d);

}  // namespace b200
