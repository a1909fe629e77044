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

// Phi(x) = 0.5 (1 + erf(x / sqrt 2)) and exp(-x^2 / 2) together, from the rational approximation 7.1.26 of Abramowitz &
// Stegun (|error of erf| <= 1.5e-7, far below bf16 resolution): one reciprocal, one exp2 and a degree-5 polynomial
// instead of the branching library erff. The exponential is the one the derivative of GELU needs as well.
__device__ __forceinline__ void normal_cdf_and_exp(float x, float& cdf, float& e) {
    const float z = fabsf(x) * 0.70710678118654752f;
    float t;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, z, 1.0f)));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * x * -0.72134752044448170f));  // exp(-x^2 / 2)
    float poly = fmaf(t, 1.061405429f, -1.453152027f);
    poly = fmaf(poly, t, 1.421413741f);
    poly = fmaf(poly, t, -0.284496736f);
    poly = fmaf(poly, t, 0.254829592f);
    const float half_tail = 0.5f * poly * t * e;  // 0.5 * (1 - erf(|x| / sqrt 2))
    cdf = x >= 0.0f ? 1.0f - half_tail : half_tail;
}
__device__ __forceinline__ float gelu_exact(float x) {
    float cdf, e;
    normal_cdf_and_exp(x, cdf, e);
    return x * cdf;
}
// d/dx [x Phi(x)] = Phi(x) + x phi(x), phi the standard normal density.
__device__ __forceinline__ float gelu_exact_grad(float x) {
    float cdf, e;
    normal_cdf_and_exp(x, cdf, e);
    return fmaf(x * 0.3989422804014327f, e, cdf);
}
__device__ __forceinline__ float gelu_tanh_approx(float x) {
    const float k = 0.7978845608028654f;  // sqrt(2/pi)
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x * x * x)));
}

__device__ __forceinline__ float epi_bias(const EpiParams& e, int n) {
    if (e.bias == nullptr) return 0.0f;
    return e.bias_f32 ? static_cast<const float*>(e.bias)[n]
                      : bf16_bits_to_float(static_cast<const uint16_t*>(e.bias)[n]);
}

// Out of line on purpose: inlined, the compiler evaluates both GELU forms for every element and selects, which
// costs ~100 instructions per output even when no activation is requested.
static __device__ __noinline__ float epi_gelu_call(float v, int tanh_form) {
    return tanh_form ? gelu_tanh_approx(v) : gelu_exact(v);
}

__device__ __forceinline__ float epi_apply(const EpiParams& e, float acc, int m, int n) {
    float v = acc * e.alpha + epi_bias(e, n);
    if (e.causal && n > m) v = e.mask_value;
    if (e.act == B200_ACT_RELU) {
        v = fmaxf(v, 0.0f);
    } else if (e.act == B200_ACT_GELU) {
        v = epi_gelu_call(v, e.gelu_tanh);
    }
    return v;
}

// The same epilogue for 32 consecutive columns n .. n+31 of one row, with every decision hoisted out of the
// element loops (uniform branches). Columns >= N are computed on clamped bias indices and discarded by the caller.
__device__ __forceinline__ void epi_apply32(const EpiParams& e, const uint32_t (&v)[32], float (&f)[32], int row, int n,
                                            int N) {
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]) * e.alpha;
    if (e.bias != nullptr) {
        if (e.bias_f32) {
            const float* b = static_cast<const float*>(e.bias);
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] += b[min(n + i, N - 1)];
        } else {
            const uint16_t* b = static_cast<const uint16_t*>(e.bias);
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] += bf16_bits_to_float(b[min(n + i, N - 1)]);
        }
    }
    if (e.causal) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (n + i > row) f[i] = e.mask_value;
    }
    if (e.act == B200_ACT_RELU) {
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] = fmaxf(f[i], 0.0f);
    } else if (e.act == B200_ACT_GELU) {
        if (e.gelu_tanh) {
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = gelu_tanh_approx(f[i]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = gelu_exact(f[i]);
        }
    }
}

// v <- the sum of the K slices of 32 accumulator columns in slice order, whichever slice the caller holds: slice `own`
// is v itself (still in registers), the others come from memory through `src_of(slice)` (8 float4, 128 apart). The fixed
// order makes the result independent of which slice happened to finish last.
template <class SrcOf>
__device__ __forceinline__ void sum_slices_in_order(uint32_t (&v)[32], int own, int k_splits, SrcOf src_of) {
    float acc[32];
    bool started = false;
    for (int sl = 0; sl < k_splits; ++sl) {
        if (sl == own) {
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = started ? acc[i] + __uint_as_float(v[i]) : __uint_as_float(v[i]);
        } else {
            const float4* src = src_of(sl);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 a = __ldcg(src + i * 128);
                acc[4 * i] = started ? acc[4 * i] + a.x : a.x;
                acc[4 * i + 1] = started ? acc[4 * i + 1] + a.y : a.y;
                acc[4 * i + 2] = started ? acc[4 * i + 2] + a.z : a.z;
                acc[4 * i + 3] = started ? acc[4 * i + 3] + a.w : a.w;
            }
        }
        started = true;
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(acc[i]);
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
    int partial_is_bf16;     // splitk_reduce_kernel only: the slices it sums are stored as bf16, not fp32
    unsigned* tickets; // pair kernel, k_splits > 1: one counter per (tile, CTA of the pair); the CTA whose slice
                       // finishes last adds the other slices' partial sums to its accumulator and writes C
    EpiParams epi;
    int* status;
    int group_m;       // tile rasterisation: row-tiles per column sweep
    // Output routing of the TMA-store epilogue (epi_mode 1). n_dst destination tensor maps receive every tile
    // (1 = the local C; g = the same column slice of C on every GPU of an all-gather). scatter_rows > 0 selects a
    // single destination per tile instead: map index m0 / scatter_rows, row coordinate relative to that block
    // (row-block owner of a reduce-scatter).
    int epi_mode;      // 0 = direct predicated stores (any alignment), 1 = shared-memory staging + TMA store,
                       // 2 = shared-memory staging + 16-byte stores by the warp to `C` (multimem.st when mc_multimem:
                       //     C is then the NVLink multicast address of the output and every store lands on all ranks)
    int mc_multimem;
    int n_dst;
    int scatter_rows;
    int dst_rotate;    // first destination each box is sent to (ranks start at different peers, so no peer is hit by all at once)
    int m_tile_rotate; // the tile order starts at this row tile and wraps around (reduce-scatter: rank r starts with the row
                       // block of rank r + 1, so that at any moment the ranks store into different owners)
};

// Destination tensor maps of the TMA-store epilogue.
struct CMaps {
    CUtensorMap m[8];
};

// Where the output tiles of one launch go when they are not the descriptor's own C.
struct GemmRoute {
    int n_dst = 0;                 // 0 = descriptor's C only
    void* dst[8] = {};             // base address of each destination matrix (already offset to this rank's slice)
    long long rows[8] = {};        // rows of each destination matrix
    int scatter_rows = 0;
    int rotate = 0;                // index of the destination to store to first
    long long m_rotate_rows = 0;   // start the tile order at this output row (wraps around)
    void* mc_dst = nullptr;        // non-null: ONE destination written with 16-byte warp stores instead of TMA stores
    int mc_multimem = 0;           // those stores are multimem.st (mc_dst is a multicast address)
};

// Host-side launchers implemented in the kernel translation units.
// block_n = 0 lets the planner pick the tile width for k_splits; group_m = 0 takes the default tile order.
int launch_gemm_tcgen05(b200_ctx* ctx, const b200_gemm_desc& d, int k_splits, cudaStream_t stream,
                        const GemmRoute* route = nullptr, int block_n = 0, int group_m = 0);
// Sums `splits` fp32 slices [splits][batch][M][N], applies the descriptor's epilogue and writes C.
int launch_splitk_reduce(b200_ctx* ctx, const b200_gemm_desc& d, const void* partial, int splits, cudaStream_t stream,
                         bool partial_bf16 = false);
// CTA-pair (cta_group::2) kernel for large products; `gemm_pair_eligible` says whether it applies.
bool gemm_pair_eligible(const b200_ctx* ctx, const b200_gemm_desc& d, const GemmRoute* route);
// Layouts the pair kernel can handle at all, whatever the tile count.
bool gemm_pair_supported(const b200_gemm_desc& d, const GemmRoute* route);
int launch_gemm_tcgen05_pair(b200_ctx* ctx, const b200_gemm_desc& d, cudaStream_t stream, const GemmRoute* route = nullptr,
                             int k_splits = 1, int group_m = 0);
// Kernel, tile width and K-slice count for one product. allow_pair = false restricts the choice to the single-CTA kernel.
struct GemmPlan {
    bool pair;   // CTA-pair kernel (256 x 256 tiles) instead of the single-CTA kernel
    int bn;      // tile width of the single-CTA kernel
    int splits;
};
GemmPlan gemm_plan(const b200_ctx* ctx, const b200_gemm_desc& d, bool allow_pair);
// Elements of K one pipeline stage (128 bytes per row) holds: 64 bf16 or 128 e4m3.
inline int gemm_bk_elems(const b200_gemm_desc& d) { return d.ab_dtype == B200_FP8_E4M3 ? 128 : 64; }
int launch_gemm_simt(b200_ctx* ctx, const b200_gemm_desc& d, cudaStream_t stream);
bool gemm_tcgen05_eligible(const b200_gemm_desc& d, const char** why);
// The descriptor checks of b200_gemm (sizes, enums, leading dimensions, batch strides); B200_OK or INVALID_ARG with text.
int gemm_validate_desc(const b200_gemm_desc* d);
// Chooses the K-slice count for the tcgen05 path (1 = no split).
int gemm_choose_split_k(const b200_ctx* ctx, const b200_gemm_desc& d);

}  // namespace b200
