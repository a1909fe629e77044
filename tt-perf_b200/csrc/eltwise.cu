// Element-wise, broadcast, reduction, layout and gather/scatter kernels around the matmuls.
// All are HBM-bandwidth bound: 16-byte vector accesses on the contiguous dimension, grid-stride loops
// sized to a multiple of the SM count, fp32 arithmetic on bf16 storage.
#include "common.cuh"
#include "gemm_common.cuh"

#include <cuda_fp8.h>

#include <algorithm>
#include <cfloat>

namespace b200 {
namespace {

constexpr int kThreads = 256;

inline int grid_for(const b200_ctx* ctx, long long work_items) {
    const long long blocks = (work_items + kThreads - 1) / kThreads;
    return static_cast<int>(std::max<long long>(1, std::min<long long>(blocks, ctx->sm_count * 16ll)));
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

// ---- 8-bit (e4m3) operands for the matmul ----------------------------------------------------------------
// max |x|: 16-byte loads, warp shuffle, one atomicMax per warp (non-negative floats order like their bit patterns).
__global__ void absmax_kernel(const __nv_bfloat16* __restrict__ x, long long n, float* __restrict__ out, int vec_ok) {
    float m = 0.0f;
    const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long nvec = vec_ok ? n / 8 : 0;
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    for (long long i = tid; i < nvec; i += nthreads) {
        float f[8];
        unpack8(__ldg(xv + i), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));
    }
    for (long long i = nvec * 8 + tid; i < n; i += nthreads) m = fmaxf(m, fabsf(__bfloat162float(x[i])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m > 0.0f) atomicMax(reinterpret_cast<int*>(out), __float_as_int(m));
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d, float s) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a * s, b * s), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c * s, d * s), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

// y = e4m3(x * scale): two 16-byte loads (16 bf16) per 16-byte store.
__global__ void quantize_e4m3_kernel(const __nv_bfloat16* __restrict__ x, long long n, float scale,
                                     uint8_t* __restrict__ y, int vec_ok) {
    const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long nvec = vec_ok ? n / 16 : 0;
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    uint4* yv = reinterpret_cast<uint4*>(y);
    for (long long i = tid; i < nvec; i += nthreads) {
        float a[8], b[8];
        unpack8(__ldg(xv + 2 * i), a);
        unpack8(__ldg(xv + 2 * i + 1), b);
        yv[i] = make_uint4(pack_e4m3x4(a[0], a[1], a[2], a[3], scale), pack_e4m3x4(a[4], a[5], a[6], a[7], scale),
                           pack_e4m3x4(b[0], b[1], b[2], b[3], scale), pack_e4m3x4(b[4], b[5], b[6], b[7], scale));
    }
    for (long long i = nvec * 16 + tid; i < n; i += nthreads)
        y[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(__bfloat162float(x[i]) * scale, __NV_SATFINITE, __NV_E4M3));
}

// y[c][r] = e4m3(x[r][c] * scale): the transposed 8-bit copy an NN or TN product needs (8-bit operands are read
// K-major only). 64 x 64 tiles through shared memory: 4-byte loads along the input rows, 4-byte stores along the
// output rows.
__global__ void quantize_e4m3_transpose_kernel(const __nv_bfloat16* __restrict__ x, int rows, int cols, long long ldx,
                                               float scale, uint8_t* __restrict__ y, long long ldy, int tiles_c,
                                               long long tiles, int vec_in, int vec_out) {
    __shared__ __align__(4) uint8_t tile[64][68];
    const int tid = threadIdx.x;
    for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int r0 = static_cast<int>(t / tiles_c) * 64, c0 = static_cast<int>(t % tiles_c) * 64;
        const int c2 = tid & 31, ty = tid >> 5;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = r0 + i * 8 + ty, c = c0 + 2 * c2;
            float v0 = 0.0f, v1 = 0.0f;
            if (r < rows) {
                const __nv_bfloat16* src = x + static_cast<long long>(r) * ldx + c;
                if (vec_in && c + 1 < cols) {
                    const uint32_t u = __ldg(reinterpret_cast<const uint32_t*>(src));
                    v0 = __uint_as_float(u << 16);
                    v1 = __uint_as_float(u & 0xffff0000u);
                } else {
                    if (c < cols) v0 = __bfloat162float(src[0]);
                    if (c + 1 < cols) v1 = __bfloat162float(src[1]);
                }
            }
            const uint32_t q = __nv_cvt_float2_to_fp8x2(make_float2(v0 * scale, v1 * scale), __NV_SATFINITE, __NV_E4M3);
            tile[2 * c2][i * 8 + ty] = static_cast<uint8_t>(q & 0xffu);
            tile[2 * c2 + 1][i * 8 + ty] = static_cast<uint8_t>(q >> 8);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = i * 256 + tid;
            const int c = idx >> 4, w = idx & 15;
            const int oc = c0 + c, orow = r0 + 4 * w;
            if (oc < cols && orow < rows) {
                uint8_t* dst = y + static_cast<long long>(oc) * ldy + orow;
                if (vec_out && orow + 3 < rows) {
                    *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(&tile[c][4 * w]);
                } else {
                    for (int j = 0; j < 4 && orow + j < rows; ++j) dst[j] = tile[c][4 * w + j];
                }
            }
        }
        __syncthreads();
    }
}

// ---- unary / scalar ops ------------------------------------------------------------------------------
enum UnaryOp : int {
    U_NEG = 0, U_RELU = 1, U_GTZ = 2, U_GELU = 3, U_RSQRT = 4, U_EXP = 5, U_LOG = 6, U_TANH = 7, U_SQRT = 8,
    U_ADD_SCALAR = 9, U_MUL_SCALAR = 10, U_RSUB_SCALAR = 11, U_COPY = 12, U_RECIP = 13, U_SQUARE = 14, U_COUNT = 15
};

__device__ __forceinline__ float unary_apply(int op, float x, float s) {
    switch (op) {
        case U_NEG: return -x;
        case U_RELU: return fmaxf(x, 0.0f);
        case U_GTZ: return x > 0.0f ? 1.0f : 0.0f;
        case U_GELU: return gelu_exact(x);
        case U_RSQRT: return rsqrtf(x);
        case U_EXP: return __expf(x);
        case U_LOG: return __logf(x);
        case U_TANH: return tanhf(x);
        case U_SQRT: return sqrtf(x);
        case U_ADD_SCALAR: return x + s;
        case U_MUL_SCALAR: return x * s;
        case U_RSUB_SCALAR: return s - x;
        case U_RECIP: return 1.0f / x;
        case U_SQUARE: return x * x;
        default: return x;
    }
}

__global__ void __launch_bounds__(kThreads) unary_kernel(const __nv_bfloat16* x, __nv_bfloat16* y, long long n, int op,
                                                          float s, int vec) {
    const long long nvec = vec ? n / 8 : 0;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += stride) {
        float f[8];
        unpack8(reinterpret_cast<const uint4*>(x)[i], f);
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = unary_apply(op, f[k], s);
        reinterpret_cast<uint4*>(y)[i] = pack8(f);
    }
    for (long long i = nvec * 8 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += stride)
        y[i] = __float2bfloat16_rn(unary_apply(op, __bfloat162float(x[i]), s));
}

// Whole-vector inputs with the operation fixed at compile time (no per-element switch) and two 16-byte loads in
// flight per thread. OP = -1 keeps the run-time switch.
template <int OP>
__global__ void __launch_bounds__(kThreads) unary_vec_kernel(const uint4* x, uint4* y, long long nvec, int op, float s) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    for (; i + stride < nvec; i += 2 * stride) {
        const uint4 u0 = x[i], u1 = x[i + stride];
        float f0[8], f1[8];
        unpack8(u0, f0);
        unpack8(u1, f1);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            f0[k] = unary_apply(OP >= 0 ? OP : op, f0[k], s);
            f1[k] = unary_apply(OP >= 0 ? OP : op, f1[k], s);
        }
        y[i] = pack8(f0);
        y[i + stride] = pack8(f1);
    }
    if (i < nvec) {
        float f[8];
        unpack8(x[i], f);
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = unary_apply(OP >= 0 ? OP : op, f[k], s);
        y[i] = pack8(f);
    }
}

// ---- binary ops with numpy-style broadcasting over up to 4 dims --------------------------------------
enum BinaryOp : int { B_ADD = 0, B_SUB = 1, B_MUL = 2, B_DIV = 3, B_RELU_BW = 4, B_GELU_BW = 5, B_MAX = 6, B_COUNT = 7 };

__device__ __forceinline__ float binary_apply(int op, float a, float b) {
    switch (op) {
        case B_ADD: return a + b;
        case B_SUB: return a - b;
        case B_MUL: return a * b;
        case B_DIV: return a / b;
        case B_RELU_BW: return b > 0.0f ? a : 0.0f;  // a = dy, b = x
        case B_GELU_BW: return a * gelu_exact_grad(b);  // a = dy, b = x; derivative of the exact (erf) GELU
        case B_MAX: return fmaxf(a, b);
        default: return a;
    }
}

struct BinaryParams {
    const __nv_bfloat16* a;
    const __nv_bfloat16* b;
    __nv_bfloat16* out;
    long long od[4];      // output dims
    long long as[4];      // element strides of a per output dim (0 = broadcast)
    long long bs[4];
    long long n;          // total output elements
    int op;
    int vec;              // last output dim % 8 == 0, all pointers 16-byte aligned, last strides in {0,1}
};

// Same-shape operands, 16-byte aligned, n % 8 == 0: flat vector loop without index arithmetic.
__global__ void __launch_bounds__(kThreads) binary_flat_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b,
                                                                __nv_bfloat16* out, long long nvec, int op) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += stride) {
        float fa[8], fb[8];
        unpack8(reinterpret_cast<const uint4*>(a)[i], fa);
        unpack8(reinterpret_cast<const uint4*>(b)[i], fb);
#pragma unroll
        for (int k = 0; k < 8; ++k) fa[k] = binary_apply(op, fa[k], fb[k]);
        reinterpret_cast<uint4*>(out)[i] = pack8(fa);
    }
}

// The same with the operation fixed at compile time and two vector pairs in flight per thread.
template <int OP>
__global__ void __launch_bounds__(kThreads) binary_vec_kernel(const uint4* a, const uint4* b, uint4* out, long long nvec) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    for (; i + stride < nvec; i += 2 * stride) {
        const uint4 a0 = a[i], b0 = b[i], a1 = a[i + stride], b1 = b[i + stride];
        float fa0[8], fb0[8], fa1[8], fb1[8];
        unpack8(a0, fa0);
        unpack8(b0, fb0);
        unpack8(a1, fa1);
        unpack8(b1, fb1);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            fa0[k] = binary_apply(OP, fa0[k], fb0[k]);
            fa1[k] = binary_apply(OP, fa1[k], fb1[k]);
        }
        out[i] = pack8(fa0);
        out[i + stride] = pack8(fa1);
    }
    if (i < nvec) {
        float fa[8], fb[8];
        unpack8(a[i], fa);
        unpack8(b[i], fb);
#pragma unroll
        for (int k = 0; k < 8; ++k) fa[k] = binary_apply(OP, fa[k], fb[k]);
        out[i] = pack8(fa);
    }
}

// a has the output's shape, b is one row [.., 1, N] broadcast over all rows (bias add): b's vector index is i mod N/8.
__global__ void __launch_bounds__(kThreads) binary_rowbcast_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b,
                                                                    __nv_bfloat16* out, long long nvec, int row_vecs, int op) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += stride) {
        float fa[8], fb[8];
        unpack8(reinterpret_cast<const uint4*>(a)[i], fa);
        unpack8(reinterpret_cast<const uint4*>(b)[static_cast<int>(i % row_vecs)], fb);
#pragma unroll
        for (int k = 0; k < 8; ++k) fa[k] = binary_apply(op, fa[k], fb[k]);
        reinterpret_cast<uint4*>(out)[i] = pack8(fa);
    }
}

__global__ void __launch_bounds__(kThreads) binary_kernel(const BinaryParams p) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    if (p.vec) {
        const long long nvec = p.n / 8;
        const long long d3v = p.od[3] / 8;
        for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += stride) {
            const long long c = (i % d3v) * 8;
            long long r = i / d3v;
            const long long i2 = r % p.od[2];
            r /= p.od[2];
            const long long i1 = r % p.od[1];
            const long long i0 = r / p.od[1];
            const long long ao = i0 * p.as[0] + i1 * p.as[1] + i2 * p.as[2] + c * p.as[3];
            const long long bo = i0 * p.bs[0] + i1 * p.bs[1] + i2 * p.bs[2] + c * p.bs[3];
            float fa[8], fb[8];
            if (p.as[3] == 1) {
                unpack8(*reinterpret_cast<const uint4*>(p.a + ao), fa);
            } else {
                const float v = __bfloat162float(p.a[ao]);
#pragma unroll
                for (int k = 0; k < 8; ++k) fa[k] = v;
            }
            if (p.bs[3] == 1) {
                unpack8(*reinterpret_cast<const uint4*>(p.b + bo), fb);
            } else {
                const float v = __bfloat162float(p.b[bo]);
#pragma unroll
                for (int k = 0; k < 8; ++k) fb[k] = v;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) fa[k] = binary_apply(p.op, fa[k], fb[k]);
            reinterpret_cast<uint4*>(p.out)[i] = pack8(fa);
        }
    } else {
        for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < p.n; i += stride) {
            const long long i3 = i % p.od[3];
            long long r = i / p.od[3];
            const long long i2 = r % p.od[2];
            r /= p.od[2];
            const long long i1 = r % p.od[1];
            const long long i0 = r / p.od[1];
            const float a = __bfloat162float(p.a[i0 * p.as[0] + i1 * p.as[1] + i2 * p.as[2] + i3 * p.as[3]]);
            const float b = __bfloat162float(p.b[i0 * p.bs[0] + i1 * p.bs[1] + i2 * p.bs[2] + i3 * p.bs[3]]);
            p.out[i] = __float2bfloat16_rn(binary_apply(p.op, a, b));
        }
    }
}

// ---- reductions over one dim of [outer, R, inner] ----------------------------------------------------
enum ReduceOp : int { R_SUM = 0, R_MEAN = 1, R_MAX = 2, R_COUNT = 3 };

// inner == 1: one warp per output (row reduction).
__global__ void __launch_bounds__(kThreads) reduce_rows_kernel(const __nv_bfloat16* x, __nv_bfloat16* y, long long outer,
                                                                long long R, int op, int vec) {
    const int lane = threadIdx.x & 31;
    const long long o = blockIdx.x * static_cast<long long>(kThreads / 32) + (threadIdx.x >> 5);
    if (o >= outer) return;
    const __nv_bfloat16* row = x + o * R;
    float acc = (op == R_MAX) ? -FLT_MAX : 0.0f;
    const long long nvec = vec ? R / 8 : 0;
    for (long long v = lane; v < nvec; v += 32) {
        float f[8];
        unpack8(reinterpret_cast<const uint4*>(row)[v], f);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc = (op == R_MAX) ? fmaxf(acc, f[k]) : acc + f[k];
    }
    for (long long i = nvec * 8 + lane; i < R; i += 32) {
        const float f = __bfloat162float(row[i]);
        acc = (op == R_MAX) ? fmaxf(acc, f) : acc + f;
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, acc, s);
        acc = (op == R_MAX) ? fmaxf(acc, other) : acc + other;
    }
    if (lane == 0) y[o] = __float2bfloat16_rn(op == R_MEAN ? acc / static_cast<float>(R) : acc);
}

// inner == 1 with few, long rows (a loss mean over a whole activation): each CTA reduces one chunk of one row and
// combines through an fp32 accumulator, so the whole GPU works on the row instead of one warp.
__global__ void __launch_bounds__(kThreads) reduce_rows_split_kernel(const __nv_bfloat16* x, float* acc_out, long long R, int op,
                                                                      long long chunk, int vec) {
    __shared__ float sh[kThreads / 32];
    const long long o = blockIdx.y;
    const long long c0 = blockIdx.x * chunk, c1 = min(R, c0 + chunk);
    const __nv_bfloat16* row = x + o * R;
    float acc = (op == R_MAX) ? -FLT_MAX : 0.0f;
    if (vec) {  // chunk and row starts are multiples of 8 elements
        for (long long v = c0 / 8 + threadIdx.x; v < c1 / 8; v += kThreads) {
            float f[8];
            unpack8(reinterpret_cast<const uint4*>(row)[v], f);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc = (op == R_MAX) ? fmaxf(acc, f[k]) : acc + f[k];
        }
        for (long long i = (c1 / 8) * 8 + threadIdx.x; i < c1; i += kThreads) {
            const float f = __bfloat162float(row[i]);
            acc = (op == R_MAX) ? fmaxf(acc, f) : acc + f;
        }
    } else {
        for (long long i = c0 + threadIdx.x; i < c1; i += kThreads) {
            const float f = __bfloat162float(row[i]);
            acc = (op == R_MAX) ? fmaxf(acc, f) : acc + f;
        }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, acc, s);
        acc = (op == R_MAX) ? fmaxf(acc, other) : acc + other;
    }
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int k = 1; k < kThreads / 32; ++k) acc = (op == R_MAX) ? fmaxf(acc, sh[k]) : acc + sh[k];
        float* dst = acc_out + o;
        if (op == R_MAX) {
            if (acc >= 0.0f)
                atomicMax(reinterpret_cast<int*>(dst), __float_as_int(acc));
            else
                atomicMin(reinterpret_cast<unsigned int*>(dst), __float_as_uint(acc));
        } else {
            atomicAdd(dst, acc);
        }
    }
}

// inner > 1: CTA = 32 column groups x 8 row lanes; a column group is 8 adjacent columns read as one 16-byte vector
// (one column when rows are not 16-byte aligned). Partial results of the row slabs are combined in fp32.
template <int VEC>
__global__ void __launch_bounds__(kThreads) reduce_cols_kernel(const __nv_bfloat16* x, float* acc_out, long long R,
                                                                long long inner, int op, long long rows_per_cta) {
    __shared__ float sh[8][32][VEC + 1];
    const long long o = blockIdx.z;
    const long long c = (blockIdx.x * 32ll + (threadIdx.x & 31)) * VEC;
    const int sub = threadIdx.x >> 5;
    const long long r0 = blockIdx.y * rows_per_cta, r1 = min(R, r0 + rows_per_cta);
    float acc[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = (op == R_MAX) ? -FLT_MAX : 0.0f;
    if (c < inner) {
        const __nv_bfloat16* base = x + o * R * inner + c;
        for (long long r = r0 + sub; r < r1; r += 8) {
            if (VEC == 8) {
                float f[8];
                unpack8(*reinterpret_cast<const uint4*>(base + r * inner), f);
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = (op == R_MAX) ? fmaxf(acc[k], f[k]) : acc[k] + f[k];
            } else {
                const float f = __bfloat162float(base[r * inner]);
                acc[0] = (op == R_MAX) ? fmaxf(acc[0], f) : acc[0] + f;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) sh[sub][threadIdx.x & 31][k] = acc[k];
    __syncthreads();
    if (sub == 0 && c < inner) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            float a = acc[k];
            for (int j = 1; j < 8; ++j) {
                const float other = sh[j][threadIdx.x][k];
                a = (op == R_MAX) ? fmaxf(a, other) : a + other;
            }
            float* dst = acc_out + o * inner + c + k;
            if (op == R_MAX) {
                // float max through integer atomics (valid for any mix of signs)
                if (a >= 0.0f)
                    atomicMax(reinterpret_cast<int*>(dst), __float_as_int(a));
                else
                    atomicMin(reinterpret_cast<unsigned int*>(dst), __float_as_uint(a));
            } else {
                atomicAdd(dst, a);
            }
        }
    }
}

// Column reduction in one launch. Each CTA reduces its slab of rows for 32 column groups into fp32 partials
// part[outer][row_block][inner]; the CTA that finishes last for a column block (a ticket counter tells it) combines the
// partials, scales, rounds to bf16 and puts the counter back to zero. No zero-fill, no atomics on the data, no cast pass,
// and the result does not depend on the order in which the CTAs ran.
// GELU_BW = true (VEC = 8, sum): the tensor that is reduced does not exist yet. x holds the pre-activations, dy the
// gradient behind the GELU; the kernel writes dx = dy * GELU'(x) (bf16) and reduces the rounded dx on the way, so that the
// bias gradient of the Linear layer in front of the GELU costs no second pass over dx.
template <int VEC, bool GELU_BW = false>
__global__ void __launch_bounds__(kThreads, 4) reduce_cols_ticket_kernel(const __nv_bfloat16* x, float* part, unsigned* tickets,
                                                                       __nv_bfloat16* y, long long R, long long inner, int op,
                                                                       long long rows_per_cta, float scale,
                                                                       const __nv_bfloat16* dy = nullptr,
                                                                       __nv_bfloat16* dx = nullptr) {
    __shared__ float sh[8][32][VEC + 1];
    __shared__ int is_last;
    const long long o = blockIdx.z;
    const int row_blocks = gridDim.y;
    const long long c = (blockIdx.x * 32ll + (threadIdx.x & 31)) * VEC;
    const int sub = threadIdx.x >> 5;
    const long long r0 = blockIdx.y * rows_per_cta, r1 = min(R, r0 + rows_per_cta);
    float acc[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = (op == R_MAX) ? -FLT_MAX : 0.0f;
    if (c < inner) {
        const __nv_bfloat16* base = x + o * R * inner + c;
        long long r = r0 + sub;
        if (GELU_BW) {
            const __nv_bfloat16* gbase = dy + o * R * inner + c;
            __nv_bfloat16* obase = dx + o * R * inner + c;
            auto one = [&](const uint4& xv, const uint4& gv, long long row) {
                float fx[8], fg[8];
                unpack8(xv, fx);
                unpack8(gv, fg);
#pragma unroll
                for (int k = 0; k < 8; ++k) fg[k] *= gelu_exact_grad(fx[k]);
                const uint4 packed = pack8(fg);
                *reinterpret_cast<uint4*>(obase + row * inner) = packed;
                unpack8(packed, fg);  // the sum of the stored values, as a reduction of dx would see them
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] += fg[k];
            };
            for (; r + 8 < r1; r += 16) {  // two row pairs in flight per thread, four CTAs per SM
                uint4 xv[2], gv[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    xv[u] = *reinterpret_cast<const uint4*>(base + (r + 8 * u) * inner);
                    gv[u] = *reinterpret_cast<const uint4*>(gbase + (r + 8 * u) * inner);
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) one(xv[u], gv[u], r + 8 * u);
            }
            for (; r < r1; r += 8)
                one(*reinterpret_cast<const uint4*>(base + r * inner), *reinterpret_cast<const uint4*>(gbase + r * inner), r);
            r = r1;
        }
        if (VEC == 8) {
            // eight independent 16-byte loads in flight per thread
            for (; r + 56 < r1; r += 64) {
                uint4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const uint4*>(base + (r + 8 * u) * inner);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    float f[8];
                    unpack8(v[u], f);
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[k] = (op == R_MAX) ? fmaxf(acc[k], f[k]) : acc[k] + f[k];
                }
            }
        }
        for (; r < r1; r += 8) {
            if (VEC == 8) {
                float f[8];
                unpack8(*reinterpret_cast<const uint4*>(base + r * inner), f);
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = (op == R_MAX) ? fmaxf(acc[k], f[k]) : acc[k] + f[k];
            } else {
                const float f = __bfloat162float(base[r * inner]);
                acc[0] = (op == R_MAX) ? fmaxf(acc[0], f) : acc[0] + f;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) sh[sub][threadIdx.x & 31][k] = acc[k];
    __syncthreads();
    // thread t now owns column t of the CTA's 32 * VEC columns: consecutive threads, consecutive columns
    constexpr int cols_here = 32 * VEC;
    float* my_part = part + (o * row_blocks + blockIdx.y) * inner;
    const long long c0 = blockIdx.x * static_cast<long long>(cols_here);
    if (threadIdx.x < cols_here && c0 + threadIdx.x < inner) {
        const int t = threadIdx.x;
        float a = sh[0][t / VEC][t % VEC];
#pragma unroll
        for (int j = 1; j < 8; ++j) {
            const float other = sh[j][t / VEC][t % VEC];
            a = (op == R_MAX) ? fmaxf(a, other) : a + other;
        }
        my_part[c0 + t] = a;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned ticket = atomicAdd(&tickets[o * gridDim.x + blockIdx.x], 1u);
        is_last = ticket == static_cast<unsigned>(row_blocks - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // The last CTA of this column block combines the partials. All 256 threads take part: a thread owns `Q` adjacent
    // columns (4 as one 16-byte load when VEC = 8) and every `groups`-th row block, 8 independent loads at a time;
    // shared memory then combines the groups.
    constexpr int Q = VEC == 8 ? 4 : 1;
    constexpr int owners = cols_here / Q;
    constexpr int groups = kThreads / owners;
    const int col = (threadIdx.x % owners) * Q, grp = threadIdx.x / owners;
    float a[Q];
#pragma unroll
    for (int q = 0; q < Q; ++q) a[q] = (op == R_MAX) ? -FLT_MAX : 0.0f;
    const bool live = c0 + col < inner;  // inner % 8 == 0 when VEC = 8, so a quad is inside or outside as a whole
    if (live) {
        const float* src = part + o * row_blocks * inner + c0 + col;
        int rb = grp;
        for (; rb + 7 * groups < row_blocks; rb += 8 * groups) {
            float v[8][Q];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float* ptr = src + static_cast<long long>(rb + u * groups) * inner;
                if (Q == 4) {
                    const float4 f = __ldcg(reinterpret_cast<const float4*>(ptr));
                    v[u][0] = f.x; v[u][Q > 1 ? 1 : 0] = f.y; v[u][Q > 2 ? 2 : 0] = f.z; v[u][Q > 3 ? 3 : 0] = f.w;
                } else {
                    v[u][0] = __ldcg(ptr);
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
                for (int q = 0; q < Q; ++q) a[q] = (op == R_MAX) ? fmaxf(a[q], v[u][q]) : a[q] + v[u][q];
        }
        for (; rb < row_blocks; rb += groups) {
#pragma unroll
            for (int q = 0; q < Q; ++q) {
                const float v = __ldcg(src + static_cast<long long>(rb) * inner + q);
                a[q] = (op == R_MAX) ? fmaxf(a[q], v) : a[q] + v;
            }
        }
    }
    float* comb = &sh[0][0][0];  // reuse: groups * cols_here <= 8 * 32 * (VEC + 1) floats
    __syncthreads();
#pragma unroll
    for (int q = 0; q < Q; ++q) comb[grp * cols_here + col + q] = a[q];
    __syncthreads();
    if (threadIdx.x < cols_here && c0 + threadIdx.x < inner) {
        float r = comb[threadIdx.x];
        for (int q = 1; q < groups; ++q) {
            const float other = comb[q * cols_here + threadIdx.x];
            r = (op == R_MAX) ? fmaxf(r, other) : r + other;
        }
        y[o * inner + c0 + threadIdx.x] = __float2bfloat16_rn(r * scale);
    }
    if (threadIdx.x == 0) tickets[o * gridDim.x + blockIdx.x] = 0u;
}

__global__ void fill_f32_kernel(float* p, long long n, float v) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += stride) p[i] = v;
}
__global__ void fill_bf16_kernel(__nv_bfloat16* p, long long n, float v) {
    const __nv_bfloat16 b = __float2bfloat16_rn(v);
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += stride) p[i] = b;
}
__global__ void fill_u32_kernel(uint32_t* p, long long n, uint32_t v) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += stride) p[i] = v;
}
__global__ void cast_f32_to_bf16_kernel(const float* x, __nv_bfloat16* y, long long n, float scale) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += stride)
        y[i] = __float2bfloat16_rn(x[i] * scale);
}
__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* x, float* y, long long n) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += stride)
        y[i] = __bfloat162float(x[i]);
}

// ---- layout: permutation of a rank-4 tensor ----------------------------------------------------------
struct PermuteParams {
    const uint16_t* x;
    uint16_t* y;
    long long od[4];   // output dims
    long long is[4];   // input element stride for each OUTPUT dim
    long long n;
    int vec;           // innermost output dim is also the input's innermost (stride 1), % 8 == 0, aligned
};

__global__ void __launch_bounds__(kThreads) permute_kernel(const PermuteParams p) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    if (p.vec) {
        const long long d3v = p.od[3] / 8, nvec = p.n / 8;
        for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += stride) {
            const long long c = (i % d3v) * 8;
            long long r = i / d3v;
            const long long i2 = r % p.od[2];
            r /= p.od[2];
            const long long i1 = r % p.od[1];
            const long long i0 = r / p.od[1];
            reinterpret_cast<uint4*>(p.y)[i] =
                *reinterpret_cast<const uint4*>(p.x + i0 * p.is[0] + i1 * p.is[1] + i2 * p.is[2] + c);
        }
    } else {
        for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < p.n; i += stride) {
            const long long i3 = i % p.od[3];
            long long r = i / p.od[3];
            const long long i2 = r % p.od[2];
            r /= p.od[2];
            const long long i1 = r % p.od[1];
            const long long i0 = r / p.od[1];
            p.y[i] = p.x[i0 * p.is[0] + i1 * p.is[1] + i2 * p.is[2] + i3 * p.is[3]];
        }
    }
}

// Batched matrix transpose [batch, R, C] -> [batch, C, R] through a padded shared-memory tile.
__global__ void __launch_bounds__(256) transpose_tile_kernel(const uint16_t* x, uint16_t* y, long long R, long long C) {
    __shared__ uint16_t tile[32][33];
    const long long b = blockIdx.z;
    const long long c0 = blockIdx.x * 32ll, r0 = blockIdx.y * 32ll;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    const uint16_t* xb = x + b * R * C;
    uint16_t* yb = y + b * R * C;
    for (int k = ty; k < 32; k += 8)
        if (r0 + k < R && c0 + tx < C) tile[k][tx] = xb[(r0 + k) * C + c0 + tx];
    __syncthreads();
    for (int k = ty; k < 32; k += 8)
        if (c0 + k < C && r0 + tx < R) yb[(c0 + k) * R + r0 + tx] = tile[tx][k];
}

// Upper-triangular part of the last two dims: y = x where col - row >= diagonal, else 0.
__global__ void triu_kernel(const __nv_bfloat16* x, __nv_bfloat16* y, long long n, long long R, long long C, int diagonal) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += stride) {
        const long long c = i % C, r = (i / C) % R;
        y[i] = (c - r >= diagonal) ? x[i] : __float2bfloat16_rn(0.0f);
    }
}

// ---- embedding ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) embedding_fw_kernel(const uint32_t* ids, const uint16_t* table, uint16_t* out,
                                                                 long long n_ids, long long dim, long long vocab, int vec) {
    const long long per_row = vec ? dim / 8 : dim;
    const long long total = n_ids * per_row;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += stride) {
        const long long r = i / per_row, c = i % per_row;
        long long id = ids[r];
        if (id >= vocab) id = vocab - 1;  // clamp instead of reading out of bounds
        if (vec)
            reinterpret_cast<uint4*>(out + r * dim)[c] = reinterpret_cast<const uint4*>(table + id * dim)[c];
        else
            out[r * dim + c] = table[id * dim + c];
    }
}
__global__ void __launch_bounds__(kThreads) embedding_bw_kernel(const uint32_t* ids, const __nv_bfloat16* dy, float* dtable,
                                                                 long long n_ids, long long dim, long long vocab) {
    const long long total = n_ids * dim;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += stride) {
        const long long r = i / dim, c = i % dim;
        const long long id = ids[r];
        if (id < vocab) atomicAdd(&dtable[id * dim + c], __bfloat162float(dy[i]));
    }
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_unary(b200_ctx* ctx, int op, const void* x, void* y, int64_t n, float scalar, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_unary: ctx is NULL");
    B200_REQUIRE(op >= 0 && op < U_COUNT, "b200_unary: unknown op %d", op);
    B200_REQUIRE(n >= 0, "b200_unary: negative size");
    if (n == 0) return B200_OK;
    B200_REQUIRE(x && y, "b200_unary: NULL buffer");
    DeviceScope scope(ctx->device);
    const int vec = al16(x) && al16(y);
    if (vec && (n % 8) == 0) {
        const auto* xv = static_cast<const uint4*>(x);
        auto* yv = static_cast<uint4*>(y);
        const int grid = grid_for(ctx, (n / 8 + 1) / 2);
        if (op == U_GELU)
            unary_vec_kernel<U_GELU><<<grid, kThreads, 0, ctx->pick(stream)>>>(xv, yv, n / 8, op, scalar);
        else
            unary_vec_kernel<-1><<<grid, kThreads, 0, ctx->pick(stream)>>>(xv, yv, n / 8, op, scalar);
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    }
    unary_kernel<<<grid_for(ctx, (n + 7) / 8), kThreads, 0, ctx->pick(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n, op, scalar, vec);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_binary(b200_ctx* ctx, int op, const void* a, const int64_t* a_shape, const void* b, const int64_t* b_shape, void* out,
                void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_binary: ctx is NULL");
    B200_REQUIRE(op >= 0 && op < B_COUNT, "b200_binary: unknown op %d", op);
    B200_REQUIRE(a_shape && b_shape, "b200_binary: NULL shape");
    BinaryParams p{};
    long long ad[4], bd[4];
    p.n = 1;
    for (int i = 0; i < 4; ++i) {
        ad[i] = a_shape[i];
        bd[i] = b_shape[i];
        B200_REQUIRE(ad[i] >= 0 && bd[i] >= 0, "b200_binary: negative dimension");
        B200_REQUIRE(ad[i] == bd[i] || ad[i] == 1 || bd[i] == 1, "b200_binary: shapes [%lld,%lld,%lld,%lld] and "
                     "[%lld,%lld,%lld,%lld] do not broadcast", (long long)a_shape[0], (long long)a_shape[1],
                     (long long)a_shape[2], (long long)a_shape[3], (long long)b_shape[0], (long long)b_shape[1],
                     (long long)b_shape[2], (long long)b_shape[3]);
        p.od[i] = (ad[i] == 1) ? bd[i] : ad[i];
        p.n *= p.od[i];
    }
    if (p.n == 0) return B200_OK;
    B200_REQUIRE(a && b && out, "b200_binary: NULL buffer");
    long long sa = 1, sb = 1;
    for (int i = 3; i >= 0; --i) {
        p.as[i] = (ad[i] == 1 && p.od[i] != 1) ? 0 : sa;
        p.bs[i] = (bd[i] == 1 && p.od[i] != 1) ? 0 : sb;
        sa *= ad[i];
        sb *= bd[i];
    }
    p.a = static_cast<const __nv_bfloat16*>(a);
    p.b = static_cast<const __nv_bfloat16*>(b);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.op = op;
    auto rows_aligned = [&](const long long* s, const long long* d) {
        // every row start of the operand must stay 16-byte aligned when its last dim is walked in vectors
        if (s[3] == 0) return true;
        return (d[3] % 8) == 0;
    };
    p.vec = (p.od[3] % 8 == 0) && al16(a) && al16(b) && al16(out) && rows_aligned(p.as, ad) && rows_aligned(p.bs, bd);
    DeviceScope scope(ctx->device);
    bool same = true;
    for (int i = 0; i < 4; ++i) same = same && ad[i] == bd[i];
    if (same && (p.n % 8 == 0) && al16(a) && al16(b) && al16(out)) {
        const auto* av = reinterpret_cast<const uint4*>(p.a);
        const auto* bv = reinterpret_cast<const uint4*>(p.b);
        auto* ov = reinterpret_cast<uint4*>(p.out);
        const int grid = grid_for(ctx, (p.n / 8 + 1) / 2);
        if (op == B_GELU_BW)
            binary_vec_kernel<B_GELU_BW><<<grid, kThreads, 0, ctx->pick(stream)>>>(av, bv, ov, p.n / 8);
        else if (op == B_ADD)
            binary_vec_kernel<B_ADD><<<grid, kThreads, 0, ctx->pick(stream)>>>(av, bv, ov, p.n / 8);
        else if (op == B_MUL)
            binary_vec_kernel<B_MUL><<<grid, kThreads, 0, ctx->pick(stream)>>>(av, bv, ov, p.n / 8);
        else
            binary_flat_kernel<<<grid_for(ctx, p.n / 8), kThreads, 0, ctx->pick(stream)>>>(p.a, p.b, p.out, p.n / 8, op);
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    }
    const bool b_is_row = bd[0] == 1 && bd[1] == 1 && bd[2] == 1 && bd[3] == p.od[3] && ad[0] == p.od[0] &&
                          ad[1] == p.od[1] && ad[2] == p.od[2] && ad[3] == p.od[3];
    if (b_is_row && (p.od[3] % 8 == 0) && al16(a) && al16(b) && al16(out) && p.od[3] / 8 < (1ll << 31)) {
        binary_rowbcast_kernel<<<grid_for(ctx, p.n / 8), kThreads, 0, ctx->pick(stream)>>>(p.a, p.b, p.out, p.n / 8,
                                                                                          static_cast<int>(p.od[3] / 8), op);
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    }
    binary_kernel<<<grid_for(ctx, p.vec ? p.n / 8 : p.n), kThreads, 0, ctx->pick(stream)>>>(p);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_reduce(b200_ctx* ctx, int op, const void* x, int64_t outer, int64_t R, int64_t inner, void* y, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_reduce: ctx is NULL");
    B200_REQUIRE(op >= 0 && op < R_COUNT, "b200_reduce: unknown op %d", op);
    B200_REQUIRE(outer >= 0 && R >= 1 && inner >= 0, "b200_reduce: bad sizes (outer %lld, R %lld, inner %lld)",
                 (long long)outer, (long long)R, (long long)inner);
    if (outer == 0 || inner == 0) return B200_OK;
    B200_REQUIRE(x && y, "b200_reduce: NULL buffer");
    DeviceScope scope(ctx->device);
    cudaStream_t s = ctx->pick(stream);
    if (inner == 1 && R >= 16384 && outer <= ctx->sm_count && outer <= 65535) {
        int rc = ensure_scratch(ctx, static_cast<size_t>(outer) * sizeof(float), s);
        if (rc != B200_OK) return rc;
        float* acc = static_cast<float*>(ctx->d_scratch);
        fill_f32_kernel<<<grid_for(ctx, outer), kThreads, 0, s>>>(acc, outer, op == R_MAX ? -FLT_MAX : 0.0f);
        long long chunks = std::max<long long>(1, std::min<long long>((ctx->sm_count * 4ll) / outer, R / 4096));
        long long chunk = ((R + chunks - 1) / chunks + 7) / 8 * 8;
        chunks = (R + chunk - 1) / chunk;
        const int vec = al16(x) && (R % 8 == 0);
        dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(outer));
        reduce_rows_split_kernel<<<grid, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), acc, R, op, chunk, vec);
        cast_f32_to_bf16_kernel<<<grid_for(ctx, outer), kThreads, 0, s>>>(acc, static_cast<__nv_bfloat16*>(y), outer,
                                                                       op == R_MEAN ? 1.0f / static_cast<float>(R) : 1.0f);
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    }
    if (inner == 1) {
        const int vec = al16(x) && (R % 8 == 0);
        const long long blocks = (outer + 7) / 8;
        B200_REQUIRE(blocks < (1ll << 31), "b200_reduce: too many rows");
        reduce_rows_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(
            static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), outer, R, op, vec);
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    }
    // column reduction
    const long long outs = outer * inner;
    const bool vec8 = al16(x) && (inner % 8 == 0);
    const long long col_blocks = vec8 ? (inner / 8 + 31) / 32 : (inner + 31) / 32;
    B200_REQUIRE(outer <= 65535, "b200_reduce: outer dimension too large for a column reduction");
    const float scale = op == R_MEAN ? 1.0f / static_cast<float>(R) : 1.0f;
    if (col_blocks * outer < kTicketCount) {
        // one launch: per-CTA partials, the last CTA of a column block combines them
        long long row_blocks = std::max<long long>(1, std::min<long long>(std::min<long long>((R + 63) / 64, 128),
                                                                           (ctx->sm_count * 4ll) / std::max<long long>(1, col_blocks * outer)));
        const long long rows_per = (R + row_blocks - 1) / row_blocks;
        row_blocks = (R + rows_per - 1) / rows_per;
        int rc = ensure_scratch(ctx, static_cast<size_t>(outs) * row_blocks * sizeof(float), s);
        if (rc != B200_OK) return rc;
        float* part = static_cast<float*>(ctx->d_scratch);
        dim3 grid(static_cast<unsigned>(col_blocks), static_cast<unsigned>(row_blocks), static_cast<unsigned>(outer));
        if (vec8)
            reduce_cols_ticket_kernel<8><<<grid, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), part, ctx_tickets(ctx),
                                                                   static_cast<__nv_bfloat16*>(y), R, inner, op, rows_per, scale);
        else
            reduce_cols_ticket_kernel<1><<<grid, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), part, ctx_tickets(ctx),
                                                                   static_cast<__nv_bfloat16*>(y), R, inner, op, rows_per, scale);
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    }
    // very wide outputs: fp32 accumulators in context scratch combined with atomics, then a cast
    int rc = ensure_scratch(ctx, static_cast<size_t>(outs) * sizeof(float), s);
    if (rc != B200_OK) return rc;
    float* acc = static_cast<float*>(ctx->d_scratch);
    fill_f32_kernel<<<grid_for(ctx, outs), kThreads, 0, s>>>(acc, outs, op == R_MAX ? -FLT_MAX : 0.0f);
    long long row_blocks = std::max<long long>(1, std::min<long long>((R + 63) / 64, (ctx->sm_count * 4ll) / std::max<long long>(1, col_blocks * outer)));
    const long long rows_per = (R + row_blocks - 1) / row_blocks;
    row_blocks = (R + rows_per - 1) / rows_per;
    B200_REQUIRE(row_blocks <= 65535, "b200_reduce: too many row blocks");
    dim3 grid(static_cast<unsigned>(col_blocks), static_cast<unsigned>(row_blocks), static_cast<unsigned>(outer));
    if (vec8)
        reduce_cols_kernel<8><<<grid, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), acc, R, inner, op, rows_per);
    else
        reduce_cols_kernel<1><<<grid, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), acc, R, inner, op, rows_per);
    cast_f32_to_bf16_kernel<<<grid_for(ctx, outs), kThreads, 0, s>>>(acc, static_cast<__nv_bfloat16*>(y), outs, scale);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_gelu_backward(b200_ctx* ctx, const void* dy, const void* x_pre, void* dx, void* dx_colsum, int64_t rows,
                       int64_t cols, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_gelu_backward: ctx is NULL");
    B200_REQUIRE(rows >= 0 && cols >= 0, "b200_gelu_backward: bad sizes (rows %lld, cols %lld)", (long long)rows, (long long)cols);
    DeviceScope scope(ctx->device);
    cudaStream_t s = ctx->pick(stream);
    if (rows == 0 || cols == 0) {
        if (dx_colsum != nullptr && cols > 0) B200_CUDA_TRY(cudaMemsetAsync(dx_colsum, 0, sizeof(__nv_bfloat16) * cols, s));
        return B200_OK;
    }
    B200_REQUIRE(dy && x_pre && dx, "b200_gelu_backward: NULL buffer");
    const long long col_blocks = (cols / 8 + 31) / 32;
    const bool fused = dx_colsum != nullptr && cols % 8 == 0 && al16(dy) && al16(x_pre) && al16(dx) && col_blocks < kTicketCount;
    if (!fused) {
        const int64_t shape[4] = {1, 1, rows, cols};
        int rc = b200_binary(ctx, B_GELU_BW, dy, shape, x_pre, shape, dx, stream);
        if (rc != B200_OK || dx_colsum == nullptr) return rc;
        return b200_reduce(ctx, R_SUM, dx, 1, rows, cols, dx_colsum, stream);
    }
    // enough CTAs for four per SM, slabs of at least 32 rows
    long long row_blocks = std::max<long long>(1, std::min<long long>(std::min<long long>((rows + 31) / 32, 256),
                                                                       (ctx->sm_count * 4ll) / col_blocks));
    const long long rows_per = (rows + row_blocks - 1) / row_blocks;
    row_blocks = (rows + rows_per - 1) / rows_per;
    int rc = ensure_scratch(ctx, static_cast<size_t>(cols) * row_blocks * sizeof(float), s);
    if (rc != B200_OK) return rc;
    dim3 grid(static_cast<unsigned>(col_blocks), static_cast<unsigned>(row_blocks), 1);
    reduce_cols_ticket_kernel<8, true><<<grid, kThreads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x_pre), static_cast<float*>(ctx->d_scratch), ctx_tickets(ctx),
        static_cast<__nv_bfloat16*>(dx_colsum), rows, cols, R_SUM, rows_per, 1.0f, static_cast<const __nv_bfloat16*>(dy),
        static_cast<__nv_bfloat16*>(dx));
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_absmax(b200_ctx* ctx, const void* x, int64_t n, float* out, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_absmax: ctx is NULL");
    B200_REQUIRE(n >= 0, "b200_absmax: negative size");
    B200_REQUIRE(out != nullptr && (n == 0 || x != nullptr), "b200_absmax: NULL buffer");
    DeviceScope scope(ctx->device);
    cudaStream_t s = ctx->pick(stream);
    B200_CUDA_TRY(cudaMemsetAsync(out, 0, sizeof(float), s));
    if (n == 0) return B200_OK;
    const int vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    absmax_kernel<<<grid_for(ctx, (n + 15) / 16), kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), n, out, vec_ok);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_quantize_fp8(b200_ctx* ctx, const void* x, int64_t n, float scale, void* y, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_quantize_fp8: ctx is NULL");
    B200_REQUIRE(n >= 0, "b200_quantize_fp8: negative size");
    if (n == 0) return B200_OK;
    B200_REQUIRE(x && y, "b200_quantize_fp8: NULL buffer");
    B200_REQUIRE(scale > 0.0f && scale <= FLT_MAX, "b200_quantize_fp8: scale must be positive and finite");
    DeviceScope scope(ctx->device);
    const int vec_ok = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0;
    quantize_e4m3_kernel<<<grid_for(ctx, (n + 15) / 16), kThreads, 0, ctx->pick(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), n, scale, static_cast<uint8_t*>(y), vec_ok);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_quantize_fp8_transposed(b200_ctx* ctx, const void* x, int64_t rows, int64_t cols, int64_t ldx, float scale,
                                 void* y, int64_t ldy, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_quantize_fp8_transposed: ctx is NULL");
    B200_REQUIRE(rows >= 0 && cols >= 0 && rows < (1ll << 31) && cols < (1ll << 31), "b200_quantize_fp8_transposed: bad shape");
    if (rows == 0 || cols == 0) return B200_OK;
    B200_REQUIRE(x && y, "b200_quantize_fp8_transposed: NULL buffer");
    B200_REQUIRE(ldx >= cols && ldy >= rows, "b200_quantize_fp8_transposed: leading dimension too small");
    B200_REQUIRE(scale > 0.0f && scale <= FLT_MAX, "b200_quantize_fp8_transposed: scale must be positive and finite");
    DeviceScope scope(ctx->device);
    const int tiles_c = static_cast<int>((cols + 63) / 64);
    const long long tiles = ((rows + 63) / 64) * tiles_c;
    const int vec_in = (reinterpret_cast<uintptr_t>(x) & 3u) == 0 && (ldx & 1) == 0;
    const int vec_out = (reinterpret_cast<uintptr_t>(y) & 3u) == 0 && (ldy & 3) == 0;
    const int grid = static_cast<int>(std::min<long long>(tiles, ctx->sm_count * 8ll));
    quantize_e4m3_transpose_kernel<<<grid, 256, 0, ctx->pick(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<int>(rows), static_cast<int>(cols), ldx, scale,
        static_cast<uint8_t*>(y), ldy, tiles_c, tiles, vec_in, vec_out);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_fill(b200_ctx* ctx, void* dst, int64_t n, int dtype, float value, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_fill: ctx is NULL");
    B200_REQUIRE(n >= 0, "b200_fill: negative size");
    if (n == 0) return B200_OK;
    B200_REQUIRE(dst != nullptr, "b200_fill: NULL buffer");
    DeviceScope scope(ctx->device);
    cudaStream_t s = ctx->pick(stream);
    if (dtype == B200_BF16)
        fill_bf16_kernel<<<grid_for(ctx, n), kThreads, 0, s>>>(static_cast<__nv_bfloat16*>(dst), n, value);
    else if (dtype == B200_F32)
        fill_f32_kernel<<<grid_for(ctx, n), kThreads, 0, s>>>(static_cast<float*>(dst), n, value);
    else if (dtype == B200_U32)
        fill_u32_kernel<<<grid_for(ctx, n), kThreads, 0, s>>>(static_cast<uint32_t*>(dst), n, static_cast<uint32_t>(value));
    else
        return fail(B200_ERR_INVALID_ARG, "b200_fill: unknown dtype %d", dtype);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_cast(b200_ctx* ctx, const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_cast: ctx is NULL");
    B200_REQUIRE(n >= 0, "b200_cast: negative size");
    if (n == 0) return B200_OK;
    B200_REQUIRE(src && dst, "b200_cast: NULL buffer");
    DeviceScope scope(ctx->device);
    cudaStream_t s = ctx->pick(stream);
    if (src_dtype == B200_F32 && dst_dtype == B200_BF16)
        cast_f32_to_bf16_kernel<<<grid_for(ctx, n), kThreads, 0, s>>>(static_cast<const float*>(src),
                                                                      static_cast<__nv_bfloat16*>(dst), n, 1.0f);
    else if (src_dtype == B200_BF16 && dst_dtype == B200_F32)
        cast_bf16_to_f32_kernel<<<grid_for(ctx, n), kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(src),
                                                                      static_cast<float*>(dst), n);
    else
        return fail(B200_ERR_INVALID_ARG, "b200_cast: only f32<->bf16 is supported (got %d -> %d)", src_dtype, dst_dtype);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_permute(b200_ctx* ctx, const void* x, const int64_t* in_shape, const int32_t* perm, void* y, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_permute: ctx is NULL");
    B200_REQUIRE(in_shape && perm, "b200_permute: NULL shape or permutation");
    bool seen[4] = {false, false, false, false};
    for (int i = 0; i < 4; ++i) {
        B200_REQUIRE(perm[i] >= 0 && perm[i] < 4 && !seen[perm[i]], "b200_permute: not a permutation of 0..3");
        seen[perm[i]] = true;
        B200_REQUIRE(in_shape[i] >= 0, "b200_permute: negative dimension");
    }
    long long istr[4];
    long long s = 1;
    for (int i = 3; i >= 0; --i) {
        istr[i] = s;
        s *= in_shape[i];
    }
    PermuteParams p{};
    p.n = s;
    if (p.n == 0) return B200_OK;
    B200_REQUIRE(x && y, "b200_permute: NULL buffer");
    for (int i = 0; i < 4; ++i) {
        p.od[i] = in_shape[perm[i]];
        p.is[i] = istr[perm[i]];
    }
    p.x = static_cast<const uint16_t*>(x);
    p.y = static_cast<uint16_t*>(y);
    DeviceScope scope(ctx->device);
    cudaStream_t st = ctx->pick(stream);
    if (perm[0] == 0 && perm[1] == 1 && perm[2] == 3 && perm[3] == 2 && in_shape[0] * in_shape[1] <= 65535) {
        const long long R = in_shape[2], Cc = in_shape[3];
        dim3 grid(static_cast<unsigned>((Cc + 31) / 32), static_cast<unsigned>((R + 31) / 32),
                  static_cast<unsigned>(in_shape[0] * in_shape[1]));
        if (grid.y <= 65535) {
            transpose_tile_kernel<<<grid, 256, 0, st>>>(p.x, p.y, R, Cc);
            B200_CUDA_TRY(cudaGetLastError());
            return B200_OK;
        }
    }
    p.vec = (perm[3] == 3) && (p.od[3] % 8 == 0) && al16(x) && al16(y);
    permute_kernel<<<grid_for(ctx, p.vec ? p.n / 8 : p.n), kThreads, 0, st>>>(p);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_triu(b200_ctx* ctx, const void* x, void* y, int64_t batch, int64_t rows, int64_t cols, int diagonal, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_triu: ctx is NULL");
    B200_REQUIRE(batch >= 0 && rows >= 0 && cols >= 0, "b200_triu: negative size");
    const long long n = batch * rows * cols;
    if (n == 0) return B200_OK;
    B200_REQUIRE(x && y, "b200_triu: NULL buffer");
    DeviceScope scope(ctx->device);
    triu_kernel<<<grid_for(ctx, n), kThreads, 0, ctx->pick(stream)>>>(static_cast<const __nv_bfloat16*>(x),
                                                                     static_cast<__nv_bfloat16*>(y), n, rows, cols, diagonal);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_embedding_forward(b200_ctx* ctx, const uint32_t* ids, int64_t n_ids, const void* table, int64_t vocab, int64_t dim,
                           void* out, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_embedding_forward: ctx is NULL");
    B200_REQUIRE(n_ids >= 0 && vocab >= 1 && dim >= 0, "b200_embedding_forward: bad sizes");
    if (n_ids == 0 || dim == 0) return B200_OK;
    B200_REQUIRE(ids && table && out, "b200_embedding_forward: NULL buffer");
    DeviceScope scope(ctx->device);
    const int vec = (dim % 8 == 0) && al16(table) && al16(out);
    embedding_fw_kernel<<<grid_for(ctx, n_ids * (vec ? dim / 8 : dim)), kThreads, 0, ctx->pick(stream)>>>(
        ids, static_cast<const uint16_t*>(table), static_cast<uint16_t*>(out), n_ids, dim, vocab, vec);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_embedding_backward(b200_ctx* ctx, const uint32_t* ids, int64_t n_ids, const void* dy, int64_t vocab, int64_t dim,
                            float* d_table_f32, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_embedding_backward: ctx is NULL");
    B200_REQUIRE(n_ids >= 0 && vocab >= 1 && dim >= 0, "b200_embedding_backward: bad sizes");
    if (dim == 0) return B200_OK;
    B200_REQUIRE(d_table_f32 != nullptr, "b200_embedding_backward: NULL output");
    DeviceScope scope(ctx->device);
    cudaStream_t s = ctx->pick(stream);
    B200_CUDA_TRY(cudaMemsetAsync(d_table_f32, 0, sizeof(float) * vocab * dim, s));
    if (n_ids == 0) return B200_OK;
    B200_REQUIRE(ids && dy, "b200_embedding_backward: NULL buffer");
    embedding_bw_kernel<<<grid_for(ctx, n_ids * dim), kThreads, 0, s>>>(ids, static_cast<const __nv_bfloat16*>(dy),
                                                                        d_table_f32, n_ids, dim, vocab);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // extern "C"
