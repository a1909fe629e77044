// Row-wise, HBM-bandwidth-bound kernels: softmax / log-softmax (forward and backward), fused
// cross-entropy (loss + d_logits in one pass over the logits) and LayerNorm (forward and backward).
//
// Layout: [rows, cols] bf16, row-major with a leading dimension. Rows of up to 1024 columns are
// handled by one warp each, the whole row held in registers between the reduction and the write
// (one read + one write of HBM per element); longer rows (vocabulary-sized) by one 256-thread CTA
// each, with an online max/sum pass followed by a write pass whose re-read is served by L2.
// All global accesses are 16-byte vectors when the row starts are 16-byte aligned, reductions are
// warp shuffles, arithmetic is fp32.
#include "common.cuh"
#include "gemm_common.cuh"

#include <algorithm>
#include <cfloat>

namespace b200 {
namespace {

constexpr int kWarp = 32;
constexpr int kBlock = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float block_sum(float v, float* sh) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) sh[w] = v;
    __syncthreads();
    float t = (threadIdx.x < (blockDim.x >> 5)) ? sh[threadIdx.x] : 0.0f;
    if (w == 0) t = warp_sum(t);
    if (threadIdx.x == 0) sh[0] = t;
    __syncthreads();
    return sh[0];
}
__device__ __forceinline__ float block_max(float v, float* sh) {
    v = warp_max(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) sh[w] = v;
    __syncthreads();
    float t = (threadIdx.x < (blockDim.x >> 5)) ? sh[threadIdx.x] : -FLT_MAX;
    if (w == 0) t = warp_max(t);
    if (threadIdx.x == 0) sh[0] = t;
    __syncthreads();
    return sh[0];
}

// 8 consecutive bf16 of a row starting at column c (c % 8 == 0) -> fp32; columns >= cols read as `fill`.
__device__ __forceinline__ void load8(const __nv_bfloat16* row, int c, int cols, bool vec_ok, float fill, float (&f)[8]) {
    if (vec_ok && c + 8 <= cols) {
        const uint4 u = *reinterpret_cast<const uint4*>(row + c);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = (c + i < cols) ? __bfloat162float(row[c + i]) : fill;
    }
}
__device__ __forceinline__ void store8(__nv_bfloat16* row, int c, int cols, bool vec_ok, const float (&f)[8]) {
    if (vec_ok && c + 8 <= cols) {
        *reinterpret_cast<uint4*>(row + c) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                                        pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (c + i < cols) row[c + i] = __float2bfloat16_rn(f[i]);
    }
}
__device__ __forceinline__ void load8f(const float* row, int c, int cols, bool vec_ok, float fill, float (&f)[8]) {
    if (vec_ok && c + 8 <= cols) {
        const float4 a = *reinterpret_cast<const float4*>(row + c);
        const float4 b = *reinterpret_cast<const float4*>(row + c + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = (c + i < cols) ? row[c + i] : fill;
    }
}

enum RowOp : int {
    OP_SOFTMAX = 0,         // y = softmax(alpha * x [causal])
    OP_LOG_SOFTMAX = 1,     // y = log softmax(x)
    OP_SOFTMAX_BW = 2,      // dx = alpha * y * (dy - sum(dy * y))          in0 = dy, in1 = y
    OP_LOG_SOFTMAX_BW = 3,  // dx = dy - exp(logy) * sum(dy)                in0 = dy, in1 = logy
    OP_CROSS_ENTROPY = 4    // loss_row = -log softmax(x)[label]; dx = (softmax(x) - onehot) * alpha
};

struct RowParams {
    const __nv_bfloat16* in0;
    const __nv_bfloat16* in1;
    __nv_bfloat16* out;       // may be nullptr for OP_CROSS_ENTROPY (loss only)
    long long ld0, ld1, ldo;
    int rows, cols;
    float alpha;
    int causal_period;        // > 0: row r may only see columns <= r % causal_period
    const uint32_t* labels;   // OP_CROSS_ENTROPY
    float* row_loss;          // OP_CROSS_ENTROPY: per-row loss (fp32) or nullptr
    float* loss_sum;          // OP_CROSS_ENTROPY: atomically accumulated alpha-scaled loss, or nullptr
    int vec0, vec1, veco;     // 16-byte access legal for in0 / in1 / out
    int stage_row;            // block kernel: keep the row in shared memory between the two passes
};

__device__ __forceinline__ int visible_cols(const RowParams& p, int r) {
    return p.causal_period > 0 ? min(p.cols, (r % p.causal_period) + 1) : p.cols;
}

// ---- one warp per row, row held in registers: cols <= 256 * VPL --------------------------------------
template <int VPL, int OP>
__global__ void __launch_bounds__(kBlock) row_warp_kernel(const RowParams p) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (kBlock / kWarp) + (threadIdx.x >> 5);
    if (r >= p.rows) return;
    const __nv_bfloat16* x0 = p.in0 + static_cast<size_t>(r) * p.ld0;
    float a[VPL][8];
    if (OP == OP_SOFTMAX || OP == OP_LOG_SOFTMAX || OP == OP_CROSS_ENTROPY) {
        const int vis = visible_cols(p, r);
        const float scale = (OP == OP_SOFTMAX) ? p.alpha : 1.0f;
        float m = -FLT_MAX;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int c = (j * kWarp + lane) * 8;
            load8(x0, c, vis, p.vec0 != 0, -FLT_MAX, a[j]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                a[j][i] = (c + i < vis) ? a[j][i] * scale : -FLT_MAX;
                m = fmaxf(m, a[j][i]);
            }
        }
        m = warp_max(m);
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < VPL; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float e = (a[j][i] == -FLT_MAX) ? 0.0f : __expf(a[j][i] - m);
                if (OP == OP_LOG_SOFTMAX) a[j][i] -= m; else a[j][i] = e;
                s += e;
            }
        s = warp_sum(s);
        if (OP == OP_SOFTMAX) {
            const float inv = 1.0f / s;
            __nv_bfloat16* y = p.out + static_cast<size_t>(r) * p.ldo;
#pragma unroll
            for (int j = 0; j < VPL; ++j) {
                const int c = (j * kWarp + lane) * 8;
#pragma unroll
                for (int i = 0; i < 8; ++i) a[j][i] *= inv;
                if (c < p.cols) store8(y, c, p.cols, p.veco != 0, a[j]);
            }
        } else if (OP == OP_LOG_SOFTMAX) {
            const float ls = __logf(s);
            __nv_bfloat16* y = p.out + static_cast<size_t>(r) * p.ldo;
#pragma unroll
            for (int j = 0; j < VPL; ++j) {
                const int c = (j * kWarp + lane) * 8;
#pragma unroll
                for (int i = 0; i < 8; ++i) a[j][i] -= ls;
                if (c < p.cols) store8(y, c, p.cols, p.veco != 0, a[j]);
            }
        } else {  // cross-entropy
            const int label = static_cast<int>(p.labels[r]);
            const float inv = 1.0f / s;
            float picked = 0.0f;
#pragma unroll
            for (int j = 0; j < VPL; ++j) {
                const int c = (j * kWarp + lane) * 8;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float prob = a[j][i] * inv;
                    if (c + i == label) picked = prob;
                    a[j][i] = (prob - ((c + i == label) ? 1.0f : 0.0f)) * p.alpha;
                }
                if (p.out != nullptr && c < p.cols)
                    store8(p.out + static_cast<size_t>(r) * p.ldo, c, p.cols, p.veco != 0, a[j]);
            }
            picked = warp_sum(picked);  // exactly one lane holds the label column
            if (lane == 0) {
                const float loss = -__logf(fmaxf(picked, 1e-38f));
                if (p.row_loss) p.row_loss[r] = loss;
                if (p.loss_sum) atomicAdd(p.loss_sum, loss * p.alpha);
            }
        }
    } else {
        const __nv_bfloat16* x1 = p.in1 + static_cast<size_t>(r) * p.ld1;
        float b[VPL][8];
        float dot = 0.0f;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int c = (j * kWarp + lane) * 8;
            load8(x0, c, p.cols, p.vec0 != 0, 0.0f, a[j]);
            load8(x1, c, p.cols, p.vec1 != 0, 0.0f, b[j]);
#pragma unroll
            for (int i = 0; i < 8; ++i) dot += (OP == OP_SOFTMAX_BW) ? a[j][i] * b[j][i] : a[j][i];
        }
        dot = warp_sum(dot);
        __nv_bfloat16* y = p.out + static_cast<size_t>(r) * p.ldo;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int c = (j * kWarp + lane) * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                a[j][i] = (OP == OP_SOFTMAX_BW) ? p.alpha * b[j][i] * (a[j][i] - dot)
                                                : a[j][i] - ((c + i < p.cols) ? __expf(b[j][i]) : 0.0f) * dot;
            if (c < p.cols) store8(y, c, p.cols, p.veco != 0, a[j]);
        }
    }
}

// ---- persistent, software-pipelined form of the warp-per-row kernel ------------------------------------
// Each warp walks rows r, r + W, r + 2W, ...; the raw 16-byte vectors of the NEXT row are requested before the current
// row is reduced, so every warp always has a row in flight (the plain kernel has nothing in flight while it reduces).
// Needs 16-byte aligned rows and cols % 8 == 0. A causal row only loads the vectors that contain visible columns.
__device__ __forceinline__ void unpack_raw(const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <int VPL, int OP>
__global__ void __launch_bounds__(kBlock) row_warp_pipe_kernel(const RowParams p) {
    constexpr bool kTwoInputs = (OP == OP_SOFTMAX_BW || OP == OP_LOG_SOFTMAX_BW);
    const int lane = threadIdx.x & 31;
    const int total_warps = gridDim.x * (kBlock / kWarp);
    int r = blockIdx.x * (kBlock / kWarp) + (threadIdx.x >> 5);
    uint4 raw0[VPL], raw1[VPL];
    auto fetch = [&](int row, uint4 (&d0)[VPL], uint4 (&d1)[VPL]) {
        const int lim = kTwoInputs ? p.cols : visible_cols(p, row);
        const uint4* s0 = reinterpret_cast<const uint4*>(p.in0 + static_cast<size_t>(row) * p.ld0);
        const uint4* s1 = kTwoInputs ? reinterpret_cast<const uint4*>(p.in1 + static_cast<size_t>(row) * p.ld1) : nullptr;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int v = j * kWarp + lane;
            if (v * 8 < lim) {
                d0[j] = s0[v];
                if (kTwoInputs) d1[j] = s1[v];
            } else {
                d0[j] = make_uint4(0, 0, 0, 0);
                if (kTwoInputs) d1[j] = make_uint4(0, 0, 0, 0);
            }
        }
    };
    if (r < p.rows) fetch(r, raw0, raw1);
    while (r < p.rows) {
        const int r_next = r + total_warps;
        uint4 nxt0[VPL], nxt1[VPL];
        if (r_next < p.rows) fetch(r_next, nxt0, nxt1);
        float a[VPL][8];
        if (OP == OP_SOFTMAX || OP == OP_LOG_SOFTMAX || OP == OP_CROSS_ENTROPY) {
            const int vis = visible_cols(p, r);
            const float scale = (OP == OP_SOFTMAX) ? p.alpha : 1.0f;
            float m = -FLT_MAX;
#pragma unroll
            for (int j = 0; j < VPL; ++j) {
                const int c = (j * kWarp + lane) * 8;
                unpack_raw(raw0[j], a[j]);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    a[j][i] = (c + i < vis) ? a[j][i] * scale : -FLT_MAX;
                    m = fmaxf(m, a[j][i]);
                }
            }
            m = warp_max(m);
            float s = 0.0f;
#pragma unroll
            for (int j = 0; j < VPL; ++j)
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float e = (a[j][i] == -FLT_MAX) ? 0.0f : __expf(a[j][i] - m);
                    if (OP == OP_LOG_SOFTMAX) a[j][i] -= m; else a[j][i] = e;
                    s += e;
                }
            s = warp_sum(s);
            if (OP == OP_SOFTMAX || OP == OP_LOG_SOFTMAX) {
                const float inv = 1.0f / s, ls = __logf(s);
                uint4* y = reinterpret_cast<uint4*>(p.out + static_cast<size_t>(r) * p.ldo);
#pragma unroll
                for (int j = 0; j < VPL; ++j) {
                    const int v = j * kWarp + lane;
                    if (v * 8 >= p.cols) continue;
#pragma unroll
                    for (int i = 0; i < 8; ++i) a[j][i] = (OP == OP_SOFTMAX) ? a[j][i] * inv : a[j][i] - ls;
                    y[v] = make_uint4(pack_bf16x2(a[j][0], a[j][1]), pack_bf16x2(a[j][2], a[j][3]),
                                      pack_bf16x2(a[j][4], a[j][5]), pack_bf16x2(a[j][6], a[j][7]));
                }
            } else {  // cross-entropy
                const int label = static_cast<int>(p.labels[r]);
                const float inv = 1.0f / s;
                float picked = 0.0f;
                uint4* y = p.out ? reinterpret_cast<uint4*>(p.out + static_cast<size_t>(r) * p.ldo) : nullptr;
#pragma unroll
                for (int j = 0; j < VPL; ++j) {
                    const int v = j * kWarp + lane;
                    const int c = v * 8;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float prob = a[j][i] * inv;
                        if (c + i == label) picked = prob;
                        a[j][i] = (prob - ((c + i == label) ? 1.0f : 0.0f)) * p.alpha;
                    }
                    if (y != nullptr && c < p.cols)
                        y[v] = make_uint4(pack_bf16x2(a[j][0], a[j][1]), pack_bf16x2(a[j][2], a[j][3]),
                                          pack_bf16x2(a[j][4], a[j][5]), pack_bf16x2(a[j][6], a[j][7]));
                }
                picked = warp_sum(picked);
                if (lane == 0) {
                    const float loss = -__logf(fmaxf(picked, 1e-38f));
                    if (p.row_loss) p.row_loss[r] = loss;
                    if (p.loss_sum) atomicAdd(p.loss_sum, loss * p.alpha);
                }
            }
        } else {
            float b[VPL][8];
            float dot = 0.0f;
#pragma unroll
            for (int j = 0; j < VPL; ++j) {
                unpack_raw(raw0[j], a[j]);
                unpack_raw(raw1[j], b[j]);
#pragma unroll
                for (int i = 0; i < 8; ++i) dot += (OP == OP_SOFTMAX_BW) ? a[j][i] * b[j][i] : a[j][i];
            }
            dot = warp_sum(dot);
            uint4* y = reinterpret_cast<uint4*>(p.out + static_cast<size_t>(r) * p.ldo);
#pragma unroll
            for (int j = 0; j < VPL; ++j) {
                const int v = j * kWarp + lane;
                if (v * 8 >= p.cols) continue;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    a[j][i] = (OP == OP_SOFTMAX_BW) ? p.alpha * b[j][i] * (a[j][i] - dot) : a[j][i] - __expf(b[j][i]) * dot;
                y[v] = make_uint4(pack_bf16x2(a[j][0], a[j][1]), pack_bf16x2(a[j][2], a[j][3]),
                                  pack_bf16x2(a[j][4], a[j][5]), pack_bf16x2(a[j][6], a[j][7]));
            }
        }
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            raw0[j] = nxt0[j];
            if (kTwoInputs) raw1[j] = nxt1[j];
        }
        r = r_next;
    }
}

// ---- one CTA per row, any length: online max/sum pass, then a write pass (re-read hits L2) -----------
template <int OP>
__global__ void __launch_bounds__(1024) row_block_kernel(const RowParams p) {
    __shared__ float sh[32];
    extern __shared__ uint4 srow[];  // p.stage_row: the row's full 16-byte vectors, so that HBM is read once
    const int r = blockIdx.x;
    const __nv_bfloat16* x0 = p.in0 + static_cast<size_t>(r) * p.ld0;
    const int nvec = (p.cols + 7) / 8;
    if (OP == OP_SOFTMAX || OP == OP_LOG_SOFTMAX || OP == OP_CROSS_ENTROPY) {
        const int vis = visible_cols(p, r);
        const float scale = (OP == OP_SOFTMAX) ? p.alpha : 1.0f;
        const bool stage = p.stage_row != 0;
        float m = -FLT_MAX, s = 0.0f;  // running max and sum of exp(x - m)
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
            float f[8];
            if (stage && v * 8 + 8 <= vis) {
                const uint4 u = reinterpret_cast<const uint4*>(x0)[v];
                srow[v] = u;
                unpack_raw(u, f);
            } else {
                load8(x0, v * 8, vis, p.vec0 != 0, -FLT_MAX, f);
            }
            float lm = m;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                f[i] = (v * 8 + i < vis) ? f[i] * scale : -FLT_MAX;
                lm = fmaxf(lm, f[i]);
            }
            if (lm > m) {
                s *= __expf(m - lm);
                m = lm;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) s += (f[i] == -FLT_MAX) ? 0.0f : __expf(f[i] - m);
        }
        const float gm = block_max(m, sh);
        s = (m == -FLT_MAX) ? 0.0f : s * __expf(m - gm);
        const float gs = block_sum(s, sh);
        const float inv = 1.0f / gs, ls = __logf(gs);
        const int label = (OP == OP_CROSS_ENTROPY) ? static_cast<int>(p.labels[r]) : -1;
        float picked = 0.0f;
        __nv_bfloat16* y = p.out ? p.out + static_cast<size_t>(r) * p.ldo : nullptr;
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
            float f[8];
            if (stage && v * 8 + 8 <= vis) {
                unpack_raw(srow[v], f);  // written by this same thread in the first pass
            } else {
                load8(x0, v * 8, vis, p.vec0 != 0, -FLT_MAX, f);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int c = v * 8 + i;
                const float xs = (c < vis) ? f[i] * scale : -FLT_MAX;
                const float e = (xs == -FLT_MAX) ? 0.0f : __expf(xs - gm);
                if (OP == OP_SOFTMAX) {
                    f[i] = e * inv;
                } else if (OP == OP_LOG_SOFTMAX) {
                    f[i] = xs - gm - ls;
                } else {
                    const float prob = e * inv;
                    if (c == label) picked = prob;
                    f[i] = (prob - ((c == label) ? 1.0f : 0.0f)) * p.alpha;
                }
            }
            if (y) store8(y, v * 8, p.cols, p.veco != 0, f);
        }
        if (OP == OP_CROSS_ENTROPY) {
            picked = block_sum(picked, sh);
            if (threadIdx.x == 0) {
                const float loss = -__logf(fmaxf(picked, 1e-38f));
                if (p.row_loss) p.row_loss[r] = loss;
                if (p.loss_sum) atomicAdd(p.loss_sum, loss * p.alpha);
            }
        }
    } else {
        const __nv_bfloat16* x1 = p.in1 + static_cast<size_t>(r) * p.ld1;
        float dot = 0.0f;
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
            float a[8], b[8];
            load8(x0, v * 8, p.cols, p.vec0 != 0, 0.0f, a);
            if (OP == OP_SOFTMAX_BW) load8(x1, v * 8, p.cols, p.vec1 != 0, 0.0f, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) dot += (OP == OP_SOFTMAX_BW) ? a[i] * b[i] : a[i];
        }
        dot = block_sum(dot, sh);
        __nv_bfloat16* y = p.out + static_cast<size_t>(r) * p.ldo;
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
            float a[8], b[8];
            load8(x0, v * 8, p.cols, p.vec0 != 0, 0.0f, a);
            load8(x1, v * 8, p.cols, p.vec1 != 0, 0.0f, b);
#pragma unroll
            for (int i = 0; i < 8; ++i)
                a[i] = (OP == OP_SOFTMAX_BW) ? p.alpha * b[i] * (a[i] - dot) : a[i] - __expf(b[i]) * dot;
            store8(y, v * 8, p.cols, p.veco != 0, a);
        }
    }
}

// Cross-entropy over long rows (a vocabulary), one CTA of 1024 threads per row, the row staged in shared memory:
//   pass 1  four 16-byte loads in flight per thread; the row goes to shared memory, running max
//   pass 2  e = exp(x - max) once per element, summed in fp32 and written back to shared memory as bf16
//   pass 3  d_logits = (e / sum - onehot) * alpha from shared memory, 16-byte stores
// One exponential per element instead of two (the special-function unit, not HBM, bounds the two-exponential form on a
// 50k vocabulary); the label's probability for the loss is computed in fp32 from the logit itself.
constexpr int kCeThreads = 1024;
__global__ void __launch_bounds__(kCeThreads, 2) cross_entropy_staged_kernel(const RowParams p) {
    __shared__ float sh[32];
    extern __shared__ uint4 srow[];
    const int r = blockIdx.x;
    const __nv_bfloat16* x0 = p.in0 + static_cast<size_t>(r) * p.ld0;
    const int cols = p.cols;
    const int full = cols / 8;            // whole vectors; a ragged tail of cols % 8 elements is handled by thread 0
    const int tail0 = full * 8;
    float m = -FLT_MAX;
    // four 16-byte loads in flight per thread (two CTAs of 1024 threads leave 32 registers per thread)
    for (int base = threadIdx.x; base < full; base += 4 * kCeThreads) {
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = base + u * kCeThreads;
            if (v < full) raw[u] = reinterpret_cast<const uint4*>(x0)[v];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = base + u * kCeThreads;
            if (v < full) {
                srow[v] = raw[u];
                float f[8];
                unpack_raw(raw[u], f);
#pragma unroll
                for (int i = 0; i < 8; ++i) m = fmaxf(m, f[i]);
            }
        }
    }
    float tail[8];
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            tail[i] = (tail0 + i < cols) ? __bfloat162float(x0[tail0 + i]) : -FLT_MAX;
            m = fmaxf(m, tail[i]);
        }
    }
    const float gm = block_max(m, sh);
    const int label = static_cast<int>(p.labels[r]);
    const float gm2 = gm * 1.4426950408889634f;
    float s = 0.0f;
    for (int v = threadIdx.x; v < full; v += kCeThreads) {
        float f[8];
        unpack_raw(srow[v], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            f[i] = exp2f(fmaf(f[i], 1.4426950408889634f, -gm2));
            s += f[i];
        }
        srow[v] = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
    }
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            tail[i] = (tail0 + i < cols) ? exp2f(fmaf(tail[i], 1.4426950408889634f, -gm2)) : 0.0f;
            s += tail[i];
        }
    }
    const float gs = block_sum(s, sh);
    const float inv = 1.0f / gs;
    if (threadIdx.x == 0) {
        const float xl = (label >= 0 && label < cols) ? __bfloat162float(x0[label]) : gm;
        const float loss = (gm - xl) + __logf(gs);   // -log(exp(xl - gm) / gs)
        if (p.row_loss) p.row_loss[r] = loss;
        if (p.loss_sum) atomicAdd(p.loss_sum, loss * p.alpha);
    }
    if (p.out == nullptr) return;
    __nv_bfloat16* y = p.out + static_cast<size_t>(r) * p.ldo;
    const float a_inv = inv * p.alpha;
    for (int v = threadIdx.x; v < full; v += kCeThreads) {
        float f[8];
        unpack_raw(srow[v], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] *= a_inv;
        if (label >= v * 8 && label < v * 8 + 8) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (v * 8 + i == label) f[i] -= p.alpha;
        }
        reinterpret_cast<uint4*>(y)[v] =
            make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
    }
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (tail0 + i < cols) y[tail0 + i] = __float2bfloat16_rn(tail[i] * a_inv - ((tail0 + i == label) ? p.alpha : 0.0f));
    }
}

template <int OP>
int launch_row_op(const RowParams& p, cudaStream_t stream) {
    if (p.rows == 0 || p.cols == 0) return B200_OK;
    constexpr bool kTwoInputs = (OP == OP_SOFTMAX_BW || OP == OP_LOG_SOFTMAX_BW);
    const bool pipe_ok = p.vec0 && (p.out == nullptr || p.veco) && (!kTwoInputs || p.vec1) && (p.cols % 8) == 0 &&
                         p.rows >= 4096;
    if (p.cols <= 1024 && pipe_ok) {
        // persistent warps: enough CTAs to fill every SM several times over, each warp streaming many rows
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const int blocks = std::min((p.rows + (kBlock / kWarp) - 1) / (kBlock / kWarp), sms * 6);
        if (p.cols <= 256)
            row_warp_pipe_kernel<1, OP><<<blocks, kBlock, 0, stream>>>(p);
        else if (p.cols <= 512)
            row_warp_pipe_kernel<2, OP><<<blocks, kBlock, 0, stream>>>(p);
        else
            row_warp_pipe_kernel<4, OP><<<blocks, kBlock, 0, stream>>>(p);
    } else if (p.cols <= 1024) {
        const int blocks = (p.rows + (kBlock / kWarp) - 1) / (kBlock / kWarp);
        if (p.cols <= 256)
            row_warp_kernel<1, OP><<<blocks, kBlock, 0, stream>>>(p);
        else if (p.cols <= 512)
            row_warp_kernel<2, OP><<<blocks, kBlock, 0, stream>>>(p);
        else
            row_warp_kernel<4, OP><<<blocks, kBlock, 0, stream>>>(p);
    } else {
        RowParams q = p;
        const size_t row_bytes = static_cast<size_t>((p.cols + 7) / 8) * 16;
        constexpr bool kForward = (OP == OP_SOFTMAX || OP == OP_LOG_SOFTMAX || OP == OP_CROSS_ENTROPY);
        q.stage_row = (kForward && p.vec0 && row_bytes <= 110 * 1024) ? 1 : 0;  // two CTAs per SM still fit
        const size_t smem = q.stage_row ? row_bytes : 0;
        if (OP == OP_CROSS_ENTROPY && q.stage_row && p.causal_period == 0 && (p.out == nullptr || p.veco) &&
            true) {
            B200_CUDA_TRY(cudaFuncSetAttribute(cross_entropy_staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024));
            B200_CUDA_TRY(cudaFuncSetAttribute(cross_entropy_staged_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                               cudaSharedmemCarveoutMaxShared));
            cross_entropy_staged_kernel<<<p.rows, kCeThreads, smem, stream>>>(q);
            B200_CUDA_TRY(cudaGetLastError());
            return B200_OK;
        }
        if (smem > 48 * 1024)  // per device function and device; cheap enough to repeat
            B200_CUDA_TRY(cudaFuncSetAttribute(row_block_kernel<OP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024));
        // a staged row allows two CTAs per SM: give each 1024 threads so the SM still has 64 warps in flight
        row_block_kernel<OP><<<p.rows, q.stage_row ? 1024 : kBlock, smem, stream>>>(q);
    }
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

inline int vec_ok(const void* p, long long ld) { return ((reinterpret_cast<uintptr_t>(p) & 15u) == 0 && (ld & 7) == 0) ? 1 : 0; }

int check_rows(const char* who, const void* a, long long lda, long long rows, long long cols) {
    B200_REQUIRE(rows >= 0 && cols >= 0, "%s: negative size", who);
    B200_REQUIRE(rows < (1ll << 31) && cols < (1ll << 31), "%s: size too large", who);
    if (rows == 0 || cols == 0) return B200_OK;
    B200_REQUIRE(a != nullptr, "%s: NULL buffer", who);
    B200_REQUIRE(lda >= cols, "%s: leading dimension %lld < cols %lld", who, lda, cols);
    return B200_OK;
}

// ---- LayerNorm -------------------------------------------------------------------------------------
// Forward: one warp per row for cols <= 2048 (row in registers), else one CTA per row.
template <int VPL>
__global__ void __launch_bounds__(kBlock, VPL <= 4 ? 3 : 2) layernorm_fw_warp_kernel(const __nv_bfloat16* x, long long ldx,
                                                                    const __nv_bfloat16* gamma, const __nv_bfloat16* beta,
                                                                    __nv_bfloat16* y, long long ldy, float* mean_out,
                                                                    float* rstd_out, int rows, int cols, float eps, int vx,
                                                                    int vy, int vg, const __nv_bfloat16* res, long long ldres,
                                                                    __nv_bfloat16* sum_out, long long ldsum, int vres) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (kBlock / kWarp) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const __nv_bfloat16* xr = x + static_cast<size_t>(r) * ldx;
    float a[VPL][8];
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const int c = (j * kWarp + lane) * 8;
        load8(xr, c, cols, vx != 0, 0.0f, a[j]);
        if (res != nullptr) {  // normalise x + res; the sum (rounded to bf16, as a separate add would) is also an output
            float rv[8];
            load8(res + static_cast<size_t>(r) * ldres, c, cols, vres != 0, 0.0f, rv);
#pragma unroll
            for (int i = 0; i < 8; ++i) a[j][i] = __bfloat162float(__float2bfloat16_rn(a[j][i] + rv[i]));
            if (c < cols) store8(sum_out + static_cast<size_t>(r) * ldsum, c, cols, vres != 0, a[j]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) s += a[j][i];
    }
    const float mean = warp_sum(s) / cols;
    float q = 0.0f;
#pragma unroll
    for (int j = 0; j < VPL; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float d = ((j * kWarp + lane) * 8 + i < cols) ? a[j][i] - mean : 0.0f;
            q += d * d;
        }
    const float rstd = rsqrtf(warp_sum(q) / cols + eps);
    if (lane == 0) {
        if (mean_out) mean_out[r] = mean;
        if (rstd_out) rstd_out[r] = rstd;
    }
    __nv_bfloat16* yr = y + static_cast<size_t>(r) * ldy;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const int c = (j * kWarp + lane) * 8;
        if (c >= cols) continue;
        float g[8], b[8];
        load8(gamma, c, cols, vg != 0, 1.0f, g);
        load8(beta, c, cols, vg != 0, 0.0f, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[j][i] = (a[j][i] - mean) * rstd * g[i] + b[i];
        store8(yr, c, cols, vy != 0, a[j]);
    }
}

__global__ void __launch_bounds__(kBlock) layernorm_fw_block_kernel(const __nv_bfloat16* x, long long ldx,
                                                                     const __nv_bfloat16* gamma, const __nv_bfloat16* beta,
                                                                     __nv_bfloat16* y, long long ldy, float* mean_out,
                                                                     float* rstd_out, int rows, int cols, float eps, int vx,
                                                                     int vy, int vg) {
    __shared__ float sh[kBlock / kWarp];
    const int r = blockIdx.x;
    const __nv_bfloat16* xr = x + static_cast<size_t>(r) * ldx;
    const int nvec = (cols + 7) / 8;
    float s = 0.0f;
    for (int v = threadIdx.x; v < nvec; v += kBlock) {
        float f[8];
        load8(xr, v * 8, cols, vx != 0, 0.0f, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) s += f[i];
    }
    const float mean = block_sum(s, sh) / cols;
    float q = 0.0f;
    for (int v = threadIdx.x; v < nvec; v += kBlock) {
        float f[8];
        load8(xr, v * 8, cols, vx != 0, 0.0f, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float d = (v * 8 + i < cols) ? f[i] - mean : 0.0f;
            q += d * d;
        }
    }
    const float rstd = rsqrtf(block_sum(q, sh) / cols + eps);
    if (threadIdx.x == 0) {
        if (mean_out) mean_out[r] = mean;
        if (rstd_out) rstd_out[r] = rstd;
    }
    __nv_bfloat16* yr = y + static_cast<size_t>(r) * ldy;
    for (int v = threadIdx.x; v < nvec; v += kBlock) {
        float f[8], g[8], b[8];
        load8(xr, v * 8, cols, vx != 0, 0.0f, f);
        load8(gamma, v * 8, cols, vg != 0, 1.0f, g);
        load8(beta, v * 8, cols, vg != 0, 0.0f, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = (f[i] - mean) * rstd * g[i] + b[i];
        store8(yr, v * 8, cols, vy != 0, f);
    }
}

// Backward, input gradient: dx = rstd * (g - mean(g) - xhat * mean(g * xhat)), g = dy * gamma. One warp per row
// (cols <= 2048) or one CTA per row.
template <int VPL>
__global__ void __launch_bounds__(kBlock, VPL <= 4 ? 3 : 2) layernorm_bw_dx_warp_kernel(const __nv_bfloat16* dy, long long lddy,
                                                                       const __nv_bfloat16* x, long long ldx,
                                                                       const __nv_bfloat16* gamma, const float* mean,
                                                                       const float* rstd, __nv_bfloat16* dx, long long lddx,
                                                                       int rows, int cols, int vdy, int vx, int vdx, int vg) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (kBlock / kWarp) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const float mu = mean[r], rs = rstd[r];
    float g[VPL][8], xh[VPL][8];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const int c = (j * kWarp + lane) * 8;
        float gm[8];
        load8(dy + static_cast<size_t>(r) * lddy, c, cols, vdy != 0, 0.0f, g[j]);
        load8(x + static_cast<size_t>(r) * ldx, c, cols, vx != 0, 0.0f, xh[j]);
        load8(gamma, c, cols, vg != 0, 0.0f, gm);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const bool in = c + i < cols;
            xh[j][i] = in ? (xh[j][i] - mu) * rs : 0.0f;
            g[j][i] = in ? g[j][i] * gm[i] : 0.0f;
            s1 += g[j][i];
            s2 += g[j][i] * xh[j][i];
        }
    }
    s1 = warp_sum(s1) / cols;
    s2 = warp_sum(s2) / cols;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const int c = (j * kWarp + lane) * 8;
        if (c >= cols) continue;
#pragma unroll
        for (int i = 0; i < 8; ++i) g[j][i] = rs * (g[j][i] - s1 - xh[j][i] * s2);
        store8(dx + static_cast<size_t>(r) * lddx, c, cols, vdx != 0, g[j]);
    }
}

// ---- fast paths: 16-byte aligned rows, cols % 8 == 0, cols <= 1024 ----------------------------------------------
__device__ __forceinline__ void unpack_bf16x8(const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float (&f)[8]) {
    return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

// Forward, one warp per row. Every load of the row (x, the residual, gamma, beta) is issued before the first use, so
// the two dependent warp reductions overlap the tail of the memory latency instead of following it.
template <int VPL>
__global__ void __launch_bounds__(kBlock, 3) layernorm_fw_vec_kernel(const __nv_bfloat16* x, long long ldx,
                                                                      const __nv_bfloat16* gamma, const __nv_bfloat16* beta,
                                                                      __nv_bfloat16* y, long long ldy, float* mean_out,
                                                                      float* rstd_out, int rows, int cols, float eps,
                                                                      const __nv_bfloat16* res, long long ldres,
                                                                      __nv_bfloat16* sum_out, long long ldsum) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (kBlock / kWarp) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    uint4 xv[VPL], rv[VPL], gv[VPL], bv[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const int c = (j * kWarp + lane) * 8;
        const bool in = c < cols;
        xv[j] = in ? *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * ldx + c) : zero;
        rv[j] = (in && res != nullptr) ? *reinterpret_cast<const uint4*>(res + static_cast<size_t>(r) * ldres + c) : zero;
        gv[j] = in ? *reinterpret_cast<const uint4*>(gamma + c) : zero;
        bv[j] = in ? *reinterpret_cast<const uint4*>(beta + c) : zero;
    }
    float a[VPL][8];
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const int c = (j * kWarp + lane) * 8;
        unpack_bf16x8(xv[j], a[j]);
        if (res != nullptr) {  // normalise x + res; the sum (rounded to bf16, as a separate add would) is also an output
            float rr[8];
            unpack_bf16x8(rv[j], rr);
#pragma unroll
            for (int i = 0; i < 8; ++i) a[j][i] += rr[i];
            const uint4 packed = pack_bf16x8(a[j]);
            unpack_bf16x8(packed, a[j]);
            if (c < cols) *reinterpret_cast<uint4*>(sum_out + static_cast<size_t>(r) * ldsum + c) = packed;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) s += a[j][i];
    }
    const float mean = warp_sum(s) / cols;
    float q = 0.0f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const bool in = (j * kWarp + lane) * 8 < cols;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float d = in ? a[j][i] - mean : 0.0f;
            q = fmaf(d, d, q);
        }
    }
    const float rstd = rsqrtf(warp_sum(q) / cols + eps);
    if (lane == 0) {
        if (mean_out) mean_out[r] = mean;
        if (rstd_out) rstd_out[r] = rstd;
    }
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const int c = (j * kWarp + lane) * 8;
        if (c >= cols) continue;
        float g[8], b[8];
        unpack_bf16x8(gv[j], g);
        unpack_bf16x8(bv[j], b);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[j][i] = fmaf((a[j][i] - mean) * rstd, g[i], b[i]);
        *reinterpret_cast<uint4*>(y + static_cast<size_t>(r) * ldy + c) = pack_bf16x8(a[j]);
    }
}

// Backward in one pass (see layernorm_bw_fused_warp_kernel below for the arithmetic), persistent grid, one warp per row
// at a time. The packed dy, x and upstream vectors of the NEXT row are requested before the current row is processed, so
// every warp has loads in flight all the time. gamma sits in shared memory as fp32. A lane only ever touches its own
// 8 * VPL columns, so the column sums for dgamma / dbeta (and of dx) stay in its registers over all rows of the warp; at
// the end every warp writes them to a shared-memory slab of its own, the CTA adds the slabs and issues one global atomic
// per column.
template <int VPL>
__global__ void __launch_bounds__(kBlock, 1) layernorm_bw_vec_kernel(
    const __nv_bfloat16* dy, long long lddy, const __nv_bfloat16* x, long long ldx, const __nv_bfloat16* gamma,
    const float* mean, const float* rstd, const __nv_bfloat16* upstream, long long ldup, __nv_bfloat16* dx, long long lddx,
    float* dgamma_out, float* dbeta_out, __nv_bfloat16* dx_colsum_out, int rows, int cols, float* stage, unsigned* ticket) {
    constexpr int WARPS = kBlock / kWarp;
    constexpr int W = VPL * kWarp * 8;
    extern __shared__ float ln_smem[];
    float* sgam = ln_smem;                 // [W]
    float* sag = sgam + W;                 // [WARPS][W]
    float* sab = sag + WARPS * W;          // [WARPS][W]
    float* sax = sab + WARPS * W;          // [WARPS][W]  column sums of the dx this kernel writes (when asked for)
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    for (int c = threadIdx.x; c < W; c += kBlock) sgam[c] = c < cols ? __bfloat162float(gamma[c]) : 0.0f;
    __syncthreads();
    float ag[VPL][8], ab[VPL][8], ax[VPL][8];
#pragma unroll
    for (int j = 0; j < VPL; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) ag[j][i] = ab[j][i] = ax[j][i] = 0.0f;
    float* my_ag = sag + warp * W;
    float* my_ab = sab + warp * W;
    float* my_ax = sax + warp * W;
    const bool colsum = dx_colsum_out != nullptr;
    const bool params = dgamma_out != nullptr || dbeta_out != nullptr;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const int stride = gridDim.x * WARPS;
    int r = blockIdx.x * WARPS + warp;
    uint4 dv[VPL], xv[VPL], uv[VPL];
    float mu = 0.0f, rs = 0.0f;
    auto fetch = [&](int row) {
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int c = (j * kWarp + lane) * 8;
            const bool in = c < cols && row < rows;
            dv[j] = in ? *reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * lddy + c) : zero;
            xv[j] = in ? *reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * ldx + c) : zero;
            uv[j] = (in && upstream != nullptr) ? *reinterpret_cast<const uint4*>(upstream + static_cast<size_t>(row) * ldup + c) : zero;
        }
        mu = row < rows ? mean[row] : 0.0f;
        rs = row < rows ? rstd[row] : 0.0f;
    };
    fetch(r);
    for (; r < rows; r += stride) {
        // move the current row out of the fetch registers, then request the next one
        uint4 cd[VPL], cx[VPL], cu[VPL];
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            cd[j] = dv[j];
            cx[j] = xv[j];
            cu[j] = uv[j];
        }
        const float cmu = mu, crs = rs;
        fetch(r + stride);
        float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int c = (j * kWarp + lane) * 8;
            if (c >= cols) continue;
            float d[8], xh[8];
            unpack_bf16x8(cd[j], d);
            unpack_bf16x8(cx[j], xh);
            const float4 g0 = *reinterpret_cast<const float4*>(sgam + c);
            const float4 g1 = *reinterpret_cast<const float4*>(sgam + c + 4);
            const float gm[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float xhat = (xh[i] - cmu) * crs;
                if (params) {
                    ab[j][i] += d[i];
                    ag[j][i] = fmaf(d[i], xhat, ag[j][i]);
                }
                const float gg = d[i] * gm[i];
                s1 += gg;
                s2 = fmaf(gg, xhat, s2);
            }
        }
        s1 = warp_sum(s1) / cols;
        s2 = warp_sum(s2) / cols;
        if (dx != nullptr) {
#pragma unroll
            for (int j = 0; j < VPL; ++j) {
                const int c = (j * kWarp + lane) * 8;
                if (c >= cols) continue;
                float d[8], xh[8], up[8], o[8];
                unpack_bf16x8(cd[j], d);
                unpack_bf16x8(cx[j], xh);
                unpack_bf16x8(cu[j], up);
                const float4 g0 = *reinterpret_cast<const float4*>(sgam + c);
                const float4 g1 = *reinterpret_cast<const float4*>(sgam + c + 4);
                const float gm[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float xhat = (xh[i] - cmu) * crs;
                    o[i] = crs * (d[i] * gm[i] - s1 - xhat * s2);
                    // the separate form rounds dx to bf16 before the add; keep that rounding
                    if (upstream != nullptr) o[i] = __bfloat162float(__float2bfloat16_rn(o[i])) + up[i];
                }
                const uint4 packed = pack_bf16x8(o);
                *reinterpret_cast<uint4*>(dx + static_cast<size_t>(r) * lddx + c) = packed;
                if (colsum) {  // sums of the rounded values, as a column reduction of the stored tensor would see them
                    float q[8];
                    unpack_bf16x8(packed, q);
#pragma unroll
                    for (int i = 0; i < 8; ++i) ax[j][i] += q[i];
                }
            }
        }
    }
    if (!params && !colsum) return;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const int c = (j * kWarp + lane) * 8;
        *reinterpret_cast<float4*>(my_ag + c) = make_float4(ag[j][0], ag[j][1], ag[j][2], ag[j][3]);
        *reinterpret_cast<float4*>(my_ag + c + 4) = make_float4(ag[j][4], ag[j][5], ag[j][6], ag[j][7]);
        *reinterpret_cast<float4*>(my_ab + c) = make_float4(ab[j][0], ab[j][1], ab[j][2], ab[j][3]);
        *reinterpret_cast<float4*>(my_ab + c + 4) = make_float4(ab[j][4], ab[j][5], ab[j][6], ab[j][7]);
        *reinterpret_cast<float4*>(my_ax + c) = make_float4(ax[j][0], ax[j][1], ax[j][2], ax[j][3]);
        *reinterpret_cast<float4*>(my_ax + c + 4) = make_float4(ax[j][4], ax[j][5], ax[j][6], ax[j][7]);
    }
    // CTA sums -> one of kLnCopies zero-initialised staging replicas (few CTAs collide on an address) -> the CTA that
    // arrives last adds the replicas, writes the outputs and leaves replicas and ticket at zero for the next launch.
    __shared__ int is_last;
    __syncthreads();
    float* mine = stage + (blockIdx.x % kLnCopies) * kLnRows * kLnMaxCols;
    // four columns per thread and one 16-byte reduction per row of the replica (cols is a multiple of 8 on this path)
    for (int c = threadIdx.x * 4; c < cols; c += kBlock * 4) {
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f), b = g, x = g;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float4 gw = *reinterpret_cast<const float4*>(sag + w * W + c);
            const float4 bw = *reinterpret_cast<const float4*>(sab + w * W + c);
            const float4 xw = *reinterpret_cast<const float4*>(sax + w * W + c);
            g.x += gw.x; g.y += gw.y; g.z += gw.z; g.w += gw.w;
            b.x += bw.x; b.y += bw.y; b.z += bw.z; b.w += bw.w;
            x.x += xw.x; x.y += xw.y; x.z += xw.z; x.w += xw.w;
        }
        if (params) {
            atomicAdd(reinterpret_cast<float4*>(mine + c), g);
            atomicAdd(reinterpret_cast<float4*>(mine + kLnMaxCols + c), b);
        }
        if (colsum) atomicAdd(reinterpret_cast<float4*>(mine + 2 * kLnMaxCols + c), x);
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int c = threadIdx.x; c < cols; c += kBlock) {
        float g = 0.0f, b = 0.0f, x = 0.0f;
#pragma unroll
        for (int k = 0; k < kLnCopies; ++k) {
            float* copy = stage + k * kLnRows * kLnMaxCols;
            g += __ldcg(copy + c);
            b += __ldcg(copy + kLnMaxCols + c);
            x += __ldcg(copy + 2 * kLnMaxCols + c);
            copy[c] = 0.0f;
            copy[kLnMaxCols + c] = 0.0f;
            copy[2 * kLnMaxCols + c] = 0.0f;
        }
        if (dgamma_out != nullptr) dgamma_out[c] = g;
        if (dbeta_out != nullptr) dbeta_out[c] = b;
        if (colsum) dx_colsum_out[c] = __float2bfloat16_rn(x);
    }
    if (threadIdx.x == 0) *ticket = 0u;
}

// Dynamic shared memory of layernorm_bw_vec_kernel<VPL>: gamma and the three per-warp accumulator slabs.
template <int VPL>
constexpr size_t ln_bw_vec_smem() {
    return sizeof(float) * (VPL * kWarp * 8) * (1 + 3 * (kBlock / kWarp));
}

// Backward in one pass for rows that fit a warp's registers: a persistent grid, one warp per row at a time.
//   dx      = rstd * (g - mean(g) - xhat * mean(g * xhat)),  g = dy * gamma   (+ `upstream`, when given: the gradient
//             that reaches the same tensor along the residual path, so that no separate add runs)
//   dgamma += sum_rows dy * xhat,  dbeta += sum_rows dy: every lane keeps fp32 partial sums for the columns it owns over
//             all the rows its warp visits; the warps of a CTA combine them in shared memory and the CTA adds one value
//             per column to the zero-initialised fp32 outputs.
template <int VPL>
__global__ void __launch_bounds__(kBlock, VPL <= 3 ? 2 : 1) layernorm_bw_fused_warp_kernel(
    const __nv_bfloat16* dy, long long lddy, const __nv_bfloat16* x, long long ldx, const __nv_bfloat16* gamma,
    const float* mean, const float* rstd, const __nv_bfloat16* upstream, long long ldup, __nv_bfloat16* dx, long long lddx,
    float* dgamma_acc, float* dbeta_acc, int rows, int cols, int vdy, int vx, int vdx, int vg, int vup) {
    constexpr int WARPS = kBlock / kWarp;
    __shared__ float red[WARPS][kWarp * 8 + 1];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    float gm[VPL][8];
    float ag[VPL][8], ab[VPL][8];
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        load8(gamma, (j * kWarp + lane) * 8, cols, vg != 0, 0.0f, gm[j]);
#pragma unroll
        for (int i = 0; i < 8; ++i) ag[j][i] = ab[j][i] = 0.0f;
    }
    const bool params = dgamma_acc != nullptr || dbeta_acc != nullptr;
    for (int r = blockIdx.x * WARPS + warp; r < rows; r += gridDim.x * WARPS) {
        const float mu = mean[r], rs = rstd[r];
        float g[VPL][8], xh[VPL][8];
        float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int c = (j * kWarp + lane) * 8;
            load8(dy + static_cast<size_t>(r) * lddy, c, cols, vdy != 0, 0.0f, g[j]);
            load8(x + static_cast<size_t>(r) * ldx, c, cols, vx != 0, 0.0f, xh[j]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const bool in = c + i < cols;
                xh[j][i] = in ? (xh[j][i] - mu) * rs : 0.0f;
                if (params) {
                    ab[j][i] += g[j][i];
                    ag[j][i] = fmaf(g[j][i], xh[j][i], ag[j][i]);
                }
                g[j][i] = in ? g[j][i] * gm[j][i] : 0.0f;
                s1 += g[j][i];
                s2 = fmaf(g[j][i], xh[j][i], s2);
            }
        }
        s1 = warp_sum(s1) / cols;
        s2 = warp_sum(s2) / cols;
        if (dx != nullptr) {
#pragma unroll
            for (int j = 0; j < VPL; ++j) {
                const int c = (j * kWarp + lane) * 8;
                if (c >= cols) continue;
                float up[8];
                if (upstream != nullptr) load8(upstream + static_cast<size_t>(r) * ldup, c, cols, vup != 0, 0.0f, up);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    g[j][i] = rs * (g[j][i] - s1 - xh[j][i] * s2);
                    // the separate form rounds dx to bf16 before the add; keep that rounding
                    if (upstream != nullptr) g[j][i] = __bfloat162float(__float2bfloat16_rn(g[j][i])) + up[i];
                }
                store8(dx + static_cast<size_t>(r) * lddx, c, cols, vdx != 0, g[j]);
            }
        }
    }
    if (!params) return;
    // combine the warps' partial sums: one column slab (32 lanes x 8 columns) at a time, dgamma then dbeta
#pragma unroll
    for (int which = 0; which < 2; ++which) {
        float* out = which == 0 ? dgamma_acc : dbeta_acc;
        if (out == nullptr) continue;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            __syncthreads();
#pragma unroll
            for (int i = 0; i < 8; ++i) red[warp][lane * 8 + i] = which == 0 ? ag[j][i] : ab[j][i];
            __syncthreads();
            // 256 threads, 256 columns of this slab: thread t sums column t over the warps
            const int t = threadIdx.x;
            const int c = j * kWarp * 8 + t;
            if (c < cols) {
                float a = 0.0f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) a += red[w][t];
                atomicAdd(&out[c], a);
            }
        }
    }
}

__global__ void __launch_bounds__(kBlock) layernorm_bw_dx_block_kernel(const __nv_bfloat16* dy, long long lddy,
                                                                        const __nv_bfloat16* x, long long ldx,
                                                                        const __nv_bfloat16* gamma, const float* mean,
                                                                        const float* rstd, __nv_bfloat16* dx, long long lddx,
                                                                        int rows, int cols, int vdy, int vx, int vdx, int vg) {
    __shared__ float sh[kBlock / kWarp];
    const int r = blockIdx.x;
    const float mu = mean[r], rs = rstd[r];
    const int nvec = (cols + 7) / 8;
    float s1 = 0.0f, s2 = 0.0f;
    for (int v = threadIdx.x; v < nvec; v += kBlock) {
        float g[8], xv[8], gm[8];
        load8(dy + static_cast<size_t>(r) * lddy, v * 8, cols, vdy != 0, 0.0f, g);
        load8(x + static_cast<size_t>(r) * ldx, v * 8, cols, vx != 0, 0.0f, xv);
        load8(gamma, v * 8, cols, vg != 0, 0.0f, gm);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (v * 8 + i < cols) {
                const float gg = g[i] * gm[i];
                s1 += gg;
                s2 += gg * (xv[i] - mu) * rs;
            }
        }
    }
    s1 = block_sum(s1, sh) / cols;
    s2 = block_sum(s2, sh) / cols;
    for (int v = threadIdx.x; v < nvec; v += kBlock) {
        float g[8], xv[8], gm[8];
        load8(dy + static_cast<size_t>(r) * lddy, v * 8, cols, vdy != 0, 0.0f, g);
        load8(x + static_cast<size_t>(r) * ldx, v * 8, cols, vx != 0, 0.0f, xv);
        load8(gamma, v * 8, cols, vg != 0, 0.0f, gm);
#pragma unroll
        for (int i = 0; i < 8; ++i) g[i] = rs * (g[i] * gm[i] - s1 - (xv[i] - mu) * rs * s2);
        store8(dx + static_cast<size_t>(r) * lddx, v * 8, cols, vdx != 0, g);
    }
}

// Backward, parameter gradients: dgamma[c] = sum_r dy[r,c] * xhat[r,c], dbeta[c] = sum_r dy[r,c].
// Each CTA owns 64 columns and a slab of rows; partial sums are combined with fp32 atomics into
// zero-initialised fp32 accumulators, which a second tiny kernel converts to bf16.
// VEC = 8: a thread owns 8 adjacent columns (16-byte loads); VEC = 1 for rows that are not 16-byte aligned.
template <int VEC>
__global__ void __launch_bounds__(256) layernorm_bw_param_kernel(const __nv_bfloat16* dy, long long lddy,
                                                                  const __nv_bfloat16* x, long long ldx, const float* mean,
                                                                  const float* rstd, float* dgamma_acc, float* dbeta_acc,
                                                                  int rows, int cols, int rows_per_cta) {
    __shared__ float sg[8][32][VEC + 1], sb[8][32][VEC + 1];
    const int lane_c = threadIdx.x & 31;
    const int c = (blockIdx.x * 32 + lane_c) * VEC;
    const int sub = threadIdx.x >> 5;  // 8 row lanes
    const int r0 = blockIdx.y * rows_per_cta;
    const int r1 = min(rows, r0 + rows_per_cta);
    float ag[VEC], ab[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) ag[k] = ab[k] = 0.0f;
    if (c < cols) {
        for (int r = r0 + sub; r < r1; r += 8) {
            float d[8], xv[8];
            if (VEC == 8) {
                load8(dy + static_cast<size_t>(r) * lddy, c, cols, true, 0.0f, d);
                load8(x + static_cast<size_t>(r) * ldx, c, cols, true, 0.0f, xv);
            } else {
                d[0] = __bfloat162float(dy[static_cast<size_t>(r) * lddy + c]);
                xv[0] = __bfloat162float(x[static_cast<size_t>(r) * ldx + c]);
            }
            const float mu = mean[r], rs = rstd[r];
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                ab[k] += d[k];
                ag[k] += d[k] * (xv[k] - mu) * rs;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        sg[sub][lane_c][k] = ag[k];
        sb[sub][lane_c][k] = ab[k];
    }
    __syncthreads();
    if (sub == 0 && c < cols) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            if (c + k >= cols) break;
            float g = 0.0f, b = 0.0f;
            for (int j = 0; j < 8; ++j) {
                g += sg[j][lane_c][k];
                b += sb[j][lane_c][k];
            }
            if (dgamma_acc) atomicAdd(&dgamma_acc[c + k], g);
            if (dbeta_acc) atomicAdd(&dbeta_acc[c + k], b);
        }
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_softmax(b200_ctx* ctx, const void* x, int64_t ldx, void* y, int64_t ldy, int64_t rows, int64_t cols, float alpha,
                 int64_t causal_period, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_softmax: ctx is NULL");
    int rc = check_rows("b200_softmax", x, ldx, rows, cols);
    if (rc == B200_OK) rc = check_rows("b200_softmax", y, ldy, rows, cols);
    if (rc != B200_OK) return rc;
    B200_REQUIRE(causal_period >= 0, "b200_softmax: causal_period must be >= 0");
    RowParams p{};
    p.in0 = static_cast<const __nv_bfloat16*>(x);
    p.out = static_cast<__nv_bfloat16*>(y);
    p.ld0 = ldx;
    p.ldo = ldy;
    p.rows = static_cast<int>(rows);
    p.cols = static_cast<int>(cols);
    p.alpha = alpha;
    p.causal_period = static_cast<int>(causal_period);
    p.vec0 = vec_ok(x, ldx);
    p.veco = vec_ok(y, ldy);
    DeviceScope scope(ctx->device);
    return launch_row_op<OP_SOFTMAX>(p, ctx->pick(stream));
}

int b200_log_softmax(b200_ctx* ctx, const void* x, int64_t ldx, void* y, int64_t ldy, int64_t rows, int64_t cols,
                     void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_log_softmax: ctx is NULL");
    int rc = check_rows("b200_log_softmax", x, ldx, rows, cols);
    if (rc == B200_OK) rc = check_rows("b200_log_softmax", y, ldy, rows, cols);
    if (rc != B200_OK) return rc;
    RowParams p{};
    p.in0 = static_cast<const __nv_bfloat16*>(x);
    p.out = static_cast<__nv_bfloat16*>(y);
    p.ld0 = ldx;
    p.ldo = ldy;
    p.rows = static_cast<int>(rows);
    p.cols = static_cast<int>(cols);
    p.alpha = 1.0f;
    p.vec0 = vec_ok(x, ldx);
    p.veco = vec_ok(y, ldy);
    DeviceScope scope(ctx->device);
    return launch_row_op<OP_LOG_SOFTMAX>(p, ctx->pick(stream));
}

static int row_backward(b200_ctx* ctx, const char* who, bool log_form, const void* dy, int64_t lddy, const void* y,
                        int64_t ldy, void* dx, int64_t lddx, int64_t rows, int64_t cols, float alpha, void* stream) {
    B200_REQUIRE(ctx != nullptr, "%s: ctx is NULL", who);
    int rc = check_rows(who, dy, lddy, rows, cols);
    if (rc == B200_OK) rc = check_rows(who, y, ldy, rows, cols);
    if (rc == B200_OK) rc = check_rows(who, dx, lddx, rows, cols);
    if (rc != B200_OK) return rc;
    RowParams p{};
    p.in0 = static_cast<const __nv_bfloat16*>(dy);
    p.in1 = static_cast<const __nv_bfloat16*>(y);
    p.out = static_cast<__nv_bfloat16*>(dx);
    p.ld0 = lddy;
    p.ld1 = ldy;
    p.ldo = lddx;
    p.rows = static_cast<int>(rows);
    p.cols = static_cast<int>(cols);
    p.alpha = alpha;
    p.vec0 = vec_ok(dy, lddy);
    p.vec1 = vec_ok(y, ldy);
    p.veco = vec_ok(dx, lddx);
    DeviceScope scope(ctx->device);
    return log_form ? launch_row_op<OP_LOG_SOFTMAX_BW>(p, ctx->pick(stream))
                    : launch_row_op<OP_SOFTMAX_BW>(p, ctx->pick(stream));
}

int b200_softmax_backward(b200_ctx* ctx, const void* dy, int64_t lddy, const void* y, int64_t ldy, void* dx, int64_t lddx,
                          int64_t rows, int64_t cols, float alpha, void* stream) {
    return row_backward(ctx, "b200_softmax_backward", false, dy, lddy, y, ldy, dx, lddx, rows, cols, alpha, stream);
}

int b200_log_softmax_backward(b200_ctx* ctx, const void* dy, int64_t lddy, const void* log_y, int64_t ldy, void* dx,
                              int64_t lddx, int64_t rows, int64_t cols, void* stream) {
    return row_backward(ctx, "b200_log_softmax_backward", true, dy, lddy, log_y, ldy, dx, lddx, rows, cols, 1.0f, stream);
}

int b200_cross_entropy(b200_ctx* ctx, const void* logits, int64_t ld, const uint32_t* labels, int64_t rows, int64_t classes,
                       float grad_scale, float* loss_sum, float* row_loss, void* d_logits, int64_t ldd, void* stream) {
    B200_REQUIRE(ctx != nullptr, "b200_cross_entropy: ctx is NULL");
    int rc = check_rows("b200_cross_entropy", logits, ld, rows, classes);
    if (rc != B200_OK) return rc;
    if (d_logits) {
        rc = check_rows("b200_cross_entropy", d_logits, ldd, rows, classes);
        if (rc != B200_OK) return rc;
    }
    if (rows == 0 || classes == 0) return B200_OK;
    B200_REQUIRE(labels != nullptr, "b200_cross_entropy: labels is NULL");
    RowParams p{};
    p.in0 = static_cast<const __nv_bfloat16*>(logits);
    p.out = static_cast<__nv_bfloat16*>(d_logits);
    p.ld0 = ld;
    p.ldo = ldd;
    p.rows = static_cast<int>(rows);
    p.cols = static_cast<int>(classes);
    p.alpha = grad_scale;
    p.labels = labels;
    p.row_loss = row_loss;
    p.loss_sum = loss_sum;
    p.vec0 = vec_ok(logits, ld);
    p.veco = d_logits ? vec_ok(d_logits, ldd) : 0;
    DeviceScope scope(ctx->device);
    if (loss_sum) B200_CUDA_TRY(cudaMemsetAsync(loss_sum, 0, sizeof(float), ctx->pick(stream)));
    return launch_row_op<OP_CROSS_ENTROPY>(p, ctx->pick(stream));
}

static int layernorm_forward_impl(const char* fn, b200_ctx* ctx, const void* x, int64_t ldx, const void* residual,
                                  int64_t ldres, void* sum_out, int64_t ldsum, const void* gamma, const void* beta, void* y,
                                  int64_t ldy, float* mean, float* rstd, int64_t rows, int64_t cols, float eps, void* stream) {
    B200_REQUIRE(ctx != nullptr, "%s: ctx is NULL", fn);
    int rc = check_rows(fn, x, ldx, rows, cols);
    if (rc == B200_OK) rc = check_rows(fn, y, ldy, rows, cols);
    if (rc == B200_OK && residual) rc = check_rows(fn, residual, ldres, rows, cols);
    if (rc == B200_OK && residual) rc = check_rows(fn, sum_out, ldsum, rows, cols);
    if (rc != B200_OK) return rc;
    if (rows == 0 || cols == 0) return B200_OK;
    B200_REQUIRE(gamma && beta, "%s: gamma or beta is NULL", fn);
    DeviceScope scope(ctx->device);
    cudaStream_t s = ctx->pick(stream);
    const auto* xp = static_cast<const __nv_bfloat16*>(x);
    const auto* gp = static_cast<const __nv_bfloat16*>(gamma);
    const auto* bp = static_cast<const __nv_bfloat16*>(beta);
    const auto* rp = static_cast<const __nv_bfloat16*>(residual);
    auto* sp = static_cast<__nv_bfloat16*>(sum_out);
    auto* yp = static_cast<__nv_bfloat16*>(y);
    const int r = static_cast<int>(rows), c = static_cast<int>(cols);
    if (residual != nullptr && c > 2048) {
        // rows too long for the register-resident kernel: add first, then normalise the sum
        const int64_t shape[4] = {1, 1, rows, cols};
        B200_REQUIRE(ldx == cols && ldres == cols && ldsum == cols, "%s: rows longer than 2048 must be contiguous", fn);
        rc = b200_binary(ctx, 0 /* add */, x, shape, residual, shape, sum_out, stream);
        if (rc != B200_OK) return rc;
        xp = sp;
        ldx = ldsum;
        rp = nullptr;
    }
    const int vx = vec_ok(xp, ldx), vy = vec_ok(y, ldy), vg = vec_ok(gamma, 8) & vec_ok(beta, 8);
    const int vres = rp ? (vec_ok(rp, ldres) & vec_ok(sp, ldsum)) : 0;
    const int blocks = (r + 7) / 8;
    if (c <= 1024 && (c % 8) == 0 && vx && vy && vg && (rp == nullptr || vres)) {
        if (c <= 512)
            layernorm_fw_vec_kernel<2><<<blocks, kBlock, 0, s>>>(xp, ldx, gp, bp, yp, ldy, mean, rstd, r, c, eps, rp, ldres, sp, ldsum);
        else if (c <= 768)
            layernorm_fw_vec_kernel<3><<<blocks, kBlock, 0, s>>>(xp, ldx, gp, bp, yp, ldy, mean, rstd, r, c, eps, rp, ldres, sp, ldsum);
        else
            layernorm_fw_vec_kernel<4><<<blocks, kBlock, 0, s>>>(xp, ldx, gp, bp, yp, ldy, mean, rstd, r, c, eps, rp, ldres, sp, ldsum);
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    }
    if (c <= 512)
        layernorm_fw_warp_kernel<2><<<blocks, kBlock, 0, s>>>(xp, ldx, gp, bp, yp, ldy, mean, rstd, r, c, eps, vx, vy, vg, rp, ldres, sp, ldsum, vres);
    else if (c <= 768)
        layernorm_fw_warp_kernel<3><<<blocks, kBlock, 0, s>>>(xp, ldx, gp, bp, yp, ldy, mean, rstd, r, c, eps, vx, vy, vg, rp, ldres, sp, ldsum, vres);
    else if (c <= 1024)
        layernorm_fw_warp_kernel<4><<<blocks, kBlock, 0, s>>>(xp, ldx, gp, bp, yp, ldy, mean, rstd, r, c, eps, vx, vy, vg, rp, ldres, sp, ldsum, vres);
    else if (c <= 2048)
        layernorm_fw_warp_kernel<8><<<blocks, kBlock, 0, s>>>(xp, ldx, gp, bp, yp, ldy, mean, rstd, r, c, eps, vx, vy, vg, rp, ldres, sp, ldsum, vres);
    else
        layernorm_fw_block_kernel<<<r, kBlock, 0, s>>>(xp, ldx, gp, bp, yp, ldy, mean, rstd, r, c, eps, vx, vy, vg);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_layernorm_forward(b200_ctx* ctx, const void* x, int64_t ldx, const void* gamma, const void* beta, void* y,
                           int64_t ldy, float* mean, float* rstd, int64_t rows, int64_t cols, float eps, void* stream) {
    return layernorm_forward_impl("b200_layernorm_forward", ctx, x, ldx, nullptr, 0, nullptr, 0, gamma, beta, y, ldy, mean,
                                  rstd, rows, cols, eps, stream);
}

int b200_add_layernorm_forward(b200_ctx* ctx, const void* x, int64_t ldx, const void* residual, int64_t ldres, void* sum_out,
                               int64_t ldsum, const void* gamma, const void* beta, void* y, int64_t ldy, float* mean,
                               float* rstd, int64_t rows, int64_t cols, float eps, void* stream) {
    B200_REQUIRE(residual != nullptr && sum_out != nullptr, "b200_add_layernorm_forward: residual or sum_out is NULL");
    return layernorm_forward_impl("b200_add_layernorm_forward", ctx, x, ldx, residual, ldres, sum_out, ldsum, gamma, beta, y,
                                  ldy, mean, rstd, rows, cols, eps, stream);
}

static int layernorm_backward_impl(const char* fn, b200_ctx* ctx, const void* dy, int64_t lddy, const void* x, int64_t ldx,
                                   const void* gamma, const float* mean, const float* rstd, const void* upstream,
                                   int64_t ldup, void* dx, int64_t lddx, float* dgamma_f32, float* dbeta_f32,
                                   void* dx_colsum_bf16, int64_t rows, int64_t cols, void* stream) {
    B200_REQUIRE(ctx != nullptr, "%s: ctx is NULL", fn);
    int rc = check_rows(fn, dy, lddy, rows, cols);
    if (rc == B200_OK) rc = check_rows(fn, x, ldx, rows, cols);
    if (rc == B200_OK && dx) rc = check_rows(fn, dx, lddx, rows, cols);
    if (rc == B200_OK && upstream) rc = check_rows(fn, upstream, ldup, rows, cols);
    if (rc != B200_OK) return rc;
    B200_REQUIRE(upstream == nullptr || dx != nullptr, "%s: upstream given without dx", fn);
    DeviceScope scope(ctx->device);
    cudaStream_t s = ctx->pick(stream);
    const int r = static_cast<int>(rows), c = static_cast<int>(cols);
    // the vector kernel writes dgamma / dbeta itself; every other path accumulates into zeroed outputs
    const bool vec_path = rows > 0 && c > 0 && c <= 1024 && (c % 8) == 0 && gamma != nullptr && vec_ok(dy, lddy) && vec_ok(x, ldx) &&
                          vec_ok(gamma, 8) && (dx == nullptr || vec_ok(dx, lddx)) && (upstream == nullptr || vec_ok(upstream, ldup)) &&
                          (dx != nullptr || dgamma_f32 || dbeta_f32);
    if (!vec_path) {
        if (dgamma_f32 && c > 0) B200_CUDA_TRY(cudaMemsetAsync(dgamma_f32, 0, sizeof(float) * c, s));
        if (dbeta_f32 && c > 0) B200_CUDA_TRY(cudaMemsetAsync(dbeta_f32, 0, sizeof(float) * c, s));
    }
    if (rows == 0 || cols == 0) {
        if (dx_colsum_bf16 && c > 0) B200_CUDA_TRY(cudaMemsetAsync(dx_colsum_bf16, 0, sizeof(__nv_bfloat16) * c, s));
        return B200_OK;
    }
    B200_REQUIRE(mean && rstd, "%s: mean or rstd is NULL", fn);
    const auto* dyp = static_cast<const __nv_bfloat16*>(dy);
    const auto* xp = static_cast<const __nv_bfloat16*>(x);
    const auto* upp = static_cast<const __nv_bfloat16*>(upstream);
    auto* dxp = static_cast<__nv_bfloat16*>(dx);
    auto* csp = static_cast<__nv_bfloat16*>(dx_colsum_bf16);
    B200_REQUIRE(dx_colsum_bf16 == nullptr || dx != nullptr, "%s: column sums of dx requested without dx", fn);
    // Paths other than the vector kernel take the column sums of dx with a reduction over the finished tensor.
    auto colsum_fallback = [&]() -> int {
        if (dx_colsum_bf16 == nullptr) return B200_OK;
        B200_REQUIRE(lddx == cols, "%s: column sums of dx need contiguous rows on this path", fn);
        return b200_reduce(ctx, 0 /* sum */, dx, 1, rows, cols, dx_colsum_bf16, stream);
    };
    if (c <= 1024 && gamma != nullptr && (dx != nullptr || dgamma_f32 || dbeta_f32)) {
        // one pass: dx, the residual add and the parameter gradients
        const auto* gp = static_cast<const __nv_bfloat16*>(gamma);
        const int vdy = vec_ok(dy, lddy), vx = vec_ok(x, ldx), vdx = dx ? vec_ok(dx, lddx) : 0, vg = gamma ? vec_ok(gamma, 8) : 0;
        const int vup = upstream ? vec_ok(upstream, ldup) : 0;
        const int blocks = std::max(1, std::min((r + 7) / 8, ctx->sm_count * (vec_path ? 1 : 2)));
        {   // the staging rows and the ticket are one set per context: keep users on different streams apart
            int rc_o = order_shared_state(ctx, s);
            if (rc_o != B200_OK) return rc_o;
        }
        if (vec_path) {
            static bool configured[64] = {};
            int dev = 0;
            B200_CUDA_TRY(cudaGetDevice(&dev));
            if (dev < 0 || dev >= 64 || !configured[dev]) {
                B200_CUDA_TRY(cudaFuncSetAttribute(layernorm_bw_vec_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ln_bw_vec_smem<2>()));
                B200_CUDA_TRY(cudaFuncSetAttribute(layernorm_bw_vec_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ln_bw_vec_smem<3>()));
                B200_CUDA_TRY(cudaFuncSetAttribute(layernorm_bw_vec_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ln_bw_vec_smem<4>()));
                // room for two CTAs per SM (the driver otherwise sizes the carve-out for one)
                B200_CUDA_TRY(cudaFuncSetAttribute(layernorm_bw_vec_kernel<2>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
                B200_CUDA_TRY(cudaFuncSetAttribute(layernorm_bw_vec_kernel<3>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
                B200_CUDA_TRY(cudaFuncSetAttribute(layernorm_bw_vec_kernel<4>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
                if (dev >= 0 && dev < 64) configured[dev] = true;
            }
            if (c <= 512)
                layernorm_bw_vec_kernel<2><<<blocks, kBlock, ln_bw_vec_smem<2>(), s>>>(dyp, lddy, xp, ldx, gp, mean, rstd, upp, ldup, dxp, lddx,
                                                                                       dgamma_f32, dbeta_f32, csp, r, c, ctx_ln_stage(ctx), ctx_tickets(ctx) + kTicketCount - 1);
            else if (c <= 768)
                layernorm_bw_vec_kernel<3><<<blocks, kBlock, ln_bw_vec_smem<3>(), s>>>(dyp, lddy, xp, ldx, gp, mean, rstd, upp, ldup, dxp, lddx,
                                                                                       dgamma_f32, dbeta_f32, csp, r, c, ctx_ln_stage(ctx), ctx_tickets(ctx) + kTicketCount - 1);
            else
                layernorm_bw_vec_kernel<4><<<blocks, kBlock, ln_bw_vec_smem<4>(), s>>>(dyp, lddy, xp, ldx, gp, mean, rstd, upp, ldup, dxp, lddx,
                                                                                       dgamma_f32, dbeta_f32, csp, r, c, ctx_ln_stage(ctx), ctx_tickets(ctx) + kTicketCount - 1);
            B200_CUDA_TRY(cudaGetLastError());
            return B200_OK;
        }
        if (c <= 512)
            layernorm_bw_fused_warp_kernel<2><<<blocks, kBlock, 0, s>>>(dyp, lddy, xp, ldx, gp, mean, rstd, upp, ldup, dxp, lddx,
                                                                        dgamma_f32, dbeta_f32, r, c, vdy, vx, vdx, vg, vup);
        else if (c <= 768)
            layernorm_bw_fused_warp_kernel<3><<<blocks, kBlock, 0, s>>>(dyp, lddy, xp, ldx, gp, mean, rstd, upp, ldup, dxp, lddx,
                                                                        dgamma_f32, dbeta_f32, r, c, vdy, vx, vdx, vg, vup);
        else
            layernorm_bw_fused_warp_kernel<4><<<blocks, kBlock, 0, s>>>(dyp, lddy, xp, ldx, gp, mean, rstd, upp, ldup, dxp, lddx,
                                                                        dgamma_f32, dbeta_f32, r, c, vdy, vx, vdx, vg, vup);
        B200_CUDA_TRY(cudaGetLastError());
        return colsum_fallback();
    }
    if (dx) {
        B200_REQUIRE(gamma != nullptr, "%s: gamma is NULL", fn);
        const auto* gp = static_cast<const __nv_bfloat16*>(gamma);
        const int vdy = vec_ok(dy, lddy), vx = vec_ok(x, ldx), vdx = vec_ok(dx, lddx), vg = vec_ok(gamma, 8);
        const int blocks = (r + 7) / 8;
        if (c <= 2048)
            layernorm_bw_dx_warp_kernel<8><<<blocks, kBlock, 0, s>>>(dyp, lddy, xp, ldx, gp, mean, rstd, dxp, lddx, r, c, vdy, vx, vdx, vg);
        else
            layernorm_bw_dx_block_kernel<<<r, kBlock, 0, s>>>(dyp, lddy, xp, ldx, gp, mean, rstd, dxp, lddx, r, c, vdy, vx, vdx, vg);
        B200_CUDA_TRY(cudaGetLastError());
        if (upstream) {
            const int64_t shape[4] = {1, 1, rows, cols};
            B200_REQUIRE(lddx == cols && ldup == cols, "%s: rows longer than 1024 must be contiguous when upstream is given", fn);
            rc = b200_binary(ctx, 0 /* add */, dx, shape, upstream, shape, dx, stream);
            if (rc != B200_OK) return rc;
        }
    }
    if (dgamma_f32 || dbeta_f32) {
        const bool vec8 = vec_ok(dy, lddy) && vec_ok(x, ldx) && (c % 8 == 0);
        const int col_blocks = vec8 ? (c / 8 + 31) / 32 : (c + 31) / 32;
        int row_blocks = std::max(1, std::min((r + 63) / 64, (ctx->sm_count * 4 + col_blocks - 1) / col_blocks));
        const int rows_per = (r + row_blocks - 1) / row_blocks;
        row_blocks = (r + rows_per - 1) / rows_per;
        dim3 grid(col_blocks, row_blocks);
        if (vec8)
            layernorm_bw_param_kernel<8><<<grid, 256, 0, s>>>(dyp, lddy, xp, ldx, mean, rstd, dgamma_f32, dbeta_f32, r, c, rows_per);
        else
            layernorm_bw_param_kernel<1><<<grid, 256, 0, s>>>(dyp, lddy, xp, ldx, mean, rstd, dgamma_f32, dbeta_f32, r, c, rows_per);
        B200_CUDA_TRY(cudaGetLastError());
    }
    return colsum_fallback();
}

int b200_layernorm_backward(b200_ctx* ctx, const void* dy, int64_t lddy, const void* x, int64_t ldx, const void* gamma,
                            const float* mean, const float* rstd, void* dx, int64_t lddx, float* dgamma_f32,
                            float* dbeta_f32, int64_t rows, int64_t cols, void* stream) {
    return layernorm_backward_impl("b200_layernorm_backward", ctx, dy, lddy, x, ldx, gamma, mean, rstd, nullptr, 0, dx, lddx,
                                   dgamma_f32, dbeta_f32, nullptr, rows, cols, stream);
}

int b200_layernorm_backward_full(b200_ctx* ctx, const void* dy, int64_t lddy, const void* x, int64_t ldx, const void* gamma,
                                 const float* mean, const float* rstd, const void* upstream, int64_t ldup, void* dx,
                                 int64_t lddx, float* dgamma_f32, float* dbeta_f32, void* dx_colsum_bf16, int64_t rows,
                                 int64_t cols, void* stream) {
    return layernorm_backward_impl("b200_layernorm_backward_full", ctx, dy, lddy, x, ldx, gamma, mean, rstd, upstream, ldup, dx,
                                   lddx, dgamma_f32, dbeta_f32, dx_colsum_bf16, rows, cols, stream);
}

int b200_layernorm_backward_add(b200_ctx* ctx, const void* dy, int64_t lddy, const void* x, int64_t ldx, const void* gamma,
                                const float* mean, const float* rstd, const void* upstream, int64_t ldup, void* dx,
                                int64_t lddx, float* dgamma_f32, float* dbeta_f32, int64_t rows, int64_t cols, void* stream) {
    B200_REQUIRE(upstream != nullptr && dx != nullptr, "b200_layernorm_backward_add: upstream or dx is NULL");
    return layernorm_backward_impl("b200_layernorm_backward_add", ctx, dy, lddy, x, ldx, gamma, mean, rstd, upstream, ldup, dx,
                                   lddx, dgamma_f32, dbeta_f32, nullptr, rows, cols, stream);
}

}  // extern "C"
