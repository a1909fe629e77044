// Fused attention for head dimension 64 on the sm_100a tensor cores (tcgen05.mma, accumulators in TMEM, operands
// brought in by TMA): forward with a running softmax, backward with recomputed probabilities. Neither pass writes an
// [S, S] matrix to memory. Replaces the matmul / scale / mask / softmax / matmul chain of
// autograd/traced/nn.hpp:164-192 (TracedCausalAttention) and transformer_train.hpp:54-70
// (SharedAttentionBuffers::attention_forward / attention_backward) of the reference.
//
// Tiles are 128 queries x 128 keys. A TMEM lane is one row of the accumulator; a warp reads the 32 lanes of its
// quarter (warp index mod 4), and several warps share a quarter by taking different columns. Both kernels are bound by
// their element-wise warps (exponentials, conversions, the latency of TMEM loads), not by the tensor pipe or by DRAM.
//
//   forward, one CTA per (batch, head, 128 queries), two CTAs per SM:
//     warp 0       TMA: Q once, the K tiles and the V tiles through two rings of two stages
//     warp 1       one thread issues every MMA: S_j = Q K_j^T and O_j = P_j V_j
//     warps 2-5    a thread owns one query row and all 128 keys of a key tile: exact row maximum, P = exp2(..) as bf16
//                  into shared memory (the 128-byte-swizzled K-major layout the P V product reads), running sum; the
//                  row's 64 output values live in registers and O_j is folded into them one tile late.
//   backward, one CTA per (batch, head, 128 keys), looping over the query tiles that see those keys:
//     warp 16      TMA and every MMA: S^T = K Q^T and dP^T = V dO^T of the NEXT query tile while the current one is
//                  evaluated; then dQ_i = dS K, dV += P^T dO, dK += dS^T Q
//     16 warps     a thread takes one row (key) and 32 columns (queries): P^T = exp(scale S^T - lse),
//                  dS^T = scale P^T (dP^T - rowsum(dO O)) into shared memory as bf16; the four warps of one column
//                  group (a different group every tile) move dQ_i from TMEM into fp32 staging boxes; dK, dV at the end
//     warp 17      one thread adds the staged dQ_i boxes to the fp32 accumulators with TMA reductions
//   The single [128 keys x 128 queries] dS^T tile in shared memory is read both as a K-major A operand (dK) and as an
//   MN-major A operand (dQ): the two readings share one physical layout.
//
// Every wait is bounded: when one runs out the CTA raises the context's status word, drains its copies and returns.
#include <algorithm>
#include <cmath>

#include "common.cuh"
#include "gemm_common.cuh"
#include "ptx.cuh"

namespace b200 {

using namespace ptx;

namespace {

constexpr int DH = 64;                    // head dimension
constexpr int BT = 128;                   // queries per tile and keys per tile
constexpr int TILE_BYTES = BT * DH * 2;   // a [128 x 64] bf16 tile, rows of 128 bytes
constexpr int PT_BYTES = BT * BT * 2;     // a [128 x 128] bf16 tile stored as two 64-column slabs of 16 KB
constexpr int UMMA_K = 16;
constexpr int BWD_COMPUTE_WARPS = 16;
constexpr int BWD_THREADS = (BWD_COMPUTE_WARPS + 2) * 32;   // + the TMA / MMA warp and the dQ store warp
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct Geom {
    int B, H, S;
    int causal;
    float scale;       // multiplies the raw scores
    float scale_log2;  // scale * log2(e)
};

struct Strided {
    __nv_bfloat16* ptr;
    long long sb, sh, ss;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Byte offset of the 16-byte unit `unit` (0..15, i.e. 8 bf16 columns each) of row `r` inside a [128 x 128] bf16 tile
// kept as two 128-byte-swizzled slabs of 64 columns.
__device__ __forceinline__ uint32_t pt_offset(int r, int unit) {
    return static_cast<uint32_t>((unit >> 3) * TILE_BYTES + r * 128 + (((unit & 7) ^ (r & 7)) << 4));
}

__device__ __forceinline__ void store_bf16x8(uint8_t* dst, const float* f) {
    *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                                                pack_bf16x2(f[6], f[7]));
}

// Two finite fp32 values to bf16x2, rounding to nearest by adding half a bf16 ulp to the bit pattern and keeping the
// upper half (ties move away from zero instead of to even: one pattern in 65536). The cvt instruction shares the
// special-function pipe with the exponentials, which the element-wise phases keep busy; these are integer adds.
__device__ __forceinline__ uint32_t pack_round_bf16x2(float lo, float hi) {
    return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
}

// Lets copies that were armed but never consumed land before the CTA's shared memory is released.
__device__ __forceinline__ void drain(uint64_t* bar, uint32_t parity) {
    const uint64_t t0 = globaltimer_ns();
    while (!mbar_try_wait(bar, parity)) {
        if (globaltimer_ns() - t0 > 100000000ull) break;
    }
}


// ------------------------------------------------------------------------------------------------------------------
// Forward
// ------------------------------------------------------------------------------------------------------------------
struct FwdParams {
    Geom g;
    Strided o;
    Strided o_lo;   // optional (ptr may be null): bf16(O - bf16(O)), what the rounding of O to bf16 drops
    float* lse;
    int* status;
};

constexpr int FWD_STAGES = 2;

// One CTA per (batch, head, 128-query tile), two CTAs per SM: the set-up, the first loads and the output epilogue of one
// CTA run under the key-tile loop of its neighbour. Roles by warp: warp 0 TMA (Q once, K tiles and V tiles through two
// rings of two stages), warp 1 one MMA-issuing thread, warps 2-5 softmax — a thread owns one query row and all 128 keys of
// a key tile. P is single-buffered (it is rewritten only after O_j-1 = P_j-1 V_j-1 has read it, which the softmax
// threads wait for anyway before they fold O_j-1), O is double-buffered in TMEM (S 128 columns, O_b 2 x 64).
constexpr int FWD_THREADS = 192;
constexpr int FWD_TMEM_COLS = 256;
constexpr int FWD_SMEM_USED = TILE_BYTES + 2 * FWD_STAGES * TILE_BYTES + PT_BYTES + 128;
// Two CTAs per SM have 2 * (FWD_SMEM + 1 KB the hardware reserves per CTA) <= 228 KB to share, which leaves no room for
// rounding the base up to 1024: the kernel relies on the base being 1024-aligned already (it is when the kernel has no
// static shared memory) and reports an error instead of running when it is not.
constexpr int FWD_SMEM = FWD_SMEM_USED;
static_assert(2 * (FWD_SMEM + 1024) <= 228 * 1024, "two forward CTAs must fit one SM");

__global__ void __launch_bounds__(FWD_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    if ((smem_u32(smem_raw) & 1023u) != 0) {  // uniform over the CTA; nothing has been set up yet
        if (threadIdx.x == 0) atomicExch(p.status, 1);
        return;
    }
    uint8_t* sQ = smem_raw;
    uint8_t* sK = sQ + TILE_BYTES;                        // FWD_STAGES tiles
    uint8_t* sV = sK + FWD_STAGES * TILE_BYTES;           // FWD_STAGES tiles
    uint8_t* sP = sV + FWD_STAGES * TILE_BYTES;           // [128 x 128] bf16
    uint64_t* q_full = reinterpret_cast<uint64_t*>(sP + PT_BYTES);
    uint64_t* k_full = q_full + 1;                        // FWD_STAGES
    uint64_t* k_empty = k_full + FWD_STAGES;              // FWD_STAGES
    uint64_t* v_full = k_empty + FWD_STAGES;              // FWD_STAGES
    uint64_t* v_empty = v_full + FWD_STAGES;              // FWD_STAGES
    uint64_t* s_full = v_empty + FWD_STAGES;              // S of a key tile is in TMEM
    uint64_t* p_ready = s_full + 1;                       // P is in shared memory and S has been read (4 arrivals)
    uint64_t* pv_full = p_ready + 1;                      // O_j is in TMEM and P_j has been read
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const Geom g = p.g;
    // The grid is [batch x head, query tile] with the first index running fastest and the tile index reversed: every
    // tile with the most key tiles is handed out before any lighter one.
    const int bh = blockIdx.x;
    const int b = bh / g.H;
    const int h = bh - b * g.H;
    const int n_q_all = (g.S + BT - 1) / BT;
    const int qt = static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y);
    const int n_kv = g.causal ? min(qt + 1, n_q_all) : n_q_all;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmV);
        mbar_init(q_full, 1);
        mbar_init(s_full, 1);
        mbar_init(p_ready, 4);
        mbar_init(pv_full, 1);
        for (int st = 0; st < FWD_STAGES; ++st) {
            mbar_init(&k_full[st], 1);
            mbar_init(&k_empty[st], 1);
            mbar_init(&v_full[st], 1);
            mbar_init(&v_empty[st], 1);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, FWD_TMEM_COLS);
        tmem_relinquish_alloc_permit();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int armed_k = 0, armed_v = 0;
            mbar_arrive_expect_tx(q_full, TILE_BYTES);
            tma_load_4d(sQ, &tmQ, q_full, 0, qt * BT, h, b);
            for (int j = 0; j < n_kv; ++j) {
                const int st = j % FWD_STAGES;
                const uint32_t reuse_parity = ((j / FWD_STAGES) - 1) & 1;
                if (j >= FWD_STAGES && !mbar_wait(&k_empty[st], reuse_parity, abort_flag)) break;
                mbar_arrive_expect_tx(&k_full[st], TILE_BYTES);
                tma_load_4d(sK + st * TILE_BYTES, &tmK, &k_full[st], 0, j * BT, h, b);
                armed_k = j + 1;
                if (j >= FWD_STAGES && !mbar_wait(&v_empty[st], reuse_parity, abort_flag)) break;
                mbar_arrive_expect_tx(&v_full[st], TILE_BYTES);
                tma_load_4d(sV + st * TILE_BYTES, &tmV, &v_full[st], 0, j * BT, h, b);
                armed_v = j + 1;
            }
            if (*abort_flag != 0) {  // let armed copies land before the shared memory is released
                drain(q_full, 0);
                for (int j = max(0, armed_k - FWD_STAGES); j < armed_k; ++j) drain(&k_full[j % FWD_STAGES], (j / FWD_STAGES) & 1);
                for (int j = max(0, armed_v - FWD_STAGES); j < armed_v; ++j) drain(&v_full[j % FWD_STAGES], (j / FWD_STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc_bf16_f32(BT, BT, 0u, 0u);   // Q (K-major) x K (K-major)
            constexpr uint32_t idesc_o = make_idesc_bf16_f32(BT, DH, 0u, 1u);   // P (K-major) x V (MN-major)
            static_assert(FWD_STAGES == 2, "the stage of key tile j is j & 1 below");
            const uint64_t d_q = make_smem_desc_sw128(smem_u32(sQ), 0, 1024);
            const uint64_t d_k[2] = {make_smem_desc_sw128(smem_u32(sK), 0, 1024), make_smem_desc_sw128(smem_u32(sK + TILE_BYTES), 0, 1024)};
            const uint64_t d_v[2] = {make_smem_desc_sw128(smem_u32(sV), BT * 128, 1024),
                                     make_smem_desc_sw128(smem_u32(sV + TILE_BYTES), BT * 128, 1024)};
            const uint64_t d_p = make_smem_desc_sw128(smem_u32(sP), 0, 1024);
            auto issue_s = [&](int j) {
                const uint64_t bb = (j & 1) ? d_k[1] : d_k[0];
#pragma unroll
                for (int k = 0; k < DH / UMMA_K; ++k) umma_f16_ss(tmem_base, d_q + 2 * k, bb + 2 * k, idesc_s, k > 0 ? 1u : 0u);
                umma_commit(s_full);
                umma_commit(&k_empty[j & 1]);
            };
            auto issue_pv = [&](int j) {
                const uint64_t vb = (j & 1) ? d_v[1] : d_v[0];
                const uint32_t dst = tmem_base + BT + (j & 1) * DH;
#pragma unroll
                for (int k = 0; k < BT / UMMA_K; ++k)
                    umma_f16_ss(dst, d_p + ((k >> 2) * (TILE_BYTES / 16) + (k & 3) * 2), vb + k * (UMMA_K * 128 / 16), idesc_o,
                                k > 0 ? 1u : 0u);
                umma_commit(pv_full);
                umma_commit(&v_empty[j & 1]);
            };
            bool ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(&k_full[0], 0, abort_flag);
            if (ok) {
                tcgen05_fence_after_sync();
                issue_s(0);
            }
            for (int j = 0; ok && j < n_kv; ++j) {
                ok = mbar_wait(p_ready, j & 1, abort_flag);
                if (!ok) break;
                if (j + 1 < n_kv) {
                    ok = mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag);
                    if (!ok) break;
                    tcgen05_fence_after_sync();
                    issue_s(j + 1);
                }
                ok = mbar_wait(&v_full[j & 1], (j >> 1) & 1, abort_flag);
                if (!ok) break;
                tcgen05_fence_after_sync();
                issue_pv(j);
            }
        }
    } else {
        const int quarter = warp & 3;          // the TMEM lane quarter a warp may read
        const int r = quarter * 32 + lane;     // row of the tile = TMEM lane
        const int row = qt * BT + r;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const uint32_t s_addr = lane_addr;
        const uint32_t o_addr = lane_addr + static_cast<uint32_t>(BT);
        const int limit = g.causal ? min(row, g.S - 1) : g.S - 1;  // last visible key of this row
        const float sl2 = g.scale_log2;
        float m = -INFINITY, l = 0.f, alpha = 0.f;
        float o[DH];
#pragma unroll
        for (int i = 0; i < DH; ++i) o[i] = 0.f;
        uint32_t va[32], vb[32];   // two TMEM reads in flight
        auto fold_pv = [&](int j, float a) {  // O = O * a + O_j
            tmem_ld_32x32b_x32(o_addr + (j & 1) * DH, va);
            tmem_ld_32x32b_x32(o_addr + (j & 1) * DH + 32, vb);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = fmaf(o[i], a, __uint_as_float(va[i]));
#pragma unroll
            for (int i = 0; i < 32; ++i) o[32 + i] = fmaf(o[32 + i], a, __uint_as_float(vb[i]));
        };
        bool ok = true;   // uniform over the warp
        for (int j = 0; ok && j < n_kv; ++j) {
            const bool got = mbar_wait(s_full, j & 1, abort_flag);
            ok = __all_sync(0xffffffffu, got);
            if (!ok) break;
            tcgen05_fence_after_sync();
            const int lim = limit - j * BT;      // index, within the tile, of the last visible key
            const bool masked = lim < BT - 1;
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            auto take_max = [&](const uint32_t* sv, int c) {
                if (!masked) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i <= lim) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
                }
            };
            tmem_ld_32x32b_x32(s_addr, va);
            tmem_ld_32x32b_x32(s_addr + 32, vb);
            tmem_ld_wait();
            take_max(va, 0);
            tmem_ld_32x32b_x32(s_addr + 64, va);
            take_max(vb, 1);
            tmem_ld_32x32b_x32(s_addr + 96, vb);
            tmem_ld_wait();
            take_max(va, 2);
            take_max(vb, 3);
            const float mx = fmaxf(m, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])));
            const float alpha_before = alpha;   // belongs to O_j-1, folded below
            alpha = ex2((m - mx) * sl2);        // 0 on the first tile (m = -inf)
            const float mb = mx * sl2;
            m = mx;
            if (j > 0) {
                // O_j-1 has read P_j-1 (the buffer about to be rewritten) and is in TMEM. Waiting here also keeps every
                // barrier at most one phase ahead of its waiter: O_j cannot be issued before P_j is handed over.
                const bool got_o = mbar_wait(pv_full, (j - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, got_o);
                if (!ok) break;
            }
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
            auto take_exp = [&](const uint32_t* sv, int c) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    float f[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const int i = u * 8 + e;
                        float pr = ex2(fmaf(__uint_as_float(sv[i]), sl2, -mb));
                        if (masked && c * 32 + i > lim) pr = 0.f;
                        rs4[e & 3] += pr;
                        f[e] = pr;
                    }
                    store_bf16x8(sP + pt_offset(r, c * 4 + u), f);
                }
            };
            take_exp(va, 2);
            tmem_ld_32x32b_x32(s_addr, va);
            take_exp(vb, 3);
            tmem_ld_32x32b_x32(s_addr + 32, vb);
            tmem_ld_wait();
            take_exp(va, 0);
            take_exp(vb, 1);
            l = l * alpha + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
            fence_proxy_async_smem();
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready);
            if (j > 0) {
                tcgen05_fence_after_sync();
                fold_pv(j - 1, alpha_before);
            }
        }
        if (ok && n_kv > 0) {
            const bool got = mbar_wait(pv_full, (n_kv - 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, got);
        }
        if (ok && n_kv > 0) {
            tcgen05_fence_after_sync();
            fold_pv(n_kv - 1, alpha);
            if (row < g.S) {
                const float inv = 1.f / l;
#pragma unroll
                for (int i = 0; i < DH; ++i) o[i] *= inv;
                uint8_t* dst = reinterpret_cast<uint8_t*>(p.o.ptr + b * p.o.sb + h * p.o.sh + static_cast<long long>(row) * p.o.ss);
#pragma unroll
                for (int u = 0; u < DH / 8; ++u) store_bf16x8(dst + u * 16, o + 8 * u);
                if (p.o_lo.ptr != nullptr) {
                    // what bf16 drops of O, for the backward pass's row term rowsum(dO * O)
#pragma unroll
                    for (int i = 0; i < DH; ++i) o[i] -= __bfloat162float(__float2bfloat16_rn(o[i]));
                    uint8_t* dst_lo = reinterpret_cast<uint8_t*>(p.o_lo.ptr + b * p.o_lo.sb + h * p.o_lo.sh +
                                                                 static_cast<long long>(row) * p.o_lo.ss);
#pragma unroll
                    for (int u = 0; u < DH / 8; ++u) store_bf16x8(dst_lo + u * 16, o + 8 * u);
                }
                p.lse[(static_cast<long long>(bh)) * g.S + row] = (m * sl2 + log2f(l)) * LN2;
            }
        }
    }

    tcgen05_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(p.status, 1);
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, FWD_TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------------------------
// Backward
// ------------------------------------------------------------------------------------------------------------------
struct BwdParams {
    Geom g;
    Strided dk, dv;
    const float* lse2;  // [B, H, S_pad]  lse * log2(e); +inf in the padding rows (probability 0)
    const float* dsc;   // [B, H, S_pad]  rowsum(dO * O) * scale; 0 in the padding rows
    int s_pad;          // S rounded up to whole tiles
    float* dq_acc;      // [B, H, S, 64] fp32, zeroed before the launch; or one such slab per key tile (dq_slabs)
    int dq_slabs;       // non-zero: key tile j stores dQ contributions into slab j (coordinate j * B * H + bh), no reduction
    int* status;
};

constexpr int BWD_TMEM_COLS = 512;  // S^T 0..127, dP^T 128..255, dK 256..319, dV 320..383, dQ_i 384..447
constexpr int DQ_BOX_BYTES = BT * 32 * 4;   // [128 queries x 32 fp32 columns], rows of 128 bytes
// K, V, Q x 2, dO x 2, P^T, dS^T, two dQ staging buffers of two boxes each, the per-query terms of two tiles, barriers.
// That is all of the 227 KB a CTA may have, with 896 bytes to spare for rounding the base up to 1024 (the kernel checks
// that this suffices).
constexpr int BWD_SMEM_USED = 6 * TILE_BYTES + 2 * PT_BYTES + 4 * DQ_BOX_BYTES + 2048 + 128;
constexpr int BWD_SMEM = 227 * 1024;
static_assert(BWD_SMEM_USED <= BWD_SMEM, "backward shared memory exceeds the per-CTA limit");

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const __grid_constant__ CUtensorMap tmdQ, const BwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
    if (pad + BWD_SMEM_USED > BWD_SMEM) {  // uniform over the CTA; nothing has been set up yet
        if (threadIdx.x == 0) atomicExch(p.status, 1);
        return;
    }
    uint8_t* smem = smem_raw + pad;
    uint8_t* sK = smem;
    uint8_t* sV = sK + TILE_BYTES;
    uint8_t* sQ = sV + TILE_BYTES;        // 2 stages
    uint8_t* sdO = sQ + 2 * TILE_BYTES;   // 2 stages
    uint8_t* sPT = sdO + 2 * TILE_BYTES;  // P^T   [keys x queries]
    uint8_t* sdST = sPT + PT_BYTES;       // dS^T  [keys x queries]
    uint8_t* sDQ = sdST + PT_BYTES;       // dQ_i as two swizzled [128 x 32] fp32 boxes on their way to the accumulators, x 2
    float* stat_s = reinterpret_cast<float*>(sDQ + 4 * DQ_BOX_BYTES);   // [column group][tile parity][lse2 | dsc][32]
    uint64_t* kv_full = reinterpret_cast<uint64_t*>(stat_s + 4 * 2 * 64);
    uint64_t* qdo_full = kv_full + 1;     // 2
    uint64_t* sdp_full = qdo_full + 2;    // S^T and dP^T of a tile are in TMEM
    uint64_t* pds_ready = sdp_full + 1;   // P^T and dS^T of a tile are in shared memory
    uint64_t* dq_full = pds_ready + 1;    // dQ_i is in TMEM
    uint64_t* acc_done = dq_full + 1;     // the dV and dK products of a tile have run
    uint64_t* sdp_free = acc_done + 1;    // S^T and dP^T of a tile are in registers: the next tile's may be written
    uint64_t* dq_staged = sdp_free + 1;   // dQ_i is in its staging boxes
    uint64_t* dq_free = dq_staged + 1;    // 2: the reduction that read a staging buffer has left it
    uint64_t* dq_read = dq_free + 2;      // dQ_i has left TMEM
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dq_read + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const Geom g = p.g;
    const int bh = blockIdx.x;
    const int b = bh / g.H;
    const int h = bh - b * g.H;
    const int jt = blockIdx.y;  // key tile; with the causal mask tile 0 has the most work, and every (batch, head) starts it first
    const int n_q = (g.S + BT - 1) / BT;
    const int i0 = g.causal ? jt : 0;
    const int n_it = n_q - i0;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmV);
        prefetch_tensormap(&tmdO);
        prefetch_tensormap(&tmdQ);
        mbar_init(kv_full, 1);
        mbar_init(&qdo_full[0], 1);
        mbar_init(&qdo_full[1], 1);
        mbar_init(sdp_full, 1);
        mbar_init(pds_ready, BWD_COMPUTE_WARPS);  // one arrival per warp
        mbar_init(dq_full, 1);
        mbar_init(acc_done, 1);
        mbar_init(sdp_free, BWD_COMPUTE_WARPS);
        mbar_init(dq_staged, 4);   // the four warps (one per TMEM lane quarter) whose turn it is
        mbar_init(dq_read, 4);
        mbar_init(&dq_free[0], 1);
        mbar_init(&dq_free[1], 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == BWD_COMPUTE_WARPS) {
        tmem_alloc(tmem_slot, BWD_TMEM_COLS);
        tmem_relinquish_alloc_permit();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == BWD_COMPUTE_WARPS) {
        if (lane == 0) {
            constexpr uint32_t idesc_nt = make_idesc_bf16_f32(BT, BT, 0u, 0u);  // both operands K-major, N = 128
            constexpr uint32_t idesc_kn = make_idesc_bf16_f32(BT, DH, 0u, 1u);  // A K-major, B MN-major, N = 64
            constexpr uint32_t idesc_mn = make_idesc_bf16_f32(BT, DH, 1u, 1u);  // A MN-major, B MN-major, N = 64
            int armed[2] = {0, 0};
            auto load_qdo = [&](int it) {
                const int st = it & 1;
                mbar_arrive_expect_tx(&qdo_full[st], 2 * TILE_BYTES);
                tma_load_4d(sQ + st * TILE_BYTES, &tmQ, &qdo_full[st], 0, (i0 + it) * BT, h, b);
                tma_load_4d(sdO + st * TILE_BYTES, &tmdO, &qdo_full[st], 0, (i0 + it) * BT, h, b);
                ++armed[st];
            };
            mbar_arrive_expect_tx(kv_full, 2 * TILE_BYTES);
            tma_load_4d(sK, &tmK, kv_full, 0, jt * BT, h, b);
            tma_load_4d(sV, &tmV, kv_full, 0, jt * BT, h, b);
            load_qdo(0);
            if (n_it > 1) load_qdo(1);
            bool ok = mbar_wait(kv_full, 0, abort_flag);
            const uint32_t ka = smem_u32(sK), va = smem_u32(sV), pta = smem_u32(sPT), dsa = smem_u32(sdST);
            auto issue_sdp = [&](int it) {   // S^T = K Q_i^T and dP^T = V dO_i^T
                const uint32_t qa = smem_u32(sQ + (it & 1) * TILE_BYTES);
                const uint32_t doa = smem_u32(sdO + (it & 1) * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < DH / UMMA_K; ++k)
                    umma_f16_ss(tmem_base, make_smem_desc_sw128(ka + k * 32, 0, 1024),
                                make_smem_desc_sw128(qa + k * 32, 0, 1024), idesc_nt, k > 0 ? 1u : 0u);
#pragma unroll
                for (int k = 0; k < DH / UMMA_K; ++k)
                    umma_f16_ss(tmem_base + 128, make_smem_desc_sw128(va + k * 32, 0, 1024),
                                make_smem_desc_sw128(doa + k * 32, 0, 1024), idesc_nt, k > 0 ? 1u : 0u);
                umma_commit(sdp_full);
            };
            if (ok) ok = mbar_wait(&qdo_full[0], 0, abort_flag);
            if (ok) {
                tcgen05_fence_after_sync();
                issue_sdp(0);
            }
            // The tensor core executes in issue order, and issuing a product takes about as long as the product before
            // it runs. So S^T and dP^T of tile i + 1 are issued as soon as the element-wise warps hold those of tile i in
            // registers, and run while the warps evaluate tile i; dQ_i, dV and dK follow when P^T and dS^T of tile i are in
            // shared memory, and run while the warps evaluate tile i + 1.
            for (int it = 0; ok && it < n_it; ++it) {
                const int st = it & 1;
                if (it + 1 < n_it) {
                    if (!mbar_wait(sdp_free, it & 1, abort_flag) ||
                        !mbar_wait(&qdo_full[(it + 1) & 1], ((it + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                    tcgen05_fence_after_sync();
                    issue_sdp(it + 1);
                }
                if (!mbar_wait(pds_ready, it & 1, abort_flag)) { ok = false; break; }
                if (it > 0 && !mbar_wait(dq_read, (it - 1) & 1, abort_flag)) { ok = false; break; }   // dQ_i-1 has left TMEM
                tcgen05_fence_after_sync();
                const uint32_t qa = smem_u32(sQ + st * TILE_BYTES);
                const uint32_t doa = smem_u32(sdO + st * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < BT / UMMA_K; ++k)   // dQ_i = dS K (reduction over the 128 keys)
                    umma_f16_ss(tmem_base + 384, make_smem_desc_sw128(dsa + k * (UMMA_K * 128), BT * 128, 1024),
                                make_smem_desc_sw128(ka + k * (UMMA_K * 128), BT * 128, 1024), idesc_mn, k > 0 ? 1u : 0u);
                umma_commit(dq_full);
#pragma unroll
                for (int k = 0; k < BT / UMMA_K; ++k)   // dV += P^T dO   (reduction over the 128 queries)
                    umma_f16_ss(tmem_base + 320, make_smem_desc_sw128(pta + (k >> 2) * TILE_BYTES + (k & 3) * 32, 0, 1024),
                                make_smem_desc_sw128(doa + k * (UMMA_K * 128), BT * 128, 1024), idesc_kn,
                                (it > 0 || k > 0) ? 1u : 0u);
#pragma unroll
                for (int k = 0; k < BT / UMMA_K; ++k)   // dK += dS^T Q
                    umma_f16_ss(tmem_base + 256, make_smem_desc_sw128(dsa + (k >> 2) * TILE_BYTES + (k & 3) * 32, 0, 1024),
                                make_smem_desc_sw128(qa + k * (UMMA_K * 128), BT * 128, 1024), idesc_kn,
                                (it > 0 || k > 0) ? 1u : 0u);
                umma_commit(acc_done);
                if (it + 2 < n_it) {
                    if (!mbar_wait(acc_done, it & 1, abort_flag)) { ok = false; break; }  // Q_i, dO_i no longer read
                    load_qdo(it + 2);
                }
            }
            if (!ok) {
                if (armed[0]) drain(&qdo_full[0], (armed[0] - 1) & 1);
                if (armed[1]) drain(&qdo_full[1], (armed[1] - 1) & 1);
                drain(kv_full, 0);
            }
        }
    } else if (warp == BWD_COMPUTE_WARPS + 1) {
        // dQ_i leaves through one thread of a warp of its own: issuing the two reductions takes this thread a microsecond
        // or so, which the element-wise warps would otherwise spend at a barrier.
        if (lane == 0) {
            for (int it = 0; it < n_it; ++it) {
                if (!mbar_wait(dq_staged, it & 1, abort_flag)) break;
                const int st = it & 1;
                if (p.dq_slabs) {
                    const int slab_bh = jt * static_cast<int>(gridDim.x) + bh;
                    tma_store_3d(&tmdQ, sDQ + (st * 2) * DQ_BOX_BYTES, 0, (i0 + it) * BT, slab_bh);
                    tma_store_3d(&tmdQ, sDQ + (st * 2 + 1) * DQ_BOX_BYTES, 32, (i0 + it) * BT, slab_bh);
                } else {
                    tma_reduce_add_3d(&tmdQ, sDQ + (st * 2) * DQ_BOX_BYTES, 0, (i0 + it) * BT, bh);
                    tma_reduce_add_3d(&tmdQ, sDQ + (st * 2 + 1) * DQ_BOX_BYTES, 32, (i0 + it) * BT, bh);
                }
                tma_store_commit();
                if (it > 0) {   // the boxes of the tile before have been read: their buffer may be refilled
                    tma_store_wait_read<1>();
                    mbar_arrive(&dq_free[(it - 1) & 1]);
                }
            }
            tma_store_wait_all<0>();
        }
    } else {
        const int quarter = warp & 3;
        const int cg = warp >> 2;            // columns [32 * cg, +32) of S^T / dP^T; [16 * cg, +16) of dQ_i, dK, dV
        const int r = quarter * 32 + lane;   // TMEM lane: key row for S^T, dP^T, dK, dV; query row for dQ_i
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const float sl2 = g.scale_log2;
        bool ok = true;   // uniform over the warp
        // The element-wise warps meet only at mbarriers, each at its own pace: no CTA-wide barrier. dQ of a tile is moved
        // out of TMEM by the four warps of one column group, a different group for every tile, so that no warp is the
        // slow one twice in a row: TMEM -> two swizzled [128 x 32] fp32 boxes in shared memory, from where one TMA
        // reduction each adds them to the fp32 accumulators (rows beyond S are dropped by the tensor map).
        auto stage_dq = [&](int itd) {
            const int sd = itd & 1;
            const bool got_dq = mbar_wait(dq_full, itd & 1, abort_flag);
            ok = __all_sync(0xffffffffu, got_dq);
            if (ok && itd >= 2) {
                const bool got_buf = mbar_wait(&dq_free[sd], ((itd - 2) >> 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, got_buf);
            }
            if (!ok) return;
            tcgen05_fence_after_sync();
#pragma unroll
            for (int box = 0; box < 2; ++box) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(lane_addr + 384 + box * 32, v);
                tmem_ld_wait();
                uint8_t* box_row = sDQ + (sd * 2 + box) * DQ_BOX_BYTES + r * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<uint4*>(box_row + ((c ^ (r & 7)) << 4)) = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
            }
            fence_proxy_async_smem();
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(dq_read);
                mbar_arrive(dq_staged);
            }
        };
        // The per-query terms of the 32 queries of this column group reach the four warps that share them through
        // shared memory: each is requested from global memory a tile ahead by one lane (lanes of quarters 0 and 1),
        // written when the tile before has been evaluated, and published by a barrier of these four warps alone.
        const float* stat_src = (quarter == 0 ? p.lse2 : p.dsc) + static_cast<long long>(bh) * p.s_pad + cg * 32 + lane;
        float* stat_mine = stat_s + cg * 128;
        float stat_next = 0.f;
        if (quarter < 2) {
            stat_mine[quarter * 32 + lane] = stat_src[i0 * BT];
            if (n_it > 1) stat_next = stat_src[(i0 + 1) * BT];
        }
        for (int it = 0; it < n_it; ++it) {   // a warp that gave up keeps walking: its three siblings wait for it at the barrier
            const int i = i0 + it;
            asm volatile("bar.sync %0, 128;" ::"r"(1 + cg) : "memory");   // the terms of tile i are in shared memory
            if (ok) {
                const bool got = mbar_wait(sdp_full, it & 1, abort_flag);
                ok = __all_sync(0xffffffffu, got);
            }
            uint32_t pp[16], dd[16];   // P^T and dS^T of this thread's 32 queries as bf16 pairs
            if (ok) {
                tcgen05_fence_after_sync();
                const bool diag = g.causal && i == jt;  // query (column) c sees key (row) r only when c >= r
                uint32_t sv[32], dp[32];
                tmem_ld_32x32b_x32(lane_addr + cg * 32, sv);
                tmem_ld_32x32b_x32(lane_addr + 128 + cg * 32, dp);
                tmem_ld_wait();
                if (it + 1 < n_it) {   // both are in registers: the tensor core may write the next tile's
                    tcgen05_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(sdp_free);
                }
                const float4* l4 = reinterpret_cast<const float4*>(stat_mine + (it & 1) * 64);
                const float4* d4 = l4 + 8;
                // P^T = exp2(S^T scale log2 e - lse log2 e); dS^T = P^T (dP^T - rowsum) scale, with rowsum * scale staged
                auto evaluate = [&](auto masked_c) {
                    constexpr bool MASKED = decltype(masked_c)::value;
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        float pf[8], df[8];
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const float4 lv = l4[t * 2 + u];
                            const float4 dv = d4[t * 2 + u];
                            const float ls[4] = {lv.x, lv.y, lv.z, lv.w};
                            const float ds[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int idx = t * 8 + u * 4 + e;
                                float pr = ex2(fmaf(__uint_as_float(sv[idx]), sl2, -ls[e]));
                                if (MASKED && cg * 32 + idx < r) pr = 0.f;
                                pf[u * 4 + e] = pr;
                                df[u * 4 + e] = pr * fmaf(__uint_as_float(dp[idx]), g.scale, -ds[e]);
                            }
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            pp[t * 4 + e] = pack_bf16x2(pf[2 * e], pf[2 * e + 1]);
                            dd[t * 4 + e] = pack_bf16x2(df[2 * e], df[2 * e + 1]);
                        }
                    }
                };
                if (diag) evaluate(std::true_type{});
                else evaluate(std::false_type{});
            }
            if (ok && it > 0 && cg == ((it - 1) & 3)) stage_dq(it - 1);   // its product was issued a whole tile ago
            if (ok && it > 0) {   // so were the dV and dK products that read the P^T and dS^T about to be replaced
                const bool got_acc = mbar_wait(acc_done, (it - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, got_acc);
            }
            if (ok) {
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const uint32_t off = pt_offset(r, cg * 4 + t);
                    *reinterpret_cast<uint4*>(sPT + off) = make_uint4(pp[t * 4], pp[t * 4 + 1], pp[t * 4 + 2], pp[t * 4 + 3]);
                    *reinterpret_cast<uint4*>(sdST + off) = make_uint4(dd[t * 4], dd[t * 4 + 1], dd[t * 4 + 2], dd[t * 4 + 3]);
                }
                fence_proxy_async_smem();
                tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(pds_ready);
            }
            if (quarter < 2 && it + 1 < n_it) {
                stat_mine[((it + 1) & 1) * 64 + quarter * 32 + lane] = stat_next;
                if (it + 2 < n_it) stat_next = stat_src[(i + 2) * BT];
            }
        }
        if (ok && cg == ((n_it - 1) & 3)) stage_dq(n_it - 1);
        if (ok) {
            const bool got = mbar_wait(acc_done, (n_it - 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, got);
        }
        if (ok) {
            tcgen05_fence_after_sync();
            const int key = jt * BT + r;
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                const Strided& dst = which == 0 ? p.dk : p.dv;
                uint32_t v[16];
                tmem_ld_32x32b_x16(lane_addr + 256 + which * 64 + cg * 16, v);
                tmem_ld_wait();
                if (key < g.S) {
                    uint8_t* out = reinterpret_cast<uint8_t*>(dst.ptr + b * dst.sb + h * dst.sh + static_cast<long long>(key) * dst.ss +
                                                              cg * 16);
                    float f[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) f[e] = __uint_as_float(v[e]);
                    store_bf16x8(out, f);
                    store_bf16x8(out + 16, f + 8);
                }
            }
        }
    }

    tcgen05_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(p.status, 1);
    if (warp == BWD_COMPUTE_WARPS) {
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, BWD_TMEM_COLS);
    }
}

struct StridedIn {
    const __nv_bfloat16* ptr;
    long long sb, sh, ss;
};

// The per-query terms of the backward pass, padded to whole tiles so that the main kernel reads them without bounds
// checks: lse2 = lse * log2(e) and dsc = scale * sum_d dO * O (O = o + o_lo when the forward pass kept the low part).
// Eight threads per row, 8 elements each.
__global__ void attn_stats_kernel(StridedIn o, StridedIn o_lo, StridedIn d_o, const float* lse, float* lse2, float* dsc, int B,
                                  int H, int S, int s_pad, float scale) {
    const long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    const long long rowi = t >> 3;   // row of the padded [B, H, s_pad] arrays
    const int part = static_cast<int>(t & 7);
    const long long rows = static_cast<long long>(B) * H * s_pad;
    const int s = static_cast<int>(rowi % s_pad);
    const long long bhh = rowi / s_pad;
    const bool real = rowi < rows && s < S;
    float acc = 0.f;
    if (real) {
        const int h = static_cast<int>(bhh % H);
        const long long b = bhh / H;
        const uint4 ov = *reinterpret_cast<const uint4*>(o.ptr + b * o.sb + h * o.sh + s * o.ss + part * 8);
        const uint4 dv = *reinterpret_cast<const uint4*>(d_o.ptr + b * d_o.sb + h * d_o.sh + s * d_o.ss + part * 8);
        const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w};
        const uint32_t dw[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            acc = fmaf(__uint_as_float(ow[e] << 16), __uint_as_float(dw[e] << 16), acc);
            acc = fmaf(__uint_as_float(ow[e] & 0xffff0000u), __uint_as_float(dw[e] & 0xffff0000u), acc);
        }
        if (o_lo.ptr != nullptr) {
            const uint4 lv = *reinterpret_cast<const uint4*>(o_lo.ptr + b * o_lo.sb + h * o_lo.sh + s * o_lo.ss + part * 8);
            const uint32_t lw[4] = {lv.x, lv.y, lv.z, lv.w};
            float lo = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                lo = fmaf(__uint_as_float(lw[e] << 16), __uint_as_float(dw[e] << 16), lo);
                lo = fmaf(__uint_as_float(lw[e] & 0xffff0000u), __uint_as_float(dw[e] & 0xffff0000u), lo);
            }
            acc += lo;
        }
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    if (rowi < rows && part == 0) {
        lse2[rowi] = real ? lse[bhh * S + s] * LOG2E : INFINITY;
        dsc[rowi] = real ? acc * scale : 0.f;
    }
}

// fp32 dQ accumulators [B, H, S, 64] -> bf16 in the caller's layout. One thread per 8 elements.
// `slabs` = 0: acc is the accumulator. Otherwise acc holds one slab per key tile and the row's dQ is their sum in key
// order over the tiles that see the row (all of them, or those up to the row's own tile with the causal mask).
__global__ void attn_dq_store_kernel(const float* acc, Strided dq, int B, int H, int S, int slabs, int causal) {
    const long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    const long long rowi = t >> 3;
    const int part = static_cast<int>(t & 7);
    const long long rows = static_cast<long long>(B) * H * S;
    if (rowi >= rows) return;
    const int s = static_cast<int>(rowi % S);
    const long long bhh = rowi / S;
    const int h = static_cast<int>(bhh % H);
    const long long b = bhh / H;
    float4 a0 = *reinterpret_cast<const float4*>(acc + rowi * DH + part * 8);
    float4 a1 = *reinterpret_cast<const float4*>(acc + rowi * DH + part * 8 + 4);
    const int n_slabs = slabs == 0 ? 1 : (causal ? s / BT + 1 : slabs);
    for (int j = 1; j < n_slabs; ++j) {
        const float* src = acc + (static_cast<long long>(j) * rows + rowi) * DH + part * 8;
        const float4 c0 = *reinterpret_cast<const float4*>(src);
        const float4 c1 = *reinterpret_cast<const float4*>(src + 4);
        a0.x += c0.x; a0.y += c0.y; a0.z += c0.z; a0.w += c0.w;
        a1.x += c1.x; a1.y += c1.y; a1.z += c1.z; a1.w += c1.w;
    }
    *reinterpret_cast<uint4*>(dq.ptr + b * dq.sb + h * dq.sh + s * dq.ss + part * 8) =
        make_uint4(pack_bf16x2(a0.x, a0.y), pack_bf16x2(a0.z, a0.w), pack_bf16x2(a1.x, a1.y), pack_bf16x2(a1.z, a1.w));
}

// 4-D tensor map {64, S, H, B} over a strided bf16 operand; box = one [128 x 64] tile, 128-byte swizzle, rows beyond S
// read as zero.
int make_attn_map(b200_ctx* ctx, CUtensorMap* out, const b200_attn_operand& t, int64_t B, int64_t H, int64_t S,
                  const char* name) {
    cuuint64_t dims[4] = {DH, static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B)};
    // A dimension of extent 1 never contributes to an address; give it a well-formed stride whatever the caller passed.
    const int64_t sh = H > 1 ? t.stride_h : DH;
    const int64_t sb = B > 1 ? t.stride_b : DH;
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(t.stride_s) * 2, static_cast<cuuint64_t>(sh) * 2,
                             static_cast<cuuint64_t>(sb) * 2};
    cuuint32_t box[4] = {DH, BT, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = ctx->encode_tiled(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t.ptr, dims, strides, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for attention operand %s: ptr %p strides {%lld,%lld,%lld}",
                    static_cast<int>(r), name, t.ptr, (long long)t.stride_b, (long long)t.stride_h, (long long)t.stride_s);
    return B200_OK;
}

int check_operand(const b200_attn_operand* t, const char* name, int64_t B, int64_t H) {
    B200_REQUIRE(t != nullptr && t->ptr != nullptr, "attention: operand %s is NULL", name);
    B200_REQUIRE((reinterpret_cast<uintptr_t>(t->ptr) & 15u) == 0, "attention: operand %s is not 16-byte aligned", name);
    B200_REQUIRE(t->stride_s >= DH && (t->stride_s % 8) == 0, "attention: %s.stride_s must be >= 64 and a multiple of 8", name);
    B200_REQUIRE(H == 1 || (t->stride_h > 0 && (t->stride_h % 8) == 0), "attention: %s.stride_h must be a positive multiple of 8", name);
    B200_REQUIRE(B == 1 || (t->stride_b > 0 && (t->stride_b % 8) == 0), "attention: %s.stride_b must be a positive multiple of 8", name);
    return B200_OK;
}

int check_geometry(int64_t B, int64_t H, int64_t S, int head_dim, float scale) {
    if (head_dim != DH)
        return fail(B200_ERR_UNSUPPORTED, "attention: head_dim %d is not supported by the fused kernels (64 only)", head_dim);
    B200_REQUIRE(B >= 0 && H >= 0 && S >= 0, "attention: negative extent");
    B200_REQUIRE(B * H <= (1 << 24), "attention: batch * heads = %lld exceeds 2^24", (long long)(B * H));
    B200_REQUIRE(S <= (1 << 22), "attention: sequence length %lld exceeds 2^22", (long long)S);
    B200_REQUIRE(scale > 0.f && std::isfinite(scale), "attention: scale must be positive and finite");
    return B200_OK;
}

template <typename K>
int configure_once(K kernel, int smem_bytes, bool (&done)[64]) {
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !done[dev]) {
        B200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        // Without this the driver sizes the shared-memory carve-out for one CTA and a second one never fits.
        B200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                           cudaSharedmemCarveoutMaxShared));
        if (dev >= 0 && dev < 64) done[dev] = true;
    }
    return B200_OK;
}

Geom make_geom(int64_t B, int64_t H, int64_t S, float scale, int causal) {
    Geom g;
    g.B = static_cast<int>(B);
    g.H = static_cast<int>(H);
    g.S = static_cast<int>(S);
    g.causal = causal != 0;
    g.scale = scale;
    g.scale_log2 = scale * LOG2E;
    return g;
}

Strided as_out(const b200_attn_operand* t) {
    return Strided{static_cast<__nv_bfloat16*>(t->ptr), t->stride_b, t->stride_h, t->stride_s};
}

StridedIn as_in(const b200_attn_operand* t) {
    return StridedIn{static_cast<const __nv_bfloat16*>(t->ptr), t->stride_b, t->stride_h, t->stride_s};
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {


int b200_attention_forward(b200_ctx* ctx, const b200_attn_operand* q, const b200_attn_operand* k, const b200_attn_operand* v,
                           const b200_attn_operand* o, float* lse, int64_t B, int64_t H, int64_t S, int head_dim,
                           float scale, int causal, void* stream_v) {
    return b200_attention_forward_hp(ctx, q, k, v, o, nullptr, lse, B, H, S, head_dim, scale, causal, stream_v);
}

int b200_attention_forward_hp(b200_ctx* ctx, const b200_attn_operand* q, const b200_attn_operand* k, const b200_attn_operand* v,
                              const b200_attn_operand* o, const b200_attn_operand* o_lo, float* lse, int64_t B, int64_t H,
                              int64_t S, int head_dim, float scale, int causal, void* stream_v) {
    B200_REQUIRE(ctx != nullptr, "b200_attention_forward: ctx is NULL");
    int rc = check_geometry(B, H, S, head_dim, scale);
    if (rc != B200_OK) return rc;
    if (B == 0 || H == 0 || S == 0) return B200_OK;
    B200_REQUIRE(lse != nullptr, "b200_attention_forward: lse is NULL");
    if ((rc = check_operand(q, "q", B, H)) != B200_OK) return rc;
    if ((rc = check_operand(k, "k", B, H)) != B200_OK) return rc;
    if ((rc = check_operand(v, "v", B, H)) != B200_OK) return rc;
    if ((rc = check_operand(o, "o", B, H)) != B200_OK) return rc;
    if (o_lo != nullptr && (rc = check_operand(o_lo, "o_lo", B, H)) != B200_OK) return rc;
    DeviceScope scope(ctx->device);
    cudaStream_t stream = ctx->pick(stream_v);
    CUtensorMap tmQ, tmK, tmV;
    if ((rc = make_attn_map(ctx, &tmQ, *q, B, H, S, "q")) != B200_OK) return rc;
    if ((rc = make_attn_map(ctx, &tmK, *k, B, H, S, "k")) != B200_OK) return rc;
    if ((rc = make_attn_map(ctx, &tmV, *v, B, H, S, "v")) != B200_OK) return rc;
    FwdParams p;
    p.g = make_geom(B, H, S, scale, causal);
    p.o = as_out(o);
    p.o_lo = o_lo != nullptr ? as_out(o_lo) : Strided{nullptr, 0, 0, 0};
    p.lse = lse;
    p.status = ctx->d_status;
    static bool configured[64] = {};
    if ((rc = configure_once(attn_fwd_kernel, FWD_SMEM, configured)) != B200_OK) return rc;
    const int64_t q_tiles = (S + BT - 1) / BT;
    const dim3 grid(static_cast<unsigned>(B * H), static_cast<unsigned>(q_tiles));
    attn_fwd_kernel<<<grid, FWD_THREADS, FWD_SMEM, stream>>>(tmQ, tmK, tmV, p);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_attention_backward(b200_ctx* ctx, const b200_attn_operand* q, const b200_attn_operand* k,
                            const b200_attn_operand* v, const b200_attn_operand* o, const b200_attn_operand* d_o,
                            const float* lse, const b200_attn_operand* d_q, const b200_attn_operand* d_k,
                            const b200_attn_operand* d_v, int64_t B, int64_t H, int64_t S, int head_dim, float scale,
                            int causal, void* stream_v) {
    return b200_attention_backward_hp(ctx, q, k, v, o, nullptr, d_o, lse, d_q, d_k, d_v, B, H, S, head_dim, scale, causal,
                                      stream_v);
}

int b200_attention_backward_hp(b200_ctx* ctx, const b200_attn_operand* q, const b200_attn_operand* k,
                               const b200_attn_operand* v, const b200_attn_operand* o, const b200_attn_operand* o_lo,
                               const b200_attn_operand* d_o, const float* lse, const b200_attn_operand* d_q,
                               const b200_attn_operand* d_k, const b200_attn_operand* d_v, int64_t B, int64_t H, int64_t S,
                               int head_dim, float scale, int causal, void* stream_v) {
    return b200_attention_backward_opts(ctx, q, k, v, o, o_lo, d_o, lse, d_q, d_k, d_v, B, H, S, head_dim, scale, causal, 0u,
                                        stream_v);
}

int b200_attention_backward_opts(b200_ctx* ctx, const b200_attn_operand* q, const b200_attn_operand* k,
                                 const b200_attn_operand* v, const b200_attn_operand* o, const b200_attn_operand* o_lo,
                                 const b200_attn_operand* d_o, const float* lse, const b200_attn_operand* d_q,
                                 const b200_attn_operand* d_k, const b200_attn_operand* d_v, int64_t B, int64_t H, int64_t S,
                                 int head_dim, float scale, int causal, unsigned flags, void* stream_v) {
    B200_REQUIRE(ctx != nullptr, "b200_attention_backward: ctx is NULL");
    B200_REQUIRE((flags & ~B200_ATTN_DETERMINISTIC) == 0, "b200_attention_backward_opts: unknown flags 0x%x", flags);
    int rc = check_geometry(B, H, S, head_dim, scale);
    if (rc != B200_OK) return rc;
    if (B == 0 || H == 0 || S == 0) return B200_OK;
    B200_REQUIRE(lse != nullptr, "b200_attention_backward: lse is NULL");
    const b200_attn_operand* ops[8] = {q, k, v, o, d_o, d_q, d_k, d_v};
    const char* names[8] = {"q", "k", "v", "o", "d_o", "d_q", "d_k", "d_v"};
    for (int i = 0; i < 8; ++i)
        if ((rc = check_operand(ops[i], names[i], B, H)) != B200_OK) return rc;
    if (o_lo != nullptr && (rc = check_operand(o_lo, "o_lo", B, H)) != B200_OK) return rc;
    DeviceScope scope(ctx->device);
    cudaStream_t stream = ctx->pick(stream_v);
    const size_t rows = static_cast<size_t>(B) * H * S;
    const int64_t key_tiles = (S + BT - 1) / BT;
    const bool slabs = (flags & B200_ATTN_DETERMINISTIC) != 0 && key_tiles > 1;
    const size_t acc_bytes = rows * DH * sizeof(float) * (slabs ? key_tiles : 1);
    const int64_t s_pad = (S + BT - 1) / BT * BT;
    const size_t rows_pad = static_cast<size_t>(B) * H * s_pad;
    if ((rc = ensure_scratch(ctx, acc_bytes + 2 * rows_pad * sizeof(float), stream)) != B200_OK) return rc;
    float* dq_acc = static_cast<float*>(ctx->d_scratch);
    float* lse2 = dq_acc + acc_bytes / sizeof(float);   // 16-byte aligned: a multiple of 64 floats before it, and s_pad is a multiple of 128
    float* dsc = lse2 + rows_pad;
    CUtensorMap tmQ, tmK, tmV, tmdO;
    if ((rc = make_attn_map(ctx, &tmQ, *q, B, H, S, "q")) != B200_OK) return rc;
    if ((rc = make_attn_map(ctx, &tmK, *k, B, H, S, "k")) != B200_OK) return rc;
    if ((rc = make_attn_map(ctx, &tmV, *v, B, H, S, "v")) != B200_OK) return rc;
    if ((rc = make_attn_map(ctx, &tmdO, *d_o, B, H, S, "d_o")) != B200_OK) return rc;

    CUtensorMap tmdQ;
    {
        // fp32 accumulators [B*H, S, 64] as boxes of [128 rows x 32 columns] (128-byte rows, swizzled like the boxes in
        // shared memory); a box that reaches beyond row S of its (batch, head) slab is clipped there
        cuuint64_t dims[3] = {DH, static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(B * H * (slabs ? key_tiles : 1))};
        cuuint64_t strides[2] = {DH * sizeof(float), static_cast<cuuint64_t>(S) * DH * sizeof(float)};
        cuuint32_t box[3] = {32, BT, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = ctx->encode_tiled(&tmdQ, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, dq_acc, dims, strides, box, estr,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for the dQ accumulators", static_cast<int>(r));
    }
    // With the causal mask key tile j never writes the rows above its own tile in slab j, and the final sum never reads
    // them; every other part of every slab is stored to. The accumulator of the default form starts at zero.
    if (!slabs) B200_CUDA_TRY(cudaMemsetAsync(dq_acc, 0, acc_bytes, stream));
    const unsigned blocks = static_cast<unsigned>((rows * 8 + 255) / 256);
    const unsigned stat_blocks = static_cast<unsigned>((rows_pad * 8 + 255) / 256);
    attn_stats_kernel<<<stat_blocks, 256, 0, stream>>>(as_in(o), o_lo != nullptr ? as_in(o_lo) : StridedIn{nullptr, 0, 0, 0}, as_in(d_o),
                                                       lse, lse2, dsc, static_cast<int>(B), static_cast<int>(H), static_cast<int>(S),
                                                       static_cast<int>(s_pad), scale);
    B200_CUDA_TRY(cudaGetLastError());

    BwdParams p;
    p.g = make_geom(B, H, S, scale, causal);
    p.dk = as_out(d_k);
    p.dv = as_out(d_v);
    p.lse2 = lse2;
    p.dsc = dsc;
    p.s_pad = static_cast<int>(s_pad);
    p.dq_acc = dq_acc;
    p.dq_slabs = slabs ? 1 : 0;
    p.status = ctx->d_status;
    static bool configured[64] = {};
    if ((rc = configure_once(attn_bwd_kernel, BWD_SMEM, configured)) != B200_OK) return rc;
    const dim3 grid(static_cast<unsigned>(B * H), static_cast<unsigned>((S + BT - 1) / BT));
    attn_bwd_kernel<<<grid, BWD_THREADS, BWD_SMEM, stream>>>(tmQ, tmK, tmV, tmdO, tmdQ, p);
    B200_CUDA_TRY(cudaGetLastError());
    attn_dq_store_kernel<<<blocks, 256, 0, stream>>>(dq_acc, as_out(d_q), static_cast<int>(B), static_cast<int>(H),
                                                     static_cast<int>(S), slabs ? static_cast<int>(key_tiles) : 0, causal != 0);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // extern "C"
