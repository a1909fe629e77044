// bf16 x bf16 -> fp32-accumulate GEMM for sm_100a: TMA-fed shared-memory ring, tcgen05.mma with the
// accumulator in TMEM, warp-specialised persistent CTAs.
//
//   warp 0      : TMA producer (one elected lane) — fills a STAGES-deep ring of {A tile, B tile}
//   warp 1      : allocates TMEM; one elected lane issues tcgen05.mma for every 64-deep K block
//   warps 2..5  : epilogue — read the finished accumulator out of TMEM (tcgen05.ld), apply
//                 alpha / bias / causal mask / activation, convert and store to global memory
//
// The accumulator is double buffered in TMEM (2 x BLOCK_N fp32 columns) so the epilogue of tile i
// overlaps the main loop of tile i+1. One CTA per SM; CTA `x` handles work items x, x+grid, ...
//
// Operand layouts. op(A) is M x K and op(B) is K x N. An operand whose K index is contiguous in
// memory ("K-major": A stored [M,K], B stored [N,K]) is loaded as one box of 64 k x ROWS with the
// 128-byte swizzle. An operand whose M/N index is contiguous ("MN-major": A stored [K,M], B stored
// [K,N]) is loaded as ROWS/64 boxes of 64 mn x 64 k. tcgen05 reads both forms directly through the
// shared-memory descriptor, so NN, NT and TN products need no transposed copy.
//
// Ragged sizes: TMA zero-fills out-of-range box elements, so any M, N, K work; the epilogue
// predicates its stores. The leading dimensions and base addresses must be multiples of 16 bytes.
#include "gemm_common.cuh"
#include "ptx.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace b200 {

using namespace ptx;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int EPI_STAGE_BYTES = 4096;  // one 32-row x 128-byte staging box per epilogue warp and buffer

template <int BN>
struct TileCfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (BN >= 192) ? 4 : (BN == 128 ? 6 : 8);
    static constexpr int TMEM_COLS = BN == 192 ? 512 : 2 * BN;  // two accumulators; allocations are powers of two
    static constexpr int EPI_BYTES = 4 * 2 * EPI_STAGE_BYTES;  // 4 epilogue warps, double buffered
    static constexpr int BARRIER_BYTES = 256;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + BARRIER_BYTES + 1024;
};

struct WorkItem {
    int b, m0, n0, kb_begin, kb_end, split;
};

__device__ __forceinline__ WorkItem decode_work(const GemmParams& p, int w, int BN) {
    WorkItem it;
    const int tiles_mn = p.num_m_tiles * p.num_n_tiles;
    const int per_split = p.batch * tiles_mn;
    it.split = w / per_split;
    int r = w - it.split * per_split;
    it.b = r / tiles_mn;
    int t = r - it.b * tiles_mn;
    const int tiles_per_group = p.group_m * p.num_n_tiles;
    const int g = t / tiles_per_group;
    const int first_m = g * p.group_m;
    const int gsz = min(p.num_m_tiles - first_m, p.group_m);
    const int rr = t - g * tiles_per_group;
    int mi = first_m + rr % gsz + p.m_tile_rotate;
    if (mi >= p.num_m_tiles) mi -= p.num_m_tiles;
    const int ni = rr / gsz;
    it.m0 = mi * BM;
    it.n0 = ni * BN;
    it.kb_begin = it.split * p.kb_per_split;
    it.kb_end = min(p.num_kb, it.kb_begin + p.kb_per_split);
    return it;
}

// FP8: A and B hold one-byte e4m3 elements. A stage is the same 128 bytes of K per row (128 elements instead of 64),
// the 32-byte step between MMA K slices is the same (32 elements instead of 16); only the TMA K coordinate, the
// instruction kind and its descriptor differ. 8-bit operands exist K-major only.
template <int BN, bool A_KMAJOR, bool B_KMAJOR, bool FP8 = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CMaps tmC, const GemmParams p) {
    using Cfg = TileCfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    static_assert(!FP8 || (A_KMAJOR && B_KMAJOR), "8-bit operands are K-major only");
    constexpr int KB_ELEMS = FP8 ? 2 * BK : BK;  // elements of K per stage

    extern __shared__ uint8_t smem_raw[];
    // 128-byte-swizzled tiles must start on a 1024-byte boundary.
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* epi_smem = smem + STAGES * Cfg::STAGE_BYTES;  // 1024-byte aligned: stage sizes are multiples of 1024
    uint8_t* bar_base = epi_smem + Cfg::EPI_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_base);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tmem_full_bar = empty_bar + STAGES;
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmB);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tmem_full_bar[a], 1);
            mbar_init(&tmem_empty_bar[a], 4);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish_alloc_permit();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int w = blockIdx.x; ok && w < p.total_work; w += gridDim.x) {
                const WorkItem it = decode_work(p, w, BN);
                const int ab = p.a_batched ? it.b : 0;
                const int bb = p.b_batched ? it.b : 0;
                for (int kb = it.kb_begin; kb < it.kb_end; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sA = smem + stage * Cfg::STAGE_BYTES;
                    uint8_t* sB = sA + Cfg::A_BYTES;
                    mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
                    if (A_KMAJOR) {
                        tma_load_3d(sA, &tmA, &full_bar[stage], kb * KB_ELEMS, it.m0, ab);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j)
                            tma_load_3d(sA + j * (64 * BK * 2), &tmA, &full_bar[stage], it.m0 + 64 * j, kb * BK, ab);
                    }
                    if (B_KMAJOR) {
                        tma_load_3d(sB, &tmB, &full_bar[stage], kb * KB_ELEMS, it.n0, bb);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_3d(sB + j * (64 * BK * 2), &tmB, &full_bar[stage], it.n0 + 64 * j, kb * BK, bb);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                // Gave up: let every copy already issued land before the CTA's shared memory goes away.
                // A stage armed in the current pass completes phase `phase`, one from the pass before `phase ^ 1`.
                for (int s = 0; s < STAGES; ++s) {
                    const uint32_t par = (s < stage) ? phase : (phase ^ 1u);
                    const uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(&full_bar[s], par)) {
                        if (globaltimer_ns() - t0 > 100000000ull) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = FP8 ? make_idesc_e4m3_f32(BM, BN)
                                           : make_idesc_bf16_f32(BM, BN, A_KMAJOR ? 0u : 1u, B_KMAJOR ? 0u : 1u);
            // Byte step between consecutive 16-deep K slices inside a stage, and the descriptor strides.
            constexpr uint32_t A_KSTEP = A_KMAJOR ? (UMMA_K * 2) : (UMMA_K * 128);
            constexpr uint32_t B_KSTEP = B_KMAJOR ? (UMMA_K * 2) : (UMMA_K * 128);
            constexpr uint32_t A_LBO = A_KMAJOR ? 0u : (BK * 128);
            constexpr uint32_t B_LBO = B_KMAJOR ? 0u : (BK * 128);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int w = blockIdx.x; ok && w < p.total_work; w += gridDim.x) {
                const WorkItem it = decode_work(p, w, BN);
                if (!mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u, abort_flag)) break;
                tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
                for (int kb = it.kb_begin; kb < it.kb_end; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + stage * Cfg::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t da = make_smem_desc_sw128(a_addr + k * A_KSTEP, A_LBO, 1024);
                        const uint64_t db = make_smem_desc_sw128(b_addr + k * B_KSTEP, B_LBO, 1024);
                        if (FP8)
                            umma_f8_ss(d_tmem, da, db, idesc, (kb > it.kb_begin || k > 0) ? 1u : 0u);
                        else
                            umma_f16_ss(d_tmem, da, db, idesc, (kb > it.kb_begin || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                umma_commit(&tmem_full_bar[acc]);  // accumulator complete
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        int ebuf = 0;  // staging buffer the next TMA-store box uses
        uint8_t* stage_base = epi_smem + (warp - 2) * 2 * EPI_STAGE_BYTES;
        for (int w = blockIdx.x; w < p.total_work; w += gridDim.x) {
            const WorkItem it = decode_work(p, w, BN);
            const bool got = mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag);
            if (!__all_sync(0xffffffffu, got)) break;
            tcgen05_fence_after_sync();
            const int row = it.m0 + q * 32 + lane;
            const bool row_ok = row < p.M;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);

            if (p.k_splits > 1) {
                // fp32 partial sums, no epilogue math: [split][batch][M][N]
                float* prow = p.partial +
                              ((static_cast<size_t>(it.split) * p.batch + it.b) * p.M + (row_ok ? row : 0)) * p.N;
                const bool vec = (p.N & 3) == 0;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    const int n = it.n0 + c;
                    if (n >= p.N) break;
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c, v);
                    tmem_ld_wait();
                    if (p.partial_round_bf16) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            v[i] = __float_as_uint(__bfloat162float(__float2bfloat16_rn(__uint_as_float(v[i]))));
                    }
                    if (row_ok) {
                        if (vec && n + 32 <= p.N) {
                            float4* dst = reinterpret_cast<float4*>(prow + n);
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                dst[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                     __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (n + i < p.N) prow[n + i] = __uint_as_float(v[i]);
                        }
                    }
                }
            } else if (p.epi_mode == 1) {
                // Staged epilogue: each warp converts a 32-row x 128-byte box (64 bf16 or 32 fp32 columns) into
                // shared memory in the 128-byte-swizzled layout and one lane hands it to TMA, which writes full
                // lines, clips the ragged edges and can target several destination matrices (peer GPUs).
                const int box_cols = p.c_f32 ? 32 : 64;
                int dst_first = 0, dst_count = p.n_dst, row_coord = it.m0 + q * 32;
                if (p.scatter_rows > 0) {
                    dst_first = it.m0 / p.scatter_rows;
                    dst_count = 1;
                    row_coord -= dst_first * p.scatter_rows;
                }
                uint32_t nx0[32], nx1[32];
                tmem_ld_32x32b_x32(taddr, nx0);
                if (box_cols == 64 && it.n0 + 32 < p.N) tmem_ld_32x32b_x32(taddr + 32, nx1);
#pragma unroll 1
                for (int c = 0; c < BN; c += box_cols) {
                    const int n = it.n0 + c;
                    if (n >= p.N) break;
                    uint8_t* sbuf = stage_base + ebuf * EPI_STAGE_BYTES;
                    if (lane == 0) tma_store_wait_read<1>();  // the box stored two iterations ago has left this buffer
                    __syncwarp();
                    uint8_t* srow = sbuf + lane * 128;
                    // The TMEM loads of the NEXT box are in flight while this one is converted and staged.
                    tmem_ld_wait();
                    uint32_t v0[32], v1[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        v0[i] = nx0[i];
                        v1[i] = nx1[i];
                    }
                    {
                        const int cn = c + box_cols;
                        if (cn < BN && it.n0 + cn < p.N) {
                            tmem_ld_32x32b_x32(taddr + cn, nx0);
                            if (box_cols == 64 && it.n0 + cn + 32 < p.N) tmem_ld_32x32b_x32(taddr + cn + 32, nx1);
                        }
                    }
#pragma unroll 1
                    for (int h = 0; h * 32 < box_cols; ++h) {
                        const int nh = n + h * 32;
                        if (nh >= p.N) break;
                        uint32_t (&v)[32] = h == 0 ? v0 : v1;
                        float f[32];
                        epi_apply32(p.epi, v, f, row, nh, p.N);
                        if (p.c_f32) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                *reinterpret_cast<float4*>(srow + ((j ^ (lane & 7)) << 4)) =
                                    make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                *reinterpret_cast<uint4*>(srow + (((h * 4 + j) ^ (lane & 7)) << 4)) =
                                    make_uint4(pack_bf16x2(f[8 * j], f[8 * j + 1]), pack_bf16x2(f[8 * j + 2], f[8 * j + 3]),
                                               pack_bf16x2(f[8 * j + 4], f[8 * j + 5]), pack_bf16x2(f[8 * j + 6], f[8 * j + 7]));
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        for (int d = 0; d < dst_count; ++d) {
                            int di = d + p.dst_rotate;
                            if (di >= dst_count) di -= dst_count;
                            tma_store_3d(&tmC.m[dst_first + di], sbuf, n, row_coord, it.b);
                        }
                        tma_store_commit();
                    }
                    ebuf ^= 1;
                }
            } else {
                const size_t crow = static_cast<size_t>(it.b) * p.stride_c + static_cast<size_t>(row_ok ? row : 0) * p.ldc;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    const int n = it.n0 + c;
                    if (n >= p.N) break;
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c, v);
                    tmem_ld_wait();
                    const bool full = (n + 32 <= p.N);
                    float f[32];
                    epi_apply32(p.epi, v, f, row, n, p.N);
                    if (row_ok) {
                        if (p.c_f32) {
                            float* dst = static_cast<float*>(p.C) + crow + n;
                            if (full && p.c_vec_ok) {
                                float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    d4[i] = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
                            } else {
#pragma unroll
                                for (int i = 0; i < 32; ++i)
                                    if (n + i < p.N) dst[i] = f[i];
                            }
                        } else {
                            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.C) + crow + n;
                            if (full && p.c_vec_ok) {
                                uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
                                for (int i = 0; i < 4; ++i)
                                    d4[i] = make_uint4(pack_bf16x2(f[8 * i], f[8 * i + 1]), pack_bf16x2(f[8 * i + 2], f[8 * i + 3]),
                                                       pack_bf16x2(f[8 * i + 4], f[8 * i + 5]),
                                                       pack_bf16x2(f[8 * i + 6], f[8 * i + 7]));
                            } else {
#pragma unroll
                                for (int i = 0; i < 32; ++i)
                                    if (n + i < p.N) dst[i] = __float2bfloat16_rn(f[i]);
                            }
                        }
                    }
                }
            }
            // Hand the accumulator buffer back to the MMA warp.
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
        // Every TMA store of this warp must have completed before the CTA (and its shared memory) goes away.
        if (lane == 0) tma_store_wait_all<0>();
    }

    // ---------------------------------------------------------------------- teardown
    tcgen05_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(p.status, 1);
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// Sums the K slices, applies the epilogue and writes C. One thread per 4 consecutive columns; 16-byte loads of the
// partial sums and one 8- or 16-byte store when the addresses allow it, element by element otherwise.
__global__ void splitk_reduce_kernel(const GemmParams p) {
    const long long cols4 = (p.N + 3) / 4;
    const long long total = static_cast<long long>(p.batch) * p.M * cols4;
    const size_t slice = static_cast<size_t>(p.batch) * p.M * p.N;
    const bool vec_in = (p.N & 3) == 0 && (reinterpret_cast<uintptr_t>(p.partial) & 15u) == 0;
    const __nv_bfloat16* partial16 = reinterpret_cast<const __nv_bfloat16*>(p.partial);
    const size_t c_es = p.c_f32 ? 4 : 2;
    const bool vec_out = (p.N & 3) == 0 && (p.ldc & 3) == 0 && (p.stride_c & 3) == 0 &&
                         (reinterpret_cast<uintptr_t>(p.C) & (4 * c_es - 1)) == 0;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c4 = static_cast<int>(i % cols4);
        const long long rm = i / cols4;
        const int m = static_cast<int>(rm % p.M);
        const int b = static_cast<int>(rm / p.M);
        const int n = c4 * 4;
        const size_t off = (static_cast<size_t>(b) * p.M + m) * p.N + n;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (p.partial_is_bf16) {
            if (vec_in) {   // 8-byte loads of four bf16 values
                for (int s = 0; s < p.k_splits; ++s) {
                    const uint2 v = *reinterpret_cast<const uint2*>(partial16 + s * slice + off);
                    acc[0] += __uint_as_float(v.x << 16);
                    acc[1] += __uint_as_float(v.x & 0xffff0000u);
                    acc[2] += __uint_as_float(v.y << 16);
                    acc[3] += __uint_as_float(v.y & 0xffff0000u);
                }
            } else {
                for (int s = 0; s < p.k_splits; ++s)
                    for (int j = 0; j < 4; ++j)
                        if (n + j < p.N) acc[j] += __bfloat162float(partial16[s * slice + off + j]);
            }
        } else if (vec_in) {
            for (int s = 0; s < p.k_splits; ++s) {
                const float4 v = *reinterpret_cast<const float4*>(p.partial + s * slice + off);
                acc[0] += v.x;
                acc[1] += v.y;
                acc[2] += v.z;
                acc[3] += v.w;
            }
        } else {
            for (int s = 0; s < p.k_splits; ++s)
                for (int j = 0; j < 4; ++j)
                    if (n + j < p.N) acc[j] += p.partial[s * slice + off + j];
        }
        const size_t coff = static_cast<size_t>(b) * p.stride_c + static_cast<size_t>(m) * p.ldc + n;
        if (vec_out) {
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = epi_apply(p.epi, acc[j], m, n + j);
            if (p.c_f32)
                *reinterpret_cast<float4*>(static_cast<float*>(p.C) + coff) = make_float4(v[0], v[1], v[2], v[3]);
            else
                *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.C) + coff) =
                    make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
            continue;
        }
        for (int j = 0; j < 4; ++j) {
            if (n + j < p.N) {
                const float v = epi_apply(p.epi, acc[j], m, n + j);
                if (p.c_f32)
                    static_cast<float*>(p.C)[coff + j] = v;
                else
                    static_cast<__nv_bfloat16*>(p.C)[coff + j] = __float2bfloat16_rn(v);
            }
        }
    }
}

// 3-D tensor map {inner, rows, batch} over a bf16 matrix with a 128-byte-swizzled box.
int make_tensor_map(b200_ctx* ctx, CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows, uint64_t batch,
                    uint64_t ld_elems, uint64_t batch_stride_elems, uint32_t box_inner, uint32_t box_rows,
                    bool f32 = false, bool u8 = false) {
    const uint64_t es = u8 ? 1 : (f32 ? 4 : 2);
    cuuint64_t dims[3] = {inner, rows, batch};
    if (batch <= 1 || batch_stride_elems == 0) {
        dims[2] = 1;
        batch_stride_elems = rows * ld_elems;
    }
    cuuint64_t strides[2] = {ld_elems * es, batch_stride_elems * es};
    cuuint32_t box[3] = {box_inner, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = ctx->encode_tiled(out, u8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail(B200_ERR_CUDA,
                    "cuTensorMapEncodeTiled failed (%d): base %p dims {%llu,%llu,%llu} strides {%llu,%llu} box {%u,%u}",
                    static_cast<int>(r), base, (unsigned long long)dims[0], (unsigned long long)dims[1],
                    (unsigned long long)dims[2], (unsigned long long)strides[0], (unsigned long long)strides[1], box_inner,
                    box_rows);
    }
    return B200_OK;
}

template <int BN, bool A_KMAJOR, bool B_KMAJOR, bool FP8 = false>
int launch_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const CMaps& tmC, const GemmParams& p, int grid,
                   cudaStream_t stream) {
    using Cfg = TileCfg<BN>;
    auto kernel = gemm_tcgen05_kernel<BN, A_KMAJOR, B_KMAJOR, FP8>;
    static bool configured[64] = {};  // per template instance and device: the attribute is per device function
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        B200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    kernel<<<grid, NUM_THREADS, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, tmC, p);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

template <int BN>
int launch_bn(bool a_kmajor, bool b_kmajor, bool fp8, const CUtensorMap& tmA, const CUtensorMap& tmB, const CMaps& tmC,
              const GemmParams& p, int grid, cudaStream_t stream) {
    if (fp8) return launch_variant<BN, true, true, true>(tmA, tmB, tmC, p, grid, stream);
    if (a_kmajor && b_kmajor) return launch_variant<BN, true, true>(tmA, tmB, tmC, p, grid, stream);
    if (a_kmajor && !b_kmajor) return launch_variant<BN, true, false>(tmA, tmB, tmC, p, grid, stream);
    if (!a_kmajor && b_kmajor) return launch_variant<BN, false, true>(tmA, tmB, tmC, p, grid, stream);
    return launch_variant<BN, false, false>(tmA, tmB, tmC, p, grid, stream);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

bool gemm_tcgen05_eligible(const b200_gemm_desc& d, const char** why) {
    const char* w = nullptr;
    const bool fp8 = d.ab_dtype == B200_FP8_E4M3;
    const int64_t mask = fp8 ? 15 : 7;  // 16 bytes
    if (!aligned16(d.A) || !aligned16(d.B))
        w = "A and B must be 16-byte aligned";
    else if ((d.lda & mask) || (d.ldb & mask))
        w = fp8 ? "lda and ldb must be multiples of 16 elements" : "lda and ldb must be multiples of 8 elements";
    else if (d.batch > 1 && ((d.stride_a & mask) || (d.stride_b & mask)))
        w = fp8 ? "batch strides of A and B must be multiples of 16 elements"
                : "batch strides of A and B must be multiples of 8 elements";
    else if (fp8 && (d.transpose_a != 0 || d.transpose_b == 0))
        w = "8-bit operands need transpose_a = 0 and transpose_b = 1";
    else if (d.M >= (1ll << 31) || d.N >= (1ll << 31) || d.K >= (1ll << 31) || d.batch >= (1ll << 31))
        w = "dimension too large";
    if (why) *why = w;
    return w == nullptr;
}

namespace {

// Normalises a requested K-slice count so that every slice gets at least one K block.
int normalise_splits(int want, int num_kb) {
    want = std::max(1, std::min(want, num_kb));
    const int per = (num_kb + want - 1) / want;
    return (num_kb + per - 1) / per;
}

// Slice counts worth trying for `tiles` work items on `slots` concurrent CTAs (or CTA pairs).
int split_candidates(const b200_gemm_desc& d, long long tiles, long long slots, int num_kb, int (&cand)[4]) {
    cand[0] = 1;
    int n = 1;
    if (d.split_k > 1) {
        cand[0] = normalise_splits(d.split_k, num_kb);
    } else if (d.split_k == 0 && tiles * 2 <= slots && num_kb >= 8) {
        const int fill = static_cast<int>(slots / tiles);              // slices that fill one round of the grid
        const int most = std::min(std::min(fill, num_kb / 4), 32);     // at least 4 K blocks per slice
        for (int want : {most, most / 2, most / 4}) {
            if (want < 2) break;
            const int s = normalise_splits(want, num_kb);
            bool seen = false;
            for (int c = 0; c < n; ++c) seen |= cand[c] == s;
            if (!seen) cand[n++] = s;
        }
    } else if (d.split_k == 0 && tiles <= 4 * slots && num_kb >= 64) {
        // A few rounds of long tiles with the last round partly empty (96 tiles on 74 CTA pairs: two rounds for 1.3
        // rounds of work): the slice count whose rounds, divided by the slices, waste least.
        const double whole = static_cast<double>((tiles + slots - 1) / slots);
        double best = whole * 0.9;  // worth the partial sums only for a tenth or more
        int pick = 0;
        for (int s = 2; s <= 6 && num_kb / s >= 32; ++s) {
            const double eff = static_cast<double>((tiles * s + slots - 1) / slots) / s;
            if (eff < best - 1e-9) {
                best = eff;
                pick = s;
            }
        }
        if (pick > 1) cand[n++] = normalise_splits(pick, num_kb);
    }
    return n;
}

}  // namespace

// Picks the kernel, the tile width and the K-slice count together from a cost model fitted to timings on B200. The
// unit is the time one 128-row tile spends on one output column of one K block at full tensor rate (about 1 ns).
//   main loop: rounds of the persistent grid x (K blocks per work item + pipeline fill) x tile width x c(width);
//              c = 1, 1.1-1.3, 1.5, 3 for 256, 192, 128, 64 columns: a narrower tile re-reads the A block more often per flop
//              and the shared-memory fill rate, not the tensor pipe, then sets the pace; 0.95 for the CTA-pair
//              kernel, whose two CTAs share the B tile;
//   K slices:  single-CTA kernel: a fixed charge for the second launch plus the fp32 partial sums written and read
//              back by it; pair kernel: the last slice to finish adds the others inside the same launch: no second
//              launch, but one CTA reads every other slice of its tile, so the charge grows with the slice count and
//              two or three slices is where it pays.
GemmPlan gemm_plan(const b200_ctx* ctx, const b200_gemm_desc& d, bool allow_pair) {
    const int bk = gemm_bk_elems(d);
    const int num_kb = static_cast<int>((d.K + bk - 1) / bk);
    const double out_elems = static_cast<double>(d.batch) * d.M * d.N;
    GemmPlan best{false, 256, 1};
    double best_cost = 0.0;
    auto offer = [&](const GemmPlan& plan, double cost) {
        if (best_cost == 0.0 || cost < best_cost * 0.97) {  // near ties go to the earlier plan
            best_cost = cost;
            best = plan;
        }
    };
    if (allow_pair && gemm_pair_supported(d, nullptr)) {
        const long long pairs = ctx->sm_count / 2;
        const long long tiles = d.batch * ((d.M + 255) / 256) * ((d.N + 255) / 256);
        int cand[4];
        const int n = split_candidates(d, tiles, pairs, num_kb, cand);
        for (int c = 0; c < n; ++c) {
            const int splits = cand[c];
            if (splits > 1 && tiles * 2 >= kTicketCount) continue;
            const long long rounds = (tiles * splits + pairs - 1) / pairs;
            const int kb_per = (num_kb + splits - 1) / splits;
            double cost = static_cast<double>(rounds) * (kb_per + 10) * 256 * 0.95;  // a pair's per-tile overhead is larger
            // long reductions (the weight-gradient products, K = tokens): measured 44-48 us for two slices against
            // 51-52 us for the single-CTA kernel's one round of 128-column tiles at 2304 x 768 x 8192 and 3072 x 768 x 8192
            if (splits > 1) cost += 1000.0 + (num_kb >= 64 ? 3000.0 : 4000.0) * splits;
            offer(GemmPlan{true, 256, splits}, cost);
        }
    }
    const long long m_tiles = d.batch * ((d.M + BM - 1) / BM);
    const int widths[4] = {256, 192, 128, 64};
    // the 192-column tile loses ground to the wider ones as K grows (measured: level at K <= 3072, 9 % behind at K = 50264)
    const double cost_per_col[4] = {1.0, 1.1 + 0.2 * std::min(1.0, num_kb / 512.0), 1.5, 3.0};
    for (int i = 0; i < 4; ++i) {
        const int bn = widths[i];
        if (i < 3 && d.N <= bn / 2) continue;  // more than half of the tile would be padding
        const long long tiles = m_tiles * ((d.N + bn - 1) / bn);
        int cand[4];
        const int n = split_candidates(d, tiles, ctx->sm_count, num_kb, cand);
        for (int c = 0; c < n; ++c) {
            const int splits = cand[c];
            const long long rounds = (tiles * splits + ctx->sm_count - 1) / ctx->sm_count;
            const int kb_per = (num_kb + splits - 1) / splits;
            double cost = static_cast<double>(rounds) * (kb_per + 6) * bn * cost_per_col[i];
            if (splits > 1) cost += 6500.0 + 2.56e-3 * splits * out_elems;
            offer(GemmPlan{false, bn, splits}, cost);
        }
    }
    return best;
}

int gemm_choose_split_k(const b200_ctx* ctx, const b200_gemm_desc& d) { return gemm_plan(ctx, d, false).splits; }

int launch_gemm_tcgen05(b200_ctx* ctx, const b200_gemm_desc& d, int k_splits, cudaStream_t stream, const GemmRoute* route,
                        int block_n, int group_m) {
    const bool a_kmajor = d.transpose_a == 0;  // A stored [M,K]
    const bool b_kmajor = d.transpose_b != 0;  // B stored [N,K]
    int bn = block_n;
    if (bn == 0) {
        b200_gemm_desc planned = d;
        planned.split_k = k_splits;  // the tile width that suits the slice count the caller settled on
        bn = gemm_plan(ctx, planned, false).bn;
    }
    B200_REQUIRE(bn == 64 || bn == 128 || bn == 192 || bn == 256, "b200_gemm: tile width %d is not one of 64, 128, 192, 256", bn);
    const bool fp8 = d.ab_dtype == B200_FP8_E4M3;
    const int bk = gemm_bk_elems(d);

    GemmParams p{};
    p.M = static_cast<int>(d.M);
    p.N = static_cast<int>(d.N);
    p.K = static_cast<int>(d.K);
    p.batch = static_cast<int>(d.batch);
    p.num_m_tiles = (p.M + BM - 1) / BM;
    p.num_n_tiles = (p.N + bn - 1) / bn;
    p.num_kb = (p.K + bk - 1) / bk;
    p.k_splits = k_splits;
    p.kb_per_split = (p.num_kb + k_splits - 1) / k_splits;
    const long long total = static_cast<long long>(k_splits) * p.batch * p.num_m_tiles * p.num_n_tiles;
    B200_REQUIRE(total < (1ll << 31), "b200_gemm: too many tiles (%lld)", total);
    p.total_work = static_cast<int>(total);
    p.a_batched = (d.batch > 1 && d.stride_a != 0) ? 1 : 0;
    p.b_batched = (d.batch > 1 && d.stride_b != 0) ? 1 : 0;
    p.C = d.C;
    p.ldc = d.ldc;
    p.stride_c = d.stride_c;
    p.c_f32 = d.c_dtype == B200_F32;
    const int cvec = p.c_f32 ? 4 : 8;
    p.c_vec_ok = aligned16(d.C) && (d.ldc % cvec) == 0 && (d.batch <= 1 || (d.stride_c % cvec) == 0);
    p.epi.alpha = d.alpha;
    p.epi.bias = d.bias;
    p.epi.bias_f32 = d.bias_dtype == B200_F32;
    p.epi.act = d.activation;
    p.epi.gelu_tanh = d.fidelity == B200_LOFI;
    p.epi.causal = d.causal_mask;
    p.epi.mask_value = d.mask_value;
    p.status = ctx->d_status;
    p.group_m = (group_m >= 1 && group_m <= 64) ? group_m : 16;
    p.partial = nullptr;
    p.partial_round_bf16 = (d.fidelity == B200_LOFI || d.fidelity == B200_HIFI2) ? 1 : 0;
    if (k_splits > 1) {
        const size_t bytes = static_cast<size_t>(k_splits) * p.batch * p.M * p.N * sizeof(float);
        int rc = ensure_scratch(ctx, bytes, stream);
        if (rc != B200_OK) return rc;
        p.partial = static_cast<float*>(ctx->d_scratch);
    }

    CUtensorMap tmA, tmB;
    int rc;
    if (a_kmajor)
        rc = make_tensor_map(ctx, &tmA, d.A, d.K, d.M, d.batch, d.lda, d.stride_a, bk, BM, false, fp8);
    else
        rc = make_tensor_map(ctx, &tmA, d.A, d.M, d.K, d.batch, d.lda, d.stride_a, 64, BK);
    if (rc != B200_OK) return rc;
    if (b_kmajor)
        rc = make_tensor_map(ctx, &tmB, d.B, d.K, d.N, d.batch, d.ldb, d.stride_b, bk, bn, false, fp8);
    else
        rc = make_tensor_map(ctx, &tmB, d.B, d.N, d.K, d.batch, d.ldb, d.stride_b, 64, BK);
    if (rc != B200_OK) return rc;

    // Output routing. The staged TMA-store epilogue needs 16-byte aligned rows of C; routed launches require it.
    CMaps tmC;
    memset(&tmC, 0, sizeof(tmC));
    p.epi_mode = 0;
    p.n_dst = 1;
    p.scatter_rows = 0;
    p.dst_rotate = 0;
    const uint32_t box_cols = p.c_f32 ? 32 : 64;
    if (k_splits == 1) {
        if (route != nullptr && route->n_dst > 0) {
            B200_REQUIRE(route->n_dst <= 8, "b200_gemm: at most 8 destinations");
            B200_REQUIRE((d.ldc % cvec) == 0, "b200_gemm: routed output needs ldc to be a multiple of %d elements", cvec);
            for (int i = 0; i < route->n_dst; ++i) {
                B200_REQUIRE(aligned16(route->dst[i]), "b200_gemm: destination %d is not 16-byte aligned", i);
                rc = make_tensor_map(ctx, &tmC.m[i], route->dst[i], d.N, route->rows[i], 1, d.ldc, 0, box_cols, 32, p.c_f32);
                if (rc != B200_OK) return rc;
            }
            p.epi_mode = 1;
            p.n_dst = route->scatter_rows > 0 ? 1 : route->n_dst;
            p.scatter_rows = route->scatter_rows;
            p.m_tile_rotate = static_cast<int>((route->m_rotate_rows / BM) % p.num_m_tiles);
            p.dst_rotate = (route->scatter_rows > 0 || route->rotate < 0 || route->rotate >= route->n_dst) ? 0 : route->rotate;
        } else if (p.c_vec_ok) {
            rc = make_tensor_map(ctx, &tmC.m[0], d.C, d.N, d.M, d.batch, d.ldc, d.stride_c, box_cols, 32, p.c_f32);
            if (rc != B200_OK) return rc;
            p.epi_mode = 1;
        }
    } else {
        B200_REQUIRE(route == nullptr || route->n_dst == 0, "b200_gemm: a routed product cannot be split along K");
    }

    const int grid = min(p.total_work, ctx->sm_count);
    if (bn == 256)
        rc = launch_bn<256>(a_kmajor, b_kmajor, fp8, tmA, tmB, tmC, p, grid, stream);
    else if (bn == 192)
        rc = launch_bn<192>(a_kmajor, b_kmajor, fp8, tmA, tmB, tmC, p, grid, stream);
    else if (bn == 128)
        rc = launch_bn<128>(a_kmajor, b_kmajor, fp8, tmA, tmB, tmC, p, grid, stream);
    else
        rc = launch_bn<64>(a_kmajor, b_kmajor, fp8, tmA, tmB, tmC, p, grid, stream);
    if (rc != B200_OK) return rc;

    if (k_splits > 1) {
        const long long work = static_cast<long long>(p.batch) * p.M * ((p.N + 3) / 4);
        const int threads = 256;
        const int blocks = static_cast<int>(std::min<long long>((work + threads - 1) / threads, ctx->sm_count * 8ll));
        splitk_reduce_kernel<<<blocks, threads, 0, stream>>>(p);
        B200_CUDA_TRY(cudaGetLastError());
    }
    return B200_OK;
}

int launch_splitk_reduce(b200_ctx* ctx, const b200_gemm_desc& d, const void* partial, int splits, cudaStream_t stream,
                         bool partial_bf16) {
    GemmParams p{};
    p.partial_is_bf16 = partial_bf16 ? 1 : 0;
    p.M = static_cast<int>(d.M);
    p.N = static_cast<int>(d.N);
    p.batch = static_cast<int>(d.batch);
    p.k_splits = splits;
    p.partial = static_cast<float*>(const_cast<void*>(partial));
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
    const long long work = static_cast<long long>(p.batch) * p.M * ((p.N + 3) / 4);
    if (work == 0) return B200_OK;
    const int threads = 256;
    const int blocks = static_cast<int>(std::min<long long>((work + threads - 1) / threads, ctx->sm_count * 8ll));
    splitk_reduce_kernel<<<blocks, threads, 0, stream>>>(p);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // namespace b200
