// CTA-pair variant of the tcgen05 GEMM for large products: two CTAs of a cluster (one SM each) share a 256 x 256
// output tile and one `tcgen05.mma.cta_group::2` instruction stream.
//
//   * each CTA loads its own 128 rows of A and 128 of the tile's 256 B columns per 64-deep K block (32 KiB per stage,
//     6 stages) — half the shared-memory fill and half the B reads per SM of the single-CTA kernel;
//   * the leader CTA (cluster rank 0) issues the MMAs (M = 256, N = 256, K = 16); the hardware reads A and B from both
//     CTAs' shared memory and writes rows 0-127 of the accumulator to the leader's TMEM, rows 128-255 to the peer's;
//   * TMA completions of both CTAs are counted on the leader's "full" barrier (cta_group::2 loads, no multicast);
//     `tcgen05.commit` with a 2-CTA multicast mask releases ring stages and publishes accumulators in both CTAs;
//   * each CTA's eight epilogue warps drain their own 128 accumulator rows (two warps per 32 rows, half of the
//     columns each) through the staged TMA-store epilogue.
//
// Same roles, ring protocol, bounded waits and output routing as gemm_tcgen05.cu; requires 16-byte aligned C rows.
#include <algorithm>
#include <cstring>

#include "gemm_common.cuh"
#include "ptx.cuh"

namespace b200 {

using namespace ptx;

namespace {

constexpr int BM_CTA = 128;   // accumulator rows per CTA
constexpr int BM_PAIR = 256;  // tile rows per CTA pair
constexpr int BN = 256;
constexpr int BN_CTA = 128;   // B columns loaded by each CTA
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int EPI_WARPS = 8;   // two warps per TMEM lane quarter, each takes half of the tile's columns
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM_CTA * BK * 2;
constexpr int B_BYTES = BN_CTA * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_STAGE_BYTES = 4096;
constexpr int EPI_BYTES = EPI_WARPS * EPI_STAGE_BYTES;  // one staging box per epilogue warp
constexpr int BARRIER_BYTES = 256;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + BARRIER_BYTES + 1024;

struct PairWork {
    int b, m0, n0;
    int split, tile;   // K slice, and the index of the output tile among batch * tiles (the ticket it uses)
    int kb_begin, kb_end;
};

__device__ __forceinline__ PairWork decode_pair(const GemmParams& p, int w) {
    PairWork it;
    const int tiles_mn = p.num_m_tiles * p.num_n_tiles;
    const int per_split = p.batch * tiles_mn;
    it.split = w / per_split;
    it.tile = w - it.split * per_split;
    it.kb_begin = it.split * p.kb_per_split;
    it.kb_end = min(p.num_kb, it.kb_begin + p.kb_per_split);
    it.b = it.tile / tiles_mn;
    const int t = it.tile - it.b * tiles_mn;
    const int tiles_per_group = p.group_m * p.num_n_tiles;
    const int g = t / tiles_per_group;
    const int first_m = g * p.group_m;
    const int gsz = min(p.num_m_tiles - first_m, p.group_m);
    const int rr = t - g * tiles_per_group;
    int mi = first_m + rr % gsz + p.m_tile_rotate;
    if (mi >= p.num_m_tiles) mi -= p.num_m_tiles;
    it.m0 = mi * BM_PAIR;
    it.n0 = (rr / gsz) * BN;
    return it;
}

// Named barrier of the eight epilogue warps (256 threads), plain and with an AND-reduction of a predicate.
__device__ __forceinline__ void epilogue_warps_sync() { asm volatile("bar.sync 2, 256;" ::: "memory"); }
__device__ __forceinline__ bool epilogue_warps_all(bool pred) {
    uint32_t out;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.u32 p, %1, 0;\n\t"
        "barrier.cta.red.and.pred q, 2, 256, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t"
        "}\n"
        : "=r"(out)
        : "r"(static_cast<uint32_t>(pred))
        : "memory");
    return out != 0;
}

// FP8: one-byte e4m3 operands, K-major only; a stage holds 128 elements of K per row in the same 128 bytes.
template <bool A_KMAJOR, bool B_KMAJOR, bool FP8 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CMaps tmC, const GemmParams p, const int tmem_cols) {
    static_assert(!FP8 || (A_KMAJOR && B_KMAJOR), "8-bit operands are K-major only");
    constexpr int KB_ELEMS = FP8 ? 2 * BK : BK;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;
    uint8_t* bar_base = epi_smem + EPI_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_base);   // used in the leader only
    uint64_t* empty_bar = full_bar + STAGES;                       // one per CTA (multicast commit)
    uint64_t* tmem_full_bar = empty_bar + STAGES;                  // one per CTA (multicast commit)
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;                  // used in the leader only: 16 arrivals (8 warps x 2 CTAs)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* last_flag = abort_flag + 1;      // split-K: this CTA drew the last ticket of its tile
    uint64_t* part_bar = reinterpret_cast<uint64_t*>(bar_base + 160);  // two K slices: the other slice's sums have landed in smem

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();       // 0 = leader
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;
    const bool two_bufs = tmem_cols >= 2 * BN;     // accumulator double buffering needs 512 TMEM columns

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmB);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tmem_full_bar[a], 1);
            mbar_init(&tmem_empty_bar[a], 2 * EPI_WARPS);  // every epilogue warp of both CTAs
        }
        mbar_init(part_bar, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, static_cast<uint32_t>(tmem_cols));
        tmem_relinquish_alloc_permit_pair();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers are initialised before anyone signals across the pair
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int w = cluster_id; ok && w < p.total_work; w += num_clusters) {
                const PairWork it = decode_pair(p, w);
                const int ab = p.a_batched ? it.b : 0;
                const int bb = p.b_batched ? it.b : 0;
                const int m_cta = it.m0 + static_cast<int>(rank) * BM_CTA;
                const int n_cta = it.n0 + static_cast<int>(rank) * BN_CTA;
                for (int kb = it.kb_begin; kb < it.kb_end; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sA = smem + stage * STAGE_BYTES;
                    uint8_t* sB = sA + A_BYTES;
                    // completions of both CTAs are counted on the leader's barrier
                    const uint32_t full_leader = mapa_shared(smem_u32(&full_bar[stage]), 0);
                    if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
                    if (A_KMAJOR) {
                        tma_load_3d_pair(sA, &tmA, full_leader, kb * KB_ELEMS, m_cta, ab);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM_CTA / 64; ++j)
                            tma_load_3d_pair(sA + j * (64 * BK * 2), &tmA, full_leader, m_cta + 64 * j, kb * BK, ab);
                    }
                    if (B_KMAJOR) {
                        tma_load_3d_pair(sB, &tmB, full_leader, kb * KB_ELEMS, n_cta, bb);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN_CTA / 64; ++j)
                            tma_load_3d_pair(sB + j * (64 * BK * 2), &tmB, full_leader, n_cta + 64 * j, kb * BK, bb);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok && rank == 0) {
                // Gave up: the leader's barriers count both CTAs' copies; let those already issued land before the
                // pair's shared memory goes away (the peer leaves only after the cluster barrier below).
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
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = FP8 ? make_idesc_e4m3_f32(BM_PAIR, BN)
                                           : make_idesc_bf16_f32(BM_PAIR, BN, A_KMAJOR ? 0u : 1u, B_KMAJOR ? 0u : 1u);
            constexpr uint32_t A_KSTEP = A_KMAJOR ? (UMMA_K * 2) : (UMMA_K * 128);
            constexpr uint32_t B_KSTEP = B_KMAJOR ? (UMMA_K * 2) : (UMMA_K * 128);
            constexpr uint32_t A_LBO = A_KMAJOR ? 0u : (BK * 128);
            constexpr uint32_t B_LBO = B_KMAJOR ? 0u : (BK * 128);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int w = cluster_id; ok && w < p.total_work; w += num_clusters) {
                const PairWork it = decode_pair(p, w);
                if (!mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u, abort_flag)) break;
                tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
                for (int kb = it.kb_begin; kb < it.kb_end; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
                    const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t da = make_smem_desc_sw128(a_addr + k * A_KSTEP, A_LBO, 1024);
                        const uint64_t db = make_smem_desc_sw128(b_addr + k * B_KSTEP, B_LBO, 1024);
                        if (FP8)
                            umma_f8_ss_pair(d_tmem, da, db, idesc, (kb > it.kb_begin || k > 0) ? 1u : 0u);
                        else
                            umma_f16_ss_pair(d_tmem, da, db, idesc, (kb > it.kb_begin || k > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(&empty_bar[stage], 3);  // frees the stage in both CTAs
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                umma_commit_pair(&tmem_full_bar[acc], 3);  // accumulator complete, both CTAs' epilogues may read
                if (two_bufs) {
                    acc ^= 1;
                    if (acc == 0) acc_phase ^= 1u;
                } else {
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
        // A warp may read the TMEM lane quarter (warp id mod 4); warps w and w + 4 share a quarter and split the tile's
        // 256 columns between them. Four warps converting and staging a whole tile took as long as a 12-K-block main
        // loop and slowed the MMAs that ran beside them; eight halve that.
        const int q = warp & 3;
        const int c_first = ((warp - 2) >> 2) * (BN / 2), c_last = c_first + BN / 2;
        int acc = 0;
        uint32_t acc_phase = 0;
        uint8_t* sbuf = epi_smem + (warp - 2) * EPI_STAGE_BYTES;
        const int box_cols = p.c_f32 ? 32 : 64;
        for (int w = cluster_id; w < p.total_work; w += num_clusters) {
            const PairWork it = decode_pair(p, w);
            const bool got = mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag);
            if (p.k_splits > 1) {
                // the epilogue warps meet at named barriers below: they must agree on whether to go on
                if (!epilogue_warps_all(__all_sync(0xffffffffu, got))) break;
            } else if (!__all_sync(0xffffffffu, got)) {
                break;
            }
            tcgen05_fence_after_sync();
            const int m_cta = it.m0 + static_cast<int>(rank) * BM_CTA;
            const int row = m_cta + q * 32 + lane;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
            int dst_first = 0, dst_count = p.n_dst, row_coord = m_cta + q * 32;
            if (p.scatter_rows > 0) {
                dst_first = m_cta / p.scatter_rows;
                dst_count = 1;
                row_coord -= dst_first * p.scatter_rows;
            }
            bool finish = true;  // this CTA writes C for the tile
            bool staged_partner = false;
            // Partial sums live in a layout of their own, [slice][tile][CTA of the pair][32-column chunk][vector j]
            // [thread]: the k-th 16-byte vector of a thread's 32 columns sits next to the same vector of its
            // neighbours, so a warp writes and reads 512 contiguous bytes per instruction (row-major fp32 would cost
            // one 128-byte line per thread per instruction).
            const size_t cta_floats = static_cast<size_t>(BM_CTA) * BN;
            const size_t tiles_total = static_cast<size_t>(p.batch) * p.num_m_tiles * p.num_n_tiles;
            const int ethread = q * 32 + lane;  // the accumulator row within the CTA: 0..127
            auto part_at = [&](int slice_idx) {
                return reinterpret_cast<float4*>(p.partial + ((static_cast<size_t>(slice_idx) * tiles_total + it.tile) * 2 + rank) * cta_floats) +
                       ethread;
            };
            if (p.k_splits > 1) {
                // K slices of one tile run in different CTA pairs. Each writes its fp32 partial sums and then draws a
                // ticket; whoever draws the last one knows that all the others are complete in memory, adds them to
                // the sums it still holds in TMEM and runs the normal epilogue. Nobody waits for anybody.
                float4* mine = part_at(it.split);
#pragma unroll 1
                for (int c = c_first; c < c_last; c += 32) {
                    if (it.n0 + c >= p.N) break;
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c, v);
                    tmem_ld_wait();
                    if (p.partial_round_bf16) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            v[i] = __float_as_uint(__bfloat162float(__float2bfloat16_rn(__uint_as_float(v[i]))));
                    }
                    float4* dst = mine + (c / 32) * 8 * 128;
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        dst[i * 128] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                   __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                }
                __threadfence();
                epilogue_warps_sync();
                // With two slices and no further work item for this CTA the operand ring is idle: the finishing slice
                // has the other slice's 128 KB of sums copied into it in bulk and adds them from shared memory. Fetched
                // with plain loads, 8 at a time per thread, the same sums cost eight L2 round trips in a row.
                staged_partner = p.k_splits == 2 && w + num_clusters >= p.total_work;
                if (threadIdx.x == 64) {
                    const unsigned t = atomicAdd(&p.tickets[it.tile * 2 + static_cast<int>(rank)], 1u);
                    *last_flag = (t == static_cast<unsigned>(p.k_splits - 1)) ? 1 : 0;
                    if (*last_flag) {
                        p.tickets[it.tile * 2 + static_cast<int>(rank)] = 0u;  // ready for the next launch
                        if (staged_partner) {
                            __threadfence();
                            fence_proxy_async_all();  // the other slice's stores (generic proxy) before this bulk read
                            constexpr uint32_t kPiece = 32768;
                            const char* src = reinterpret_cast<const char*>(part_at(1 - it.split) - ethread);
                            mbar_arrive_expect_tx(part_bar, static_cast<uint32_t>(cta_floats * sizeof(float)));
                            for (uint32_t off = 0; off < cta_floats * sizeof(float); off += kPiece)
                                bulk_load_g2s(smem + off, src + off, kPiece, part_bar);
                        }
                    }
                }
                epilogue_warps_sync();
                finish = *last_flag != 0;
                if (finish) {
                    __threadfence();
                    if (staged_partner) {  // all lanes of a warp agree on whether the copy landed
                        const bool landed = mbar_wait(part_bar, 0, abort_flag);
                        if (!__all_sync(0xffffffffu, landed)) finish = false;
                    }
                }
            }
            if (finish && m_cta < p.M) {  // a CTA whose 128 rows lie entirely below the matrix has nothing to store
#pragma unroll 1
                for (int c = c_first; c < c_last; c += box_cols) {
                    const int n = it.n0 + c;
                    if (n >= p.N) break;
                    uint32_t v0[32], v1[32];
                    tmem_ld_32x32b_x32(taddr + c, v0);
                    if (box_cols == 64 && n + 32 < p.N) tmem_ld_32x32b_x32(taddr + c + 32, v1);
                    if (p.epi_mode == 1 && lane == 0) tma_store_wait_read<0>();  // the box this warp stored before has left its buffer
                    __syncwarp();
                    uint8_t* srow = sbuf + lane * 128;
                    tmem_ld_wait();
#pragma unroll 1
                    for (int h = 0; h * 32 < box_cols; ++h) {
                        const int nh = n + h * 32;
                        if (nh >= p.N) break;
                        uint32_t (&v)[32] = h == 0 ? v0 : v1;
                        if (p.k_splits > 1 && p.partial_round_bf16) {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                v[i] = __float_as_uint(__bfloat162float(__float2bfloat16_rn(__uint_as_float(v[i]))));
                        }
                        if (staged_partner) {
                            // two terms: a + b is the same number in either order
                            const float4* ps = reinterpret_cast<const float4*>(smem) + ((c + h * 32) / 32) * 8 * 128 + ethread;
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float4 a = ps[i * 128];
                                v[4 * i] = __float_as_uint(__uint_as_float(v[4 * i]) + a.x);
                                v[4 * i + 1] = __float_as_uint(__uint_as_float(v[4 * i + 1]) + a.y);
                                v[4 * i + 2] = __float_as_uint(__uint_as_float(v[4 * i + 2]) + a.z);
                                v[4 * i + 3] = __float_as_uint(__uint_as_float(v[4 * i + 3]) + a.w);
                            }
                        } else if (p.k_splits > 1) {
                            sum_slices_in_order(v, it.split, p.k_splits,
                                                [&](int sl) { return part_at(sl) + ((c + h * 32) / 32) * 8 * 128; });
                        }
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
                    if (p.epi_mode == 2) {
                        // The warp writes its box itself, 16 bytes per lane and instruction (four 128-byte rows per
                        // instruction): to a multicast address one such store reaches every rank's C.
                        __syncwarp();
                        const size_t es = p.c_f32 ? 4 : 2;
                        const int per16 = p.c_f32 ? 4 : 8;   // elements per 16-byte chunk
                        char* gbase = static_cast<char*>(p.C) + (static_cast<size_t>(row_coord) * p.ldc + n) * es;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int ci = i * 32 + lane;
                            const int r = ci >> 3, ch = ci & 7;
                            if (row_coord + r < p.M && n + ch * per16 < p.N) {
                                const uint4 val = *reinterpret_cast<const uint4*>(sbuf + r * 128 + ((ch ^ (r & 7)) << 4));
                                char* dst = gbase + static_cast<size_t>(r) * p.ldc * es + ch * 16;
                                if (p.mc_multimem)
                                    multimem_st_v4(dst, val);
                                else
                                    *reinterpret_cast<uint4*>(dst) = val;
                            }
                        }
                        continue;
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
                }
            }
            // Hand the accumulator buffer back to the leader's MMA warp (remote arrive from the peer CTA).
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty_bar[acc]), 0));
            if (two_bufs) {
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            } else {
                acc_phase ^= 1u;
            }
        }
        if (lane == 0) tma_store_wait_all<0>();
    }

    // ---------------------------------------------------------------------- teardown
    tcgen05_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // the peer may still be signalling this CTA's barriers or reading its shared memory
    if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(p.status, 1);
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc_pair(tmem_base, static_cast<uint32_t>(tmem_cols));
    }
}

template <bool A_KMAJOR, bool B_KMAJOR, bool FP8 = false>
int launch_pair_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const CMaps& tmC, const GemmParams& p, int grid,
                        int tmem_cols, cudaStream_t stream) {
    auto kernel = gemm_tcgen05_2cta_kernel<A_KMAJOR, B_KMAJOR, FP8>;
    static bool configured[64] = {};
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        B200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, tmC, p, tmem_cols);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int encode_map(b200_ctx* ctx, CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows, uint64_t batch,
               uint64_t ld_elems, uint64_t batch_stride_elems, uint32_t box_inner, uint32_t box_rows, bool f32,
               bool u8 = false) {
    const uint64_t es = u8 ? 1 : (f32 ? 4 : 2);
    cuuint64_t dims[3] = {inner, rows, batch};
    if (batch <= 1 || batch_stride_elems == 0) {
        dims[2] = 1;
        batch_stride_elems = rows * ld_elems;
    }
    cuuint64_t strides[2] = {ld_elems * es, batch_stride_elems * es};
    cuuint32_t box[3] = {box_inner, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = ctx->encode_tiled(out, u8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
    return B200_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// Accumulator columns the pair kernel allocates in each CTA's TMEM: two 256-column buffers, so that the epilogue of one
// tile runs under the main loop of the next.
static int pair_tmem_cols() { return 512; }

// Row-tiles (of 256 rows) per column sweep of the tile order. Measured: 8 is best up to 8192 rows, 16 at 16384.
static int pair_group_m(int num_m_tiles) { return num_m_tiles >= 64 ? 16 : 8; }

// Operand and output layouts the pair kernel can handle at all (its epilogue always stores through TMA).
bool gemm_pair_supported(const b200_gemm_desc& d, const GemmRoute* route) {
    if (!gemm_tcgen05_eligible(d, nullptr)) return false;
    const int cvec = d.c_dtype == B200_F32 ? 4 : 8;
    if ((d.ldc % cvec) != 0 || (d.batch > 1 && (d.stride_c % cvec) != 0)) return false;
    if (route == nullptr || route->n_dst == 0) {
        if (!aligned16(d.C)) return false;
    } else if (route->scatter_rows > 0 && (route->scatter_rows % BM_CTA) != 0) {
        return false;
    }
    return d.N >= 256 && d.M >= 256;
}

bool gemm_pair_eligible(const b200_ctx* ctx, const b200_gemm_desc& d, const GemmRoute* route) {
    if (!gemm_pair_supported(d, route)) return false;
    // worth it only when the 256 x 256 tiles keep all CTA pairs busy
    const long long tiles = d.batch * ((d.M + BM_PAIR - 1) / BM_PAIR) * ((d.N + BN - 1) / BN);
    if (tiles < (ctx->sm_count / 2)) return false;
    // Both kernels give a CTA 128 x 256 outputs per round; the pair kernel must not need more rounds (an odd number
    // of 128-row blocks, or a tile count just above a multiple of the pair count, costs it one).
    const long long pairs = ctx->sm_count / 2;
    const long long tiles_single = d.batch * ((d.M + BM_CTA - 1) / BM_CTA) * ((d.N + BN - 1) / BN);
    return (tiles + pairs - 1) / pairs <= (tiles_single + ctx->sm_count - 1) / ctx->sm_count;
}

int launch_gemm_tcgen05_pair(b200_ctx* ctx, const b200_gemm_desc& d, cudaStream_t stream, const GemmRoute* route,
                             int k_splits, int group_m) {
    const bool a_kmajor = d.transpose_a == 0;
    const bool b_kmajor = d.transpose_b != 0;
    const bool fp8 = d.ab_dtype == B200_FP8_E4M3;
    const int bk = gemm_bk_elems(d);
    GemmParams p{};
    p.M = static_cast<int>(d.M);
    p.N = static_cast<int>(d.N);
    p.K = static_cast<int>(d.K);
    p.batch = static_cast<int>(d.batch);
    p.num_m_tiles = (p.M + BM_PAIR - 1) / BM_PAIR;
    p.num_n_tiles = (p.N + BN - 1) / BN;
    p.num_kb = (p.K + bk - 1) / bk;
    k_splits = std::max(1, std::min(k_splits, p.num_kb));
    p.kb_per_split = (p.num_kb + k_splits - 1) / k_splits;
    p.k_splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;  // every slice gets at least one K block
    const long long tiles = static_cast<long long>(p.batch) * p.num_m_tiles * p.num_n_tiles;
    const long long total = tiles * p.k_splits;
    B200_REQUIRE(total < (1ll << 31), "b200_gemm: too many tiles (%lld)", total);
    p.total_work = static_cast<int>(total);
    p.partial = nullptr;
    p.tickets = nullptr;
    if (p.k_splits > 1) {
        B200_REQUIRE(route == nullptr || route->n_dst == 0, "b200_gemm: routed outputs cannot be combined with K slices");
        B200_REQUIRE(tiles * 2 < kTicketCount, "b200_gemm: %lld tiles exceed the ticket counters of the sliced pair kernel", tiles);
        const size_t bytes = static_cast<size_t>(p.k_splits) * tiles * BM_PAIR * BN * sizeof(float);  // whole tiles
        int rc_s = ensure_scratch(ctx, bytes, stream);
        if (rc_s != B200_OK) return rc_s;
        p.partial = static_cast<float*>(ctx->d_scratch);
        p.tickets = ctx_tickets(ctx);
    }
    p.a_batched = (d.batch > 1 && d.stride_a != 0) ? 1 : 0;
    p.b_batched = (d.batch > 1 && d.stride_b != 0) ? 1 : 0;
    p.C = d.C;
    p.ldc = d.ldc;
    p.stride_c = d.stride_c;
    p.c_f32 = d.c_dtype == B200_F32;
    p.c_vec_ok = 1;
    p.epi.alpha = d.alpha;
    p.epi.bias = d.bias;
    p.epi.bias_f32 = d.bias_dtype == B200_F32;
    p.epi.act = d.activation;
    p.epi.gelu_tanh = d.fidelity == B200_LOFI;
    p.epi.causal = d.causal_mask;
    p.epi.mask_value = d.mask_value;
    p.partial_round_bf16 = (d.fidelity == B200_LOFI || d.fidelity == B200_HIFI2) ? 1 : 0;
    p.status = ctx->d_status;
    p.group_m = (group_m >= 1 && group_m <= 64) ? group_m : pair_group_m(p.num_m_tiles);
    p.epi_mode = 1;
    p.n_dst = 1;

    CUtensorMap tmA, tmB;
    CMaps tmC;
    memset(&tmC, 0, sizeof(tmC));
    int rc;
    if (a_kmajor)
        rc = encode_map(ctx, &tmA, d.A, d.K, d.M, d.batch, d.lda, d.stride_a, bk, BM_CTA, false, fp8);
    else
        rc = encode_map(ctx, &tmA, d.A, d.M, d.K, d.batch, d.lda, d.stride_a, 64, BK, false);
    if (rc != B200_OK) return rc;
    if (b_kmajor)
        rc = encode_map(ctx, &tmB, d.B, d.K, d.N, d.batch, d.ldb, d.stride_b, bk, BN_CTA, false, fp8);
    else
        rc = encode_map(ctx, &tmB, d.B, d.N, d.K, d.batch, d.ldb, d.stride_b, 64, BK, false);
    if (rc != B200_OK) return rc;
    const uint32_t box_cols = p.c_f32 ? 32 : 64;
    if (route != nullptr && route->mc_dst != nullptr) {
        B200_REQUIRE(aligned16(route->mc_dst) && d.batch == 1, "b200_gemm: the multicast destination must be 16-byte aligned, batch 1");
        p.C = route->mc_dst;
        p.epi_mode = 2;
        p.mc_multimem = route->mc_multimem;
        rc = encode_map(ctx, &tmC.m[0], d.C, d.N, d.M, 1, d.ldc, 0, box_cols, 32, p.c_f32);  // unused by this mode; kept valid
        if (rc != B200_OK) return rc;
    } else if (route != nullptr && route->n_dst > 0) {
        B200_REQUIRE(route->n_dst <= 8, "b200_gemm: at most 8 destinations");
        for (int i = 0; i < route->n_dst; ++i) {
            B200_REQUIRE(aligned16(route->dst[i]), "b200_gemm: destination %d is not 16-byte aligned", i);
            rc = encode_map(ctx, &tmC.m[i], route->dst[i], d.N, route->rows[i], 1, d.ldc, 0, box_cols, 32, p.c_f32);
            if (rc != B200_OK) return rc;
        }
        p.n_dst = route->scatter_rows > 0 ? 1 : route->n_dst;
        p.scatter_rows = route->scatter_rows;
        p.m_tile_rotate = static_cast<int>((route->m_rotate_rows / BM_PAIR) % p.num_m_tiles);
        p.dst_rotate = (route->scatter_rows > 0 || route->rotate < 0 || route->rotate >= route->n_dst) ? 0 : route->rotate;
    } else {
        rc = encode_map(ctx, &tmC.m[0], d.C, d.N, d.M, d.batch, d.ldc, d.stride_c, box_cols, 32, p.c_f32);
        if (rc != B200_OK) return rc;
    }
    const int clusters = std::min(p.total_work, ctx->sm_count / 2);
    const int grid = 2 * clusters;
    const int cols = pair_tmem_cols();
    if (fp8) return launch_pair_variant<true, true, true>(tmA, tmB, tmC, p, grid, cols, stream);
    if (a_kmajor && b_kmajor) return launch_pair_variant<true, true>(tmA, tmB, tmC, p, grid, cols, stream);
    if (a_kmajor && !b_kmajor) return launch_pair_variant<true, false>(tmA, tmB, tmC, p, grid, cols, stream);
    if (!a_kmajor && b_kmajor) return launch_pair_variant<false, true>(tmA, tmB, tmC, p, grid, cols, stream);
    return launch_pair_variant<false, false>(tmA, tmB, tmC, p, grid, cols, stream);
}

}  // namespace b200
