// igemm_sparse_pair.cuh — 2:4-sparse WEIGHT GEMM on CTA pairs: tcgen05.mma.sp.cta_group::2.
//
// D^T = W_sparse * X^T with 256 output channels x 240 tokens per CTA pair.  CTA r of the pair
// stages, per 256-wide K block: its 128 weight rows (kept values 128 x 128 B, TMA, 128-byte
// swizzle), their 4 KiB of position metadata (one untiled TMA box of 32 rows x 128 B over the contiguous tiled array) and HALF of the
// token tile (120 rows x 256 B as two swizzled boxes) — 50 KiB per stage and CTA against 84 KiB for
// a lone CTA with a 256-token tile.  The leader's MMA lane copies the metadata of BOTH CTAs into
// tensor memory (tcgen05.cp.cta_group::2) and issues four sparse MMAs (M = 256, N = 240, K = 64
// logical) per stage.  Accumulators: 2 x 240 columns, metadata 8 columns per stage behind them
// (480 + 32 = the whole tensor memory; a 256-token tile would leave no room for the metadata).
// Lanes are output channels, accumulator columns are tokens, so the epilogue writes D[m][n] with
// 32 adjacent channels per warp store.  Barrier protocol as in igemm_dense_pair.cuh; no copy is
// multicast.
#pragma once
#include "epilogue.cuh"
#include "igemm_dense.cuh"
#include "igemm_sparse.cuh"
#include "sm100_ptx.cuh"

namespace bm {

// LEFT = true is the reference orientation (igemm_sparse_tiled.cu:88-96, hgemm_sparse_tiled.cu:122-129):
// the sparse operand on the left, out[r][c], the dense operand B[K x C] row-major taken as an MN-major
// MMA operand.  A pair then computes 256 rows x 224 columns: each CTA stages ONE 128-byte-wide box of
// B per K block at column offset 112 * rank (16-byte aligned; the MMA reads 112 of its 128 columns),
// 52 KiB per stage and CTA, accumulators 2 x 224 + 32 metadata columns = 480.  F16 = true (LEFT only)
// is the fp16 form: a stage covers 128 logical K, B is two boxes of 64 fp16 columns, one
// tcgen05.cp of metadata and four tcgen05.mma.sp.kind::f16 of K = 32 (column pair + selector).
template <bool LEFT>
struct SpPairCfg {
    static constexpr int BN = LEFT ? 224 : 240;
    static constexpr int HALF_N = BN / 2;
    static constexpr int A_BYTES = 128 * 128;
    static constexpr int B_BYTES = LEFT ? 128 * 256 : HALF_N * 256;          // 32 / 30 KiB
    static constexpr int STAGE_BYTES = A_BYTES + kSpMetaBytes + B_BYTES;      // 52 / 50 KiB
    // LEFT gives one ring stage to 8 x 4 KiB of store staging: its row-major fp32 / int32 output leaves
    // through TMA stores (a lane per output row makes direct stores touch 32 lines per instruction:
    // 541 us instead of 373 us for the lone-CTA kernel at 8192^3 before this)
    static constexpr int STAGES = LEFT ? 3 : 4;
    static constexpr int E_BASE = 2 * BN;
    static constexpr int NC = 128;
    static constexpr int STORE_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int BAR_OFFSET = STORE_OFFSET + (LEFT ? kEpiWarps * kStoreBoxBytes : 0);
    static constexpr int STRIP_OFFSET = BAR_OFFSET + (2 * STAGES + 5) * 8 + 16;
    static constexpr int SMEM_BYTES = STRIP_OFFSET + kEpiWarps * (int)sizeof(EpiStrip<NC>) + 1024;
    static_assert(E_BASE + STAGES * 8 <= 512, "tensor memory over-subscribed");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory over-subscribed");
};

// the sparse-weight orientation's figures under the names the launchers use
constexpr int kSpPairBN = SpPairCfg<false>::BN;               // tokens per pair tile (MMA N): 2 x 240 + 32 = all 512 TMEM columns
constexpr int kSpPairHalfN = SpPairCfg<false>::HALF_N;        // token rows staged per CTA
constexpr int kSpPairABytes = SpPairCfg<false>::A_BYTES;      // kept values
constexpr int kSpPairTmemCols = 512;
constexpr int kSpPairNC = SpPairCfg<false>::NC;               // accumulator columns per epilogue warp (second half: 112 / 96 live)
constexpr int kSpPairSmemBytes = SpPairCfg<false>::SMEM_BYTES;

__device__ __forceinline__ void tmem_cp_128x128b_pair(uint32_t taddr, uint64_t smem_desc) {
    asm volatile("tcgen05.cp.cta_group::2.128x128b [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}
__device__ __forceinline__ void mma_i8_sp_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t e_tmem,
                                               uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.sp.cta_group::2.kind::i8 [%0], %1, %2, [%3], %4, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void mma_f16_sp_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t e_tmem,
                                                uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.sp.cta_group::2.kind::f16 [%0], %1, %2, [%3], %4, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
        : "memory");
}

// map_w: kept values (byte map); map_e: tiled metadata as rows of 128 B = 8 units (box: 32 rows, 16 for fp16);
// map_x: the dense operand — tokens [M x K] (K-major), or B[K x C] as a byte map when LEFT
template <int EPI, bool LEFT = false, bool F16 = false>
__global__ void __launch_bounds__(kDenseThreads, 1)
igemm_sparse_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_e,
                         const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_out,
                         const SparseParams p) {
    using PC = SpPairCfg<LEFT>;
    constexpr int kSpPairStages = PC::STAGES;
    static_assert(!F16 || (LEFT && EPI == EPI_I32), "fp16: reference orientation, accumulator bits stored as they are");
    constexpr int kSpPairBN = PC::BN, kSpPairHalfN = PC::HALF_N, kSpPairBBytes = PC::B_BYTES;
    constexpr int kSpPairEBase = PC::E_BASE, kSpPairBarOffset = PC::BAR_OFFSET;
    constexpr int kSpPairStripOffset = PC::STRIP_OFFSET;
    constexpr int kKRows = F16 ? 128 : kSpKLogical;          // logical K per stage
    constexpr int kMetaStage = F16 ? 2048 : kSpMetaBytes;
    constexpr int kStageTx = PC::A_BYTES + kMetaStage + PC::B_BYTES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t a_smem0 = smem_base;
    const uint32_t b_smem0 = a_smem0 + kSpPairStages * kSpPairABytes;
    const uint32_t e_smem0 = b_smem0 + kSpPairStages * kSpPairBBytes;
    const uint32_t bar0 = smem_base + kSpPairBarOffset;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kSpPairStages + s); };
    auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * kSpPairStages + a); };
    auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * kSpPairStages + 2 + a); };
    const uint32_t drain_bar = bar0 + 8u * (2 * kSpPairStages + 4);
    const uint32_t tmem_slot = bar0 + 8u * (2 * kSpPairStages + 5);
    volatile uint32_t* tmem_slot_gen =
        reinterpret_cast<volatile uint32_t*>(smem_gen + kSpPairBarOffset + 8 * (2 * kSpPairStages + 5));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot_gen + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;
    const int num_tiles = p.tiles_r * p.tiles_c;        // tiles of 256 channels x 240 tokens
    auto tile_rb = [&](int tile) { return p.col_first ? tile / p.tiles_c : tile % p.tiles_r; };   // 256-row block
    auto tile_cb = [&](int tile) { return p.col_first ? tile % p.tiles_c : tile / p.tiles_r; };   // column tile

    if (threadIdx.x == 0) {
        for (int s = 0; s < kSpPairStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full_bar(a), 1);
            mbar_init(acc_empty_bar(a), 2 * kEpiWarps);
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, kSpPairTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_gen;
    pdl_launch_dependents();      // the next kernel of the stream may start its own set-up
    pdl_wait_prior_grid();        // nothing global is touched before the previous grid is complete

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (both CTAs)
        if (lane == 0) {
            prefetch_tensormap(&map_w);
            prefetch_tensormap(&map_e);
            prefetch_tensormap(&map_x);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                const int rb = tile_rb(tile) * 2 + static_cast<int>(rank);       // 128-row block of the sparse operand
                const int t0 = tile_cb(tile) * kSpPairBN + static_cast<int>(rank) * kSpPairHalfN;
                // metadata chunks of 128 rows x 16 B (= 128 logical K): 2 per int8 K block, 1 per fp16 K block;
                // a row block holds 2 * ceil(K / 256) of them
                const int chunks_per_rb = F16 ? ((p.k_blocks + 1) / 2) * 2 : p.k_blocks * 2;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!bounded_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status,
                                      DEV_TIMEOUT_PRODUCER_EMPTY)) { ok = false; break; }
                    const uint32_t leader_full = mapa_shared(full_bar(stage), 0);
                    if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * kStageTx);
                    tma_load_2d_pair(a_smem0 + stage * kSpPairABytes, &map_w, leader_full, kb * 128, rb * 128);
                    tma_load_2d_pair(e_smem0 + stage * kSpMetaBytes, &map_e, leader_full, 0,
                                     (rb * chunks_per_rb + kb * (F16 ? 1 : 2)) * 16);       // a chunk = 128 units = 16 rows
                    const uint32_t b_addr = b_smem0 + stage * kSpPairBBytes;
                    if constexpr (F16) {
#pragma unroll
                        for (int j = 0; j < 2; ++j)          // [128 K rows x 64 fp16 columns] per box, byte map
                            tma_load_2d_pair(b_addr + j * (128 * 128), &map_x, leader_full, t0 * 2 + j * 128, kb * kKRows);
                    } else if constexpr (LEFT) {
                        tma_load_2d_pair(b_addr, &map_x, leader_full, t0, kb * kKRows);   // [256 K rows x 128 columns]
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j)
                            tma_load_2d_pair(b_addr + j * (kSpPairHalfN * 128), &map_x, leader_full,
                                             kb * kSpKLogical + j * 128, t0);
                    }
                    if (++stage == kSpPairStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = F16 ? make_idesc_f16(256, kSpPairBN, true, true) : make_idesc_i8(256, kSpPairBN, LEFT, true);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                if (!bounded_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort_flag, p.status,
                                  DEV_TIMEOUT_MMA_ACC_EMPTY)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * kSpPairBN;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!bounded_wait(full_bar(stage), phase, abort_flag, p.status, DEV_TIMEOUT_MMA_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = a_smem0 + stage * kSpPairABytes;
                    const uint32_t b_addr = b_smem0 + stage * kSpPairBBytes;
                    const uint32_t e_addr = e_smem0 + stage * kSpMetaBytes;
                    const uint32_t e_tmem = tmem_base + kSpPairEBase + stage * 8;
#pragma unroll
                    for (int j = 0; j < (F16 ? 1 : 2); ++j)
                        tmem_cp_128x128b_pair(e_tmem + 4 * j, make_smem_desc(e_addr + j * 2048, 0, 128, SWIZZLE_NONE_DESC));
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint64_t a_desc = make_smem_desc(a_addr + ks * 32, 0, 1024, SWIZZLE_128B_DESC);
                        if constexpr (F16) {
                            // 32 K rows per MMA; the second 64-column group is one box (128 x 128 B) further
                            const uint64_t b_desc = make_smem_desc(b_addr + ks * (32 * 128), 128 * 128, 1024, SWIZZLE_128B_DESC);
                            mma_f16_sp_pair(d_tmem, a_desc, b_desc, e_tmem + (ks & ~1), idesc | static_cast<uint32_t>(ks & 1),
                                            (kb | ks) != 0 ? 1u : 0u);
                        } else if constexpr (LEFT) {
                            // 64 K rows of 128 B per MMA, a single 128-column group per CTA
                            const uint64_t b_desc = make_smem_desc(b_addr + ks * (64 * 128), 128 * kKRows, 1024, SWIZZLE_128B_DESC);
                            mma_i8_sp_pair(d_tmem, a_desc, b_desc, e_tmem + 2 * ks, idesc, (kb | ks) != 0 ? 1u : 0u);
                        } else {
                            const uint64_t b_desc = make_smem_desc(b_addr + (ks >> 1) * (kSpPairHalfN * 128) + (ks & 1) * 64,
                                                                   0, 1024, SWIZZLE_128B_DESC);
                            mma_i8_sp_pair(d_tmem, a_desc, b_desc, e_tmem + 2 * ks, idesc, (kb | ks) != 0 ? 1u : 0u);
                        }
                    }
                    tc_commit_pair(empty_bar(stage));
                    tc_commit_pair(mapa_shared(empty_bar(stage), 1));
                    if (++stage == kSpPairStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc_commit_pair(acc_full_bar(acc));
                tc_commit_pair(mapa_shared(acc_full_bar(acc), 1));
                acc ^= 1u;
                if (acc == 0) acc_phase ^= 1u;
            }
            if (!ok) {
                tc_commit_pair(drain_bar);
                uint64_t t0 = global_timer_ns();
                while (!mbar_try_wait(drain_bar, 0) && global_timer_ns() - t0 < 20000000ull) {}
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps (both CTAs)
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        EpiStrip<kSpPairNC>* strip = reinterpret_cast<EpiStrip<kSpPairNC>*>(smem_gen + kSpPairStripOffset) + (warp - 2);
        uint32_t acc = 0, acc_phase = 0;
        [[maybe_unused]] uint32_t box_count = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs) {
            const int n0 = tile_rb(tile) * 256 + static_cast<int>(rank) * 128;           // first sparse row (channel) of this CTA
            const int tile_t0 = tile_cb(tile) * kSpPairBN;
            const int t0 = tile_t0 + half * kSpPairNC;                                         // first accumulator column of this warp
            const int cross_extent = LEFT ? p.epi.cols : p.epi.rows;
            const int t_limit = cross_extent < tile_t0 + kSpPairBN ? cross_extent : tile_t0 + kSpPairBN;
            const int channel = n0 + quarter * 32 + lane;
            stage_strip<EPI, kSpPairNC, !LEFT>(p.epi, strip, t0, lane);
            const float lane_s = lane_scale_of<EPI, !LEFT>(p.epi, channel);
            if (!bounded_wait(acc_full_bar(acc), acc_phase, abort_flag, p.status, DEV_TIMEOUT_EPI_ACC_FULL))
                break;
            tc_fence_after_sync();
            const uint32_t taddr =
                tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kSpPairBN + half * kSpPairNC;
            bool stored = false;
            if constexpr (LEFT) {
                if (p.epi.tma_ok) {
                    drain_tma_from<EPI, kSpPairNC, 1>(p.epi, &map_out, 1, TmemSource{taddr}, n0 + quarter * 32, lane, t0, strip,
                                                      lane_s, smem_base + PC::STORE_OFFSET + (warp - 2) * kStoreBoxBytes,
                                                      box_count, t_limit);
                    stored = true;
                }
            }
            if (!stored) drain_accumulator<EPI, kSpPairNC, !LEFT>(p.epi, taddr, channel, t0, t_limit, strip, lane_s);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(acc_empty_bar(acc), 0));
            acc ^= 1u;
            if (acc == 0) acc_phase ^= 1u;
        }
        if constexpr (LEFT) {
            if (lane == 0) bulk_wait_all();          // the staging strips are read by stores still in flight
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {}
    }
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kSpPairTmemCols);
    }
}

}  // namespace bm
