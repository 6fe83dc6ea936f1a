// igemm_dense_pair.cuh — dense INT8 GEMM on CTA PAIRS: tcgen05.mma.cta_group::2, M = 256.
//
// Two CTAs of a 2-CTA cluster (two neighbouring SMs) compute one 256 x 256 output tile.  CTA r
// of the pair owns accumulator rows [128 r, 128 r + 128) in ITS tensor memory and stages, per
// K block, only ITS halves of the operands: 128 rows of A and 128 of the 256 columns of B.
// The MMA, issued by one lane of the leader CTA (rank 0), reads A from each CTA's own shared
// memory and the two B halves from both.  Per SM and K byte that is 256 operand bytes for
// 32768 MACs (4 tensor clocks) — 64 B/clk, against 96 B/clk for a lone 128 x 256 CTA, whose
// measured fill rate (~65 B/clk/SM) is what caps it.  No copy is multicast: each CTA issues
// plain TMA loads into its own shared memory.
//
// Synchronisation across the pair
//   full[s]      lives in the LEADER: both producers' TMA bytes are counted there (the peer
//                names the leader's barrier through its shared::cluster address); the leader's
//                producer arms it with the byte count of both CTAs.
//   empty[s]     one per CTA: the leader's MMA lane commits to both when the stage's MMAs retire.
//   acc_full[a]  one per CTA: committed to both when a tile's last MMA retires.
//   acc_empty[a] lives in the LEADER: one arrival per epilogue warp of either CTA.
// Every wait is bounded as in the single-CTA kernel; the CTAs meet at a cluster barrier
// before tensor memory is freed, so neither exits while its peer can still touch it.
#pragma once
#include "epilogue.cuh"
#include "igemm_dense.cuh"
#include "sm100_ptx.cuh"

namespace bm {

constexpr int kPairBN = 256;                       // tile columns (MMA N)
constexpr int kPairHalfN = kPairBN / 2;            // B columns staged per CTA
constexpr int kPairBBytes = kPairHalfN * kBK;      // 16 KiB
constexpr int kPairStageBytes = kABytes + kPairBBytes;   // 32 KiB per CTA and stage
#ifndef BM_PAIR_STAGES
#define BM_PAIR_STAGES 4
#define BM_PAIR_STORE_BUFS 2
#endif
constexpr int kPairStages = BM_PAIR_STAGES;        // 128 KiB ring
constexpr int kPairStoreBufs = BM_PAIR_STORE_BUFS; // staging strips per epilogue warp
constexpr int kPairTmemCols = 2 * kPairBN;         // two accumulators
constexpr int kPairStoreOffset = kPairStages * kPairStageBytes;   // per-warp TMA-store staging
constexpr int kPairBarOffset = kPairStoreOffset + kEpiWarps * kPairStoreBufs * kStoreBoxBytes;
constexpr int kPairNC = kPairBN / 2;                // columns drained per epilogue warp
constexpr int kPairStripOffset = kPairBarOffset + (2 * kPairStages + 5) * 8 + 16;
constexpr int kPairSmemBytes = kPairStripOffset + kEpiWarps * (int)sizeof(EpiStrip<kPairNC>) + 1024;

// Work of one CTA pair: whole tiles pair, pair+P, ... below `tail_first`, then (half-height tail) one
// 128-row half of one tile of the partly filled last wave.
struct PairWork {
    int tile;
    int nhalf;                          // < 0: all 256 rows; 0 / 1: rows [128 nhalf, +128) of the tile only (a half-height unit)
};
struct PairWorkIter {
    int next_tile, pairs, tiles, tail_first, pair;
    bool tail_done, narrow;
    __device__ PairWorkIter(int pair_, int pairs_, int tiles_, int tail_first_, bool narrow_)
        : next_tile(pair_), pairs(pairs_), tiles(tiles_), tail_first(narrow_ ? tail_first_ : tiles_), pair(pair_),
          tail_done(false), narrow(narrow_) {}
    __device__ bool next(PairWork& w) {
        w.nhalf = -1;
        if (next_tile < tail_first) {
            w.tile = next_tile;
            next_tile += pairs;
            return true;
        }
        if (narrow && !tail_done) {
            tail_done = true;
            if (pair < (tiles - tail_first) * 2) {                   // pair u takes row half u % 2 of tail tile u / 2
                w.tile = tail_first + pair / 2;
                w.nhalf = pair % 2;
                return true;
            }
        }
        return false;
    }
};

template <bool B_MN, int EPI>
__global__ void __launch_bounds__(kDenseThreads, 1)
igemm_dense_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ CUtensorMap map_a_short, const __grid_constant__ OutMaps maps_out,
                        const DenseParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t a_smem0 = smem_base;
    const uint32_t b_smem0 = smem_base + kPairStages * kABytes;
    const uint32_t bar0 = smem_base + kPairBarOffset;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kPairStages + s); };
    auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * kPairStages + a); };
    auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * kPairStages + 2 + a); };
    const uint32_t drain_bar = bar0 + 8u * (2 * kPairStages + 4);
    const uint32_t tmem_slot = bar0 + 8u * (2 * kPairStages + 5);
    volatile uint32_t* tmem_slot_gen =
        reinterpret_cast<volatile uint32_t*>(smem_gen + kPairBarOffset + 8 * (2 * kPairStages + 5));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot_gen + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();        // 0 = leader
    const uint32_t peer = rank ^ 1u;
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;
    const int num_tiles = p.tiles_m * p.tiles_n;    // tiles of 256 x 256

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPairStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full_bar(a), 1);
            mbar_init(acc_empty_bar(a), 2 * kEpiWarps);   // the epilogue warps of both CTAs (used in the leader)
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, kPairTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_arrive();                                // the peer's barriers exist before anyone signals them
    cluster_wait();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_gen;
    pdl_launch_dependents();      // the next kernel of the stream may start its own set-up
    pdl_wait_prior_grid();        // nothing global is touched before the previous grid is complete

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            prefetch_tensormap(&map_a);
            prefetch_tensormap(&map_b);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            PairWorkIter work(pair, num_pairs, num_tiles, p.tail_first, p.tail_narrow != 0);
            PairWork w;
            while (ok && work.next(w)) {
                int tm, tn;
                pair_tile_coords(p, w.tile, tm, tn);
                const int m0 = tm * 256 + static_cast<int>(rank) * kBM;
                // half-height unit: 128 rows of the tile, 64 per CTA (an M = 128 pair MMA); B as for a whole tile
                const bool narrow = w.nhalf >= 0;
                const int n0 = tn * kPairBN + static_cast<int>(rank) * kPairHalfN;
                const int m0s = tm * 256 + w.nhalf * 128 + static_cast<int>(rank) * 64;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!bounded_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status,
                                      DEV_TIMEOUT_PRODUCER_EMPTY)) { ok = false; break; }
                    const uint32_t leader_full = mapa_shared(full_bar(stage), 0);
                    if (rank == 0) mbar_expect_tx(full_bar(stage), narrow ? 2 * (kABytes / 2 + kPairBBytes) : 2 * kPairStageBytes);
                    if (narrow) tma_load_2d_pair(a_smem0 + stage * kABytes, &map_a_short, leader_full, kb * kBK, m0s);
                    else        tma_load_2d_pair(a_smem0 + stage * kABytes, &map_a, leader_full, kb * kBK, m0);
                    if constexpr (B_MN)
                        tma_load_2d_pair(b_smem0 + stage * kPairBBytes, &map_b, leader_full, n0, kb * kBK);
                    else
                        tma_load_2d_pair(b_smem0 + stage * kPairBBytes, &map_b, leader_full, kb * kBK, n0);
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc_full = make_idesc_i8(256, kPairBN, B_MN, false);
            constexpr uint32_t idesc_narrow = make_idesc_i8(128, kPairBN, B_MN, false);   // 64 rows per CTA
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            PairWorkIter work(pair, num_pairs, num_tiles, p.tail_first, p.tail_narrow != 0);
            PairWork w;
            while (ok && work.next(w)) {
                if (!bounded_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort_flag, p.status,
                                  DEV_TIMEOUT_MMA_ACC_EMPTY)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * kPairBN;
                const uint32_t idesc = w.nhalf >= 0 ? idesc_narrow : idesc_full;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!bounded_wait(full_bar(stage), phase, abort_flag, p.status, DEV_TIMEOUT_MMA_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = a_smem0 + stage * kABytes;
                    const uint32_t b_addr = b_smem0 + stage * kPairBBytes;
#pragma unroll
                    for (int ks = 0; ks < kBK / kUmmaK; ++ks) {
                        const uint64_t a_desc = make_smem_desc(a_addr + ks * kUmmaK, 0, 1024, SWIZZLE_128B_DESC);
                        const uint64_t b_desc =
                            B_MN ? make_smem_desc(b_addr + ks * (kUmmaK * 128), 128 * kBK, 1024, SWIZZLE_128B_DESC)
                                 : make_smem_desc(b_addr + ks * kUmmaK, 0, 1024, SWIZZLE_128B_DESC);
                        mma_i8_pair(d_tmem, a_desc, b_desc, idesc, (kb | ks) != 0 ? 1u : 0u);
                    }
                    tc_commit_pair(empty_bar(stage));                       // this CTA's producer
                    tc_commit_pair(mapa_shared(empty_bar(stage), 1));       // the peer's producer
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
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
        EpiStrip<kPairNC>* strip = reinterpret_cast<EpiStrip<kPairNC>*>(smem_gen + kPairStripOffset) + (warp - 2);
        uint32_t acc = 0, acc_phase = 0, box_count = 0;
        PairWorkIter work(pair, num_pairs, num_tiles, p.tail_first, p.tail_narrow != 0);
        PairWork w;
        while (work.next(w)) {
            int tm, tn;
            pair_tile_coords(p, w.tile, tm, tn);
            const int m0 = tm * 256 + static_cast<int>(rank) * kBM;
            // Whole tile: lanes = the CTA's 128 rows, this warp drains TMEM columns [128 half, +128).
            // Half-height unit (M = 128 on the pair): the CTA's 64 rows sit in lanes 0-63 for output columns
            // [0,128) and again in lanes 64-127 for output columns [128,256); 128 TMEM columns are in use and
            // this warp drains 64 of them.
            const bool narrow = w.nhalf >= 0;
            const int row_base = narrow ? tm * 256 + w.nhalf * 128 + static_cast<int>(rank) * 64 + (quarter & 1) * 32
                                        : m0 + quarter * 32;
            const int n0 = tn * kPairBN + (narrow ? (quarter >> 1) * 128 + half * 64 : half * kPairNC);
            const int row = row_base + lane;
            const int col_limit = narrow ? (p.epi.cols < n0 + 64 ? p.epi.cols : n0 + 64) : p.epi.cols;
            stage_strip<EPI, kPairNC, false>(p.epi, strip, n0, lane);
            const float lane_s = lane_scale_of<EPI, false>(p.epi, row);
            if (!bounded_wait(acc_full_bar(acc), acc_phase, abort_flag, p.status, DEV_TIMEOUT_EPI_ACC_FULL))
                break;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kPairBN +
                                   (narrow ? half * 64 : half * kPairNC);
            const uint32_t my_stage = smem_base + kPairStoreOffset + (warp - 2) * kPairStoreBufs * kStoreBoxBytes;
            if (p.epi.tma_ok)
                drain_accumulator_tma<EPI, kPairNC, kPairStoreBufs>(p.epi, maps_out.m, p.n_out, taddr, row_base, lane,
                                                                    n0, strip, lane_s, my_stage, box_count, col_limit, p.pace);
            else
                drain_accumulator<EPI, kPairNC, false>(p.epi, taddr, row, n0, col_limit, strip, lane_s);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(acc_empty_bar(acc), 0));
            acc ^= 1u;
            if (acc == 0) acc_phase ^= 1u;
        }
        if (lane == 0) bulk_wait_all();
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // aborting: give copies still in flight (their completion is counted in the leader) time to land
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {}
    }
    __syncthreads();
    cluster_arrive();                                // neither CTA leaves while its peer may still use it
    cluster_wait();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kPairTmemCols);
    }
    (void)peer;
}

}  // namespace bm
