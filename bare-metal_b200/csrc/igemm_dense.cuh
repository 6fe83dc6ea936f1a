// igemm_dense.cuh — dense INT8 GEMM for sm_100a: s8 x s8 -> s32 on the tcgen05 tensor cores.
//
// One persistent CTA per SM walks output tiles of 128 x BN.  Three warp roles:
//   warp 0      TMA producer  — one lane streams 128-byte-swizzled operand tiles into a
//                               ring of shared-memory stages (mbarrier full/empty pairs)
//   warp 1      MMA issuer    — one lane issues tcgen05.mma.kind::i8 (M=128, N=BN, K=32),
//                               four per stage; accumulators live in tensor memory, two of
//                               them, so tile t+1 accumulates while tile t is drained
//   warps 2..9  epilogue      — two warps per tensor-memory lane quarter, each draining half of
//                               the tile's columns: double-buffered tcgen05.ld, fused
//                               dequantise and cast, vectorised stores
//
// Operand layouts
//   A        [M x K] row-major (K-major), always
//   B_MN=0   W[N x K] row-major: K-major right-hand side, the tensor core's natural form
//   B_MN=1   B[K x N] row-major: the reference ABI; loaded as [K rows x 128 N-bytes] boxes
//            and described to the MMA as an MN-major operand (no transpose pass)
// Out-of-range parts of a TMA box read as zero, so ragged M/N/K need no special mainloop;
// the epilogue masks stores.
//
// HBM traffic per launch (algorithmic): M*K + K*N bytes in, M*N*sizeof(out) out.
#pragma once
#include "epilogue.cuh"
#include "sm100_ptx.cuh"

namespace bm {

constexpr int kBM = 128;          // tile rows = tensor-memory lanes
constexpr int kBK = 128;          // K bytes per stage = one 128-byte swizzle span
constexpr int kUmmaK = 32;        // K per tcgen05.mma for 8-bit operands
constexpr int kEpiWarps = 8;            // two per tensor-memory lane quarter
constexpr int kDenseThreads = 64 + 32 * kEpiWarps;
constexpr int kABytes = kBM * kBK;               // 16 KiB
constexpr int kSmemBudget = 160 * 1024;          // operand ring budget (the rest: store staging, strips)

template <int BN>
struct DenseCfg {
    static constexpr int B_BYTES = BN * kBK;
    static constexpr int STAGE_BYTES = kABytes + B_BYTES;
    static constexpr int STAGES_RAW = kSmemBudget / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int TMEM_COLS_RAW = 2 * BN;
    static constexpr int TMEM_COLS = TMEM_COLS_RAW < 32 ? 32 : TMEM_COLS_RAW;   // 64..512: powers of two
    static constexpr int STORE_OFFSET = STAGES * STAGE_BYTES;     // per-warp TMA-store staging, 1 KiB aligned
    static constexpr int BAR_OFFSET = STORE_OFFSET + kEpiWarps * kStoreBoxBytes;
    // full[STAGES] empty[STAGES] acc_full[2] acc_empty[2] drain[1], then tmem slot + abort flag,
    // then one strip of column-side epilogue parameters per epilogue warp
    static constexpr int NC = BN / 2;                              // columns drained per epilogue warp
    static constexpr int STRIP_OFFSET = BAR_OFFSET + (2 * STAGES + 5) * 8 + 16;
    static constexpr int SMEM_BYTES = STRIP_OFFSET + kEpiWarps * (int)sizeof(EpiStrip<NC>) + 1024 /*alignment slack*/;
};

struct DenseParams {
    EpilogueParams epi;
    int tiles_m, tiles_n, k_blocks;
    int* status;
    int n_out;                 // number of output destinations in the OutMaps argument (1 unless gathering)
    StorePace pace;            // gathering: which destinations are remote and how their stores are paced
    // half-height tail (CTA-pair kernel): tiles [0, tail_first) run whole, wave after wave; the tiles of
    // the partly filled last wave are computed as two 128 x 256 halves by different pairs — no
    // reduction, just shorter units for pairs that would otherwise idle.
    int tail_first, tail_narrow;
    // tile order of the CTA-pair kernel: 0 = row tiles fastest over the whole matrix; G > 0 = bands of G
    // row tiles, inside a band row tiles fastest (a wave then touches G row tiles x pairs/G column tiles)
    int group_m;
};

// (row tile, column tile) of linear tile index `tile` under DenseParams::group_m
__device__ __forceinline__ void pair_tile_coords(const DenseParams& p, int tile, int& tm, int& tn) {
    if (p.group_m <= 0) {
        tm = tile % p.tiles_m;
        tn = tile / p.tiles_m;
        return;
    }
    const int band_tiles = p.group_m * p.tiles_n;
    const int band = tile / band_tiles, r = tile - band * band_tiles;
    const int left = p.tiles_m - band * p.group_m;
    const int rows = left < p.group_m ? left : p.group_m;       // the last band may be short
    tm = band * p.group_m + r % rows;
    tn = r / rows;
}

template <int BN, bool B_MN, int EPI>
__global__ void __launch_bounds__(kDenseThreads, 1)
igemm_dense_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ OutMaps maps_out, const DenseParams p) {
    using Cfg = DenseCfg<BN>;
    static_assert(!B_MN || BN % 128 == 0, "MN-major B is loaded in 128-column boxes");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzle atoms are 1 KiB
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t a_smem0 = smem_base;
    const uint32_t b_smem0 = smem_base + Cfg::STAGES * kABytes;
    const uint32_t bar0 = smem_base + Cfg::BAR_OFFSET;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (Cfg::STAGES + s); };
    auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * Cfg::STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * Cfg::STAGES + 2 + a); };
    const uint32_t drain_bar = bar0 + 8u * (2 * Cfg::STAGES + 4);
    const uint32_t tmem_slot = bar0 + 8u * (2 * Cfg::STAGES + 5);
    volatile uint32_t* tmem_slot_gen =
        reinterpret_cast<volatile uint32_t*>(smem_gen + Cfg::BAR_OFFSET + 8 * (2 * Cfg::STAGES + 5));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot_gen + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_tiles = p.tiles_m * p.tiles_n;
    constexpr uint32_t nstages = Cfg::STAGES;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full_bar(a), 1);
            mbar_init(acc_empty_bar(a), kEpiWarps);   // one arrival per epilogue warp
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_gen;
    pdl_launch_dependents();      // the next kernel of the stream may start its own set-up
    pdl_wait_prior_grid();        // nothing global is touched before the previous grid is complete

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            prefetch_tensormap(&map_a);
            prefetch_tensormap(&map_b);
            uint32_t stage = 0, phase = 0, issued = 0, issued_parity = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const int m0 = (tile % p.tiles_m) * kBM;
                const int n0 = (tile / p.tiles_m) * BN;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!bounded_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status,
                                      DEV_TIMEOUT_PRODUCER_EMPTY)) { ok = false; break; }
                    const uint32_t bar = full_bar(stage);
                    mbar_expect_tx(bar, Cfg::STAGE_BYTES);
                    tma_load_2d(a_smem0 + stage * kABytes, &map_a, bar, kb * kBK, m0);
                    if constexpr (B_MN) {
#pragma unroll
                        for (int j = 0; j < BN / 128; ++j)
                            tma_load_2d(b_smem0 + stage * Cfg::B_BYTES + j * (128 * kBK), &map_b, bar,
                                        n0 + j * 128, kb * kBK);
                    } else {
                        tma_load_2d(b_smem0 + stage * Cfg::B_BYTES, &map_b, bar, kb * kBK, n0);
                    }
                    issued |= 1u << stage;
                    issued_parity = (issued_parity & ~(1u << stage)) | (phase << stage);
                    if (++stage == nstages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // aborting: let the copies already in flight land before the CTA gives up its smem
                for (int s = 0; s < Cfg::STAGES; ++s)
                    if (issued & (1u << s)) {
                        uint64_t t0 = global_timer_ns();
                        while (!mbar_try_wait(full_bar(s), (issued_parity >> s) & 1u) &&
                               global_timer_ns() - t0 < 20000000ull) {}
                    }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_i8(kBM, BN, B_MN, false);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                if (!bounded_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort_flag, p.status,
                                  DEV_TIMEOUT_MMA_ACC_EMPTY)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!bounded_wait(full_bar(stage), phase, abort_flag, p.status, DEV_TIMEOUT_MMA_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = a_smem0 + stage * kABytes;
                    const uint32_t b_addr = b_smem0 + stage * Cfg::B_BYTES;
#pragma unroll
                    for (int ks = 0; ks < kBK / kUmmaK; ++ks) {
                        // K-major, 128B swizzle: 8-row groups are 1 KiB apart; a K step of 32 bytes
                        // moves the start address inside the swizzle span.
                        const uint64_t a_desc = make_smem_desc(a_addr + ks * kUmmaK, 0, 1024, SWIZZLE_128B_DESC);
                        uint64_t b_desc;
                        if constexpr (B_MN) {
                            // MN-major, 128B swizzle: 128 N-bytes contiguous, 8 K-rows per 1 KiB atom
                            // (stride-dimension offset), next 128-column block one box (16 KiB) on
                            // (leading-dimension offset); a K step of 32 rows is 4 KiB.
                            b_desc = make_smem_desc(b_addr + ks * (kUmmaK * 128), 128 * kBK, 1024,
                                                    SWIZZLE_128B_DESC);
                        } else {
                            b_desc = make_smem_desc(b_addr + ks * kUmmaK, 0, 1024, SWIZZLE_128B_DESC);
                        }
                        mma_i8(d_tmem, a_desc, b_desc, idesc, (kb | ks) != 0 ? 1u : 0u);
                    }
                    tc_commit(empty_bar(stage));            // frees the stage when these MMAs retire
                    if (++stage == nstages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc_commit(acc_full_bar(acc));               // accumulator complete
                acc ^= 1u;
                if (acc == 0) acc_phase ^= 1u;
            }
            if (!ok) {
                // aborting: wait for MMAs in flight before tensor memory is released
                tc_commit(drain_bar);
                uint64_t t0 = global_timer_ns();
                while (!mbar_try_wait(drain_bar, 0) && global_timer_ns() - t0 < 20000000ull) {}
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3;                        // tensor-memory lanes 32q .. 32q+31
        const int half = (warp - 2) >> 2;                    // which half of the tile's columns
        EpiStrip<Cfg::NC>* strip =
            reinterpret_cast<EpiStrip<Cfg::NC>*>(smem_gen + Cfg::STRIP_OFFSET) + (warp - 2);
        uint32_t acc = 0, acc_phase = 0, box_count = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            const int m0 = (tile % p.tiles_m) * kBM;
            const int n0 = (tile / p.tiles_m) * BN + half * Cfg::NC;
            const int row = m0 + quarter * 32 + lane;
            // column-side parameters of this tile, fetched while its MMAs are still running
            stage_strip<EPI, Cfg::NC, false>(p.epi, strip, n0, lane);
            const float lane_s = lane_scale_of<EPI, false>(p.epi, row);
            if (!bounded_wait(acc_full_bar(acc), acc_phase, abort_flag, p.status, DEV_TIMEOUT_EPI_ACC_FULL))
                break;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN + half * Cfg::NC;
            bool stored = false;
            if constexpr (Cfg::NC * sizeof(typename OutType<EPI>::type) >= 128) {
                if (p.epi.tma_ok) {
                    drain_accumulator_tma<EPI, Cfg::NC, 1>(p.epi, maps_out.m, p.n_out, taddr, m0 + quarter * 32, lane, n0, strip,
                                                           lane_s, smem_base + Cfg::STORE_OFFSET + (warp - 2) * kStoreBoxBytes,
                                                           box_count, p.epi.cols, p.pace);
                    stored = true;
                }
            }
            if (!stored) drain_accumulator<EPI, Cfg::NC, false>(p.epi, taddr, row, n0, p.epi.cols, strip, lane_s);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(acc));
            acc ^= 1u;
            if (acc == 0) acc_phase ^= 1u;
        }
        if (lane == 0) bulk_wait_all();                      // TMA stores of this warp have landed
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

}  // namespace bm
