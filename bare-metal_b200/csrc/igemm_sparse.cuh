// igemm_sparse.cuh — 2:4 structured-sparse INT8 GEMM for sm_100a on tcgen05.mma.sp.kind::i8.
//
// The sparse operand S [R x K] (stored as its kept half, comp [R x K/2], plus 4-bit-per-group
// position metadata) always sits in the tensor core's A slot, so its rows are the 128
// tensor-memory lanes of a tile.  The dense operand takes the B slot, either
//   DENSE_MN=0  X[C x K] row-major (K-major): rows are the tile's BN accumulator columns
//   DENSE_MN=1  B[K x C] row-major (the reference ABI, igemm_sparse_tiled.cu:88-96), described
//               to the MMA as MN-major
// Output orientation
//   TRANSPOSED=0  out[r][c]  — sparse operand on the left (reference sparse kernels)
//   TRANSPOSED=1  out[c][r]  — sparse WEIGHTS W[N x K]: lanes are output channels, accumulator
//                              columns are tokens (D^T = W * X^T), decode shapes use a narrow BN
//
// Per k-block (256 logical K) a stage holds: comp tile 128 x 128 B (128B swizzle, TMA),
// dense tile BN x 256 B (two 128B-swizzled boxes) and 4 KiB of metadata (one bulk copy).
// The MMA lane copies the metadata shared -> tensor memory with two tcgen05.cp.128x128b
// (each: 128 rows x 16 B = 128 logical K) and issues four tcgen05.mma.sp (K = 64 logical);
// each reads its 2 metadata columns.  Metadata has its own tensor-memory columns per stage.
//
// Metadata, tiled order (what bm_sp_pack_meta writes): for row block rb (128 rows) and
// k-block kb (256 logical K): 2 chunks x 128 rows x 16 bytes, chunk-major; byte b of a
// row's 16 covers logical K [8b, 8b+8): low nibble = first group of 4, high nibble = second;
// nibble = (idx1 << 2) | idx0.
//
// HBM traffic per launch (algorithmic): R*K/2 + R*K/8 + C*K bytes in, R*C*sizeof(out) out.
#pragma once
#include "epilogue.cuh"
#include "igemm_dense.cuh"
#include "sm100_ptx.cuh"

namespace bm {

constexpr int kSpKLogical = 256;                 // logical K per stage
constexpr int kSpMetaBytes = 4096;               // metadata bytes per (128-row block, k-block)
constexpr int kSpSmemBudget = 216 * 1024;         // one CTA per SM
constexpr int kSpSmemBudgetNarrow = 100 * 1024;   // narrow token tiles (decode): two CTAs per SM

// ROWS < 128 (packed weights, row-balanced decode tiles only): a stage holds at most ROWS rows of the sparse
// operand, so the ring is deeper — a CTA that was dealt a few dozen rows (a slab of an N-split layer) walks its
// K blocks with up to 12 of them in flight instead of 4.  The MMA still spans 128 lanes; what it reads beyond the
// stage's rows (the following stages' bytes) lands in accumulator lanes nobody stores.
template <int BN, int ROWS = kBM>
struct SparseCfg {
    static constexpr int A_BYTES = ROWS * 128;                    // compressed values (16 KiB for 128 rows)
    static constexpr int B_BYTES = BN * kSpKLogical;              // dense operand
    static constexpr int E_BYTES = ROWS * 32;                     // metadata (kSpMetaBytes for 128 rows)
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + E_BYTES;
    // Decode-shaped tiles (BN <= 64) take half an SM each: two CTAs per SM keep twice as many
    // independent streams in flight and let the CTAs of the next launch settle in while the last
    // ones of this launch drain.
    static constexpr int CTAS_PER_SM = BN <= 64 ? 2 : 1;
    static constexpr int STAGES_RAW = (BN <= 32 ? kSpSmemBudgetNarrow : BN == 64 ? 108 * 1024 : kSpSmemBudget) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > (ROWS < kBM ? 12 : 8) ? (ROWS < kBM ? 12 : 8) : STAGES_RAW;
    static constexpr int E_COLS = STAGES * 8;                     // 2 x tcgen05.cp of 4 columns per stage
    static constexpr int ACC_BUFS = (2 * BN + E_COLS <= 512) ? 2 : 1;
    static constexpr int E_BASE = ACC_BUFS * BN;
    static constexpr int COLS_NEEDED = E_BASE + E_COLS;
    static constexpr int TMEM_COLS = COLS_NEEDED <= 32 ? 32 : COLS_NEEDED <= 64 ? 64 : COLS_NEEDED <= 128 ? 128
                                   : COLS_NEEDED <= 256 ? 256 : 512;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int EPI_WARPS = BN >= 64 ? 8 : 4;            // two per lane quarter from 64 columns up
    static constexpr int NC = BN >= 64 ? BN / 2 : 32;             // accumulator columns drained per warp
    static constexpr int THREADS = 64 + 32 * EPI_WARPS;
    static constexpr int STRIP_OFFSET = BAR_OFFSET + (2 * STAGES + 5) * 8 + 16;
    static constexpr int SMEM_BYTES = STRIP_OFFSET + EPI_WARPS * (int)sizeof(EpiStrip<NC>) + 1024;
    static_assert(STAGES >= 2, "tile too large for the shared-memory ring");
    static_assert(ROWS == kBM || (ROWS % 8 == 0 && STAGES * B_BYTES >= kBM * 128), "short stages: over-read must stay inside the ring");
    static_assert(COLS_NEEDED <= 512, "tensor memory over-subscribed");
};

// Packed weights (what the decode-shaped GEMM streams): for every 256-wide K block kb one slice of
// rows_padded x 160 bytes — first the compressed values of ALL rows (128 B per row, pre-swizzled), then the
// metadata of all rows in groups of 8 rows (256 B per group: the 16 bytes of K half 0 of the 8 rows, then
// those of K half 1).  Any range of rows that starts on a multiple of 8 is then two contiguous pieces per K
// block, whatever 128-row block it starts in: one bulk copy of values and one of metadata per pipeline stage.
constexpr int kSpPackedRowBytes = 160;

struct SparseParams {
    EpilogueParams epi;
    const uint8_t* meta_tiled;         // tiled metadata, or the packed weight blocks when PACKED
    int tiles_r, tiles_c, k_blocks;    // row blocks of the sparse operand, column tiles of the dense one
    int* status;
    // row-balanced mode (packed weights, one column tile — the decode shapes): the rows of the
    // sparse operand are dealt out evenly in multiples of 8, so a CTA's last tile may hold fewer
    // than 128 rows and only those rows are fetched (packed weights are row-contiguous within a K block).
    int row_balanced;
    int sparse_rows;                   // rows of the sparse operand (R)
    // tile order of the pair kernel: 0 = row blocks of the sparse operand fastest (consecutive pairs share
    // a tile of the dense operand), 1 = column tiles fastest (consecutive pairs share a block of the
    // sparse operand — for weights larger than L2 and few column tiles, so each block leaves HBM once)
    int col_first;
};

// One piece of work: a tile over its whole K range; the tile covers rows [row0, row0 + nrows) of the
// sparse operand (nrows = 128 except in row-balanced mode).
struct WorkSegment {
    int tile, row0, nrows;
};

// Deals work to CTA `cta` of `ctas`: whole tiles cta, cta+ctas, ..., or (row-balanced mode) one
// contiguous range of rows cut into tiles of at most 128.
struct WorkIter {
    int tile, tiles, step, tiles_r;
    int row, row_end;                  // row-balanced mode
    bool row_balanced;
    int tile_rows;                     // rows per tile in row-balanced mode (128, or the kernel's shorter stage)
    __device__ WorkIter(const SparseParams& p, int cta, int ctas, int tiles_, int tile_rows_ = 128)
        : tile(cta), tiles(tiles_), step(ctas), tiles_r(p.tiles_r), row_balanced(p.row_balanced != 0),
          tile_rows(tile_rows_) {
        const long long r8 = (p.sparse_rows + 7) / 8;
        row = static_cast<int>(r8 * cta / ctas) * 8;
        row_end = static_cast<int>(r8 * (cta + 1) / ctas) * 8;
    }
    __device__ bool next(WorkSegment& s) {
        if (row_balanced) {
            if (row >= row_end) return false;
            s.tile = 0;
            s.row0 = row;
            s.nrows = row_end - row < tile_rows ? row_end - row : tile_rows;
            row += s.nrows;
            return true;
        }
        if (tile >= tiles) return false;
        s.tile = tile;
        s.row0 = (tile % tiles_r) * 128;
        s.nrows = 128;
        tile += step;
        return true;
    }
};

// F16 = true turns the same pipeline into the FP16 2:4 GEMM of kernels/gemm/hgemm_sparse
// (hgemm_sparse_tiled.cu:122-129: fp16 A_comp[M x K/2], fp16 B[K x N], fp32 C): in BYTES a stage
// looks the same — 128 rows x 128 B of compressed values, BN x 256 B of the dense operand — but
// covers 128 logical K instead of 256, carries half the metadata (16 B per row: one
// tcgen05.cp.128x128b, one 32-bit column per MMA of K = 32, named as column pair + selector) and its four MMAs are
// tcgen05.mma.sp.kind::f16 with fp32 accumulators, whose bits the EPI_I32 epilogue stores as they
// are.  BN counts fp16 elements; the tensor maps are byte maps (inner extents doubled).  Only the
// reference orientation is built: DENSE_MN, not TRANSPOSED, not PACKED.
template <int BN, bool DENSE_MN, bool TRANSPOSED, int EPI, bool PACKED = false, bool F16 = false, int ROWS = kBM>
__global__ void __launch_bounds__(SparseCfg<BN, ROWS>::THREADS, SparseCfg<BN, ROWS>::CTAS_PER_SM)
igemm_sparse_kernel(const __grid_constant__ CUtensorMap map_s, const __grid_constant__ CUtensorMap map_d,
                    const SparseParams p) {
    using Cfg = SparseCfg<BN, ROWS>;
    static_assert(ROWS == kBM || (PACKED && TRANSPOSED), "short stages are for row-balanced tiles of packed weights");
    static_assert(!DENSE_MN || BN % 128 == 0, "MN-major dense operand is loaded in 128-column boxes");
    static_assert(!F16 || (DENSE_MN && !TRANSPOSED && !PACKED && EPI == EPI_I32), "fp16: reference orientation only");
    constexpr bool ROTATE_K = TRANSPOSED && BN <= 64;         // decode shapes: per-CTA starting K block (see the producer)
    constexpr int kKRows = F16 ? 128 : kSpKLogical;          // logical K (= rows of B[K x N]) per stage
    constexpr int kMetaStage = F16 ? 2048 : kSpMetaBytes;    // metadata bytes fetched per stage
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    // ring order: values, dense operand, metadata — with short stages metadata first, so that what the 128-lane
    // MMA and metadata copy read beyond a short stage is always ring memory (values, then the dense operand)
    const uint32_t e_short0 = smem_base;
    const uint32_t a_smem0 = ROWS == kBM ? smem_base : e_short0 + Cfg::STAGES * Cfg::E_BYTES;
    const uint32_t b_smem0 = a_smem0 + Cfg::STAGES * Cfg::A_BYTES;
    const uint32_t e_smem0 = ROWS == kBM ? b_smem0 + Cfg::STAGES * Cfg::B_BYTES : e_short0;
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
    const int num_tiles = p.tiles_r * p.tiles_c;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full_bar(a), 1);
            mbar_init(acc_empty_bar(a), Cfg::EPI_WARPS);
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
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            if constexpr (!PACKED) prefetch_tensormap(&map_s);
            prefetch_tensormap(&map_d);
            uint32_t stage = 0, phase = 0, issued = 0, issued_parity = 0;
            bool ok = true;
            WorkIter work(p, blockIdx.x, gridDim.x, num_tiles, ROWS);
            WorkSegment seg;
            while (ok && work.next(seg)) {
                const int r0 = seg.row0;
                const int c0 = (seg.tile / p.tiles_r) * BN;
                // tiled metadata is laid out in 4 KiB blocks of 256 logical K; an fp16 k-block is half of one
                const uint8_t* meta_row = p.meta_tiled + static_cast<size_t>(r0 / kBM) *
                                                             (F16 ? (p.k_blocks + 1) / 2 : p.k_blocks) * kSpMetaBytes;
                // packed weights: one slice of (padded rows) x 160 bytes per K block, values first
                const size_t rows_padded = static_cast<size_t>(p.tiles_r) * kBM;
                // Decode shapes: every CTA walks the K blocks of its tile from a different starting block and wraps
                // around (exact integer sums do not care about the order).  All CTAs read the SAME few tokens; in
                // lockstep they would all ask the L2 for the same 16 KiB of activations at the same moment.
                const int rot = ROTATE_K ? static_cast<int>((blockIdx.x * 7u) % static_cast<unsigned>(p.k_blocks)) : 0;
                for (int kb_seq = 0; kb_seq < p.k_blocks; ++kb_seq) {
                    const int kb = kb_seq + rot < p.k_blocks ? kb_seq + rot : kb_seq + rot - p.k_blocks;
                    if (!bounded_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status,
                                      DEV_TIMEOUT_PRODUCER_EMPTY)) { ok = false; break; }
                    const uint32_t bar = full_bar(stage);
                    if constexpr (PACKED) {
                        // pre-swizzled and row-contiguous within the K block: one linear copy of the values and
                        // one of the metadata of exactly the rows of this tile (row0 is a multiple of 8, so the
                        // swizzle phase of a row in the tile is the one it was packed with)
                        mbar_expect_tx(bar, static_cast<uint32_t>(seg.nrows) * kSpPackedRowBytes + Cfg::B_BYTES);
                        const uint8_t* slice = p.meta_tiled + static_cast<size_t>(kb) * rows_padded * kSpPackedRowBytes;
                        bulk_load(a_smem0 + stage * Cfg::A_BYTES, slice + static_cast<size_t>(r0) * 128, seg.nrows * 128, bar);
                        bulk_load(e_smem0 + stage * Cfg::E_BYTES, slice + rows_padded * 128 + static_cast<size_t>(r0) * 32,
                                  seg.nrows * 32, bar);
                    } else {
                        mbar_expect_tx(bar, Cfg::A_BYTES + Cfg::B_BYTES + kMetaStage);
                        tma_load_2d(a_smem0 + stage * Cfg::A_BYTES, &map_s, bar, kb * 128, r0);
                    }
                    const uint32_t b_addr = b_smem0 + stage * Cfg::B_BYTES;
                    if constexpr (F16) {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)    // [128 K rows x 64 fp16 columns] per box, byte map
                            tma_load_2d(b_addr + j * (128 * kKRows), &map_d, bar, (c0 + j * 64) * 2, kb * kKRows);
                    } else if constexpr (DENSE_MN) {
#pragma unroll
                        for (int j = 0; j < BN / 128; ++j)   // [256 K rows x 128 C bytes] per box
                            tma_load_2d(b_addr + j * (128 * kSpKLogical), &map_d, bar, c0 + j * 128,
                                        kb * kSpKLogical);
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j)          // [BN rows x 128 K bytes] per box
                            tma_load_2d(b_addr + j * (BN * 128), &map_d, bar, kb * kSpKLogical + j * 128, c0);
                    }
                    if constexpr (!PACKED)
                        bulk_load(e_smem0 + stage * Cfg::E_BYTES, meta_row + static_cast<size_t>(kb) * kMetaStage,
                                  kMetaStage, bar);
                    issued |= 1u << stage;
                    issued_parity = (issued_parity & ~(1u << stage)) | (phase << stage);
                    if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
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
            constexpr uint32_t idesc = F16 ? make_idesc_f16(kBM, BN, DENSE_MN, true) : make_idesc_i8(kBM, BN, DENSE_MN, true);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            WorkIter work(p, blockIdx.x, gridDim.x, num_tiles, ROWS);
            WorkSegment seg;
            while (ok && work.next(seg)) {
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
                    const uint32_t a_addr = a_smem0 + stage * Cfg::A_BYTES;
                    const uint32_t b_addr = b_smem0 + stage * Cfg::B_BYTES;
                    const uint32_t e_addr = e_smem0 + stage * Cfg::E_BYTES;
                    const uint32_t e_tmem = tmem_base + Cfg::E_BASE + stage * 8;
                    // metadata: rows are 16 B apart, 8-row groups 128 B apart, no swizzle
#pragma unroll
                    for (int j = 0; j < (F16 ? 1 : 2); ++j)
                        tmem_cp_128x128b(e_tmem + 4 * j,
                                         PACKED ? make_smem_desc(e_addr + j * 128, 0, 256, SWIZZLE_NONE_DESC)   // halves interleaved per 8 rows
                                                : make_smem_desc(e_addr + j * 2048, 0, 128, SWIZZLE_NONE_DESC));
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint64_t a_desc = make_smem_desc(a_addr + ks * 32, 0, 1024, SWIZZLE_128B_DESC);
                        uint64_t b_desc;
                        if constexpr (F16) {
                            // 32 K rows of 128 B per MMA; 64-column groups are one box (128 x 128 B) apart
                            b_desc = make_smem_desc(b_addr + ks * (32 * 128), 128 * kKRows, 1024, SWIZZLE_128B_DESC);
                            // metadata is addressed in pairs of 32-bit columns (what one kind::i8 MMA of
                            // K = 64 consumes); a K = 32 fp16 MMA takes one column of the pair, chosen by
                            // the selector in bits [0,2) of the instruction descriptor
                            mma_f16_sp(d_tmem, a_desc, b_desc, e_tmem + (ks & ~1), idesc | static_cast<uint32_t>(ks & 1),
                                       (kb != 0 || ks != 0) ? 1u : 0u);
                            continue;
                        } else if constexpr (DENSE_MN) {
                            b_desc = make_smem_desc(b_addr + ks * (64 * 128), 128 * kSpKLogical, 1024,
                                                    SWIZZLE_128B_DESC);
                        } else {
                            b_desc = make_smem_desc(b_addr + (ks >> 1) * (BN * 128) + (ks & 1) * 64, 0, 1024,
                                                    SWIZZLE_128B_DESC);
                        }
                        mma_i8_sp(d_tmem, a_desc, b_desc, e_tmem + 2 * ks, idesc, (kb != 0 || ks != 0) ? 1u : 0u);
                    }
                    tc_commit(empty_bar(stage));
                    if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc_commit(acc_full_bar(acc));
                if (++acc == Cfg::ACC_BUFS) { acc = 0; acc_phase ^= 1u; }
            }
            if (!ok) {
                tc_commit(drain_bar);
                uint64_t t0 = global_timer_ns();
                while (!mbar_try_wait(drain_bar, 0) && global_timer_ns() - t0 < 20000000ull) {}
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;                     // 0 unless the tile is drained by 8 warps
        EpiStrip<Cfg::NC>* strip = reinterpret_cast<EpiStrip<Cfg::NC>*>(smem_gen + Cfg::STRIP_OFFSET) + (warp - 2);
        uint32_t acc = 0, acc_phase = 0;
        WorkIter work(p, blockIdx.x, gridDim.x, num_tiles, ROWS);
        WorkSegment seg;
        while (work.next(seg)) {
            const int r0 = seg.row0;
            const int c0 = (seg.tile / p.tiles_r) * BN + half * Cfg::NC;
            const int lane_coord = r0 + quarter * 32 + lane;      // row of the sparse operand
            EpilogueParams epi = p.epi;                           // rows beyond this tile's share are not ours to write
            if (seg.nrows < kBM) {
                if (TRANSPOSED) epi.cols = epi.cols < r0 + seg.nrows ? epi.cols : r0 + seg.nrows;
                else            epi.rows = epi.rows < r0 + seg.nrows ? epi.rows : r0 + seg.nrows;
            }
            // never write past this tile's own columns when the tile is narrower than a 32-column chunk
            int c_limit = TRANSPOSED ? p.epi.rows : p.epi.cols;
            if (BN < 32 && c_limit > c0 + BN) c_limit = c0 + BN;
            stage_strip<EPI, Cfg::NC, TRANSPOSED>(p.epi, strip, c0, lane);
            const float lane_s = lane_scale_of<EPI, TRANSPOSED>(p.epi, lane_coord);
            if (!bounded_wait(acc_full_bar(acc), acc_phase, abort_flag, p.status, DEV_TIMEOUT_EPI_ACC_FULL))
                break;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN + half * Cfg::NC;
            drain_accumulator<EPI, Cfg::NC, TRANSPOSED>(epi, taddr, lane_coord, c0, c_limit, strip, lane_s);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(acc));
            if (++acc == Cfg::ACC_BUFS) { acc = 0; acc_phase ^= 1u; }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

}  // namespace bm
