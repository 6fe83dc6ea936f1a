// epilogue.cuh — fused dequantise-and-store epilogues shared by the dense and the sparse
// tcgen05 kernels.  A thread owns ONE accumulator lane and receives 32 consecutive columns
// of it straight from tensor memory; which output coordinate a (lane, column) pair means is
// decided by the kernel (normal: lane = output row; transposed: lane = output column).
//
// Arithmetic (must match the CPU checker bit for bit in fp32, then round once to fp16):
//   EPI_I32          C = acc
//   EPI_F32_TENSOR   C = (float)acc * s,            s = scale_a * scale_b computed on the host
//                    (igemm.cu:104-110 multiplies the two scales first, then the accumulator)
//   EPI_F32_CHANNEL  C = ((float)acc - (float)zp[n]) * scale[n]
//                    (igemm_pipelined_cpasync_perchannel.cu:276-281)
//   EPI_F16_ROWCOL   D = half_rn((float)acc * (sa[m] * sw[n]))
//   EPI_F32_ROWCOL   C = (float)acc * (sa[m] * sw[n])            (online-quant GEMM: block scales
//                    expanded per row / column, igemm_online_quant.cu:128,340-347)
// __fmul_rn / __fsub_rn keep the compiler from contracting anything into an FMA.
//
// Latency structure: the parameters that vary along the accumulator COLUMNS of a tile (sw[n] and
// zp[n] in the normal orientation, sa[m] in the transposed one) are staged once per tile into a
// per-warp strip of shared memory BEFORE the warp waits for the accumulator, and the tensor-
// memory loads are double-buffered (chunk c+1 is in flight while chunk c is converted), so the
// drain of a tile is a short dependent chain instead of eight.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>

#include "sm100_ptx.cuh"

namespace bm {

enum : int { EPI_I32 = 0, EPI_F32_TENSOR = 1, EPI_F32_CHANNEL = 2, EPI_F16_ROWCOL = 3, EPI_F32_ROWCOL = 4 };
__host__ __device__ constexpr bool epi_rowcol(int epi) { return epi == EPI_F16_ROWCOL || epi == EPI_F32_ROWCOL; }

struct EpilogueParams {
    void* out;                 // C / D
    long long ld;              // row pitch of the output in elements
    int rows, cols;            // logical output extent [rows x cols] (rows = tokens M, cols = channels N)
    float tensor_scale;        // EPI_F32_TENSOR
    const float* row_scale;    // EPI_F16_ROWCOL : sa[rows]
    const float* col_scale;    // EPI_F16_ROWCOL : sw[cols];  EPI_F32_CHANNEL : scale[cols]
    const int* col_zero;       // EPI_F32_CHANNEL : zero_point[cols]
    int vec_ok;                // output base and pitch allow 16-byte vector stores
    int tma_ok;                // ... and a tensor map of the output exists: drain through TMA stores
};

template <int EPI>
struct OutType { using type = float; };
template <>
struct OutType<EPI_I32> { using type = int32_t; };
template <>
struct OutType<EPI_F16_ROWCOL> { using type = __half; };

// `lane_s` is the scale attached to the accumulator lane, `cross_s` / `cross_z` the scale and
// zero point attached to the accumulator column (fp32 multiplication commutes, so the product
// sa*sw has the same bits in either orientation).
template <int EPI>
__device__ __forceinline__ typename OutType<EPI>::type
convert_acc(int32_t acc, float tensor_scale, float lane_s, float cross_s, int cross_z) {
    if constexpr (EPI == EPI_I32) {
        return acc;
    } else if constexpr (EPI == EPI_F32_TENSOR) {
        return __fmul_rn(__int2float_rn(acc), tensor_scale);
    } else if constexpr (EPI == EPI_F32_CHANNEL) {
        return __fmul_rn(__fsub_rn(__int2float_rn(acc), __int2float_rn(cross_z)), cross_s);
    } else if constexpr (EPI == EPI_F32_ROWCOL) {
        return __fmul_rn(__int2float_rn(acc), __fmul_rn(lane_s, cross_s));
    } else {
        return __float2half_rn(__fmul_rn(__int2float_rn(acc), __fmul_rn(lane_s, cross_s)));
    }
}

// Per-warp strip of column-side parameters for NC accumulator columns.
template <int NC>
struct EpiStrip {
    float scale[NC];
    int zero[NC];
};

// Fill the strip for accumulator columns [cross0, cross0 + NC) of the coming tile.
template <int EPI, int NC, bool TRANSPOSED>
__device__ __forceinline__ void stage_strip(const EpilogueParams& p, EpiStrip<NC>* strip, int cross0, int lane) {
    if constexpr (epi_rowcol(EPI) || EPI == EPI_F32_CHANNEL) {
        const float* src = TRANSPOSED ? p.row_scale : p.col_scale;
        const int limit = TRANSPOSED ? p.rows : p.cols;
#pragma unroll
        for (int i = lane; i < NC; i += 32) {
            const int c = cross0 + i;
            strip->scale[i] = c < limit ? __ldg(src + c) : 0.f;
            if constexpr (EPI == EPI_F32_CHANNEL) strip->zero[i] = c < limit ? __ldg(p.col_zero + c) : 0;
        }
        __syncwarp();
    }
}

template <int EPI, bool TRANSPOSED>
__device__ __forceinline__ float lane_scale_of(const EpilogueParams& p, int lane_coord) {
    if constexpr (epi_rowcol(EPI)) {
        const float* src = TRANSPOSED ? p.col_scale : p.row_scale;
        const int limit = TRANSPOSED ? p.cols : p.rows;
        return lane_coord < limit ? __ldg(src + lane_coord) : 0.f;
    } else {
        return 0.f;
    }
}

// Normal orientation: the thread holds columns [col0, col0+32) of output row `row`.
template <int EPI>
__device__ __forceinline__ void emit_row_chunk(const EpilogueParams& p, int row, int col0, const uint32_t (&r)[32],
                                               const float* s_scale, const int* s_zero, float lane_s) {
    using T = typename OutType<EPI>::type;
    if (row >= p.rows || col0 >= p.cols) return;
    T* dst = reinterpret_cast<T*>(p.out) + static_cast<long long>(row) * p.ld + col0;
    if (p.vec_ok && col0 + 32 <= p.cols) {
        constexpr int PER_VEC = 16 / sizeof(T);
#pragma unroll
        for (int v = 0; v < 32 / PER_VEC; ++v) {
            alignas(16) T tmp[PER_VEC];
#pragma unroll
            for (int j = 0; j < PER_VEC; ++j) {
                const int k = v * PER_VEC + j;
                tmp[j] = convert_acc<EPI>(static_cast<int32_t>(r[k]), p.tensor_scale, lane_s,
                                          (epi_rowcol(EPI) || EPI == EPI_F32_CHANNEL) ? s_scale[k] : 0.f,
                                          EPI == EPI_F32_CHANNEL ? s_zero[k] : 0);
            }
            *reinterpret_cast<uint4*>(dst + v * PER_VEC) = *reinterpret_cast<const uint4*>(tmp);
        }
    } else {
#pragma unroll
        for (int k = 0; k < 32; ++k)
            if (col0 + k < p.cols)
                dst[k] = convert_acc<EPI>(static_cast<int32_t>(r[k]), p.tensor_scale, lane_s,
                                          (epi_rowcol(EPI) || EPI == EPI_F32_CHANNEL) ? s_scale[k] : 0.f,
                                          EPI == EPI_F32_CHANNEL ? s_zero[k] : 0);
    }
}

// Transposed orientation: the thread holds output column `col` (a channel) for the 32
// consecutive output rows (tokens) [row0, row0+32); per token the 32 lanes of the warp write 32
// adjacent channels.  `row_limit` clips to the tile's own tokens for tiles narrower than 32.
template <int EPI>
__device__ __forceinline__ void emit_col_chunk(const EpilogueParams& p, int col, int row0, int row_limit,
                                               const uint32_t (&r)[32], const float* s_scale, float lane_s) {
    using T = typename OutType<EPI>::type;
    if (col >= p.cols) return;
    T* dst = reinterpret_cast<T*>(p.out) + col + static_cast<long long>(row0) * p.ld;
    // all conversions first (independent, so they overlap), then the stores: with both in one loop every store
    // waited for its own scale load and conversions
    T v[32];
#pragma unroll
    for (int k = 0; k < 32; ++k)
        v[k] = convert_acc<EPI>(static_cast<int32_t>(r[k]), p.tensor_scale, lane_s, epi_rowcol(EPI) ? s_scale[k] : 0.f, 0);
    const int live = row_limit - row0;            // rows of this chunk inside the output
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        if (k < live) *dst = v[k];
        dst += p.ld;
    }
}

// Drain NC accumulator columns starting at tensor-memory address `taddr` (lane quarter and first
// column already applied).  `cross0` is the output coordinate of the first column.
template <int EPI, int NC, bool TRANSPOSED>
__device__ __forceinline__ void drain_accumulator(const EpilogueParams& p, uint32_t taddr, int lane_coord, int cross0,
                                                  int cross_limit, const EpiStrip<NC>* strip, float lane_s) {
    static_assert(NC % 32 == 0, "drained in chunks of 32 columns");
    constexpr int CHUNKS = NC / 32;
    uint32_t ra[32], rb[32];
    if (cross0 < cross_limit) tmem_ld_32x32(taddr, ra);
#pragma unroll
    for (int c = 0; c < CHUNKS; c += 2) {
        if (cross0 + c * 32 < cross_limit) {                       // warp-uniform
            tmem_ld_wait();
            if (c + 1 < CHUNKS && cross0 + (c + 1) * 32 < cross_limit) tmem_ld_32x32(taddr + (c + 1) * 32, rb);
            if constexpr (TRANSPOSED)
                emit_col_chunk<EPI>(p, lane_coord, cross0 + c * 32, cross_limit, ra, strip->scale + c * 32, lane_s);
            else
                emit_row_chunk<EPI>(p, lane_coord, cross0 + c * 32, ra, strip->scale + c * 32, strip->zero + c * 32, lane_s);
        }
        if (c + 1 < CHUNKS && cross0 + (c + 1) * 32 < cross_limit) {
            tmem_ld_wait();
            if (c + 2 < CHUNKS && cross0 + (c + 2) * 32 < cross_limit) tmem_ld_32x32(taddr + (c + 2) * 32, ra);
            if constexpr (TRANSPOSED)
                emit_col_chunk<EPI>(p, lane_coord, cross0 + (c + 1) * 32, cross_limit, rb, strip->scale + (c + 1) * 32, lane_s);
            else
                emit_row_chunk<EPI>(p, lane_coord, cross0 + (c + 1) * 32, rb, strip->scale + (c + 1) * 32,
                                    strip->zero + (c + 1) * 32, lane_s);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// TMA-store drain (normal orientation).  Direct stores from the accumulator layout make every
// lane of a warp write a different output ROW (16 bytes each, a pitch apart); with power-of-two
// pitches those land on few L2 slices and the drain, not the MMA, bounds the tile.  Here each warp
// converts a 32-row x 128-byte box into a 4 KiB strip of shared memory (128-byte swizzle, so the
// 16-byte pieces of 8 rows never share a bank) and one lane hands it to the TMA engine, which writes
// whole 128-byte lines and clips rows/columns beyond the output.  The strip is single-buffered:
// before it is rewritten the lane waits until the previous store has finished reading it.
// ------------------------------------------------------------------------------------------------
constexpr int kStoreBoxBytes = 32 * 128;          // per-warp staging strip

// Up to kMaxOutMaps destinations of one output tile: the local matrix, or the same column slab of
// the output on every GPU of an N-split group (peer-mapped buffers) — the all-gather of the slab is
// then nothing but extra TMA stores of the box that is already staged in shared memory.
constexpr int kMaxOutMaps = 8;
struct OutMaps {
    CUtensorMap m[kMaxOutMaps];
};

// Pacing of stores that leave the GPU over NVLink.  Measured on two B200s: when SMs offer peer stores faster
// than the link takes them (~770 GB/s per direction), the stores back up towards the SMs and the
// operand LOADS of the same SMs collapse from ~23 TB/s to ~1 TB/s until the backlog is gone — TMA stores
// and plain st.global alike — so an unpaced fused gather computes OR sends, never both.  Offered at up to
// ~720 GB/s the same stores leave the loads untouched.  All CTAs of a GPU therefore draw their remote
// stores from one token bucket: a virtual clock in global memory (1/16 ns units) that every remote
// 4 KiB store advances by `cost`; a store waits until the wall clock reaches its slot.  The bucket holds
// 1 us of credit, so an idle link takes a short burst at once.  The wait is bounded (2 ms): pacing is an
// optimisation, never a condition for correctness.
struct StorePace {
    unsigned long long* clock;      // shared by every launch on this GPU
    unsigned cost;                  // virtual-clock units per remote box store; 0 = no pacing
    unsigned remote_mask;           // bit d set: destination d is another GPU's memory
    int first;                      // destination served first (the GPU's own buffer); the others follow in ring order
};

__device__ __forceinline__ unsigned long long pace_now() {
    return (global_timer_ns() & 0x00FFFFFFFFFFFFFFull) << 4;
}
__device__ __forceinline__ void pace_remote_store(unsigned long long* clock, unsigned cost) {
    constexpr unsigned long long kCredit = 16ull * 1000;            // 1 us
    constexpr unsigned long long kGiveUp = 16ull * 2000000;         // 2 ms
    unsigned long long now = pace_now();
    atomicMax(clock, now > kCredit ? now - kCredit : 0ull);
    const unsigned long long slot = atomicAdd(clock, static_cast<unsigned long long>(cost));
    if (slot > now + 16ull * 1000000000) {                          // a clock from another epoch: restart it
        atomicExch(clock, now);
        return;
    }
    const unsigned long long t0 = now;
    while (now < slot && now - t0 < kGiveUp) now = pace_now();
}

// The 32-column chunks of a drain come from tensor memory: asynchronous loads, waited for just before use.
struct TmemSource {
    uint32_t taddr;
    __device__ __forceinline__ void issue(int c, uint32_t (&r)[32]) const { tmem_ld_32x32(taddr + c * 32, r); }
    __device__ __forceinline__ void wait() const { tmem_ld_wait(); }
};

// NBUF staging strips per warp (1 or 2), used round-robin over the boxes of all tiles (`box_count`
// runs on across tiles).  With two strips a box is converted while the previous one is still being
// read by its stores — what keeps the epilogue going when the stores go to other GPUs over NVLink.
template <int EPI, int NC, int NBUF, class Source>
__device__ __forceinline__ void drain_tma_from(const EpilogueParams& p, const CUtensorMap* maps, int n_maps, const Source& src,
                                               int row0, int lane, int col0, const EpiStrip<NC>* strip, float lane_s,
                                               uint32_t stage_smem0, uint32_t& box_count, int col_limit,
                                               const StorePace& pace = StorePace{nullptr, 0u, 0u, 0}) {
    using T = typename OutType<EPI>::type;
    static_assert(NC % 32 == 0, "drained in chunks of 32 columns");
    constexpr int CHUNKS = NC / 32;
    constexpr int COLS_PER_BOX = 128 / sizeof(T);            // 64 fp16 or 32 fp32/int32 columns
    constexpr int CHUNKS_PER_BOX = COLS_PER_BOX / 32;        // 2 or 1
    constexpr int PIECES_PER_CHUNK = 32 * sizeof(T) / 16;    // 16-byte pieces a thread writes per chunk
    constexpr int PER_VEC = 16 / sizeof(T);
    const int sw = lane & 7;                                 // 128-byte swizzle: piece index ^ (row % 8)
    uint32_t stage_smem = stage_smem0 + (NBUF > 1 ? (box_count & 1u) * kStoreBoxBytes : 0u);

    uint32_t rr[2][32];
    if (col0 < col_limit) src.issue(0, rr[0]);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int cur = c & 1;
        const bool live = col0 + c * 32 < col_limit;            // warp-uniform
        if (live) {
            src.wait();
            if (c + 1 < CHUNKS && col0 + (c + 1) * 32 < col_limit) src.issue(c + 1, rr[cur ^ 1]);
            if (c % CHUNKS_PER_BOX == 0) {
                // the strip may still be read by the store issued NBUF boxes ago
                stage_smem = stage_smem0 + (NBUF > 1 ? (box_count & 1u) * kStoreBoxBytes : 0u);
                if (lane == 0) {
                    if constexpr (NBUF > 1) bulk_wait_read_all_but_one();
                    else bulk_wait_read_all();
                }
                __syncwarp();
            }
            const uint32_t my_row = stage_smem + lane * 128;
#pragma unroll
            for (int v = 0; v < PIECES_PER_CHUNK; ++v) {
                alignas(16) T tmp[PER_VEC];
#pragma unroll
                for (int j = 0; j < PER_VEC; ++j) {
                    const int k = v * PER_VEC + j;
                    tmp[j] = convert_acc<EPI>(static_cast<int32_t>(rr[cur][k]), p.tensor_scale, lane_s,
                                              (epi_rowcol(EPI) || EPI == EPI_F32_CHANNEL) ? strip->scale[c * 32 + k] : 0.f,
                                              EPI == EPI_F32_CHANNEL ? strip->zero[c * 32 + k] : 0);
                }
                const int piece = (c % CHUNKS_PER_BOX) * PIECES_PER_CHUNK + v;
                const uint4 val = *reinterpret_cast<const uint4*>(tmp);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_row + ((piece ^ sw) << 4)), "r"(val.x),
                             "r"(val.y), "r"(val.z), "r"(val.w)
                             : "memory");
            }
        }
        const bool box_done = (c % CHUNKS_PER_BOX == CHUNKS_PER_BOX - 1) || c == CHUNKS - 1;
        const int box_c0 = col0 + (c / CHUNKS_PER_BOX) * COLS_PER_BOX;
        if (box_done && box_c0 < col_limit) {
            fence_proxy_async_smem();                        // generic-proxy writes -> visible to the TMA engine
            __syncwarp();
            if (lane == 0) {
                for (int i = 0; i < n_maps; ++i) {
                    int d = pace.first + i;
                    if (d >= n_maps) d -= n_maps;
                    if (pace.cost != 0 && ((pace.remote_mask >> d) & 1u)) pace_remote_store(pace.clock, pace.cost);
                    tma_store_2d(maps + d, stage_smem, box_c0, row0);
                }
                bulk_commit_group();
            }
            ++box_count;
        }
    }
}

template <int EPI, int NC, int NBUF>
__device__ __forceinline__ void drain_accumulator_tma(const EpilogueParams& p, const CUtensorMap* maps, int n_maps,
                                                      uint32_t taddr, int row0, int lane, int col0,
                                                      const EpiStrip<NC>* strip, float lane_s, uint32_t stage_smem0,
                                                      uint32_t& box_count, int col_limit,
                                                      const StorePace& pace = StorePace{nullptr, 0u, 0u, 0}) {
    drain_tma_from<EPI, NC, NBUF>(p, maps, n_maps, TmemSource{taddr}, row0, lane, col0, strip, lane_s, stage_smem0,
                                  box_count, col_limit, pace);
}

}  // namespace bm
