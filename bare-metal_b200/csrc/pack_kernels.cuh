// pack_kernels.cuh — one-time operand repacks (excluded from GEMM timing):
//   * 2:4 position metadata -> the sparse kernel's tiled order, from the reference's uint32
//     word format (kernels/gemm/igemm/sparse_meta_int8.h:13-31,166-175: one word per
//     (16-row tile, 32-wide K step, gid), rows gid and gid+8 share it) or from plain per-row
//     nibble bytes;
//   * B[K x N] -> W[N x K] byte transpose.
// All three are pure HBM streaming: each source byte is read once, each output byte written once.
#pragma once
#include <cstdint>

#include "igemm_sparse.cuh"      // kSpPackedRowBytes

namespace bm {

// Tiled order: [row block rb][k-block kb][chunk j in 0..1][row r in 0..127][16 bytes].
// Chunk (kb, j) covers logical K [256 kb + 128 j, +128); padding rows / K get the valid
// pattern 0x44 (positions 0 and 1) — their values are zero-filled by TMA.
__device__ __forceinline__ void tiled_coords(size_t unit, int k_blocks, int& row, int& k_byte0) {
    const int r = static_cast<int>(unit & 127);
    const size_t chunk = unit >> 7;                 // (rb * k_blocks + kb) * 2 + j
    const int j = static_cast<int>(chunk & 1);
    const size_t blk = chunk >> 1;
    const int kb = static_cast<int>(blk % k_blocks);
    const int rb = static_cast<int>(blk / k_blocks);
    row = rb * 128 + r;
    k_byte0 = (kb * 2 + j) * 16;                    // first metadata byte of this row's 16
}

// Where unit u of the tiled metadata goes: blocks of 4 KiB (256 units) packed back to back
// (rows_padded = 0), or the metadata part of the packed weight format above.
struct MetaDest {
    int k_blocks;
    int rows_padded;                // 0: plain tiled blocks; else rows of the packed weights (multiple of 128)
};
__device__ __forceinline__ size_t meta_unit_offset(size_t unit, const MetaDest& d) {
    if (d.rows_padded == 0) return unit * 16;
    const size_t blk = unit >> 8;
    const size_t kb = blk % d.k_blocks, rb = blk / d.k_blocks;
    const size_t j = (unit >> 7) & 1, row = rb * 128 + (unit & 127);
    return kb * static_cast<size_t>(d.rows_padded) * kSpPackedRowBytes + static_cast<size_t>(d.rows_padded) * 128 +
           (row >> 3) * 256 + j * 128 + (row & 7) * 16;
}

// How tcgen05.mma.sp.kind::f16 reads its metadata (found by probing single nibbles on a B200): within
// a 16-row block, tensor-memory lane i < 8 holds in each 32-bit column the nibbles of K groups 0-3 of
// row i (bits 15:0) and of row i + 8 (bits 31:16); lane i + 8 holds groups 4-7 of the same two rows.
// (kind::i8 reads row-per-lane, groups in order.)  `f16_lanes` applies that regrouping to the tiled
// order: a 2 x 2 exchange of 16-bit halves between the natural words of rows i and i + 8.
template <class NatWord>
__device__ __forceinline__ uint32_t lane_word(const NatWord& nat, int row, int q, int f16_lanes) {
    if (!f16_lanes) return nat(row, q);
    const int lo_row = row - (row % 16) + (row % 8);
    const uint32_t a = nat(lo_row, q), b = nat(lo_row + 8, q);
    return (row % 16) >= 8 ? ((a >> 16) | (b & 0xFFFF0000u)) : ((a & 0xFFFFu) | (b << 16));
}

// per-row nibble bytes [R x K/8] -> tiled; one thread per 16-byte unit
__global__ void pack_meta_rows_kernel(const uint8_t* __restrict__ rows_meta, uint8_t* __restrict__ tiled,
                                      int R, int K, int k_blocks, size_t units,
                                      MetaDest dest, int f16_lanes) {
    const size_t unit = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (unit >= units) return;
    int row, b0;
    tiled_coords(unit, k_blocks, row, b0);
    const int row_bytes = K / 8;
    auto nat = [&](int r, int q) -> uint32_t {
        const int b = b0 + 4 * q;                  // K % 32 == 0, so rows are whole 4-byte words
        return (r < R && b < row_bytes)
                   ? *reinterpret_cast<const uint32_t*>(rows_meta + static_cast<size_t>(r) * row_bytes + b)
                   : 0x44444444u;
    };
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) w[q] = lane_word(nat, row, q, f16_lanes);
    *reinterpret_cast<uint4*>(tiled + meta_unit_offset(unit, dest)) =
        make_uint4(w[0], w[1], w[2], w[3]);
}

// reference uint32 words -> tiled; one thread per 16-byte unit (4 K steps of 32)
__global__ void pack_meta_ref_kernel(const uint32_t* __restrict__ meta_ref, uint8_t* __restrict__ tiled,
                                     int R, int K, int k_blocks, size_t units,
                                     MetaDest dest) {
    const size_t unit = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (unit >= units) return;
    int row, b0;
    tiled_coords(unit, k_blocks, row, b0);
    const int k_steps = K / 32;
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int s = b0 / 4 + q;
        w[q] = (row < R && s < k_steps)
                   ? meta_ref[(static_cast<size_t>(row / 16) * k_steps + s) * 8 + (row % 16) % 8]
                   : 0x44444444u;
    }
    *reinterpret_cast<uint4*>(tiled + meta_unit_offset(unit, dest)) =
        make_uint4(w[0], w[1], w[2], w[3]);
}

// FP16 reference words (kernels/gemm/hgemm_sparse/sparse_meta.h:10-30,185: one uint32 per (16-row tile,
// 16-wide K step, gid), 4 nibbles in bits 15:0, duplicated into 31:16) -> tiled in the lane order of
// kind::f16; one thread per 16-byte unit = 8 K steps of 16
__global__ void pack_meta_ref_f16_kernel(const uint32_t* __restrict__ meta_ref, uint8_t* __restrict__ tiled,
                                         int R, int K, int k_blocks, size_t units,
                                         MetaDest dest) {
    const size_t unit = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (unit >= units) return;
    int row, b0;
    tiled_coords(unit, k_blocks, row, b0);
    const int k_steps = K / 16;
    auto nat = [&](int r, int q) -> uint32_t {
        uint32_t v = 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int s = b0 / 2 + 2 * q + h;
            const uint32_t half = (r < R && s < k_steps)
                                      ? (meta_ref[(static_cast<size_t>(r / 16) * k_steps + s) * 8 + (r % 16) % 8] & 0xFFFFu)
                                      : 0x4444u;
            v |= half << (16 * h);
        }
        return v;
    };
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) w[q] = lane_word(nat, row, q, 1);
    *reinterpret_cast<uint4*>(tiled + meta_unit_offset(unit, dest)) =
        make_uint4(w[0], w[1], w[2], w[3]);
}

// tiled metadata (4 KiB blocks) -> the metadata part of packed weights
__global__ void pack_meta_copy_kernel(const uint8_t* __restrict__ tiled_in, uint8_t* __restrict__ packed,
                                      size_t units, MetaDest dest) {
    const size_t unit = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (unit >= units) return;
    *reinterpret_cast<uint4*>(packed + meta_unit_offset(unit, dest)) =
        *reinterpret_cast<const uint4*>(tiled_in + unit * 16);
}

// Compressed 2:4 values comp[R x K/2] -> the values part of packed weights.  Within K block kb, row r holds
// compressed bytes [128 kb, +128) laid out exactly as a TMA load with 128-byte swizzle would leave the row in
// shared memory when the copied range starts on a multiple of 8 rows (16-byte chunk c of row r sits at
// r*128 + ((c ^ (r & 7)) << 4)), so the GEMM fetches any such range with one linear bulk copy.
// Rows / bytes beyond the operand are zero.  One thread per 16-byte chunk.
__global__ void pack_comp_blocks_kernel(const int8_t* __restrict__ comp, uint8_t* __restrict__ packed,
                                        int R, int K, int k_blocks, size_t chunks, int rows_padded) {
    const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (idx >= chunks) return;
    const int c = static_cast<int>(idx & 7);
    const int r = static_cast<int>((idx >> 3) & 127);
    const size_t blk = idx >> 10;
    const int kb = static_cast<int>(blk % k_blocks);
    const int rb = static_cast<int>(blk / k_blocks);
    const int row = rb * 128 + r;
    const int byte0 = kb * 128 + c * 16;
    const int row_bytes = K / 2;                   // K % 32 == 0, so rows are whole 16-byte chunks
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < R && byte0 < row_bytes)
        v = *reinterpret_cast<const uint4*>(comp + static_cast<size_t>(row) * row_bytes + byte0);
    *reinterpret_cast<uint4*>(packed + static_cast<size_t>(kb) * rows_padded * kSpPackedRowBytes +
                              static_cast<size_t>(row) * 128 + ((c ^ (r & 7)) << 4)) = v;
}

// Magnitude pruning of a dense int8 matrix W[R x K] to 2:4 along K, compression included: of every
// aligned group of 4 the two entries of largest |w| are kept (ties: the lower position wins), written
// lower position first into comp[R x K/2], and their positions go into the per-row nibble bytes
// nib[R x K/8] ((idx1 << 2) | idx0; byte j = groups 2j in the low nibble, 2j + 1 in the high one) —
// the layout compress_2_4_int8 of the reference produces for a matrix that is already 2:4
// (kernels/gemm/igemm/sparse_meta_int8.h:137-167), with the keep mask taken from the magnitudes
// instead of from "value != 0".  One thread per 32 input bytes: two 16-byte loads, one 16-byte store
// of values, one 4-byte store of positions.  Streams at HBM speed: 1.625 bytes per element.
__device__ __forceinline__ uint32_t prune_group(uint32_t word, uint32_t& kept) {
    // key = |w| * 4 + (3 - position): distinct per position, larger key = kept first, so equal
    // magnitudes resolve to the lower position.  __vabs4 maps -128 to 128 (no saturation).
    const uint32_t mag = __vabs4(word);
    const uint32_t k0 = ((mag & 0xFFu) << 2) | 3u, k1 = (((mag >> 8) & 0xFFu) << 2) | 2u;
    const uint32_t k2 = (((mag >> 16) & 0xFFu) << 2) | 1u, k3 = ((mag >> 24) << 2);
    const uint32_t hi01 = max(k0, k1), lo01 = min(k0, k1), hi23 = max(k2, k3), lo23 = min(k2, k3);
    const uint32_t first = max(hi01, hi23);
    const uint32_t second = hi01 > hi23 ? max(hi23, lo01) : max(hi01, lo23);
    const uint32_t pa = 3u - (first & 3u), pb = 3u - (second & 3u);
    const uint32_t idx0 = min(pa, pb), idx1 = max(pa, pb);
    kept = ((word >> (8 * idx0)) & 0xFFu) | (((word >> (8 * idx1)) & 0xFFu) << 8);
    return (idx1 << 2) | idx0;
}

__global__ void prune_2_4_kernel(const int8_t* __restrict__ W, int8_t* __restrict__ comp, uint8_t* __restrict__ nib,
                                 size_t units) {
    for (size_t u = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; u < units;
         u += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint4 lo = reinterpret_cast<const uint4*>(W)[2 * u];
        const uint4 hi = reinterpret_cast<const uint4*>(W)[2 * u + 1];
        const uint32_t in[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        uint32_t out[4] = {0, 0, 0, 0}, nibbles = 0;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            uint32_t kept;
            nibbles |= prune_group(in[g], kept) << (4 * g);
            out[g >> 1] |= kept << (16 * (g & 1));
        }
        reinterpret_cast<uint4*>(comp)[u] = make_uint4(out[0], out[1], out[2], out[3]);
        reinterpret_cast<uint32_t*>(nib)[u] = nibbles;
    }
}

// B[K x N] -> W[N x K], 64 x 64 byte tiles through shared memory
__global__ void transpose_kn_to_nk_kernel(const int8_t* __restrict__ src, int8_t* __restrict__ dst, int K, int N) {
    __shared__ int8_t tile[64][65];
    const int k0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    for (int i = threadIdx.y; i < 64; i += blockDim.y) {
        const int k = k0 + i, n = n0 + threadIdx.x;
        tile[i][threadIdx.x] = (k < K && n < N) ? src[static_cast<size_t>(k) * N + n] : int8_t(0);
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 64; i += blockDim.y) {
        const int n = n0 + i, k = k0 + threadIdx.x;
        if (n < N && k < K) dst[static_cast<size_t>(n) * K + k] = tile[threadIdx.x][i];
    }
}

}  // namespace bm
