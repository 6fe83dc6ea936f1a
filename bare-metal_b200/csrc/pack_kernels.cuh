// pack_kernels.cuh — one-time operand repacks (excluded from GEMM timing):
//   * 2:4 position metadata -> the sparse kernel's tiled order, from the reference's uint32
//     word format (kernels/gemm/igemm/sparse_meta_int8.h:13-31,166-175: one word per
//     (16-row tile, 32-wide K step, gid), rows gid and gid+8 share it) or from plain per-row
//     nibble bytes;
//   * B[K x N] -> W[N x K] byte transpose.
// All three are pure HBM streaming: each source byte is read once, each output byte written once.
#pragma once
#include <cstdint>

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

// per-row nibble bytes [R x K/8] -> tiled; one thread per 16-byte unit
__global__ void pack_meta_rows_kernel(const uint8_t* __restrict__ rows_meta, uint8_t* __restrict__ tiled,
                                      int R, int K, int k_blocks, size_t units) {
    const size_t unit = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (unit >= units) return;
    int row, b0;
    tiled_coords(unit, k_blocks, row, b0);
    const int row_bytes = K / 8;
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int b = b0 + 4 * q;                  // K % 32 == 0, so rows are whole 4-byte words
        w[q] = (row < R && b < row_bytes)
                   ? *reinterpret_cast<const uint32_t*>(rows_meta + static_cast<size_t>(row) * row_bytes + b)
                   : 0x44444444u;
    }
    *reinterpret_cast<uint4*>(tiled + unit * 16) = make_uint4(w[0], w[1], w[2], w[3]);
}

// reference uint32 words -> tiled; one thread per 16-byte unit (4 K steps of 32)
__global__ void pack_meta_ref_kernel(const uint32_t* __restrict__ meta_ref, uint8_t* __restrict__ tiled,
                                     int R, int K, int k_blocks, size_t units) {
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
    *reinterpret_cast<uint4*>(tiled + unit * 16) = make_uint4(w[0], w[1], w[2], w[3]);
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
