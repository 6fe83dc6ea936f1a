// gather_kernels.cuh — all-gather of an fp16 column slab by plain peer stores.
//
// For the N-split layers whose GEMM has no store-fused gather (the 2:4-sparse kernels write their
// transposed accumulators with direct stores): the rank's slab D[:, n0 : n0 + n_len] already sits in
// its own [M x N_total] output; this kernel copies it to the same place in every other GPU's output.
// 16-byte loads from local memory, 16-byte stores to peer-mapped memory; no load ever touches a
// peer, nothing is multicast.  Stores that leave the GPU draw on the same token bucket as the
// GEMM-fused gather (StorePace in epilogue.cuh), one token per 4 KiB.
#pragma once
#include <cstdint>

#include "epilogue.cuh"

namespace bm {

constexpr int kGatherThreads = 256;
constexpr int kGatherMaxPeers = 8;

struct GatherDests {
    uint16_t* ptr[kGatherMaxPeers];     // slab's first column in every GPU's output (entry `self` is the source)
};

// One CTA moves tiles of 8 rows x 512 bytes (4 KiB): warp w takes row w of the tile, lane l bytes [16 l, 16 l + 16).
__global__ void __launch_bounds__(kGatherThreads)
gather_slab_kernel(const GatherDests dests, int n_dests, int self, int rows, int row_bytes, long long pitch_bytes,
                   unsigned long long* clock, unsigned cost) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col_tiles = (row_bytes + 511) / 512;
    const long long tiles = static_cast<long long>((rows + 7) / 8) * col_tiles;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(dests.ptr[self]);
    for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int r = static_cast<int>(t / col_tiles) * 8 + warp;
        const int c = static_cast<int>(t % col_tiles) * 512 + lane * 16;
        const bool live = r < rows && c < row_bytes;              // row_bytes is a multiple of 16
        uint4 v = make_uint4(0, 0, 0, 0);
        if (live) v = *reinterpret_cast<const uint4*>(src + r * pitch_bytes + c);
        for (int i = 1; i < n_dests; ++i) {
            int d = self + i;
            if (d >= n_dests) d -= n_dests;
            if (cost != 0 && threadIdx.x == 0) pace_remote_store(clock, cost);
            __syncthreads();
            if (live) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(dests.ptr[d]) + r * pitch_bytes + c) = v;
        }
    }
}

}  // namespace bm
