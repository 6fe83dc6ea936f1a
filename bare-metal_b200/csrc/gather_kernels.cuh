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

// One CTA moves tiles of 32 rows x 512 bytes (16 KiB): warp w takes rows w, w + 8, w + 16, w + 24 of the tile,
// lane l bytes [16 l, 16 l + 16) of each; the four loads are in flight together, then each destination gets the
// four stores (4 tokens of the pacer per destination and tile).
__global__ void __launch_bounds__(kGatherThreads)
gather_slab_kernel(const GatherDests dests, int n_dests, int self, int rows, int row_bytes, long long pitch_bytes,
                   unsigned long long* clock, unsigned cost) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col_tiles = (row_bytes + 511) / 512;
    const long long tiles = static_cast<long long>((rows + 31) / 32) * col_tiles;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(dests.ptr[self]);
    for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int r0 = static_cast<int>(t / col_tiles) * 32 + warp;
        const int c = static_cast<int>(t % col_tiles) * 512 + lane * 16;
        uint4 v[4];
        bool live[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            live[q] = (r0 + 8 * q) < rows && c < row_bytes;            // row_bytes is a multiple of 16
            v[q] = live[q] ? *reinterpret_cast<const uint4*>(src + (r0 + 8 * q) * pitch_bytes + c) : make_uint4(0, 0, 0, 0);
        }
        for (int i = 1; i < n_dests; ++i) {
            int d = self + i;
            if (d >= n_dests) d -= n_dests;
            if (cost != 0) {
                if (threadIdx.x == 0) pace_remote_store(clock, 4u * cost);
                __syncthreads();
            }
            uint8_t* dst = reinterpret_cast<uint8_t*>(dests.ptr[d]);
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (live[q]) *reinterpret_cast<uint4*>(dst + (r0 + 8 * q) * pitch_bytes + c) = v[q];
        }
    }
}

// Group barrier over peer-mapped flag words, for the step after a peer-store gather (no reference counterpart).
// flags.ptr[d] is GPU d's array of 32-bit words: words [0, n) are written by the peers (word s only by GPU s), word
// 32 is this GPU's own round counter.  The round number is taken from that counter ON THE DEVICE (and advanced), so
// a launch recorded in a CUDA graph signals a new round on every replay.  Thread d of the single CTA tells GPU d
// "my stores of this round are complete" (release, system scope) and then waits until GPU d has said the same here.
// Launched with programmatic stream serialization it is resident before the kernel in front of it ends;
// griddepcontrol.wait holds it until that kernel has completed and its stores are visible.  The wait is bounded
// (1 s): on expiry it records DEV_TIMEOUT_PEER in the status word and returns.
constexpr int kBarrierRoundWord = 32;
struct BarrierFlags {
    unsigned* ptr[kGatherMaxPeers];
};
__global__ void __launch_bounds__(32)
peer_barrier_kernel(const BarrierFlags flags, int n, int self, int* status) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    unsigned seq = 0;
    if (threadIdx.x == 0) {
        unsigned* round = flags.ptr[self] + kBarrierRoundWord;
        seq = *round + 1u;
        *round = seq;
    }
    seq = __shfl_sync(0xFFFFFFFFu, seq, 0);
    const int d = threadIdx.x;
    if (d >= n || d == self) return;
    __threadfence_system();
    unsigned* theirs = flags.ptr[d] + self;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(seq) : "memory");
    const unsigned* mine = flags.ptr[self] + d;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if (static_cast<int>(v - seq) >= 0) break;                    // rounds only move forward (wrap-safe compare)
        if (global_timer_ns() - t0 > BM_WAIT_LIMIT_NS) {
            if (status) atomicCAS(status, 0, DEV_TIMEOUT_PEER);
            break;
        }
    }
}

}  // namespace bm
