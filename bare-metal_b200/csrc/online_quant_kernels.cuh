// online_quant_kernels.cuh — the quantisation step of the reference's FP16-in GEMMs
// (kernels/gemm/igemm/igemm_online_quant.cu and its _inplace / _bankfree / _bf_128x256 /
// warp_specialized variants), restated as two streaming kernels in front of the tcgen05 GEMM.
//
// What the reference computes (igemm_online_quant.cu:66-142,255,393): every thread block owns a
// 128 x 128 output tile (128 x 256 in _bf_128x256).  It takes max|A| over its 128 rows x the FIRST
// 32 columns of K and max|B| over the first 32 rows of K x its 128 (256) columns, sets
// inv = 127 / max (1 if max == 0), and quantises EVERY K tile with those two factors
// (QUANTIZE_TILE on tile 0, QUANTIZE_TILE_FAST afterwards): q = clamp(rint(x * inv), -128, 127).
// Each K tile's int32 sum is folded into an fp32 accumulator with tile_scale =
// (max_a / 127) * (max_b / 127).  So the scales are per 128-row block of A and per 128 (256)
// column block of B — a block-scaled W8A8 GEMM whose int32 sums can be kept exactly over all of K
// and multiplied by tile_scale once.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>

namespace bm {

constexpr int kOqRowBlock = 128;
constexpr int kOqKTile = 32;

// One launch does both steps.  A CTA owns a chunk of 32768 elements inside ONE scale block — 128 rows x
// 256 columns of A, or 256 (128) rows x 128 (256) columns of B — first takes the block's maximum over
// the first K tile itself (4096 / 8192 elements, an L2 hit for all but the first CTA of a block), then
// converts its chunk: 16 elements per thread and step, two 16-byte loads, one 16-byte store.  The CTAs
// of chunk 0 also publish the dequantisation scale max / 127 per row / column for the GEMM epilogue.
// K % 16 == 0 and N % 16 == 0, so a 16-element unit never straddles an edge.
constexpr int kOqChunkElems = 32768;
constexpr int kOqThreads = 256;

__device__ __forceinline__ float oq_unit_max(const __half* p) {
    const uint4 lo = reinterpret_cast<const uint4*>(p)[0], hi = reinterpret_cast<const uint4*>(p)[1];
    const uint32_t in[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const __half2 h = *reinterpret_cast<const __half2*>(&in[j]);
        m = fmaxf(m, fmaxf(fabsf(__low2float(h)), fabsf(__high2float(h))));
    }
    return m;
}

__device__ __forceinline__ void oq_unit_convert(const __half* src, int8_t* dst, float inv) {
    const uint4 lo = reinterpret_cast<const uint4*>(src)[0], hi = reinterpret_cast<const uint4*>(src)[1];
    const uint32_t in[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const __half h = __ushort_as_half(static_cast<unsigned short>((in[j >> 1] >> (16 * (j & 1))) & 0xFFFFu));
        int q = __float2int_rn(__fmul_rn(__half2float(h), inv));
        q = max(-128, min(127, q));
        out[j >> 2] |= (static_cast<uint32_t>(q) & 0xFFu) << (8 * (j & 3));
    }
    *reinterpret_cast<uint4*>(dst) = make_uint4(out[0], out[1], out[2], out[3]);
}

__global__ void __launch_bounds__(kOqThreads)
oq_quantize_kernel(const __half* __restrict__ A, const __half* __restrict__ B, int8_t* __restrict__ Aq,
                   int8_t* __restrict__ Bq, float* __restrict__ row_scale, float* __restrict__ col_scale, int M, int N,
                   int K, int col_block, int chunks_a, int a_chunks_per_block, int b_chunks_per_block) {
    __shared__ float warp_max[kOqThreads / 32];
    const int kt = K < kOqKTile ? K : kOqKTile;
    const int tid = threadIdx.x;
    const bool is_a = static_cast<int>(blockIdx.x) < chunks_a;
    const int id = is_a ? blockIdx.x : blockIdx.x - chunks_a;
    const int per = is_a ? a_chunks_per_block : b_chunks_per_block;
    const int blk = id / per, chunk = id % per;
    // operand-independent view: `rows` x `cols` matrix with pitch `pitch`, the chunk at (r0, c0) is
    // ch_rows x ch_cols, the first-K-tile window at (w_r0, w_c0) is w_rows x w_cols
    const __half* X = is_a ? A : B;
    int8_t* Xq = is_a ? Aq : Bq;
    const int rows = is_a ? M : K, cols = is_a ? K : N;
    const int ch_cols = is_a ? 256 : col_block, ch_rows = kOqChunkElems / ch_cols;
    const int r0 = is_a ? blk * kOqRowBlock : chunk * ch_rows, c0 = is_a ? chunk * ch_cols : blk * col_block;
    const int w_r0 = is_a ? r0 : 0, w_c0 = is_a ? 0 : c0;
    const int w_rows = is_a ? kOqRowBlock : kt, w_cols = is_a ? kt : col_block;
    const int w_units_per_row = (w_cols + 15) / 16;

    float m = 0.f;
    for (int u = tid; u < w_rows * w_units_per_row; u += kOqThreads) {
        const int r = w_r0 + u / w_units_per_row, c = w_c0 + (u % w_units_per_row) * 16;
        if (r < rows && c < cols && c < w_c0 + w_cols) m = fmaxf(m, oq_unit_max(X + static_cast<size_t>(r) * cols + c));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
    if ((tid & 31) == 0) warp_max[tid >> 5] = m;
    __syncthreads();
    float bmax = warp_max[0];
#pragma unroll
    for (int w = 1; w < kOqThreads / 32; ++w) bmax = fmaxf(bmax, warp_max[w]);
    const float inv = bmax > 0.f ? __fdiv_rn(127.0f, bmax) : 1.0f;
    if (chunk == 0) {
        const float scale = __fdiv_rn(bmax, 127.0f);
        float* dst = is_a ? row_scale : col_scale;
        const int first = is_a ? r0 : c0, count = is_a ? kOqRowBlock : col_block, limit = is_a ? M : N;
        for (int i = tid; i < count; i += kOqThreads)
            if (first + i < limit) dst[first + i] = scale;
    }
    const int units_per_row = ch_cols / 16;
#pragma unroll 4
    for (int u = tid; u < kOqChunkElems / 16; u += kOqThreads) {
        const int r = r0 + u / units_per_row, c = c0 + (u % units_per_row) * 16;
        if (r < rows && c < cols) {
            const size_t e = static_cast<size_t>(r) * cols + c;
            oq_unit_convert(X + e, Xq + e, inv);
        }
    }
}

}  // namespace bm
