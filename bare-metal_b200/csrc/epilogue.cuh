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
// __fmul_rn / __fsub_rn keep the compiler from contracting anything into an FMA.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>

namespace bm {

enum : int { EPI_I32 = 0, EPI_F32_TENSOR = 1, EPI_F32_CHANNEL = 2, EPI_F16_ROWCOL = 3 };

struct EpilogueParams {
    void* out;                 // C / D
    long long ld;              // row pitch of the output in elements
    int rows, cols;            // logical output extent [rows x cols] (rows = tokens M, cols = channels N)
    float tensor_scale;        // EPI_F32_TENSOR
    const float* row_scale;    // EPI_F16_ROWCOL : sa[rows]
    const float* col_scale;    // EPI_F16_ROWCOL : sw[cols];  EPI_F32_CHANNEL : scale[cols]
    const int* col_zero;       // EPI_F32_CHANNEL : zero_point[cols]
    int vec_ok;                // output base and pitch allow 16-byte vector stores
};

template <int EPI>
struct OutType { using type = float; };
template <>
struct OutType<EPI_I32> { using type = int32_t; };
template <>
struct OutType<EPI_F16_ROWCOL> { using type = __half; };

template <int EPI>
__device__ __forceinline__ typename OutType<EPI>::type
convert_one(const EpilogueParams& p, int32_t acc, int row, int col, float row_s) {
    if constexpr (EPI == EPI_I32) {
        return acc;
    } else if constexpr (EPI == EPI_F32_TENSOR) {
        return __fmul_rn(__int2float_rn(acc), p.tensor_scale);
    } else if constexpr (EPI == EPI_F32_CHANNEL) {
        return __fmul_rn(__fsub_rn(__int2float_rn(acc), __int2float_rn(__ldg(p.col_zero + col))),
                         __ldg(p.col_scale + col));
    } else {
        float s = __fmul_rn(row_s, __ldg(p.col_scale + col));
        return __float2half_rn(__fmul_rn(__int2float_rn(acc), s));
    }
}

// Lane = output ROW.  The thread holds columns [col0, col0+32) of row `row`.
template <int EPI>
__device__ __forceinline__ void store_row_chunk(const EpilogueParams& p, int row, int col0,
                                                const uint32_t (&r)[32]) {
    using T = typename OutType<EPI>::type;
    if (row >= p.rows || col0 >= p.cols) return;
    float row_s = 0.f;
    if constexpr (EPI == EPI_F16_ROWCOL) row_s = __ldg(p.row_scale + row);
    T* dst = reinterpret_cast<T*>(p.out) + static_cast<long long>(row) * p.ld + col0;
    if (p.vec_ok && col0 + 32 <= p.cols) {
        constexpr int PER_VEC = 16 / sizeof(T);
#pragma unroll
        for (int v = 0; v < 32 / PER_VEC; ++v) {
            alignas(16) T tmp[PER_VEC];
#pragma unroll
            for (int j = 0; j < PER_VEC; ++j)
                tmp[j] = convert_one<EPI>(p, static_cast<int32_t>(r[v * PER_VEC + j]), row,
                                          col0 + v * PER_VEC + j, row_s);
            *reinterpret_cast<uint4*>(dst + v * PER_VEC) = *reinterpret_cast<const uint4*>(tmp);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col0 + j < p.cols)
                dst[j] = convert_one<EPI>(p, static_cast<int32_t>(r[j]), row, col0 + j, row_s);
    }
}

// Lane = output COLUMN (channel); the 32 accumulator columns are 32 consecutive output ROWS
// (tokens).  For a fixed token the 32 lanes of a warp write 32 adjacent channels.
template <int EPI>
__device__ __forceinline__ void store_col_chunk(const EpilogueParams& p, int col, int row0,
                                                const uint32_t (&r)[32]) {
    using T = typename OutType<EPI>::type;
    if (col >= p.cols) return;
    T* dst = reinterpret_cast<T*>(p.out) + col;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        int row = row0 + j;
        if (row < p.rows) {
            float row_s = 0.f;
            if constexpr (EPI == EPI_F16_ROWCOL) row_s = __ldg(p.row_scale + row);
            dst[static_cast<long long>(row) * p.ld] =
                convert_one<EPI>(p, static_cast<int32_t>(r[j]), row, col, row_s);
        }
    }
}

}  // namespace bm
