// quantize_kernels.cuh — per-token dynamic quantisation fp16 -> int8, the step BEFORE the W8A8 GEMM.
//
// The reference's online-quant kernels (kernels/gemm/igemm/igemm_online_quant*.cu) take fp16 operands
// and quantise them tile by tile inside the GEMM with scale = max|x| / 127 (igemm_online_quant.cu:66-120).
// On B200 the W8A8 kernels want int8 operands with one fp32 scale per token, so the quantisation is
// its own HBM-bound pass with the arithmetic of the reference's host quantiser
// (kernels/gemm/igemm/bench.cu:28-51) applied per row:
//     scale[m] = max_k |x[m][k]| / 127   (1 if the row is all zero)
//     q[m][k]  = clamp((int)roundf(x[m][k] * (1 / scale[m])), -128, 127)
// One warp per row; the row is read once (16-byte loads, kept in registers while the maximum is
// reduced) and written once: 3 bytes of HBM traffic per element.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>

namespace bm {

constexpr int kQuantThreads = 256;             // 8 warps = 8 rows per CTA
constexpr int kQuantHeld = 16;                 // 16 x 8 halves x 32 lanes = 4096 columns held in registers

// One WARP per row: all of the row's 16-byte loads are issued before the first is used (up to 8 KiB
// in flight per warp, 64 warps per SM), the maximum is reduced with shuffles, no block barrier.
__global__ void __launch_bounds__(kQuantThreads)
quantize_rows_f16_kernel(const __half* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scale, int M, int K) {
    const int row = blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= M) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * K);
    const int vecs = K / 8;                    // K % 16 == 0

    uint4 held[kQuantHeld];
#pragma unroll
    for (int i = 0; i < kQuantHeld; ++i) {
        const int v = lane + i * 32;
        held[i] = v < vecs ? __ldg(src + v) : make_uint4(0, 0, 0, 0);
    }
    float mx = 0.f;
#pragma unroll
    for (int i = 0; i < kQuantHeld; ++i) {
        const __half2* h = reinterpret_cast<const __half2*>(&held[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
    }
    for (int v = lane + kQuantHeld * 32; v < vecs; v += 32) {          // rows longer than 4096: rest of the row
        const uint4 d = __ldg(src + v);
        const __half2* h = reinterpret_cast<const __half2*>(&d);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));

    const float s = mx == 0.f ? 1.0f : __fdiv_rn(mx, 127.0f);
    const float inv = __fdiv_rn(1.0f, s);
    if (lane == 0) scale[row] = s;

    uint2* dst = reinterpret_cast<uint2*>(q + static_cast<size_t>(row) * K);
    auto emit = [&](const uint4& d, int v) {
        const __half* h = reinterpret_cast<const __half*>(&d);
        uint32_t packed[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int r = static_cast<int>(roundf(__fmul_rn(__half2float(h[j]), inv)));
            r = r > 127 ? 127 : (r < -128 ? -128 : r);
            packed[j >> 2] |= (static_cast<uint32_t>(r) & 0xFFu) << (8 * (j & 3));
        }
        dst[v] = make_uint2(packed[0], packed[1]);
    };
#pragma unroll
    for (int i = 0; i < kQuantHeld; ++i) {
        const int v = lane + i * 32;
        if (v < vecs) emit(held[i], v);
    }
    for (int v = lane + kQuantHeld * 32; v < vecs; v += 32) emit(__ldg(src + v), v);   // second read hits L2
}

}  // namespace bm
