// sparse_host.h — host-side pieces shared by the 2:4 sparse bench drivers: the reference's seeded generator,
// compressor, dense-operand fill and exact int32 CPU GEMM (kernels/gemm/igemm/sparse_meta_int8.h:65-208,
// bench_sparse.cu:57-60), restated so the drivers build without the reference checkout.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <cstring>

// 2 of every 4 positions non-zero; rows r and r+8 of a 16-row tile share positions — sparse_meta_int8.h:65-105
static inline void gen_sparse(int8_t* A, int M, int K, unsigned seed) {
    srand(seed);
    memset(A, 0, (size_t)M * K);
    for (int mt = 0; mt < M / 16; ++mt)
        for (int gid = 0; gid < 8; ++gid) {
            const int lo = mt * 16 + gid, hi = lo + 8;
            for (int g = 0; g < K / 4; ++g) {
                int perm[4] = {0, 1, 2, 3};
                for (int i = 3; i >= 2; --i) { int j = rand() % (i + 1); int t = perm[i]; perm[i] = perm[j]; perm[j] = t; }
                int p0 = perm[2], p1 = perm[3];
                if (p0 > p1) { int t = p0; p0 = p1; p1 = t; }
                int8_t v[4];
                for (int i = 0; i < 4; ++i) do { v[i] = (int8_t)((rand() % 255) - 127); } while (v[i] == 0);
                A[(size_t)lo * K + g * 4 + p0] = v[0]; A[(size_t)lo * K + g * 4 + p1] = v[1];
                A[(size_t)hi * K + g * 4 + p0] = v[2]; A[(size_t)hi * K + g * 4 + p1] = v[3];
            }
        }
}
// kept values + one metadata word per (16-row tile, 32-wide K step, gid) — sparse_meta_int8.h:116-178
static inline void compress(const int8_t* A, int M, int K, int8_t* comp, uint32_t* meta) {
    const int ks = K / 32;
    memset(meta, 0, (size_t)(M / 16) * ks * 8 * 4);
    for (int m = 0; m < M; ++m)
        for (int s = 0; s < ks; ++s) {
            uint32_t nib = 0;
            for (int g = 0; g < 8; ++g) {
                const int8_t* v = &A[(size_t)m * K + s * 32 + g * 4];
                int i0 = -1, i1 = -1;
                for (int i = 0; i < 4; ++i)
                    if (v[i] != 0) { if (i0 < 0) i0 = i; else if (i1 < 0) { i1 = i; break; } }
                if (i0 < 0) i0 = 0;
                if (i1 < 0) i1 = 1;
                comp[(size_t)m * (K / 2) + s * 16 + g * 2] = v[i0];
                comp[(size_t)m * (K / 2) + s * 16 + g * 2 + 1] = v[i1];
                nib |= (((uint32_t)i1 << 2) | (uint32_t)i0) << (g * 4);
            }
            if (m % 16 < 8) meta[((size_t)(m / 16) * ks + s) * 8 + (m % 16) % 8] = nib;
        }
}

// dense operand: libc rand() values in [-127, 127] without zeros — bench_sparse.cu:57-60
static inline void fill_nonzero_i8(int8_t* B, size_t n, unsigned seed) {
    srand(seed);
    for (size_t i = 0; i < n; ++i) { int8_t v; do { v = (int8_t)((rand() % 255) - 127); } while (v == 0); B[i] = v; }
}
// exact int32 GEMM in row x k x column order, zeros of A skipped — sparse_meta_int8.h:190-208
static inline void cpu_sparse_gemm(const int8_t* A, const int8_t* B, int32_t* C, int M, int N, int K) {
    memset(C, 0, (size_t)M * N * sizeof(int32_t));
    for (int r = 0; r < M; ++r)
        for (int k = 0; k < K; ++k) {
            const int8_t a = A[(size_t)r * K + k];
            if (a == 0) continue;
            const int8_t* b = &B[(size_t)k * N];
            int32_t* c = &C[(size_t)r * N];
            for (int n = 0; n < N; ++n) c[n] += (int32_t)a * (int32_t)b[n];
        }
}
