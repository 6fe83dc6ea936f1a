/*
 * igemm_oracle.c — CPU restatement of the bare-metal INT8 GEMM hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared against (and the "port" CPU baseline the benchmark times beside
 * them).  Nothing in the shipped library or its host-side wrappers may call
 * into it; the product path has no CPU fallback.
 *
 * Parity status: PINNED.  Every function that restates reference code is
 * checked, bit for bit, against the reference's own headers compiled in place
 * (see ref_shim.cpp / Makefile target `ref`) and against the fixtures
 * generated from them under tests/golden/.
 *
 * Each function cites the reference file:line (paths relative to the
 * reference project's root) whose behaviour it follows.  Functions marked
 * "NEW" have no reference counterpart: they are the seeded generators and the
 * fp16 / per-row formats that the B200 workloads need.
 *
 * Plain C99 + pthreads (the row-parallel GEMM used as a timed multi-core
 * baseline splits rows over threads; the arithmetic per row is unchanged).
 */
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#include <pthread.h>
#include <unistd.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------
 * LCG fill in [-1, 1)            — kernels/_common/check.h:98-106
 * ---------------------------------------------------------------------- */
ORC_API void orc_fill_random(float *matrix, int num_elements, unsigned int seed)
{
    unsigned int state = seed;
    for (int i = 0; i < num_elements; i++) {
        state = state * 1664525u + 1013904223u;
        float unit = (float)(state >> 8) / (float)(1 << 24);
        matrix[i] = unit * 2.0f - 1.0f;
    }
}

/* ------------------------------------------------------------------------
 * Symmetric per-tensor quantisation — kernels/gemm/igemm/bench.cu:28-51
 * ---------------------------------------------------------------------- */
ORC_API float orc_compute_scale(const float *data, int num_elements)
{
    float max_abs = 0.0f;
    for (int i = 0; i < num_elements; i++) {
        float a = fabsf(data[i]);
        if (a > max_abs) max_abs = a;
    }
    if (max_abs == 0.0f) return 1.0f;
    return max_abs / 127.0f;
}

ORC_API void orc_quantize_symmetric(const float *src, int8_t *dst, int num_elements, float scale)
{
    float inv_scale = 1.0f / scale;
    for (int i = 0; i < num_elements; i++) {
        int q = (int)roundf(src[i] * inv_scale);
        if (q > 127) q = 127;
        if (q < -128) q = -128;
        dst[i] = (int8_t)q;
    }
}

/* ------------------------------------------------------------------------
 * Per-channel parameters as the dense bench draws them (libc rand()):
 * scale[n] = sa*sb*(0.8+0.4u), zp[n] in [-2,2] — bench.cu:280-289
 * ---------------------------------------------------------------------- */
ORC_API void orc_gen_per_channel_params(float *scale, int *zero_point, int N,
                                        float scale_a, float scale_b, unsigned int seed)
{
    float sym = scale_a * scale_b;
    srand(seed);
    for (int n = 0; n < N; n++) {
        scale[n] = sym * (0.8f + 0.4f * ((float)rand() / RAND_MAX));
        zero_point[n] = (rand() % 5) - 2;
    }
}

/* ------------------------------------------------------------------------
 * fp32 reference GEMM (m, n, k order) — kernels/_common/check.h:76-93
 * ---------------------------------------------------------------------- */
ORC_API void orc_sgemm(int M, int N, int K, float alpha, const float *A, int lda,
                       const float *B, int ldb, float beta, float *C, int ldc)
{
    for (int row = 0; row < M; row++) {
        for (int col = 0; col < N; col++) {
            float acc = 0.0f;
            for (int k = 0; k < K; k++) acc += A[row * lda + k] * B[k * ldb + col];
            C[row * ldc + col] = alpha * acc + beta * C[row * ldc + col];
        }
    }
}

/* ------------------------------------------------------------------------
 * Exact int32 GEMM, row x k x col order, zero multiplicands skipped
 *                    — kernels/gemm/igemm/sparse_meta_int8.h:190-208
 * B is [K x N] row-major.  Rows [row_begin, row_end) only, so callers can
 * time or check a slab; (0, M) reproduces the reference function.
 * ---------------------------------------------------------------------- */
ORC_API void orc_igemm_rows(const int8_t *A, const int8_t *B, int32_t *C,
                            int M, int N, int K, int row_begin, int row_end)
{
    (void)M;
    for (int row = row_begin; row < row_end; row++) {
        int32_t *c_row = &C[(size_t)row * N];
        memset(c_row, 0, (size_t)N * sizeof(int32_t));
        for (int k = 0; k < K; k++) {
            int8_t a = A[(size_t)row * K + k];
            if (a == 0) continue;
            const int8_t *b_row = &B[(size_t)k * N];
            for (int col = 0; col < N; col++) c_row[col] += (int32_t)a * (int32_t)b_row[col];
        }
    }
}

ORC_API void orc_igemm(const int8_t *A, const int8_t *B, int32_t *C, int M, int N, int K)
{
    orc_igemm_rows(A, B, C, M, N, K, 0, M);
}

/* Same arithmetic with the rows dealt out to `threads` pthreads in contiguous
 * slabs (the multi-core timed baseline).  threads <= 0 means all online cores.
 * Returns the thread count used. */
struct slab_job {
    const int8_t *A, *B; int32_t *C; int M, N, K, row_begin, row_end; int nt;
};

static void *slab_main(void *arg)
{
    struct slab_job *j = (struct slab_job *)arg;
    if (j->nt) {
        for (int m = j->row_begin; m < j->row_end; m++) {
            const int8_t *a = &j->A[(size_t)m * j->K];
            for (int n = 0; n < j->N; n++) {
                const int8_t *w = &j->B[(size_t)n * j->K];
                int32_t acc = 0;
                for (int k = 0; k < j->K; k++) acc += (int32_t)a[k] * (int32_t)w[k];
                j->C[(size_t)m * j->N + n] = acc;
            }
        }
    } else {
        orc_igemm_rows(j->A, j->B, j->C, j->M, j->N, j->K, j->row_begin, j->row_end);
    }
    return NULL;
}

static int run_slabs(const int8_t *A, const int8_t *B, int32_t *C, int M, int N, int K,
                     int row_begin, int row_end, int threads, int nt)
{
    if (threads <= 0) threads = (int)sysconf(_SC_NPROCESSORS_ONLN);
    int rows = row_end - row_begin;
    if (threads > rows) threads = rows > 0 ? rows : 1;
    if (threads > 256) threads = 256;
    pthread_t tid[256];
    struct slab_job job[256];
    for (int t = 0; t < threads; t++) {
        int b = row_begin + (int)((long long)rows * t / threads);
        int e = row_begin + (int)((long long)rows * (t + 1) / threads);
        struct slab_job j = { A, B, C, M, N, K, b, e, nt };
        job[t] = j;
        pthread_create(&tid[t], NULL, slab_main, &job[t]);
    }
    for (int t = 0; t < threads; t++) pthread_join(tid[t], NULL);
    return threads;
}

ORC_API int orc_igemm_parallel(const int8_t *A, const int8_t *B, int32_t *C,
                               int M, int N, int K, int row_begin, int row_end, int threads)
{
    return run_slabs(A, B, C, M, N, K, row_begin, row_end, threads, 0);
}

/* ------------------------------------------------------------------------
 * Dense integer reference in (m, n, k) order as the per-channel check writes
 * it inline — kernels/gemm/igemm/bench.cu:460-467.  Same integers as
 * orc_igemm; kept because the reference times/uses this order at M <= 512.
 * ---------------------------------------------------------------------- */
ORC_API void orc_igemm_mnk(const int8_t *A, const int8_t *B, int32_t *C, int M, int N, int K)
{
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            int acc = 0;
            for (int k = 0; k < K; k++) acc += (int)A[(size_t)m * K + k] * (int)B[(size_t)k * N + n];
            C[(size_t)m * N + n] = acc;
        }
}

/* NEW: weights given K-major, W[N x K]; C[m][n] = sum_k A[m][k] * W[n][k].
 * Integer arithmetic is order-independent, so this equals orc_igemm on the
 * transposed weights; used where the workload stores weights [N x K]. */
ORC_API int orc_igemm_nt_rows(const int8_t *A, const int8_t *W, int32_t *C,
                              int M, int N, int K, int row_begin, int row_end, int threads)
{
    return run_slabs(A, W, C, M, N, K, row_begin, row_end, threads, 1);
}

/* ------------------------------------------------------------------------
 * Epilogues
 * ---------------------------------------------------------------------- */
/* per-tensor: (float)acc * (scale_a*scale_b) — kernels/gemm/igemm/igemm.cu:104-110,
 * igemm_tiled.cu:153,167, igemm_sparse_tiled.cu:365-380 */
ORC_API void orc_dequant_per_tensor(const int32_t *acc, float *out, size_t count,
                                    float scale_a, float scale_b)
{
    float dequant = scale_a * scale_b;
    for (size_t i = 0; i < count; i++) out[i] = (float)acc[i] * dequant;
}

/* per-channel: ((float)acc - (float)zp[n]) * scale[n]
 *            — kernels/gemm/igemm/igemm_pipelined_cpasync_perchannel.cu:276-281,
 *              kernels/gemm/igemm/bench.cu:466 */
ORC_API void orc_dequant_per_channel(const int32_t *acc, float *out, int M, int N,
                                     const float *scale, const int *zero_point)
{
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++)
            out[(size_t)m * N + n] =
                ((float)acc[(size_t)m * N + n] - (float)zero_point[n]) * scale[n];
}

/* NEW: fp32 -> IEEE binary16, round to nearest even (what __float2half_rn does). */
static uint16_t f32_to_f16_rn(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t abs = x & 0x7FFFFFFFu;
    if (abs >= 0x7F800000u) {                       /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((abs > 0x7F800000u) ? 0x0200u : 0u));
    }
    if (abs >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);   /* rounds to inf */
    if (abs < 0x33000001u) return (uint16_t)sign;                /* rounds to zero */
    int exp = (int)(abs >> 23) - 127;
    uint32_t man = (abs & 0x007FFFFFu) | 0x00800000u;
    int shift;
    uint32_t half_exp;
    if (exp < -14) { shift = 13 + (-14 - exp); half_exp = 0; }   /* subnormal half */
    else { shift = 13; half_exp = (uint32_t)(exp + 15); }
    uint32_t kept = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (kept & 1u))) kept++;
    uint32_t h;
    if (half_exp == 0) h = kept;                    /* may carry into exponent 1: fine */
    else h = ((half_exp - 1) << 10) + kept;         /* kept includes the hidden bit */
    return (uint16_t)(sign | h);
}

ORC_API uint16_t orc_f32_to_f16(float f) { return f32_to_f16_rn(f); }

/* NEW: W8A8 epilogue of the B200 workloads:
 * s = sa[m]*sw[n] (fp32), y = (float)acc * s (fp32), D = half_rn(y). */
ORC_API void orc_dequant_w8a8_f16(const int32_t *acc, uint16_t *out, int M, int N,
                                  const float *sa, const float *sw)
{
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            float s = sa[m] * sw[n];
            float y = (float)acc[(size_t)m * N + n] * s;
            out[(size_t)m * N + n] = f32_to_f16_rn(y);
        }
}

/* ------------------------------------------------------------------------
 * AND-logic comparator — kernels/_common/check.h:25-58.
 * Returns the number of wrong elements; optional outputs mirror CheckResult.
 * ---------------------------------------------------------------------- */
ORC_API int orc_check_fp32(const float *gpu, const float *ref, int num_elements,
                           float abs_tol, float rel_tol,
                           float *max_abs_out, float *max_rel_out, int *first_error_out)
{
    int errors = 0, first = -1;
    float max_abs = 0.0f, max_rel = 0.0f;
    for (int i = 0; i < num_elements; i++) {
        float abs_err = fabsf(gpu[i] - ref[i]);
        float ref_abs = fabsf(ref[i]);
        float rel_err = (ref_abs > 1e-8f) ? (abs_err / ref_abs) : abs_err;
        max_abs = fmaxf(max_abs, abs_err);
        max_rel = fmaxf(max_rel, rel_err);
        if (abs_err > abs_tol && rel_err > rel_tol) {
            errors++;
            if (first < 0) first = i;
        }
    }
    if (max_abs_out) *max_abs_out = max_abs;
    if (max_rel_out) *max_rel_out = max_rel;
    if (first_error_out) *first_error_out = first;
    return errors;
}

/* ------------------------------------------------------------------------
 * Reference 2:4 INT8 operand format — kernels/gemm/igemm/sparse_meta_int8.h
 * ---------------------------------------------------------------------- */
/* :46-50 */
ORC_API size_t orc_sparse_meta_count(int M, int K)
{
    return (size_t)(M / 16) * (size_t)(K / 32) * 8;
}

/* :65-105 — libc rand() generator; rows r and r+8 of a 16-row tile share positions */
ORC_API void orc_gen_sparse_2_4_ref(int8_t *A_dense, int M, int K, unsigned int seed)
{
    srand(seed);
    memset(A_dense, 0, (size_t)M * K);
    int m_tiles = M / 16, k_groups = K / 4;
    for (int mt = 0; mt < m_tiles; mt++)
        for (int gid = 0; gid < 8; gid++) {
            int row_lo = mt * 16 + gid, row_hi = row_lo + 8;
            for (int g = 0; g < k_groups; g++) {
                int perm[4] = {0, 1, 2, 3};
                for (int i = 3; i >= 2; i--) {
                    int j = rand() % (i + 1);
                    int t = perm[i]; perm[i] = perm[j]; perm[j] = t;
                }
                int p0 = perm[2], p1 = perm[3];
                if (p0 > p1) { int t = p0; p0 = p1; p1 = t; }
                int8_t v[4];
                for (int i = 0; i < 4; i++) {
                    do { v[i] = (int8_t)((rand() % 255) - 127); } while (v[i] == 0);
                }
                A_dense[(size_t)row_lo * K + g * 4 + p0] = v[0];
                A_dense[(size_t)row_lo * K + g * 4 + p1] = v[1];
                A_dense[(size_t)row_hi * K + g * 4 + p0] = v[2];
                A_dense[(size_t)row_hi * K + g * 4 + p1] = v[3];
            }
        }
}

/* :116-178 — positions found by value != 0, fall-backs idx0=0 / idx1=1,
 * metadata word written only from the lower row of each (r, r+8) pair */
ORC_API void orc_compress_2_4_ref(const int8_t *A_dense, int M, int K,
                                  int8_t *A_comp, uint32_t *meta)
{
    int k_stored = K / 2, k_steps = K / 32;
    memset(meta, 0, orc_sparse_meta_count(M, K) * sizeof(uint32_t));
    for (int m = 0; m < M; m++) {
        int m_tile = m / 16, tile_row = m % 16, gid = tile_row % 8;
        for (int ks = 0; ks < K; ks += 32) {
            uint32_t nibbles = 0;
            for (int g = 0; g < 8; g++) {
                const int8_t *v = &A_dense[(size_t)m * K + ks + g * 4];
                int idx0 = -1, idx1 = -1;
                for (int i = 0; i < 4; i++) {
                    if (v[i] != 0) {
                        if (idx0 < 0) idx0 = i;
                        else if (idx1 < 0) { idx1 = i; break; }
                    }
                }
                if (idx0 < 0) idx0 = 0;
                if (idx1 < 0) idx1 = 1;
                A_comp[(size_t)m * k_stored + ks / 2 + g * 2 + 0] = v[idx0];
                A_comp[(size_t)m * k_stored + ks / 2 + g * 2 + 1] = v[idx1];
                nibbles |= (((uint32_t)idx1 << 2) | (uint32_t)idx0) << (g * 4);
            }
            if (tile_row < 8) meta[(m_tile * k_steps + ks / 32) * 8 + gid] = nibbles;
        }
    }
}

/* Inverse of the format described at :13-31 (decompress compressed values +
 * reference metadata back to a dense [M x K] matrix). */
ORC_API void orc_decompress_2_4_ref(const int8_t *A_comp, const uint32_t *meta,
                                    int M, int K, int8_t *A_dense)
{
    int k_stored = K / 2, k_steps = K / 32;
    memset(A_dense, 0, (size_t)M * K);
    for (int m = 0; m < M; m++) {
        int m_tile = m / 16, gid = (m % 16) % 8;
        for (int s = 0; s < k_steps; s++) {
            uint32_t word = meta[(m_tile * k_steps + s) * 8 + gid];
            for (int g = 0; g < 8; g++) {
                uint32_t nib = (word >> (4 * g)) & 0xFu;
                /* += keeps the sum right even for a degenerate nibble with idx0 == idx1 */
                A_dense[(size_t)m * K + 32 * s + 4 * g + (nib & 3u)] += A_comp[(size_t)m * k_stored + 16 * s + 2 * g];
                A_dense[(size_t)m * K + 32 * s + 4 * g + (nib >> 2)] += A_comp[(size_t)m * k_stored + 16 * s + 2 * g + 1];
            }
        }
    }
}

/* ------------------------------------------------------------------------
 * NEW: per-row 2:4 format of the B200 workloads.
 *   comp [R x K/2]  : kept values, lower index first
 *   nib  [R x K/8]  : one byte per 8 logical K = two groups;
 *                     low nibble = group 2j, high nibble = group 2j+1,
 *                     each nibble (idx1 << 2) | idx0 with idx0 < idx1.
 * Any of the 6 patterns per (row, group); rows are independent.
 * ---------------------------------------------------------------------- */
ORC_API void orc_decompress_rows(const int8_t *comp, const uint8_t *nib, int R, int K, int8_t *dense)
{
    memset(dense, 0, (size_t)R * K);
    for (int r = 0; r < R; r++)
        for (int g = 0; g < K / 4; g++) {
            uint8_t byte = nib[(size_t)r * (K / 8) + g / 2];
            uint32_t n = (g & 1) ? (byte >> 4) : (byte & 0xF);
            dense[(size_t)r * K + 4 * g + (n & 3u)] += comp[(size_t)r * (K / 2) + 2 * g];
            dense[(size_t)r * K + 4 * g + (n >> 2)] += comp[(size_t)r * (K / 2) + 2 * g + 1];
        }
}

/* NEW (the reference has a compressor but no pruner): magnitude pruning to 2:4 with compression.
 * Keeps the two largest |w| of every aligned group of 4 (ties: lower position), lower position first,
 * nibble (idx1 << 2) | idx0 as compress_2_4_int8 writes it (:137-138,166-167).  On a matrix that is
 * already 2:4 with non-zero kept values it must reproduce orc_compress_2_4_ref — tested. */
ORC_API void orc_prune_2_4_rows(const int8_t *W, int R, int K, int8_t *comp, uint8_t *nib)
{
    memset(nib, 0, (size_t)R * (K / 8));
    for (int r = 0; r < R; r++)
        for (int g = 0; g < K / 4; g++) {
            const int8_t *v = &W[(size_t)r * K + 4 * g];
            int best = -1, second = -1;
            for (int i = 0; i < 4; i++) {           /* strict > keeps the lower position on ties */
                int a = abs((int)v[i]);
                if (best < 0 || a > abs((int)v[best])) { second = best; best = i; }
                else if (second < 0 || a > abs((int)v[second])) second = i;
            }
            int idx0 = best < second ? best : second, idx1 = best < second ? second : best;
            comp[(size_t)r * (K / 2) + 2 * g] = v[idx0];
            comp[(size_t)r * (K / 2) + 2 * g + 1] = v[idx1];
            uint8_t n = (uint8_t)((idx1 << 2) | idx0);
            nib[(size_t)r * (K / 8) + g / 2] |= (uint8_t)((g & 1) ? (n << 4) : n);
        }
}

/* Reference metadata words -> per-row nibble bytes (rows r and r+8 share). */
ORC_API void orc_meta_ref_to_rows(const uint32_t *meta, int M, int K, uint8_t *nib)
{
    int k_steps = K / 32;
    for (int m = 0; m < M; m++) {
        int m_tile = m / 16, gid = (m % 16) % 8;
        for (int s = 0; s < k_steps; s++) {
            uint32_t word = meta[(m_tile * k_steps + s) * 8 + gid];
            memcpy(&nib[(size_t)m * (K / 8) + 4 * s], &word, 4);   /* little endian: byte j = groups 2j, 2j+1 */
        }
    }
}

/* ------------------------------------------------------------------------
 * NEW: counter-based generators (identical bytes from C, Python-via-ctypes
 * and any other caller): value i of stream s under seed = mix(seed, s, i).
 * ---------------------------------------------------------------------- */
static inline uint64_t mix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

static inline uint64_t draw(uint64_t seed, uint64_t stream, uint64_t index)
{
    return mix64(mix64(seed * 0xD1342543DE82EF95ull + stream) + index);
}

/* int8 i.i.d. uniform on the integers [-127, 127] */
ORC_API void orc_gen_int8_uniform(int8_t *out, size_t count, uint64_t seed, uint64_t stream)
{
    for (size_t i = 0; i < count; i++) out[i] = (int8_t)((int)(draw(seed, stream, i) % 255u) - 127);
}

/* fp32 uniform on [lo, lo+span): lo + u*span with u a 24-bit fraction, one fused rounding */
ORC_API void orc_gen_f32_uniform(float *out, size_t count, float lo, float span,
                                 uint64_t seed, uint64_t stream)
{
    for (size_t i = 0; i < count; i++) {
        float u = (float)(draw(seed, stream, i) >> 40) * (1.0f / 16777216.0f);
        out[i] = fmaf(u, span, lo);
    }
}

/* per-row 2:4 operand: pattern uniform over the 6 pairs, values uniform on
 * [-127,127] \ {0}; writes the compressed values and the per-row nibbles */
ORC_API void orc_gen_sparse_rows(int8_t *comp, uint8_t *nib, int R, int K,
                                 uint64_t seed, uint64_t stream)
{
    static const uint8_t pattern[6] = { (1 << 2) | 0, (2 << 2) | 0, (3 << 2) | 0,
                                        (2 << 2) | 1, (3 << 2) | 1, (3 << 2) | 2 };
    size_t groups_per_row = (size_t)K / 4;
    for (int r = 0; r < R; r++) {
        for (size_t g = 0; g < groups_per_row; g++) {
            uint64_t h = draw(seed, stream, (size_t)r * groups_per_row + g);
            uint8_t n = pattern[h % 6u];
            unsigned v0 = (unsigned)((h >> 16) % 254u), v1 = (unsigned)((h >> 40) % 254u);
            comp[(size_t)r * (K / 2) + 2 * g]     = (int8_t)(v0 < 127 ? (int)v0 - 127 : (int)v0 - 126);
            comp[(size_t)r * (K / 2) + 2 * g + 1] = (int8_t)(v1 < 127 ? (int)v1 - 127 : (int)v1 - 126);
            uint8_t *b = &nib[(size_t)r * (K / 8) + g / 2];
            if (g & 1) *b = (uint8_t)((*b & 0x0F) | (n << 4));
            else       *b = (uint8_t)((*b & 0xF0) | n);
        }
    }
}

/* ------------------------------------------------------------------------
 * kernels/gemm/igemm/igemm_online_quant.cu (FP16 in, per-tile int8 quantisation, fp32 out),
 * also _inplace, _bankfree, igemm_warp_specialized (col_block 128) and _bf_128x256 (256).
 * Per 128 x col_block output tile (:170-173): max|A| over the tile's rows x K[0,32) and max|B|
 * over K[0,32) x the tile's columns (QUANTIZE_TILE on tile 0, :66-98,255); inv = 127/max or 1
 * (:100-101); every K tile is quantised with those factors (QUANTIZE_TILE_FAST, :127-142,393):
 * q = clamp(rint(x * inv), -128, 127) (:103-116); per K tile the int32 sum is folded into an fp32
 * running value, running += (float)acc * tile_scale (:340-347,396-433), tile_scale =
 * (max_a/127) * (max_b/127) (:120).  nvcc contracts that update into one FMA, so fmaf here.
 * Elements outside the matrices read as zero (:206-220).
 * ---------------------------------------------------------------------- */
static float half_bits_to_float(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 112u) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static int8_t oq_quant(float v, float inv)
{
    volatile float prod = v * inv;                 /* one fp32 multiply, no contraction */
    long q = lrintf(prod);                         /* round to nearest even, like __float2int_rn */
    if (q < -128) q = -128;
    if (q > 127) q = 127;
    return (int8_t)q;
}

ORC_API void orc_online_quant_gemm(const uint16_t *A, const uint16_t *B, float *C,
                                   int M, int N, int K, int col_block)
{
    const int BMr = 128, BK = 32;
    int blocks_a = (M + BMr - 1) / BMr, blocks_b = (N + col_block - 1) / col_block;
    int tiles = (K + BK - 1) / BK;
    float *max_a = (float *)calloc((size_t)blocks_a, sizeof(float));
    float *max_b = (float *)calloc((size_t)blocks_b, sizeof(float));
    int8_t *Aq = (int8_t *)malloc((size_t)M * K), *Bq = (int8_t *)malloc((size_t)K * N);
    for (int m = 0; m < M; m++)
        for (int k = 0; k < BK && k < K; k++)
            max_a[m / BMr] = fmaxf(max_a[m / BMr], fabsf(half_bits_to_float(A[(size_t)m * K + k])));
    for (int k = 0; k < BK && k < K; k++)
        for (int n = 0; n < N; n++)
            max_b[n / col_block] = fmaxf(max_b[n / col_block], fabsf(half_bits_to_float(B[(size_t)k * N + n])));
    for (int m = 0; m < M; m++) {
        float mx = max_a[m / BMr], inv = mx > 0.0f ? 127.0f / mx : 1.0f;
        for (int k = 0; k < K; k++) Aq[(size_t)m * K + k] = oq_quant(half_bits_to_float(A[(size_t)m * K + k]), inv);
    }
    for (int n = 0; n < N; n++) {
        float mx = max_b[n / col_block], inv = mx > 0.0f ? 127.0f / mx : 1.0f;
        for (int k = 0; k < K; k++) Bq[(size_t)k * N + n] = oq_quant(half_bits_to_float(B[(size_t)k * N + n]), inv);
    }
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            float tile_scale = (max_a[m / BMr] / 127.0f) * (max_b[n / col_block] / 127.0f);
            float running = 0.0f;
            for (int t = 0; t < tiles; t++) {
                int32_t acc = 0;
                for (int k = t * BK; k < (t + 1) * BK && k < K; k++)
                    acc += (int32_t)Aq[(size_t)m * K + k] * (int32_t)Bq[(size_t)k * N + n];
                running = fmaf((float)acc, tile_scale, running);
            }
            C[(size_t)m * N + n] = running;
        }
    free(max_a); free(max_b); free(Aq); free(Bq);
}

/* ------------------------------------------------------------------------
 * kernels/gemm/hgemm_sparse/sparse_meta.h — FP16 sibling of the 2:4 utilities (K step 16).
 * ---------------------------------------------------------------------- */
/* :46-50 */
ORC_API size_t orc_h_sparse_meta_count(int M, int K)
{
    return (size_t)(M / 16) * (size_t)(K / 16) * 8;
}

/* :65-105 — libc rand(); rows gid and gid+8 of a 16-row tile share positions; values in (-1,1) \ {0} */
static float h_rval(void)
{
    float v;
    do { v = ((float)rand() / RAND_MAX) * 2.0f - 1.0f; } while (v == 0.0f);
    return v;
}

ORC_API void orc_h_gen_sparse_2_4(float *A_dense, int M, int K, unsigned int seed)
{
    srand(seed);
    memset(A_dense, 0, (size_t)M * K * sizeof(float));
    for (int mt = 0; mt < M / 16; mt++)
        for (int gid = 0; gid < 8; gid++) {
            int row_lo = mt * 16 + gid, row_hi = row_lo + 8;
            for (int g = 0; g < K / 4; g++) {
                int perm[4] = {0, 1, 2, 3};
                for (int i = 3; i >= 2; i--) {
                    int j = rand() % (i + 1);
                    int t = perm[i]; perm[i] = perm[j]; perm[j] = t;
                }
                int p0 = perm[2], p1 = perm[3];
                if (p0 > p1) { int t = p0; p0 = p1; p1 = t; }
                A_dense[(size_t)row_lo * K + g * 4 + p0] = h_rval();
                A_dense[(size_t)row_lo * K + g * 4 + p1] = h_rval();
                A_dense[(size_t)row_hi * K + g * 4 + p0] = h_rval();
                A_dense[(size_t)row_hi * K + g * 4 + p1] = h_rval();
            }
        }
}

/* :128-190 — positions by value != 0 (fall-backs 0 / 1), values rounded to fp16, one word per
 * (16-row tile, K step of 16, gid) from the lower row, nibbles duplicated into bits 31:16 */
ORC_API void orc_h_compress_2_4(const float *A_dense, int M, int K, uint16_t *A_comp, uint32_t *meta)
{
    int k_stored = K / 2, k_steps = K / 16;
    memset(meta, 0, orc_h_sparse_meta_count(M, K) * sizeof(uint32_t));
    for (int m = 0; m < M; m++) {
        int m_tile = m / 16, tile_row = m % 16, gid = tile_row % 8;
        for (int ks = 0; ks < K; ks += 16) {
            uint32_t nibbles = 0;
            for (int g = 0; g < 4; g++) {
                const float *v = &A_dense[(size_t)m * K + ks + g * 4];
                int idx0 = -1, idx1 = -1;
                for (int i = 0; i < 4; i++)
                    if (v[i] != 0.0f) {
                        if (idx0 < 0) idx0 = i;
                        else if (idx1 < 0) { idx1 = i; break; }
                    }
                if (idx0 < 0) idx0 = 0;
                if (idx1 < 0) idx1 = 1;
                A_comp[(size_t)m * k_stored + ks / 2 + g * 2 + 0] = f32_to_f16_rn(v[idx0]);
                A_comp[(size_t)m * k_stored + ks / 2 + g * 2 + 1] = f32_to_f16_rn(v[idx1]);
                nibbles |= (((uint32_t)idx1 << 2) | (uint32_t)idx0) << (g * 4);
            }
            if (tile_row < 8) meta[(m_tile * k_steps + ks / 16) * 8 + gid] = nibbles | (nibbles << 16);
        }
    }
}

/* :207-223 — fp32 reference, row x k x col, zeros skipped */
ORC_API void orc_h_cpu_sparse_gemm(const float *A_dense, const float *B, float *C, int M, int N, int K)
{
    memset(C, 0, (size_t)M * N * sizeof(float));
    for (int row = 0; row < M; row++)
        for (int k = 0; k < K; k++) {
            float a = A_dense[(size_t)row * K + k];
            if (a == 0.0f) continue;
            const float *b_row = &B[(size_t)k * N];
            float *c_row = &C[(size_t)row * N];
            for (int col = 0; col < N; col++) {
                volatile float prod = a * b_row[col];      /* product and sum round separately (host code, -O2, no FMA) */
                c_row[col] += prod;
            }
        }
}

/* inverse of the format: compressed fp16 + reference words -> dense fp16 bits (NEW, for tests) */
ORC_API void orc_h_decompress_2_4(const uint16_t *A_comp, const uint32_t *meta, int M, int K, uint16_t *A_dense)
{
    int k_stored = K / 2, k_steps = K / 16;
    memset(A_dense, 0, (size_t)M * K * sizeof(uint16_t));
    for (int m = 0; m < M; m++)
        for (int s = 0; s < k_steps; s++) {
            uint32_t word = meta[((m / 16) * k_steps + s) * 8 + (m % 16) % 8];
            for (int g = 0; g < 4; g++) {
                uint32_t nib = (word >> (4 * g)) & 0xFu;
                A_dense[(size_t)m * K + 16 * s + 4 * g + (nib & 3u)] = A_comp[(size_t)m * k_stored + 8 * s + 2 * g];
                A_dense[(size_t)m * K + 16 * s + 4 * g + (nib >> 2)] = A_comp[(size_t)m * k_stored + 8 * s + 2 * g + 1];
            }
        }
}

/* [R x C] -> [C x R] byte transpose (layout helper for tests) */
ORC_API void orc_transpose_i8(const int8_t *src, int8_t *dst, int R, int C)
{
    for (int r = 0; r < R; r++)
        for (int c = 0; c < C; c++) dst[(size_t)c * R + r] = src[(size_t)r * C + c];
}

ORC_API int orc_num_threads(void) { return (int)sysconf(_SC_NPROCESSORS_ONLN); }
