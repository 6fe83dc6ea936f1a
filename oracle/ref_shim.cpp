/*
 * ref_shim.cpp — C-ABI handles onto the reference project's OWN CPU code.
 *
 * TEST INFRASTRUCTURE ONLY.  This translation unit contains no arithmetic of
 * its own: it includes the reference headers where they lie (the include
 * path is given on the command line by the Makefile; nothing is copied into
 * this repository) and forwards to them.  The resulting shared object
 * (oracle/_ref/libbm_ref.so) is used to pin igemm_oracle.c and to generate
 * the fixtures under tests/golden/, and as the "reference" CPU baseline the
 * benchmark times.
 *
 * Headers used: kernels/_common/check.h (cpu_sgemm, fill_random, check_fp32)
 * and kernels/gemm/igemm/sparse_meta_int8.h (sparse_meta_count_int8,
 * gen_random_sparse_2_4_int8, compress_2_4_int8, cpu_sparse_gemm_int8).
 */
#include "check.h"
#include "sparse_meta_int8.h"

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API void ref_fill_random(float *m, int n, unsigned int seed) { fill_random(m, n, seed); }

REF_API void ref_cpu_sgemm(int M, int N, int K, float alpha, const float *A, int lda,
                           const float *B, int ldb, float beta, float *C, int ldc)
{
    cpu_sgemm(M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
}

REF_API int ref_check_fp32(const float *gpu, const float *ref, int n, float abs_tol, float rel_tol,
                           float *max_abs, float *max_rel, int *first_error)
{
    CheckResult r = check_fp32(gpu, ref, n, abs_tol, rel_tol, false);
    if (max_abs) *max_abs = r.max_abs_error;
    if (max_rel) *max_rel = r.max_rel_error;
    if (first_error) *first_error = r.first_error_index;
    return r.num_errors;
}

REF_API size_t ref_sparse_meta_count_int8(int M, int K) { return sparse_meta_count_int8(M, K); }

REF_API void ref_gen_random_sparse_2_4_int8(int8_t *A, int M, int K, unsigned int seed)
{
    gen_random_sparse_2_4_int8(A, M, K, seed);
}

REF_API void ref_compress_2_4_int8(const int8_t *A, int M, int K, int8_t *A_comp, uint32_t *meta)
{
    compress_2_4_int8(A, M, K, A_comp, meta);
}

REF_API void ref_cpu_sparse_gemm_int8(const int8_t *A, const int8_t *B, int32_t *C, int M, int N, int K)
{
    cpu_sparse_gemm_int8(A, B, C, M, N, K);
}
