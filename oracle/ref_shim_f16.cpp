/*
 * ref_shim_f16.cpp — C-ABI handles onto the reference project's FP16 2:4 host utilities.
 *
 * TEST INFRASTRUCTURE ONLY, no arithmetic of its own: includes
 * kernels/gemm/hgemm_sparse/sparse_meta.h where it lies (include path from the Makefile; needs
 * cuda_fp16.h from the CUDA toolkit for __half on the host) and forwards to sparse_meta_count,
 * gen_random_sparse_2_4, compress_2_4_arbitrary and cpu_sparse_gemm_arbitrary.  Built into
 * oracle/_ref/libbm_ref_f16.so; pins the restatement in igemm_oracle.c.
 */
#include "sparse_meta.h"

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API size_t ref_h_sparse_meta_count(int M, int K) { return sparse_meta_count(M, K); }

REF_API void ref_h_gen_sparse_2_4(float *A, int M, int K, unsigned int seed) { gen_random_sparse_2_4(A, M, K, seed); }

REF_API void ref_h_compress_2_4(const float *A, int M, int K, uint16_t *A_comp, uint32_t *meta)
{
    compress_2_4_arbitrary(A, M, K, reinterpret_cast<__half *>(A_comp), meta);
}

REF_API void ref_h_cpu_sparse_gemm(const float *A, const float *B, float *C, int M, int N, int K)
{
    cpu_sparse_gemm_arbitrary(A, B, C, M, N, K);
}
