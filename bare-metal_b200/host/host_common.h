// host_common.h — shared pieces of the C++ bench drivers: CUDA error check, event timer,
// throughput formula and the AND-logic comparator, with the reference's printing formats so that
// the reference's stdout-parsing gate reads these drivers' output unchanged
// (kernels/_common/bench.h:21-75, kernels/_common/check.h:25-69).
#pragma once
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>

#include "bm_igemm.h"

#define CHECK_CUDA(call)                                                                           \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) {                                                                   \
            fprintf(stderr, "CUDA error at %s:%d — %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
            exit(EXIT_FAILURE);                                                                    \
        }                                                                                          \
    } while (0)

#define CHECK_BM(call)                                                                             \
    do {                                                                                           \
        int rc_ = (call);                                                                          \
        if (rc_ != BM_OK) {                                                                        \
            fprintf(stderr, "libbm_igemm error at %s:%d — %d (%s)\n", __FILE__, __LINE__, rc_,    \
                    bm_last_error_string());                                                       \
            exit(EXIT_FAILURE);                                                                    \
        }                                                                                          \
    } while (0)

struct EventTimer {
    cudaEvent_t a, b;
    EventTimer() { CHECK_CUDA(cudaEventCreate(&a)); CHECK_CUDA(cudaEventCreate(&b)); }
    ~EventTimer() { cudaEventDestroy(a); cudaEventDestroy(b); }
    void start() { CHECK_CUDA(cudaEventRecord(a, nullptr)); }
    float stop_ms() {
        float ms = 0.f;
        CHECK_CUDA(cudaEventRecord(b, nullptr));
        CHECK_CUDA(cudaEventSynchronize(b));
        CHECK_CUDA(cudaEventElapsedTime(&ms, a, b));
        return ms;
    }
};

// 2*M*N*K operations in `ms`, in units of 1e9 per second (the reference labels this "TOPS")
inline double gemm_gops(int M, int N, int K, float ms) { return 2.0 * M * N * K / (ms / 1000.0) / 1e9; }

struct CheckOutcome { int errors, total; float max_abs, max_rel; };

// wrong only when BOTH the absolute and the relative error exceed their limits
inline CheckOutcome check_and_logic(const float* gpu, const float* ref, int n, float abs_tol, float rel_tol) {
    CheckOutcome r{0, n, 0.f, 0.f};
    for (int i = 0; i < n; ++i) {
        float abs_err = fabsf(gpu[i] - ref[i]), ref_abs = fabsf(ref[i]);
        float rel_err = ref_abs > 1e-8f ? abs_err / ref_abs : abs_err;
        r.max_abs = fmaxf(r.max_abs, abs_err);
        r.max_rel = fmaxf(r.max_rel, rel_err);
        if (abs_err > abs_tol && rel_err > rel_tol) ++r.errors;
    }
    return r;
}

inline void print_check(const char* label, const CheckOutcome& r) {
    if (r.errors == 0)
        printf("  %-30s PASS  (max_abs=%.2e  max_rel=%.2e)\n", label, r.max_abs, r.max_rel);
    else
        printf("  %-30s FAIL  %d/%d wrong  (max_abs=%.2e  max_rel=%.2e)\n", label, r.errors, r.total, r.max_abs, r.max_rel);
}
