// bench_sparse.cpp — C++ driver for the 2:4 sparse INT8 GEMM, the counterpart of the reference's
// kernels/gemm/igemm/bench_sparse.cu with its cubin load replaced by a call into libbm_igemm.so.
//
//   ./bench_sparse [M] [N] [K]         (default 256 256 256; M, N % 16 == 0, K % 32 == 0)
//
// Same flow and stdout contract (bench_sparse.cu:19-103): libc-rand() 2:4 generator with seed 42,
// compressor to values + uint32 metadata words, B from srand(137) without zeros, exact int32 CPU
// reference scaled by (1/127)^2, 0.5/0.1 AND-logic check, and for M >= 512 a timed run (5 warm-up,
// 50 launches) printed as "<ms> ms  <eff> eff GFLOPS  <dense> dense-equiv GFLOPS".
#include <cstdint>
#include <cstring>
#include <vector>

#include "host_common.h"
#include "sparse_host.h"

int main(int argc, char** argv) {
    int M = argc > 1 ? atoi(argv[1]) : 256, N = argc > 2 ? atoi(argv[2]) : M, K = argc > 3 ? atoi(argv[3]) : M;
    if (M % 16 != 0 || N % 16 != 0 || K % 32 != 0) {
        fprintf(stderr, "M, N must be multiples of 16; K must be multiple of 32\n");
        return 1;
    }
    printf("=== Sparse INT8 GEMM Benchmark (libbm_igemm, sm_100a tcgen05.mma.sp) ===\n");
    printf("M=%d  N=%d  K=%d\n\n", M, N, K);
    cudaDeviceProp prop;
    CHECK_CUDA(cudaGetDeviceProperties(&prop, 0));
    printf("Device: %s\n\n", prop.name);

    const size_t na = (size_t)M * K, nb = (size_t)K * N, nc = (size_t)M * N, nmeta = (size_t)(M / 16) * (K / 32) * 8;
    std::vector<int8_t> A(na), comp(na / 2), B(nb);
    std::vector<uint32_t> meta(nmeta);
    std::vector<int32_t> ref_i(nc, 0);
    std::vector<float> ref(nc), out(nc);
    const float sa = 1.0f / 127.0f, sb = 1.0f / 127.0f;
    gen_sparse(A.data(), M, K, 42);
    compress(A.data(), M, K, comp.data(), meta.data());
    fill_nonzero_i8(B.data(), nb, 137);
    cpu_sparse_gemm(A.data(), B.data(), ref_i.data(), M, N, K);
    const float dq = sa * sb;
    for (size_t i = 0; i < nc; ++i) ref[i] = (float)ref_i[i] * dq;

    int8_t *dComp, *dB;
    float* dC;
    uint32_t* dMeta;
    CHECK_CUDA(cudaMalloc(&dComp, na / 2)); CHECK_CUDA(cudaMalloc(&dB, nb)); CHECK_CUDA(cudaMalloc(&dC, nc * 4));
    CHECK_CUDA(cudaMalloc(&dMeta, nmeta * 4));
    CHECK_CUDA(cudaMemcpy(dComp, comp.data(), na / 2, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dB, B.data(), nb, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dMeta, meta.data(), nmeta * 4, cudaMemcpyHostToDevice));
    auto launch = [&]() { CHECK_BM(bm_igemm_sparse_f32(dComp, dB, dC, dMeta, M, N, K, sa, sb, nullptr)); };

    CHECK_CUDA(cudaMemset(dC, 0, nc * 4));
    launch();
    CHECK_CUDA(cudaDeviceSynchronize());
    CHECK_CUDA(cudaMemcpy(out.data(), dC, nc * 4, cudaMemcpyDeviceToHost));
    const CheckOutcome r = check_and_logic(out.data(), ref.data(), (int)nc, 0.5f, 0.1f);
    print_check("igemm_sparse_tiled (INT8)", r);

    if (M >= 512) {
        for (int i = 0; i < 5; ++i) launch();
        CHECK_CUDA(cudaDeviceSynchronize());
        EventTimer t;
        t.start();
        for (int i = 0; i < 50; ++i) launch();
        const float ms = t.stop_ms() / 50.f;
        const double eff = 2.0 * M * N * (K / 2.0) / (ms / 1000.0) / 1e9, dense = 2.0 * M * N * (double)K / (ms / 1000.0) / 1e9;
        printf("  %-34s %9.3f ms  %8.0f eff GFLOPS  %8.0f dense-equiv GFLOPS\n", "igemm_sparse_tiled", ms, eff, dense);
    }
    int code = 0;
    CHECK_BM(bm_last_device_status(&code));
    if (code != 0) { fprintf(stderr, "device status %d\n", code); return EXIT_FAILURE; }
    cudaFree(dComp); cudaFree(dB); cudaFree(dC); cudaFree(dMeta);
    bm_shutdown();
    return r.errors ? EXIT_FAILURE : EXIT_SUCCESS;
}
