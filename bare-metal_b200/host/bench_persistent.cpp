// bench_persistent.cpp — C++ driver for the persistent 2:4 sparse INT8 GEMM, the counterpart of the reference's
// kernels/gemm/igemm/bench_persistent.cu with its cubin load replaced by a call into libbm_igemm.so.
//
//   ./bench_persistent [M] [N] [K]     (default 512 512 512; M, N % 16 == 0, K % 32 == 0)
//
// Same flow and stdout contract (bench_persistent.cu:6-55): seed-42 2:4 generator, compressor, B from
// srand(137), 5 synchronised warm-up launches, then 50 launches enqueued back to back with one synchronisation
// at the end, printed as "  igemm_sparse_tiled_persistent  <ms> ms  <eff> eff GFLOPS  (grid=<g>x1)".  The
// reference hands its kernel one zeroed tile counter per launch for an atomic scheduler (:28-31,43-47); every
// kernel of this library is persistent with a STATIC tile schedule (min(tiles, SMs) CTAs walk the tiles), so
// there is no counter to pass and `grid` reports that CTA count.  Unlike the reference driver, the output of the
// first launch is also checked against the exact CPU product (0.5 / 0.1 AND-logic, as bench_sparse does).
#include <cstdint>
#include <vector>

#include "host_common.h"
#include "sparse_host.h"

int main(int argc, char** argv) {
    int M = argc > 1 ? atoi(argv[1]) : 512, N = argc > 2 ? atoi(argv[2]) : M, K = argc > 3 ? atoi(argv[3]) : M;
    if (M % 16 || N % 16 || K % 32) { printf("bad align\n"); return 1; }
    cudaDeviceProp prop;
    CHECK_CUDA(cudaGetDeviceProperties(&prop, 0));
    const size_t na = (size_t)M * K, nb = (size_t)K * N, nc = (size_t)M * N, nmeta = (size_t)(M / 16) * (K / 32) * 8;
    std::vector<int8_t> A(na), comp(na / 2), B(nb);
    std::vector<uint32_t> meta(nmeta);
    std::vector<int32_t> ref_i(nc);
    std::vector<float> ref(nc), out(nc);
    const float sa = 1.0f / 127, sb = 1.0f / 127;
    gen_sparse(A.data(), M, K, 42);
    compress(A.data(), M, K, comp.data(), meta.data());
    fill_nonzero_i8(B.data(), nb, 137);
    const bool check = (double)M * N * K <= 1024.0 * 1024 * 1024;       // the CPU product of larger problems takes minutes
    if (check) {
        cpu_sparse_gemm(A.data(), B.data(), ref_i.data(), M, N, K);
        const float dq = sa * sb;
        for (size_t i = 0; i < nc; ++i) ref[i] = (float)ref_i[i] * dq;
    }
    int8_t *dComp, *dB;
    float* dC;
    uint32_t* dMeta;
    CHECK_CUDA(cudaMalloc(&dComp, na / 2)); CHECK_CUDA(cudaMalloc(&dB, nb)); CHECK_CUDA(cudaMalloc(&dC, nc * 4));
    CHECK_CUDA(cudaMalloc(&dMeta, nmeta * 4));
    CHECK_CUDA(cudaMemcpy(dComp, comp.data(), na / 2, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dB, B.data(), nb, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dMeta, meta.data(), nmeta * 4, cudaMemcpyHostToDevice));
    auto launch = [&]() { CHECK_BM(bm_igemm_sparse_f32(dComp, dB, dC, dMeta, M, N, K, sa, sb, nullptr)); };

    int errors = 0;
    for (int w = 0; w < 5; ++w) {                                        // warm-up, synchronised as in the reference
        launch();
        CHECK_CUDA(cudaDeviceSynchronize());
    }
    if (check) {
        CHECK_CUDA(cudaMemcpy(out.data(), dC, nc * 4, cudaMemcpyDeviceToHost));
        const CheckOutcome r = check_and_logic(out.data(), ref.data(), (int)nc, 0.5f, 0.1f);
        print_check("igemm_sparse_tiled_persistent", r);
        errors = r.errors;
    }
    const int NUM_ITERS = 50;
    EventTimer t;
    t.start();
    for (int i = 0; i < NUM_ITERS; ++i) launch();                        // batch of launches, one synchronisation at the end
    const float ms = t.stop_ms() / NUM_ITERS;
    const int tiles = ((M + 127) / 128) * ((N + 127) / 128);
    const int grid = tiles < prop.multiProcessorCount ? tiles : prop.multiProcessorCount;
    const double eff = 2.0 * M * N * (K / 2.0) / (ms / 1000.0) / 1e9;
    printf("  %-40s %9.3f ms  %8.0f eff GFLOPS  (grid=%dx1)\n", "igemm_sparse_tiled_persistent", ms, eff, grid);
    int code = 0;
    CHECK_BM(bm_last_device_status(&code));
    if (code != 0) { fprintf(stderr, "device status %d\n", code); return EXIT_FAILURE; }
    cudaFree(dComp); cudaFree(dB); cudaFree(dC); cudaFree(dMeta);
    bm_shutdown();
    return errors ? EXIT_FAILURE : EXIT_SUCCESS;
}
