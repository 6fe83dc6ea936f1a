// bm_noalloc.cu — bm_igemm_sparse_f32_noalloc: the reference-format 2:4 sparse GEMM for callers
// that are not allowed to allocate device memory.
//
// Who needs this: code that runs where cudaMalloc / cudaFree are forbidden or would stall —
// inside a latency-critical serving loop that has promised its allocator a fixed footprint,
// under a memory pool that owns every byte of the device, or in a host process whose policy is
// "no driver allocations after start-up".  The regular entry point bm_igemm_sparse_f32 re-tiles
// the reference's metadata words into scratch that the library obtains with cudaMalloc on
// first use (and grows on demand); this variant keeps that scratch in a fixed array that is
// part of the library image instead, so nothing is ever allocated or freed on its behalf.
//
// The price is a capacity limit and shared state:
//   * the re-tiled metadata must fit BM_NOALLOC_META_BYTES (2 MiB): ceil(M/128) * ceil(K/256)
//     * 4096 bytes, i.e. up to M = K = 4096 (or any M*K of that area in whole tiles).  Larger
//     problems are rejected with BM_ERR_TOO_LARGE before anything is launched;
//   * the 2 MiB array (plus two status words) is part of the library's device image: a GPU holds it
//     from the moment the CUDA runtime loads that image on it until the process exits.  With the
//     runtime's default lazy loading that moment is this entry point's FIRST CALL on the device
//     (with CUDA_MODULE_LOADING=EAGER it is context creation).  A process whose pool is about to
//     claim the whole device must therefore make one call — any small problem — BEFORE the pool
//     takes the memory, or run with eager loading; afterwards no call reserves anything;
//   * all calls on a device share the one array.  It still holds the previous call's metadata
//     when the next call starts; that is harmless because the packing kernel rewrites every
//     byte the GEMM will read before the GEMM starts (same stream, so ordered), so nothing has
//     to be cleared.  Two calls that overlap on the GPU (different streams, no dependency)
//     race on the array and produce garbage: serialise them.
//
// Set-up: the array's name is only a host-side handle.  The first call on each device, made
// with that device current, asks the runtime for the array's device address
// (cudaGetSymbolAddress) and raises the kernel's shared-memory limit; later calls reuse the
// cached address.  Make that first call outside any stream capture.
//
// Errors inside a launch: the GEMM's bounded waits record a give-up in g_noalloc_status, a word
// of this file (not the cudaMalloc'ed word of the other entry points).  Read and clear it with
// bm_noalloc_last_device_status, which allocates nothing either; bm_last_device_status reports
// it too, but creates the library's regular per-device state on first use (a 4-byte cudaMalloc).
#include <cstdlib>

#include "host_common.cuh"
#include "igemm_sparse.cuh"

#define BM_NOALLOC_META_BYTES (2u * 1024u * 1024u)

namespace bm {

// Fixed scratch for the tiled metadata and the timeout status of this entry point's launches.
static __device__ __align__(256) unsigned char g_noalloc_meta[BM_NOALLOC_META_BYTES];
static __device__ int g_noalloc_status;
static __device__ int g_noalloc_selftest;      // outcome word of bm_noalloc_selftest_bounded_wait

// Reference uint32 metadata words -> tiled order, written straight into the fixed array
// (device code may name the array directly).  Same mapping as bm_sp_pack_meta with BM_META_REF:
// unit = 16 bytes = 4 K-steps of 32 for one row; rows / K beyond the operand get the valid
// pattern 0x44 (their values are zero-filled by the TMA loads).
static __global__ void noalloc_pack_meta_ref_kernel(const uint32_t* __restrict__ meta_ref, int R, int K, int k_blocks,
                                                    size_t units) {
    const size_t unit = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (unit >= units) return;
    const int r = static_cast<int>(unit & 127);
    const size_t chunk = unit >> 7;
    const int j = static_cast<int>(chunk & 1);
    const size_t blk = chunk >> 1;
    const int kb = static_cast<int>(blk % k_blocks);
    const int rb = static_cast<int>(blk / k_blocks);
    const int row = rb * 128 + r;
    const int s0 = (kb * 2 + j) * 4;
    const int k_steps = K / 32;
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int s = s0 + q;
        w[q] = (row < R && s < k_steps) ? meta_ref[(static_cast<size_t>(row / 16) * k_steps + s) * 8 + (row % 16) % 8]
                                        : 0x44444444u;
    }
    *reinterpret_cast<uint4*>(g_noalloc_meta + unit * 16) = make_uint4(w[0], w[1], w[2], w[3]);
}

struct NoAllocDevice {
    bool ready = false;
    unsigned char* meta = nullptr;     // device address of g_noalloc_meta on this device
    int* status = nullptr;             // device address of g_noalloc_status on this device
    int* selftest = nullptr;           // device address of g_noalloc_selftest on this device
    int sm_count = 0;
};

static NoAllocDevice* noalloc_devices() {
    static NoAllocDevice devices[kMaxDevices];
    return devices;
}

static std::mutex& noalloc_mutex() {
    static std::mutex m;
    return m;
}

// Once per device, with that device current: resolve the device addresses of the fixed arrays.
static int noalloc_device(NoAllocDevice** out) {
    int dev = 0;
    BM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail_msg(BM_ERR_CUDA, "device index out of range");
    std::lock_guard<std::mutex> lock(noalloc_mutex());
    NoAllocDevice& d = noalloc_devices()[dev];
    if (!d.ready) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_meta);
        if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(g_noalloc_meta)");
        d.meta = static_cast<unsigned char*>(p);
        e = cudaGetSymbolAddress(&p, g_noalloc_status);
        if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(g_noalloc_status)");
        d.status = static_cast<int*>(p);
        e = cudaGetSymbolAddress(&p, g_noalloc_selftest);
        if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(g_noalloc_selftest)");
        d.selftest = static_cast<int*>(p);
        BM_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        BM_CUDA_TRY(cudaFuncSetAttribute(igemm_sparse_kernel<128, true, false, EPI_F32_TENSOR>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SparseCfg<128>::SMEM_BYTES));
        d.ready = true;
    }
    *out = &d;
    return BM_OK;
}

// Declared in host_common.cuh.  The caller has synchronised the device.  Nothing is allocated:
// cudaMemcpy / cudaMemset on an existing address, and only when this file's set-up has run here.
int noalloc_read_status(int* code) {
    *code = 0;
    int dev = 0;
    BM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail_msg(BM_ERR_CUDA, "device index out of range");
    std::lock_guard<std::mutex> lock(noalloc_mutex());
    const NoAllocDevice& d = noalloc_devices()[dev];
    if (!d.ready) return BM_OK;
    BM_CUDA_TRY(cudaMemcpy(code, d.status, sizeof(int), cudaMemcpyDeviceToHost));
    if (*code != 0) BM_CUDA_TRY(cudaMemset(d.status, 0, sizeof(int)));
    return BM_OK;
}

// A wait that nothing satisfies, with a short limit, recording into the status word it is given:
// the give-up path of the pipeline waits, exercised without hanging or faulting anything.
static __global__ void noalloc_selftest_kernel(int* status, unsigned long long limit_ns, int* returned) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool ok = bounded_wait(smem_u32(&bar), 0, &abort_flag, status, DEV_TIMEOUT_DRAIN, limit_ns);
        *returned = ok ? 1 : 2;                     // 2 = gave up cleanly
    }
}

}  // namespace bm

using namespace bm;

extern "C" int bm_noalloc_last_device_status(int* code) {
    if (!code) return fail_msg(BM_ERR_NULL, "code pointer is NULL");
    BM_CUDA_TRY(cudaDeviceSynchronize());
    return noalloc_read_status(code);
}

extern "C" int bm_noalloc_selftest_bounded_wait(unsigned limit_us, int* outcome) {
    if (!outcome) return fail_msg(BM_ERR_NULL, "outcome pointer is NULL");
    if (limit_us == 0 || limit_us > 2000000u) return fail_msg(BM_ERR_SHAPE, "limit must be 1 us .. 2 s");
    NoAllocDevice* dev = nullptr;
    if (int rc = noalloc_device(&dev)) return rc;
    BM_CUDA_TRY(cudaMemset(dev->selftest, 0, sizeof(int)));
    noalloc_selftest_kernel<<<1, 32>>>(dev->status, static_cast<unsigned long long>(limit_us) * 1000ull, dev->selftest);
    BM_CUDA_TRY(cudaGetLastError());
    BM_CUDA_TRY(cudaDeviceSynchronize());
    BM_CUDA_TRY(cudaMemcpy(outcome, dev->selftest, sizeof(int), cudaMemcpyDeviceToHost));
    return BM_OK;
}

extern "C" int bm_igemm_sparse_f32_noalloc(const int8_t* A_comp, const int8_t* B, float* C, const uint32_t* meta, int M,
                                           int N, int K, float scale_a, float scale_b, void* stream_v) {
    if (!A_comp || !B || !C || !meta) return fail_msg(BM_ERR_NULL, "operand pointer is NULL");
    if (M <= 0 || N <= 0 || K <= 0) return fail_msg(BM_ERR_SHAPE, "M, N, K must be positive");
    if (M % 16 != 0) return fail_msg(BM_ERR_SHAPE, "M must be a multiple of 16 (reference metadata format)");
    if (K % 32 != 0) return fail_msg(BM_ERR_SHAPE, "K must be a multiple of 32 for the 2:4 format");
    if (N % 16 != 0) return fail_msg(BM_ERR_SHAPE, "N must be a multiple of 16 for B[K x N]");
    if (!aligned16(A_comp) || !aligned16(B) || (reinterpret_cast<uintptr_t>(meta) & 3u))
        return fail_msg(BM_ERR_ALIGN, "operands must be 16-byte aligned (metadata 4-byte)");
    const int tiles_r = (M + 127) / 128, k_blocks = (K + kSpKLogical - 1) / kSpKLogical;
    const size_t need = static_cast<size_t>(tiles_r) * k_blocks * kSpMetaBytes;
    if (need > BM_NOALLOC_META_BYTES) {
        snprintf(error_buffer(), 256,
                 "tiled metadata needs %zu bytes but the fixed scratch of the no-alloc entry point holds %u "
                 "(ceil(M/128)*ceil(K/256)*4096 must not exceed 2 MiB, e.g. M = K = 4096)",
                 need, BM_NOALLOC_META_BYTES);
        return BM_ERR_TOO_LARGE;
    }
    NoAllocDevice* dev = nullptr;
    if (int rc = noalloc_device(&dev)) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    // 1. re-tile the metadata into the fixed array (every byte the GEMM reads is rewritten)
    const size_t units = need / 16;
    noalloc_pack_meta_ref_kernel<<<static_cast<unsigned>((units + 255) / 256), 256, 0, stream>>>(meta, M, K, k_blocks,
                                                                                                units);
    BM_CUDA_TRY(cudaGetLastError());

    // 2. the sparse GEMM itself: same kernel as bm_igemm_sparse_f32, 128 x 128 tiles
    constexpr int BN = 128;
    CUtensorMap map_s, map_d;
    if (int rc = make_tensor_map_u8(&map_s, A_comp, K / 2, M, K / 2, 128, kBM, true)) return rc;
    if (int rc = make_tensor_map_u8(&map_d, B, N, K, N, 128, kSpKLogical, true)) return rc;
    SparseParams p{};
    p.epi.out = C;
    p.epi.ld = N;
    p.epi.rows = M;
    p.epi.cols = N;
    volatile float dequant = scale_a * scale_b;                 // igemm_sparse_tiled.cu:365
    p.epi.tensor_scale = dequant;
    p.epi.vec_ok = aligned16(C) && (static_cast<size_t>(N) * 4) % 16 == 0;
    p.meta_tiled = dev->meta;
    p.tiles_r = tiles_r;
    p.tiles_c = (N + BN - 1) / BN;
    p.k_blocks = k_blocks;
    p.status = dev->status;
    const int num_tiles = p.tiles_r * p.tiles_c;
    const int grid = num_tiles < dev->sm_count ? num_tiles : dev->sm_count;
    igemm_sparse_kernel<BN, true, false, EPI_F32_TENSOR>
        <<<grid, SparseCfg<BN>::THREADS, SparseCfg<BN>::SMEM_BYTES, stream>>>(map_s, map_d, p);
    BM_CUDA_TRY(cudaGetLastError());
    return BM_OK;
}
