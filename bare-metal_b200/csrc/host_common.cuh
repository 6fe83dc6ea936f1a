// host_common.cuh — host-side plumbing shared by the launchers: error capture, per-device
// state (SM count, status word, scratch), and TMA tensor-map encoding through the driver
// entry point (resolved at run time, so the library links against cudart only and still
// loads on a machine without a driver).
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/bm_igemm.h"

namespace bm {

// ---- last host-side error text (per thread) ---------------------------------------------
inline char* error_buffer() {
    static thread_local char buf[256] = "";
    return buf;
}
inline int fail_cuda(cudaError_t e, const char* what) {
    snprintf(error_buffer(), 256, "%s: %s", what, cudaGetErrorString(e));
    return BM_ERR_CUDA;
}
inline int fail_msg(int code, const char* what) {
    snprintf(error_buffer(), 256, "%s", what);
    return code;
}
#define BM_CUDA_TRY(expr)                                              \
    do {                                                               \
        cudaError_t _e = (expr);                                       \
        if (_e != cudaSuccess) return ::bm::fail_cuda(_e, #expr);      \
    } while (0)

// ---- per-device state -------------------------------------------------------------------
constexpr int kMaxDevices = 16;

struct DeviceState {
    bool ready = false;
    int sm_count = 0;
    int* status = nullptr;          // device int: first bounded-wait failure code, 0 = none
    void* scratch = nullptr;        // library-owned staging (tiled metadata for reference-format calls)
    size_t scratch_bytes = 0;
    void* sk_workspace = nullptr;   // split-K partial sums (stream-K launches)
    size_t sk_workspace_bytes = 0;
    int* sk_counters = nullptr;     // split-K arrival counters, kept at zero between launches
    size_t sk_counter_ints = 0;
};

inline std::mutex& state_mutex() {
    static std::mutex m;
    return m;
}
inline DeviceState* device_states() {
    static DeviceState s[kMaxDevices];
    return s;
}

// state of the CURRENT device, created on first use (allocates the 4-byte status word)
inline int current_device_state(DeviceState** out) {
    int dev = 0;
    BM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail_msg(BM_ERR_CUDA, "device index out of range");
    std::lock_guard<std::mutex> lock(state_mutex());
    DeviceState& s = device_states()[dev];
    if (!s.ready) {
        BM_CUDA_TRY(cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev));
        BM_CUDA_TRY(cudaMalloc(&s.status, sizeof(int)));
        BM_CUDA_TRY(cudaMemset(s.status, 0, sizeof(int)));
        s.ready = true;
    }
    *out = &s;
    return BM_OK;
}

// grow-only scratch of the current device
inline int ensure_scratch(DeviceState* s, size_t bytes) {
    std::lock_guard<std::mutex> lock(state_mutex());
    if (s->scratch_bytes >= bytes) return BM_OK;
    if (s->scratch) {
        BM_CUDA_TRY(cudaDeviceSynchronize());
        BM_CUDA_TRY(cudaFree(s->scratch));
        s->scratch = nullptr;
        s->scratch_bytes = 0;
    }
    BM_CUDA_TRY(cudaMalloc(&s->scratch, bytes));
    s->scratch_bytes = bytes;
    return BM_OK;
}

// grow-only split-K buffers of the current device (counters are zero-filled when (re)allocated)
inline int ensure_split_k(DeviceState* s, size_t workspace_bytes, size_t counter_ints) {
    std::lock_guard<std::mutex> lock(state_mutex());
    if (s->sk_workspace_bytes < workspace_bytes) {
        if (s->sk_workspace) {
            BM_CUDA_TRY(cudaDeviceSynchronize());
            BM_CUDA_TRY(cudaFree(s->sk_workspace));
            s->sk_workspace = nullptr;
            s->sk_workspace_bytes = 0;
        }
        BM_CUDA_TRY(cudaMalloc(&s->sk_workspace, workspace_bytes));
        s->sk_workspace_bytes = workspace_bytes;
    }
    if (s->sk_counter_ints < counter_ints) {
        if (s->sk_counters) {
            BM_CUDA_TRY(cudaDeviceSynchronize());
            BM_CUDA_TRY(cudaFree(s->sk_counters));
            s->sk_counters = nullptr;
            s->sk_counter_ints = 0;
        }
        BM_CUDA_TRY(cudaMalloc(&s->sk_counters, counter_ints * sizeof(int)));
        BM_CUDA_TRY(cudaMemset(s->sk_counters, 0, counter_ints * sizeof(int)));
        s->sk_counter_ints = counter_ints;
    }
    return BM_OK;
}

// ---- TMA tensor maps --------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// 2-D byte matrix [rows x cols] with `pitch` bytes between rows, box = box_cols x box_rows,
// 128-byte swizzle (box_cols must be 128) or none.  Out-of-range parts of a box read as zero.
inline int make_tensor_map_u8(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                              uint64_t pitch, uint32_t box_cols, uint32_t box_rows, bool swizzle128) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail_msg(BM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t elem_strides[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                    elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(error_buffer(), 256, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
        return BM_ERR_CUDA;
    }
    return BM_OK;
}

// Output matrix [rows x cols] of 2- or 4-byte elements for TMA stores: box = 128 bytes x 32 rows,
// 128-byte swizzle (matches the staging strips of the epilogue); stores are clipped to the extent.
inline int make_tensor_map_out(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                               uint64_t pitch_bytes, int elem_size) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail_msg(BM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elem_size), 32};
    cuuint32_t elem_strides[2] = {1, 1};
    CUresult r = fn(map, elem_size == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2,
                    const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(error_buffer(), 256, "cuTensorMapEncodeTiled (output) failed with CUresult %d", static_cast<int>(r));
        return BM_ERR_CUDA;
    }
    return BM_OK;
}

// Launch with programmatic stream serialization (and optionally a 2-CTA cluster): the kernel may be
// scheduled while the previous kernel of the stream drains; it synchronises itself with
// griddepcontrol.wait.  BM_NO_PDL=1 falls back to plain stream order (testing hook).
template <class Kernel, class... Args>
inline cudaError_t launch_pdl(Kernel kern, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_x,
                              Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    static const bool no_pdl = getenv("BM_NO_PDL") != nullptr;
    if (!no_pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace bm
