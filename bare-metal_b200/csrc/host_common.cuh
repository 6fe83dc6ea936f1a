// host_common.cuh — host-side plumbing shared by the launchers: error capture, per-device
// state (SM count, status word, scratch), and TMA tensor-map encoding through the driver
// entry point (resolved at run time, so the library links against cudart only and still
// loads on a machine without a driver).
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <cstring>
#include <mutex>
#include <unordered_map>

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

// ---- launcher options -------------------------------------------------------------------
// Tuning and testing switches of the launchers (bm_set_option / bm_get_option).  Each starts from the
// environment variable BM_<NAME IN CAPITALS>, read ONCE when the first launcher runs, or from its
// default; no launcher reads the environment on the launch path.  -1 means "let the launcher decide".
enum : int {
    OPT_FORCE_BN = 0,        // pin the tile width (0 = choose); 240 / 224 select the sparse pair kernels
    OPT_DENSE_PAIR,          // 0 keeps dense problems on the single-CTA kernel
    OPT_SPARSE_PAIR,         // 0 keeps sparse problems on the single-CTA kernel
    OPT_ROW_BALANCED,        // decode shapes on packed weights: rows dealt out in multiples of 8 (0 = whole tiles)
    OPT_TMA_STORE,           // 0 forces the direct-store epilogue
    OPT_DENSE_GROUP_M,       // -1 automatic; G >= 0 pins the band height of the pair kernel's tile order
    OPT_SPARSE_COL_FIRST,    // -1 automatic; 0 / 1 pins the tile order of the sparse pair kernel
    OPT_TAIL_NARROW,         // 0 switches the half-height tiles of a partly filled last wave off
    OPT_PDL,                 // 0 launches without programmatic stream serialization
    OPT_GATHER_GBS,          // fused all-gather: GB/s of peer stores a GPU may send (0 = unpaced)
    OPT_DECODE_TILE_ROWS,    // row-balanced decode tiles: rows per ring stage (0 automatic; 32 / 64 / 128 pins it)
    OPT_COUNT
};
struct OptionSpec { const char* name; const char* env; int def; };
inline const OptionSpec* option_specs() {
    static const OptionSpec specs[OPT_COUNT] = {
        {"force_bn", "BM_FORCE_BN", 0},           {"dense_pair", "BM_DENSE_PAIR", 1},
        {"sparse_pair", "BM_SPARSE_PAIR", 1},     {"row_balanced", "BM_ROW_BALANCED", 1},
        {"tma_store", "BM_TMA_STORE", 1},         {"dense_group_m", "BM_DENSE_GROUP_M", -1},
        {"sparse_col_first", "BM_SPARSE_COL_FIRST", -1}, {"tail_narrow", "BM_TAIL_NARROW", 1},
        {"pdl", "BM_PDL", 1},                     {"gather_gbs", "BM_GATHER_GBS", 680},
        {"decode_tile_rows", "BM_DECODE_TILE_ROWS", 0},
    };
    return specs;
}
inline std::atomic<int>* option_values() {
    static std::atomic<int> values[OPT_COUNT];
    static std::once_flag once;
    std::call_once(once, [] {
        for (int i = 0; i < OPT_COUNT; ++i) {
            const char* e = getenv(option_specs()[i].env);
            values[i].store(e ? atoi(e) : option_specs()[i].def, std::memory_order_relaxed);
        }
    });
    return values;
}
inline int opt(int which) { return option_values()[which].load(std::memory_order_relaxed); }

// ---- per-device state -------------------------------------------------------------------
constexpr int kMaxDevices = 16;

inline std::mutex& state_mutex();

// Raises a kernel's dynamic shared-memory limit once per device.  One ConfiguredFlags object per kernel
// instantiation (a function-local static of its launcher); the flag is published with release / acquire
// so concurrent host threads either see it set or take the mutex.
struct ConfiguredFlags {
    std::atomic<bool> done[kMaxDevices];
};

struct DeviceState {
    bool ready = false;
    int sm_count = 0;
    int* status = nullptr;          // device int: first bounded-wait failure code, 0 = none
    unsigned long long* link_clock = nullptr;   // device word: virtual clock of the NVLink store pacer (same allocation)
    void* scratch = nullptr;        // library-owned staging (tiled metadata for reference-format calls)
    size_t scratch_bytes = 0;
};

inline std::mutex& state_mutex() {
    static std::mutex m;
    return m;
}
template <class Kernel>
inline int ensure_smem_limit(ConfiguredFlags& flags, Kernel kern, int bytes) {
    int dev = 0;
    BM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail_msg(BM_ERR_CUDA, "device index out of range");
    if (flags.done[dev].load(std::memory_order_acquire)) return BM_OK;
    std::lock_guard<std::mutex> lock(state_mutex());
    if (!flags.done[dev].load(std::memory_order_relaxed)) {
        BM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
        flags.done[dev].store(true, std::memory_order_release);
    }
    return BM_OK;
}
inline DeviceState* device_states() {
    static DeviceState s[kMaxDevices];
    return s;
}

// state of the CURRENT device, created on first use (allocates 16 bytes: status word + pacer clock)
inline int current_device_state(DeviceState** out) {
    int dev = 0;
    BM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail_msg(BM_ERR_CUDA, "device index out of range");
    std::lock_guard<std::mutex> lock(state_mutex());
    DeviceState& s = device_states()[dev];
    if (!s.ready) {
        BM_CUDA_TRY(cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev));
        BM_CUDA_TRY(cudaMalloc(&s.status, 16));
        BM_CUDA_TRY(cudaMemset(s.status, 0, 16));
        s.link_clock = reinterpret_cast<unsigned long long*>(s.status + 2);
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

// Tensor-map cache.  A CUtensorMap is a pure function of (base, extents, pitch, box, element type,
// swizzle), so a map encoded once is valid for every later launch with the same key — also after the
// buffer was freed and another one of the same shape landed on the same address.  Launchers look their
// maps up here (one mutex, shared by all host threads) instead of calling cuTensorMapEncodeTiled three
// to ten times per launch.  The cache is bounded: when it is full it is emptied and refilled.
struct MapKey {
    const void* base;
    uint64_t d0, d1, d2, pitch;
    uint32_t b0, b1, b2, kind;           // kind: element size | swizzle << 8 | rank << 16 | L2 promotion << 24
    bool operator==(const MapKey& o) const {
        return base == o.base && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && pitch == o.pitch && b0 == o.b0 &&
               b1 == o.b1 && b2 == o.b2 && kind == o.kind;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
        auto mix = [&h](uint64_t v) { h = (h ^ v) * 0x100000001B3ull; h ^= h >> 29; };
        mix(k.d0); mix(k.d1); mix(k.d2); mix(k.pitch);
        mix((static_cast<uint64_t>(k.b0) << 32) | k.b1);
        mix((static_cast<uint64_t>(k.b2) << 32) | k.kind);
        return static_cast<size_t>(h);
    }
};
constexpr size_t kMapCacheCapacity = 4096;
struct MapCache {
    std::mutex mutex;
    std::unordered_map<MapKey, CUtensorMap, MapKeyHash> maps;
    std::atomic<unsigned long long> hits{0}, misses{0};
};
inline MapCache& map_cache() {
    static MapCache c;
    return c;
}

// Encodes (or fetches) a tiled map of rank 2 or 3.  dims / box are innermost first; `pitch` is the byte
// stride of dimension 1 for rank 2, of dimension 2 for rank 3 (dimension 1 of a rank-3 map is 128 bytes).
inline int cached_tensor_map(CUtensorMap* map, const void* base, int rank, CUtensorMapDataType type, int elem_size,
                             const uint64_t (&dims)[3], uint64_t pitch, const uint32_t (&box)[3], bool swizzle128,
                             bool l2_promote) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail_msg(BM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    MapKey key{base, dims[0], dims[1], rank == 3 ? dims[2] : 0, pitch, box[0], box[1], rank == 3 ? box[2] : 0,
               static_cast<uint32_t>(elem_size) | (swizzle128 ? 1u << 8 : 0u) | (static_cast<uint32_t>(rank) << 16) |
                   (l2_promote ? 1u << 24 : 0u)};
    MapCache& cache = map_cache();
    {
        std::lock_guard<std::mutex> lock(cache.mutex);
        auto it = cache.maps.find(key);
        if (it != cache.maps.end()) {
            *map = it->second;
            cache.hits.fetch_add(1, std::memory_order_relaxed);
            return BM_OK;
        }
    }
    cuuint64_t gdims[3] = {dims[0], dims[1], dims[2]};
    cuuint64_t strides[2] = {pitch, 0};
    if (rank == 3) { strides[0] = 128; strides[1] = pitch; }
    cuuint32_t gbox[3] = {box[0], box[1], box[2]};
    cuuint32_t elem_strides[3] = {1, 1, 1};
    CUresult r = fn(map, type, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims, strides, gbox, elem_strides,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    l2_promote ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(error_buffer(), 256, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
        return BM_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lock(cache.mutex);
    if (cache.maps.size() >= kMapCacheCapacity) cache.maps.clear();
    cache.maps.emplace(key, *map);
    cache.misses.fetch_add(1, std::memory_order_relaxed);
    return BM_OK;
}

// 2-D byte matrix [rows x cols] with `pitch` bytes between rows, box = box_cols x box_rows,
// 128-byte swizzle (box_cols must be 128) or none.  Out-of-range parts of a box read as zero.
inline int make_tensor_map_u8(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                              uint64_t pitch, uint32_t box_cols, uint32_t box_rows, bool swizzle128) {
    const uint64_t dims[3] = {cols, rows, 1};
    const uint32_t box[3] = {box_cols, box_rows, 1};
    return cached_tensor_map(map, base, 2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, dims, pitch, box, swizzle128, true);
}

// Output matrix [rows x cols] of 2- or 4-byte elements for TMA stores: box = 128 bytes x 32 rows,
// 128-byte swizzle (matches the staging strips of the epilogue); stores are clipped to the extent.
inline int make_tensor_map_out(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                               uint64_t pitch_bytes, int elem_size) {
    const uint64_t dims[3] = {cols, rows, 1};
    const uint32_t box[3] = {static_cast<uint32_t>(128 / elem_size), 32, 1};
    return cached_tensor_map(map, base, 2, elem_size == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32,
                             elem_size, dims, pitch_bytes, box, true, false);
}

// Launch with programmatic stream serialization (and optionally a 2-CTA cluster): the kernel may be
// scheduled while the previous kernel of the stream drains; it synchronises itself with
// griddepcontrol.wait.  Option "pdl" = 0 falls back to plain stream order (testing hook).
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
    if (opt(OPT_PDL) != 0) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Status word of the no-alloc entry point (bm_noalloc.cu) on the current device: copies it to *code and
// clears it when set; *code = 0 when that entry point was never used on this device.  Allocates nothing.
// The caller has synchronised the device.
int noalloc_read_status(int* code);

}  // namespace bm
