// linkprobe.cu — what can the SMs of one B200 push into a PEER GPU's memory over NVLink, and what does that do to
// the operand loads of the same SMs?  The measurement behind the pacing of the fused all-gather (option
// "gather_gbs", StorePace in csrc/epilogue.cuh); run it on a new box to see where that box's knee is.
//
//   ./linkprobe            (needs two GPUs with peer access; with one GPU only the local rows are printed)
//
// Single process, two devices.  Part 1: 148 CTAs x 8 warps store staged 8 KiB strips (the epilogue's 32-row boxes)
// with different instructions and row lengths, to local memory, to the peer one way, and both ways at once; the
// copy engine's peer memcpy is printed beside them.  Part 2 ("MIX"): a ninth warp per CTA streams 32 KiB TMA boxes
// from an L2-resident matrix into a 4-stage ring, as a GEMM mainloop does, while the other eight store to the
// peer — unpaced, then paced by a per-warp timer to a given aggregate rate; per role the device-side duration is
// reported.  No reference counterpart (the reference is single-GPU).  Every mbarrier wait is bounded; nothing is
// multicast; the kernel only ever STORES to the peer.
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "../csrc/host_common.cuh"
#include "../csrc/sm100_ptx.cuh"
using namespace bm;

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); exit(1);} } while (0)

constexpr int ROWS = 65536, COLS = 4096;          // fp16 matrix, pitch 8192 B, 512 MiB
constexpr int PITCH = COLS * 2;

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(reinterpret_cast<uint64_t>(dst)), "r"(src), "r"(bytes) : "memory");
}

// mode 0: 2 x TMA 2-D boxes (64 cols x 32 rows, 128-byte rows)     [what the GEMM epilogue does]
// mode 1: 1 x TMA 3-D box {64, 2, 32} (256 contiguous bytes per row)
// mode 2: 32 x cp.async.bulk of 256 B (one row per lane)
// mode 3: 16 x cp.async.bulk of 512 B (box = 16 rows x 512 B)
// mode 4: st.global.v4, a warp instruction writes 512 contiguous bytes (box = 16 rows x 512 B)
// mode 5: st.global.v4, a warp instruction writes 2 rows x 256 B
// mode 6: 8 x cp.async.bulk of 1024 B
// mode 7: 2 x cp.async.bulk of 4096 B (fully contiguous, upper bound for bulk stores)
__global__ void __launch_bounds__(256, 1)
probe_kernel(const __grid_constant__ CUtensorMap map2d, const __grid_constant__ CUtensorMap map3d, uint8_t* dst, int mode,
             int iters, int depth) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t strip = smem_base + warp * 8192;
    // fill the strip once
    for (int i = lane; i < 8192 / 16; i += 32)
        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(strip + i * 16), "r"(warp * 1000 + i) : "memory");
    fence_proxy_async_smem();
    __syncwarp();
    uint4 regs = make_uint4(lane, warp, blockIdx.x, 7);
    for (int it = 0; it < iters; ++it) {
        const int t = it * gridDim.x + blockIdx.x;
        const int band = (t / 16) % (ROWS / 128), ct = t % 16;
        const int row0 = band * 128 + (warp & 3) * 32;
        const int col0 = ct * 256 + (warp >> 2) * 128;             // fp16 column
        uint8_t* base = dst + static_cast<size_t>(row0) * PITCH + col0 * 2;
        if (mode <= 3 || mode >= 6) {
            if (lane == 0 || mode == 2 || mode == 3 || mode == 6 || mode == 7) {
                if (depth <= 1) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                else asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            }
            __syncwarp();
        }
        if (mode == 0) {
            if (lane == 0) {
                tma_store_2d(&map2d, strip, col0, row0);
                tma_store_2d(&map2d, strip + 4096, col0 + 64, row0);
                bulk_commit_group();
            }
        } else if (mode == 1) {
            if (lane == 0) {
                tma_store_3d(&map3d, strip, 0, col0 / 64, row0);
                bulk_commit_group();
            }
        } else if (mode == 2) {
            bulk_store(base + static_cast<size_t>(lane) * PITCH, strip + lane * 256, 256);
            bulk_commit_group();
        } else if (mode == 3) {
            // 16 rows x 512 B: pretend the warp owns 256 columns of 16 rows
            uint8_t* b3 = dst + static_cast<size_t>(band * 128 + warp * 16) * PITCH + ct * 512;
            if (lane < 16) bulk_store(b3 + static_cast<size_t>(lane) * PITCH, strip + lane * 512, 512);
            bulk_commit_group();
        } else if (mode == 4) {
            uint8_t* b3 = dst + static_cast<size_t>(band * 128 + warp * 16) * PITCH + ct * 512;
#pragma unroll
            for (int r = 0; r < 16; ++r) *reinterpret_cast<uint4*>(b3 + static_cast<size_t>(r) * PITCH + lane * 16) = regs;
        } else if (mode == 5) {
#pragma unroll
            for (int r = 0; r < 32; r += 2)
                *reinterpret_cast<uint4*>(base + static_cast<size_t>(r + (lane >> 4)) * PITCH + (lane & 15) * 16) = regs;
        } else if (mode == 6) {
            uint8_t* b3 = dst + static_cast<size_t>(band * 128 + warp * 8) * PITCH + ct * 1024;   // 8 rows x 1024 B (cols 0..8191 B)
            if (lane < 8 && ct < 8) bulk_store(b3 + static_cast<size_t>(lane) * PITCH, strip + lane * 1024, 1024);
            else if (lane < 8) bulk_store(dst + static_cast<size_t>(band * 128 + 64 + warp * 8 + lane) * PITCH + (ct - 8) * 1024, strip + lane * 1024, 1024);
            bulk_commit_group();
        } else if (mode == 7) {
            // contiguous 8 KiB per warp: row (t*8+warp) of the matrix viewed as 8 KiB rows
            uint8_t* b3 = dst + (static_cast<size_t>(t) * 8 + warp) % ROWS * PITCH;
            if (lane < 2) bulk_store(b3 + lane * 4096, strip + lane * 4096, 4096);
            bulk_commit_group();
        }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}


// ---- interference probe: a TMA LOAD stream (L2-resident operand tiles into a ring, as a GEMM mainloop
// does) next to remote stores of the flavours above.  store_mode -1 = no stores; load_iters 0 = no loads.
constexpr int LD_STAGES = 4, LD_BOX = 32768;
__global__ void __launch_bounds__(320, 1)
mix_kernel(const __grid_constant__ CUtensorMap map2d, const __grid_constant__ CUtensorMap map_ld, uint8_t* dst,
           int store_mode, int iters, int load_iters, int* status, unsigned long long* stamps, unsigned pace_ns,
           int done_wait) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ring = smem_base + 65536;
    const uint32_t bar0 = ring + LD_STAGES * LD_BOX;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + 65536 + LD_STAGES * LD_BOX + 128);
    if (threadIdx.x == 0) {
        for (int s = 0; s < 2 * LD_STAGES; ++s) mbar_init(bar0 + 8 * s, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    const unsigned long long t0 = global_timer_ns();
    if (warp < 8) {
        if (store_mode < 0) return;
        const uint32_t strip = smem_base + warp * 8192;
        for (int i = lane; i < 8192 / 16; i += 32)
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(strip + i * 16), "r"(warp * 1000 + i) : "memory");
        fence_proxy_async_smem();
        __syncwarp();
        unsigned long long next_t = t0 + (pace_ns / 8) * warp;        // warps of a CTA take turns
        for (int it = 0; it < iters; ++it) {
            const int t = it * gridDim.x + blockIdx.x;
            const int band = (t / 16) % (ROWS / 128), ct = t % 16;
            const int row0 = band * 128 + (warp & 3) * 32;
            const int col0 = ct * 256 + (warp >> 2) * 128;
            uint8_t* base = dst + static_cast<size_t>(row0) * PITCH + col0 * 2;
            if (pace_ns) {
                while (global_timer_ns() < next_t) {}
                next_t += pace_ns;
            }
            if (store_mode == 0) {
                if (lane == 0) {
                    if (done_wait) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    tma_store_2d(&map2d, strip, col0, row0);
                    tma_store_2d(&map2d, strip + 4096, col0 + 64, row0);
                    bulk_commit_group();
                }
                __syncwarp();
            } else {
                // staged strip -> registers -> remote: a warp instruction writes 2 rows x 256 B
#pragma unroll 4
                for (int r = 0; r < 32; r += 2) {
                    uint4 v;
                    const uint32_t src = strip + (r + (lane >> 4)) * 256 + (lane & 15) * 16;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(src));
                    *reinterpret_cast<uint4*>(base + static_cast<size_t>(r + (lane >> 4)) * PITCH + (lane & 15) * 16) = v;
                }
            }
        }
        if (store_mode == 0 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        if (warp == 0 && lane == 0) stamps[blockIdx.x * 2] = global_timer_ns() - t0;
    } else if (warp == 8) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            for (int i = 0; i < load_iters; ++i) {
                if (!bounded_wait(bar0 + 8 * (LD_STAGES + stage), phase ^ 1u, abort_flag, status, 1)) break;
                mbar_expect_tx(bar0 + 8 * stage, LD_BOX);
                const int box = (i * gridDim.x + blockIdx.x) % 1024;          // 1024 boxes of 32 KiB = 32 MiB, L2-resident
                tma_load_2d(ring + stage * LD_BOX, &map_ld, bar0 + 8 * stage, 0, box * 256);
                if (++stage == LD_STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            for (int i = 0; i < load_iters; ++i) {
                if (!bounded_wait(bar0 + 8 * stage, phase, abort_flag, status, 2)) break;
                mbar_arrive(bar0 + 8 * (LD_STAGES + stage));
                if (++stage == LD_STAGES) { stage = 0; phase ^= 1u; }
            }
            stamps[blockIdx.x * 2 + 1] = global_timer_ns() - t0;
        }
    }
}

static int make3d(CUtensorMap* map, void* base) {
    EncodeTiledFn fn = encode_tiled_fn();
    cuuint64_t dims[3] = {64, COLS / 64, ROWS};
    cuuint64_t strides[2] = {128, PITCH};
    cuuint32_t box[3] = {64, 2, 32};
    cuuint32_t es[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { printf("encode 3d failed %d\n", (int)r); return 1; }
    return 0;
}

struct Side { int dev; uint8_t* local; uint8_t* remote; CUtensorMap m2l, m3l, m2r, m3r; cudaStream_t st; cudaEvent_t e0, e1; };

int main(int argc, char** argv) {
    int ndev = 0;
    CK(cudaGetDeviceCount(&ndev));
    printf("devices: %d\n", ndev);
    const size_t bytes = static_cast<size_t>(ROWS) * PITCH;
    Side s[2];
    for (int d = 0; d < 2 && d < ndev; ++d) {
        CK(cudaSetDevice(d));
        CK(cudaMalloc(&s[d].local, bytes));
        CK(cudaMemset(s[d].local, 0, bytes));
        CK(cudaStreamCreate(&s[d].st));
        CK(cudaEventCreate(&s[d].e0));
        CK(cudaEventCreate(&s[d].e1));
        s[d].dev = d;
        CK(cudaFuncSetAttribute(probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 66 * 1024));
    }
    const bool two = ndev >= 2;
    if (two) {
        int can = 0;
        CK(cudaDeviceCanAccessPeer(&can, 0, 1));
        printf("peer access 0->1: %d\n", can);
        if (!can) return 0;
        CK(cudaSetDevice(0)); CK(cudaDeviceEnablePeerAccess(1, 0));
        CK(cudaSetDevice(1)); CK(cudaDeviceEnablePeerAccess(0, 0));
        s[0].remote = s[1].local;
        s[1].remote = s[0].local;
    }
    for (int d = 0; d < (two ? 2 : 1); ++d) {
        CK(cudaSetDevice(d));
        if (make_tensor_map_out(&s[d].m2l, s[d].local, COLS, ROWS, PITCH, 2)) return 1;
        if (make3d(&s[d].m3l, s[d].local)) return 1;
        if (two) {
            if (make_tensor_map_out(&s[d].m2r, s[d].remote, COLS, ROWS, PITCH, 2)) return 1;
            if (make3d(&s[d].m3r, s[d].remote)) return 1;
        }
    }
    const int grid = 148, iters = 96;
    const double total = static_cast<double>(grid) * iters * 65536.0;
    auto run = [&](int d, bool remote, int mode, int depth) {
        CK(cudaSetDevice(d));
        probe_kernel<<<grid, 256, 66 * 1024, s[d].st>>>(remote ? s[d].m2r : s[d].m2l, remote ? s[d].m3r : s[d].m3l,
                                                       remote ? s[d].remote : s[d].local, mode, iters, depth);
    };
    const char* names[8] = {"tma2d 128B rows", "tma3d 256B rows", "bulk 256B rows", "bulk 512B rows", "st.v4 512B rows",
                            "st.v4 256B rows", "bulk 1024B rows", "bulk 4096B contiguous"};
    for (int remote = 0; remote <= (two ? 1 : 0); ++remote)
        for (int bidir = 0; bidir <= remote; ++bidir)
            for (int mode = 0; mode < 8; ++mode) {
                float best = 1e30f;
                for (int rep = 0; rep < 4; ++rep) {
                    for (int d = 0; d <= bidir; ++d) { CK(cudaSetDevice(d)); CK(cudaEventRecord(s[d].e0, s[d].st)); }
                    for (int d = 0; d <= bidir; ++d) run(d, remote, mode, 1);
                    for (int d = 0; d <= bidir; ++d) { CK(cudaSetDevice(d)); CK(cudaEventRecord(s[d].e1, s[d].st)); }
                    float worst = 0;
                    for (int d = 0; d <= bidir; ++d) {
                        CK(cudaSetDevice(d)); CK(cudaStreamSynchronize(s[d].st));
                        float ms; CK(cudaEventElapsedTime(&ms, s[d].e0, s[d].e1));
                        worst = ms > worst ? ms : worst;
                    }
                    if (rep > 0 && worst < best) best = worst;
                }
                printf("%s %s mode %d (%s): %.3f ms  %.1f GB/s per direction\n", remote ? "REMOTE" : "local ",
                       bidir ? "bidir" : "unidir", mode, names[mode], best, total / best / 1e6);
            }
    if (two) {
        // copy-engine reference: peer memcpy of the same bytes, one direction and both
        for (int bidir = 0; bidir <= 1; ++bidir) {
            float best = 1e30f;
            for (int rep = 0; rep < 4; ++rep) {
                for (int d = 0; d <= bidir; ++d) { CK(cudaSetDevice(d)); CK(cudaEventRecord(s[d].e0, s[d].st)); }
                for (int d = 0; d <= bidir; ++d) { CK(cudaSetDevice(d)); CK(cudaMemcpyPeerAsync(s[d].remote, 1 - d, s[d].local, d, bytes, s[d].st)); }
                for (int d = 0; d <= bidir; ++d) { CK(cudaSetDevice(d)); CK(cudaEventRecord(s[d].e1, s[d].st)); }
                float worst = 0;
                for (int d = 0; d <= bidir; ++d) {
                    CK(cudaSetDevice(d)); CK(cudaStreamSynchronize(s[d].st));
                    float ms; CK(cudaEventElapsedTime(&ms, s[d].e0, s[d].e1));
                    worst = ms > worst ? ms : worst;
                }
                if (rep > 0 && worst < best) best = worst;
            }
            printf("copy engine peer memcpy %s: %.3f ms  %.1f GB/s per direction\n", bidir ? "bidir" : "unidir", best, bytes / best / 1e6);
        }
    }

    if (two) {
        CK(cudaSetDevice(0));
        CK(cudaFuncSetAttribute(mix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        uint8_t* ldsrc; int* status; unsigned long long* stamps;
        CK(cudaMalloc(&ldsrc, 32u << 20)); CK(cudaMemset(ldsrc, 1, 32u << 20));
        CK(cudaMalloc(&status, 4)); CK(cudaMemset(status, 0, 4));
        CK(cudaMalloc(&stamps, 148 * 16)); 
        CUtensorMap map_ld;
        if (make_tensor_map_u8(&map_ld, ldsrc, 128, 262144, 128, 128, 256, true)) return 1;
        std::vector<unsigned long long> h(296);
        auto mix = [&](const char* what, bool remote, int store_mode, int it, int lit, unsigned pace_ns = 0, int done_wait = 0) {
            float best = 1e30f; double st_us = 0, ld_us = 0;
            for (int rep = 0; rep < 3; ++rep) {
                CK(cudaMemset(stamps, 0, 148 * 16));
                CK(cudaEventRecord(s[0].e0, s[0].st));
                mix_kernel<<<148, 320, 200 * 1024, s[0].st>>>(remote ? s[0].m2r : s[0].m2l, map_ld, remote ? s[0].remote : s[0].local,
                                                             store_mode, it, lit, status, stamps, pace_ns, done_wait);
                CK(cudaEventRecord(s[0].e1, s[0].st));
                CK(cudaStreamSynchronize(s[0].st));
                float ms; CK(cudaEventElapsedTime(&ms, s[0].e0, s[0].e1));
                if (rep > 0 && ms < best) {
                    best = ms;
                    CK(cudaMemcpy(h.data(), stamps, 148 * 16, cudaMemcpyDeviceToHost));
                    st_us = ld_us = 0;
                    for (int c = 0; c < 148; ++c) { st_us += h[2 * c] / 1e3 / 148; ld_us += h[2 * c + 1] / 1e3 / 148; }
                }
            }
            const double sb = store_mode >= 0 ? 148.0 * it * 65536 : 0, lb = 148.0 * lit * LD_BOX;
            printf("MIX %-44s kernel %.3f ms | stores: avg %.0f us -> %.0f GB/s | loads: avg %.0f us -> %.0f GB/s (%.1f B/clk/SM at 1.9 GHz)\n",
                   what, best, st_us, st_us > 0 ? sb / st_us / 1e3 : 0.0, ld_us, ld_us > 0 ? lb / ld_us / 1e3 : 0.0,
                   ld_us > 0 ? lb / 148 / (ld_us * 1e-6) / 1.9e9 : 0.0);
        };
        const int IT = 96, LIT = 5000;
        mix("loads only", true, -1, 0, LIT);
        mix("remote TMA stores only", true, 0, IT, 0);
        mix("remote st.global stores only", true, 1, IT, 0);
        mix("loads + remote TMA stores", true, 0, IT, LIT);
        mix("loads + remote st.global stores", true, 1, IT, LIT);
        mix("loads + remote TMA stores, wait for completion", true, 0, IT, LIT, 0, 1);
        for (int gbs : {300, 450, 550, 620, 680, 720}) {
            // every warp-iteration sends 8 KiB; 148 x 8 warps share the link
            const unsigned pace = static_cast<unsigned>(8192.0 * 148 * 8 / (gbs * 1e9) * 1e9);
            char name[96];
            snprintf(name, sizeof name, "loads + remote TMA stores paced to %d GB/s", gbs);
            mix(name, true, 0, IT, LIT, pace);
            snprintf(name, sizeof name, "loads + remote st.global paced to %d GB/s", gbs);
            mix(name, true, 1, IT, LIT, pace);
        }
        int hs = 0; CK(cudaMemcpy(&hs, status, 4, cudaMemcpyDeviceToHost));
        printf("mix status word: %d\n", hs);
    }
    // verify something landed (mode 1 pattern differs from mode 0 only in layout; just check non-zero)
    CK(cudaSetDevice(0));
    std::vector<uint32_t> h(16);
    CK(cudaMemcpy(h.data(), two ? s[1].local : s[0].local, 64, cudaMemcpyDeviceToHost));
    printf("first words at destination: %u %u %u %u\n", h[0], h[1], h[2], h[3]);
    printf("done\n");
    return 0;
}
