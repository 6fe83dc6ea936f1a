// bm_api.cu — the extern "C" launchers declared in include/bm_igemm.h.
// Argument validation, tensor-map encoding, tile-shape choice and the kernel launch; no
// arithmetic happens on the host.
#include <cstdlib>

#include "host_common.cuh"
#include "igemm_dense.cuh"
#include "igemm_dense_pair.cuh"
#include "igemm_sparse.cuh"
#include "igemm_sparse_pair.cuh"
#include "pack_kernels.cuh"
#include "online_quant_kernels.cuh"
#include "quantize_kernels.cuh"
#include "gather_kernels.cuh"

namespace bm {

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Testing hook: option "force_bn" pins the tile width so every instantiation can be exercised
// on small problems.  0 (the default) lets the launcher choose.
static int forced_bn() { return opt(OPT_FORCE_BN); }

static int validate_epilogue(int epi, const void* out, long long ld, int cols, const float* row_scale,
                             const float* col_scale, const int* col_zero) {
    if (!out) return fail_msg(BM_ERR_NULL, "output pointer is NULL");
    if (ld < cols) return fail_msg(BM_ERR_SHAPE, "output pitch is smaller than the row length");
    if (epi == EPI_F32_CHANNEL && (!col_scale || !col_zero)) return fail_msg(BM_ERR_NULL, "scale / zero_point is NULL");
    if (epi_rowcol(epi) && (!row_scale || !col_scale)) return fail_msg(BM_ERR_NULL, "row / column scale is NULL");
    return BM_OK;
}

static size_t out_elem_size(int epi) { return epi == EPI_F16_ROWCOL ? 2 : 4; }

// =========================================================================================
// dense
// =========================================================================================
template <int BN, bool B_MN, int EPI>
static int launch_dense_inst(const CUtensorMap& ma, const CUtensorMap& mb, const OutMaps& mo,
                             const DenseParams& p, int grid, cudaStream_t stream) {
    using Cfg = DenseCfg<BN>;
    auto kern = igemm_dense_kernel<BN, B_MN, EPI>;
    static ConfiguredFlags flags;
    if (int rc = ensure_smem_limit(flags, kern, Cfg::SMEM_BYTES)) return rc;
    BM_CUDA_TRY(launch_pdl(kern, dim3(grid), dim3(kDenseThreads), Cfg::SMEM_BYTES, stream, 1, ma, mb, mo, p));
    return BM_OK;
}

// CTA-pair kernel: 2-CTA clusters, one pair per two SMs, 256 x 256 tiles
template <bool B_MN, int EPI>
static int launch_dense_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mbn, const OutMaps& mo,
                             const DenseParams& p, int pairs, cudaStream_t stream) {
    auto kern = igemm_dense_pair_kernel<B_MN, EPI>;
    static ConfiguredFlags flags;
    if (int rc = ensure_smem_limit(flags, kern, kPairSmemBytes)) return rc;
    BM_CUDA_TRY(launch_pdl(kern, dim3(2 * pairs), dim3(kDenseThreads), kPairSmemBytes, stream, 2, ma, mb, mbn, mo, p));
    return BM_OK;
}

// option "dense_pair" = 0 keeps large problems on the single-CTA kernel (testing hook; default on)
static bool pair_enabled() { return opt(OPT_DENSE_PAIR) != 0; }

template <bool B_MN, int EPI>
static int launch_dense_bn(int bn, const CUtensorMap& ma, const CUtensorMap& mb, const OutMaps& mo,
                           const DenseParams& p, int grid, cudaStream_t stream) {
    switch (bn) {
        case 256: return launch_dense_inst<256, B_MN, EPI>(ma, mb, mo, p, grid, stream);
        case 128: return launch_dense_inst<128, B_MN, EPI>(ma, mb, mo, p, grid, stream);
        case 64:
            if constexpr (!B_MN) return launch_dense_inst<64, B_MN, EPI>(ma, mb, mo, p, grid, stream);
        default: return fail_msg(BM_ERR_SHAPE, "unsupported tile width");
    }
}

static int dense_gemm(int epi, const int8_t* A, const int8_t* B, void* C, int M, int N, int K, long long ldc,
                      int b_layout, float tensor_scale, const float* row_scale, const float* col_scale,
                      const int* col_zero, void* stream_v, void* const* peers = nullptr, int n_peers = 0,
                      int self_index = -1) {
    if (!A || !B) return fail_msg(BM_ERR_NULL, "operand pointer is NULL");
    if (M <= 0 || N <= 0 || K <= 0) return fail_msg(BM_ERR_SHAPE, "M, N, K must be positive");
    if (b_layout != BM_B_KN && b_layout != BM_B_NK) return fail_msg(BM_ERR_LAYOUT, "unknown B layout tag");
    if (K % 16 != 0) return fail_msg(BM_ERR_SHAPE, "K must be a multiple of 16 (16-byte row pitch of A)");
    if (b_layout == BM_B_KN && N % 16 != 0)
        return fail_msg(BM_ERR_SHAPE, "N must be a multiple of 16 for B[K x N] (16-byte row pitch of B)");
    if (!aligned16(A) || !aligned16(B)) return fail_msg(BM_ERR_ALIGN, "operands must be 16-byte aligned");
    if (int rc = validate_epilogue(epi, C, ldc, N, row_scale, col_scale, col_zero)) return rc;

    DeviceState* dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;

    const bool b_mn = (b_layout == BM_B_KN);
    const int tiles_m = ceil_div(M, kBM);
    int bn = forced_bn();
    bool pair_ok = pair_enabled() && dev->sm_count >= 2;
    if (bn == 0) {
        // Tile choice by a wave count model: cost = start-up + waves x (time of one tile per 4096 of K).
        // The per-wave figures (us at K = 4096, W8A8 fp16 out, one B200) were measured on problems from
        // 64 x 512 to 4352 x 8192: narrow tiles move more operand bytes per MAC but finish a wave sooner,
        // so they win while the wide tiles would leave SMs idle, and lose once they need a second wave.
        struct Cand { int bn; bool pair; float wave_us, start_us; };
        const Cand cands[4] = {{256, true, 12.0f, 3.6f}, {256, false, 12.3f, 3.0f}, {128, false, 9.8f, 2.8f},
                               {64, false, 9.3f, 2.6f}};
        const int min_bn = (b_mn || n_peers > 0) ? 128 : 64;
        float best = 0.f;
        bool best_pair = false;
        for (const Cand& c : cands) {
            if (c.bn < min_bn || (c.pair && !pair_ok)) continue;
            const long long tiles = static_cast<long long>(ceil_div(M, c.pair ? 256 : kBM)) * ceil_div(N, c.bn);
            const long long slots = c.pair ? dev->sm_count / 2 : dev->sm_count;
            const float cost = c.start_us + static_cast<float>((tiles + slots - 1) / slots) * c.wave_us;
            if (bn == 0 || cost < best) { best = cost; bn = c.bn; best_pair = c.pair; }
        }
        pair_ok = best_pair;
    }
    if (b_mn && bn < 128) bn = 128;
    if (n_peers > 0 && bn < 128) bn = 128;          // the gather rides on the TMA-store epilogue (tiles >= 128 wide)

    const bool use_pair = (bn == 256) && pair_ok;

    CUtensorMap map_a, map_b;
    if (int rc = make_tensor_map_u8(&map_a, A, K, M, K, kBK, kBM, true)) return rc;
    if (b_mn) {
        if (int rc = make_tensor_map_u8(&map_b, B, N, K, N, 128, kBK, true)) return rc;
    } else {
        if (int rc = make_tensor_map_u8(&map_b, B, K, N, K, kBK, use_pair ? kPairHalfN : bn, true)) return rc;
    }

    DenseParams p{};
    p.epi.out = C;
    p.epi.ld = ldc;
    p.epi.rows = M;
    p.epi.cols = N;
    p.epi.tensor_scale = tensor_scale;
    p.epi.row_scale = row_scale;
    p.epi.col_scale = col_scale;
    p.epi.col_zero = col_zero;
    p.epi.vec_ok = aligned16(C) && (static_cast<size_t>(ldc) * out_elem_size(epi)) % 16 == 0;
    OutMaps map_out{};
    p.n_out = 1;
    if (n_peers > 0) {
        // the same slab goes to every GPU of the group: one tensor map per destination buffer
        if (n_peers > kMaxOutMaps) return fail_msg(BM_ERR_TOO_LARGE, "at most 8 gather destinations");
        for (int d = 0; d < n_peers; ++d) {
            if (!peers[d] || !aligned16(peers[d])) return fail_msg(BM_ERR_ALIGN, "gather destinations must be 16-byte aligned");
            if (int rc = make_tensor_map_out(&map_out.m[d], peers[d], N, M, static_cast<size_t>(ldc) * out_elem_size(epi),
                                             static_cast<int>(out_elem_size(epi))))
                return rc;
        }
        if ((static_cast<size_t>(ldc) * out_elem_size(epi)) % 16 != 0)
            return fail_msg(BM_ERR_ALIGN, "gather needs a 16-byte aligned output pitch");
        p.n_out = n_peers;
        p.epi.tma_ok = 1;
        p.epi.vec_ok = 1;
        // every destination but the GPU's own buffer is reached over NVLink: those stores are paced
        const bool self_ok = self_index >= 0 && self_index < n_peers;
        p.pace.first = self_ok ? self_index : 0;
        p.pace.remote_mask = ((1u << n_peers) - 1u) & ~(self_ok ? 1u << self_index : 0u);
        p.pace.clock = dev->link_clock;
        const int gbs = opt(OPT_GATHER_GBS);
        // one remote store = one 32-row x 128-byte box = 4 KiB; virtual-clock units are 1/16 ns
        p.pace.cost = gbs > 0 ? static_cast<unsigned>((4096.0 * 16.0) / gbs + 0.5) : 0u;
    } else if (p.epi.vec_ok && opt(OPT_TMA_STORE) != 0) {
        if (int rc = make_tensor_map_out(&map_out.m[0], C, N, M, static_cast<size_t>(ldc) * out_elem_size(epi),
                                         static_cast<int>(out_elem_size(epi))))
            return rc;
        p.epi.tma_ok = 1;
    }
    p.tiles_m = tiles_m;
    p.tiles_n = ceil_div(N, bn);
    p.k_blocks = ceil_div(K, kBK);
    p.status = dev->status;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int grid = num_tiles < dev->sm_count ? num_tiles : dev->sm_count;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    CUtensorMap map_a_short = map_a;
    if (use_pair) {
        p.tiles_m = ceil_div(M, 256);
        const int pair_tiles = p.tiles_m * p.tiles_n;
        const int max_pairs = dev->sm_count / 2;
        const int pairs = pair_tiles < max_pairs ? pair_tiles : max_pairs;
        // Tile order: with many more row tiles than column tiles a wave of row-tiles-first order streams
        // 74 different A tiles against one or two B tiles; bands of 8 row tiles give every wave ~8 x 9
        // tiles to reuse.  Measured (medians, interleaved): 16384 x 4096 x 4096 +4.4 %, 8192 x 4096 x 11008
        // +5.7 %, 8192 x 4096 x 4096 +1.6 %; wide problems (8192 x 22016 x 4096: -1.8 %) keep the plain order.
        p.group_m = (p.tiles_m >= 2 * p.tiles_n && p.tiles_m >= 16) ? 8 : 0;
        if (opt(OPT_DENSE_GROUP_M) >= 0) p.group_m = opt(OPT_DENSE_GROUP_M);
        // Half-height tail: when at most half of the pairs would work in the last wave, its tiles are
        // computed as two 128 x 256 halves by different pairs (M = 128 pair MMAs, 64 rows per CTA; no
        // reduction).  Worth only ~1 % (4096^3: 48.1 -> 47.8 us): a K = 32 MMA step chained on one
        // accumulator takes ~128 clocks whether it is 256 x 256, 256 x 128 or 128 x 256, so a smaller unit
        // saves operand waits, not MMA time.  Option "tail_narrow" = 0 switches it off.  (Cutting the tail
        // tiles along K instead — partial sums parked in global memory, last arrival finishes — was
        // measured 15 % SLOWER at 4096^3, 69.5 vs 60.3 us, and is not built.)
        {
            const int rem = pair_tiles % pairs;
            if (rem > 0 && pair_tiles > pairs && 2 * rem <= pairs && opt(OPT_TAIL_NARROW) != 0) {
                if (int rc = make_tensor_map_u8(&map_a_short, A, K, M, K, kBK, 64, true)) return rc;
                p.tail_first = pair_tiles - rem;
                p.tail_narrow = 1;
            }
        }
#define BM_PAIR_CASE(E)                                                                         \
    case E:                                                                                     \
        return b_mn ? launch_dense_pair<true, E>(map_a, map_b, map_a_short, map_out, p, pairs, stream)   \
                    : launch_dense_pair<false, E>(map_a, map_b, map_a_short, map_out, p, pairs, stream);
        switch (epi) {
            BM_PAIR_CASE(EPI_I32)
            BM_PAIR_CASE(EPI_F32_TENSOR)
            BM_PAIR_CASE(EPI_F32_CHANNEL)
            BM_PAIR_CASE(EPI_F16_ROWCOL)
            case EPI_F32_ROWCOL:                       // online-quant GEMM: B stays [K x N]
                if (!b_mn) return fail_msg(BM_ERR_LAYOUT, "fp32 row x column scaling is built for B[K x N] only");
                return launch_dense_pair<true, EPI_F32_ROWCOL>(map_a, map_b, map_a_short, map_out, p, pairs, stream);
        }
#undef BM_PAIR_CASE
    }

#define BM_DENSE_CASE(E)                                                                        \
    case E:                                                                                     \
        return b_mn ? launch_dense_bn<true, E>(bn, map_a, map_b, map_out, p, grid, stream)      \
                    : launch_dense_bn<false, E>(bn, map_a, map_b, map_out, p, grid, stream);
    switch (epi) {
        BM_DENSE_CASE(EPI_I32)
        BM_DENSE_CASE(EPI_F32_TENSOR)
        BM_DENSE_CASE(EPI_F32_CHANNEL)
        BM_DENSE_CASE(EPI_F16_ROWCOL)
        case EPI_F32_ROWCOL:
            if (!b_mn) return fail_msg(BM_ERR_LAYOUT, "fp32 row x column scaling is built for B[K x N] only");
            return launch_dense_bn<true, EPI_F32_ROWCOL>(bn, map_a, map_b, map_out, p, grid, stream);
    }
#undef BM_DENSE_CASE
    return fail_msg(BM_ERR_LAYOUT, "unknown epilogue");
}

// =========================================================================================
// sparse
// =========================================================================================
static size_t meta_tiled_bytes(int R, int K) {
    return static_cast<size_t>(ceil_div(R, 128)) * ceil_div(K, kSpKLogical) * kSpMetaBytes;
}

static int pack_meta(const void* meta_in, int fmt, void* tiled, int R, int K, cudaStream_t stream,
                     bool into_packed_weights = false) {
    if (!meta_in || !tiled) return fail_msg(BM_ERR_NULL, "metadata pointer is NULL");
    if (R <= 0 || K <= 0 || K % (fmt == BM_META_REF_F16 ? 16 : 32) != 0)
        return fail_msg(BM_ERR_SHAPE, "K must be a positive multiple of 32 (16 for the fp16 reference format)");
    if ((fmt == BM_META_REF || fmt == BM_META_REF_F16) && R % 16 != 0)
        return fail_msg(BM_ERR_SHAPE, "reference metadata needs rows % 16 == 0");
    if (!aligned16(tiled) || (reinterpret_cast<uintptr_t>(meta_in) & 3u))
        return fail_msg(BM_ERR_ALIGN, "metadata buffers are misaligned");
    const int k_blocks = ceil_div(K, kSpKLogical);
    const size_t units = meta_tiled_bytes(R, K) / 16;
    const unsigned blocks = static_cast<unsigned>((units + 255) / 256);
    const MetaDest dest{k_blocks, into_packed_weights ? ceil_div(R, 128) * 128 : 0};
    if (fmt == BM_META_ROWS || fmt == BM_META_ROWS_F16)
        pack_meta_rows_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(meta_in),
                                                          static_cast<uint8_t*>(tiled), R, K, k_blocks, units,
                                                          dest, fmt == BM_META_ROWS_F16 ? 1 : 0);
    else if (fmt == BM_META_REF)
        pack_meta_ref_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint32_t*>(meta_in),
                                                         static_cast<uint8_t*>(tiled), R, K, k_blocks, units,
                                                         dest);
    else if (fmt == BM_META_REF_F16)
        pack_meta_ref_f16_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint32_t*>(meta_in),
                                                             static_cast<uint8_t*>(tiled), R, K, k_blocks, units,
                                                             dest);
    else if (fmt == BM_META_TILED && into_packed_weights)
        pack_meta_copy_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(meta_in),
                                                          static_cast<uint8_t*>(tiled), units, dest);
    else
        return fail_msg(BM_ERR_LAYOUT, "unknown metadata format tag");
    BM_CUDA_TRY(cudaGetLastError());
    return BM_OK;
}

template <int BN, bool DENSE_MN, bool TRANSPOSED, int EPI, bool PACKED = false, int ROWS = kBM>
static int launch_sparse_inst(const CUtensorMap& ms, const CUtensorMap& md, const SparseParams& p, int grid,
                              cudaStream_t stream) {
    using Cfg = SparseCfg<BN, ROWS>;
    auto kern = igemm_sparse_kernel<BN, DENSE_MN, TRANSPOSED, EPI, PACKED, false, ROWS>;
    static ConfiguredFlags flags;
    if (int rc = ensure_smem_limit(flags, kern, Cfg::SMEM_BYTES)) return rc;
    BM_CUDA_TRY(launch_pdl(kern, dim3(grid), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, stream, 1, ms, md, p));
    return BM_OK;
}

// CTA-pair kernel for sparse weights: 256 channels x 240 tokens per pair
template <int EPI>
static int launch_sparse_pair(const CUtensorMap& mw, const CUtensorMap& me, const CUtensorMap& mx, const SparseParams& p,
                              int pairs, cudaStream_t stream) {
    auto kern = igemm_sparse_pair_kernel<EPI>;
    static ConfiguredFlags flags;
    if (int rc = ensure_smem_limit(flags, kern, kSpPairSmemBytes)) return rc;
    BM_CUDA_TRY(launch_pdl(kern, dim3(2 * pairs), dim3(kDenseThreads), kSpPairSmemBytes, stream, 2, mw, me, mx, mw, p));
    return BM_OK;                                   // (no output tensor map in this orientation: mw fills the slot)
}

// the reference orientation (sparse operand on the left, B[K x C]) on CTA pairs: 256 rows x 224 columns
template <int EPI, bool F16>
static int launch_sparse_pair_left(const CUtensorMap& mw, const CUtensorMap& me, const CUtensorMap& mx,
                                   const CUtensorMap& mo, const SparseParams& p, int pairs, cudaStream_t stream) {
    auto kern = igemm_sparse_pair_kernel<EPI, true, F16>;
    constexpr int smem = SpPairCfg<true>::SMEM_BYTES;
    static ConfiguredFlags flags;
    if (int rc = ensure_smem_limit(flags, kern, smem)) return rc;
    BM_CUDA_TRY(launch_pdl(kern, dim3(2 * pairs), dim3(kDenseThreads), smem, stream, 2, mw, me, mx, mo, p));
    return BM_OK;
}

// Sets up and launches the pair kernel in the reference orientation.  `elem` = bytes per operand element
// (1: int8, 2: fp16); K counts logical elements, the tensor maps are byte maps.
static int sparse_pair_left(int epi, bool f16, const void* S_comp, const uint8_t* meta_tiled, const void* B, void* out,
                            int R, int Cn, int K, long long ld, float tensor_scale, DeviceState* dev,
                            cudaStream_t stream) {
    const int elem = f16 ? 2 : 1;
    CUtensorMap map_w, map_e, map_x;
    const size_t comp_bytes = static_cast<size_t>(K / 2) * elem;
    if (int rc = make_tensor_map_u8(&map_w, S_comp, comp_bytes, R, comp_bytes, 128, kBM, true)) return rc;
    const size_t units = meta_tiled_bytes(R, K) / 16;
    // the tiled metadata is one contiguous run of 16-byte units: described as rows of 128 bytes, a box of 32 rows (16
    // for fp16) lands in shared memory byte for byte as 256 (128) units would, with an eighth of the requests
    if (int rc = make_tensor_map_u8(&map_e, meta_tiled, 128, units / 8, 128, 128, f16 ? 16 : 32, false)) return rc;
    const size_t row_bytes = static_cast<size_t>(Cn) * elem;
    if (int rc = make_tensor_map_u8(&map_x, B, row_bytes, K, row_bytes, 128, f16 ? 128 : kSpKLogical, true)) return rc;
    SparseParams p{};
    p.epi.out = out;
    p.epi.ld = ld;
    p.epi.rows = R;
    p.epi.cols = Cn;
    p.epi.tensor_scale = tensor_scale;
    p.epi.vec_ok = aligned16(out) && (static_cast<size_t>(ld) * 4) % 16 == 0;
    CUtensorMap map_o = map_w;                       // placeholder unless the output qualifies for TMA stores
    if (p.epi.vec_ok && opt(OPT_TMA_STORE) != 0) {
        if (int rc = make_tensor_map_out(&map_o, out, Cn, R, static_cast<size_t>(ld) * 4, 4)) return rc;
        p.epi.tma_ok = 1;
    }
    p.meta_tiled = meta_tiled;
    p.tiles_r = ceil_div(R, 256);
    p.tiles_c = ceil_div(Cn, SpPairCfg<true>::BN);
    p.k_blocks = ceil_div(K, f16 ? 128 : kSpKLogical);
    p.status = dev->status;
    p.sparse_rows = R;
    const int pair_tiles = p.tiles_r * p.tiles_c;
    const int max_pairs = dev->sm_count / 2;
    const int pairs = pair_tiles < max_pairs ? pair_tiles : max_pairs;
    if (f16) return launch_sparse_pair_left<EPI_I32, true>(map_w, map_e, map_x, map_o, p, pairs, stream);
    if (epi == EPI_I32) return launch_sparse_pair_left<EPI_I32, false>(map_w, map_e, map_x, map_o, p, pairs, stream);
    if (epi == EPI_F32_TENSOR) return launch_sparse_pair_left<EPI_F32_TENSOR, false>(map_w, map_e, map_x, map_o, p, pairs, stream);
    return fail_msg(BM_ERR_LAYOUT, "unsupported epilogue for the sparse pair kernel");
}

// When the reference orientation runs on CTA pairs.  Measured against the lone-CTA kernel with 128-column
// tiles: int8 is no faster on pairs (4096^3: 67.6 vs 58.4 us; 8192^3: 395 vs 371 us), so pairs are used
// for int8 only when the tile width is forced to 224; fp16 gains 6-18 % once there are two waves of pair tiles
// (4096^3: 90.7 vs 96.4 us; 8192 x 8192 x 4096: 315 vs 370 us).
static bool sparse_pair_left_wanted(int R, int Cn, const DeviceState* dev, int forced, bool f16) {
    if (forced == 224) return dev->sm_count >= 2;
    if (forced != 0 || dev->sm_count < 2 || !f16) return false;
    if (opt(OPT_SPARSE_PAIR) == 0) return false;
    return static_cast<long long>(ceil_div(R, 256)) * ceil_div(Cn, SpPairCfg<true>::BN) >= dev->sm_count;
}

// option "sparse_pair" = 0 keeps large sparse-weight problems on the single-CTA kernel (testing hook)
static bool sparse_pair_enabled() { return opt(OPT_SPARSE_PAIR) != 0; }

// mode 0: sparse operand on the left, out[r][c];  mode 1: sparse weights, out[c][r]
static int sparse_gemm(int mode, int epi, const int8_t* S_comp, const uint8_t* meta_tiled, const int8_t* Dn,
                       void* out, int R, int Cn, int K, long long ld, int dense_layout, float tensor_scale,
                       const float* row_scale, const float* col_scale, void* stream_v, bool packed = false) {
    if ((!S_comp && !packed) || !meta_tiled || !Dn) return fail_msg(BM_ERR_NULL, "operand pointer is NULL");
    if (R <= 0 || Cn <= 0 || K <= 0) return fail_msg(BM_ERR_SHAPE, "dimensions must be positive");
    if (K % 32 != 0) return fail_msg(BM_ERR_SHAPE, "K must be a multiple of 32 for the 2:4 format");
    const bool dense_mn = (dense_layout == BM_B_KN);
    if (dense_mn && Cn % 16 != 0) return fail_msg(BM_ERR_SHAPE, "N must be a multiple of 16 for B[K x N]");
    if ((!packed && !aligned16(S_comp)) || !aligned16(Dn) || !aligned16(meta_tiled))
        return fail_msg(BM_ERR_ALIGN, "operands must be 16-byte aligned");
    const int out_rows = mode == 0 ? R : Cn, out_cols = mode == 0 ? Cn : R;
    if (int rc = validate_epilogue(epi, out, ld, out_cols, row_scale, col_scale, nullptr)) return rc;

    DeviceState* dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;

    const int tiles_r = ceil_div(R, kBM);
    int bn = forced_bn();

    // large token counts with sparse weights: CTA pairs (256 channels x 240 tokens per pair)
    if (mode == 1 && !dense_mn && !packed && sparse_pair_enabled() && dev->sm_count >= 2 &&
        (bn == 240 || (bn == 0 && Cn >= 192 && ceil_div(R, 256) * ceil_div(Cn, kSpPairBN) >= dev->sm_count / 2))) {
        CUtensorMap map_w, map_e, map_x;
        if (int rc = make_tensor_map_u8(&map_w, S_comp, K / 2, R, K / 2, 128, kBM, true)) return rc;
        const size_t units = meta_tiled_bytes(R, K) / 16;
        if (int rc = make_tensor_map_u8(&map_e, meta_tiled, 128, units / 8, 128, 128, 32, false)) return rc;   // see sparse_pair_left
        if (int rc = make_tensor_map_u8(&map_x, Dn, K, Cn, K, 128, kSpPairHalfN, true)) return rc;
        SparseParams p{};
        p.epi.out = out;
        p.epi.ld = ld;
        p.epi.rows = out_rows;
        p.epi.cols = out_cols;
        p.epi.tensor_scale = tensor_scale;
        p.epi.row_scale = row_scale;
        p.epi.col_scale = col_scale;
        p.epi.vec_ok = aligned16(out) && (static_cast<size_t>(ld) * out_elem_size(epi)) % 16 == 0;
        p.meta_tiled = meta_tiled;
        p.tiles_r = ceil_div(R, 256);
        p.tiles_c = ceil_div(Cn, kSpPairBN);
        p.k_blocks = ceil_div(K, kSpKLogical);
        p.status = dev->status;
        // Tile order.  Weights that do not fit in L2 with few token tiles (prefill chunks against a wide
        // layer): column tiles fastest, so the pairs working at the same time share a block of weights and
        // every block leaves HBM once — N = 28672, K = 8192 (147 MB): 3001 -> 3662 TOPS at 1024 tokens,
        // 3305 -> 4142 at 2048.  Otherwise row blocks fastest (8192^3: 4284 vs 3722 TOPS).
        // Option "sparse_col_first" = 0/1 overrides.
        {
            const double w_bytes = 0.625 * static_cast<double>(R) * K, x_bytes = static_cast<double>(Cn) * K;
            p.col_first = (w_bytes > 96e6 && 2.0 * x_bytes <= w_bytes) ? 1 : 0;
            if (opt(OPT_SPARSE_COL_FIRST) >= 0) p.col_first = opt(OPT_SPARSE_COL_FIRST) != 0;
        }
        const int pair_tiles = p.tiles_r * p.tiles_c;
        const int max_pairs = dev->sm_count / 2;
        const int pairs = pair_tiles < max_pairs ? pair_tiles : max_pairs;
        cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
        if (epi == EPI_I32) return launch_sparse_pair<EPI_I32>(map_w, map_e, map_x, p, pairs, stream);
        if (epi == EPI_F16_ROWCOL) return launch_sparse_pair<EPI_F16_ROWCOL>(map_w, map_e, map_x, p, pairs, stream);
        return fail_msg(BM_ERR_LAYOUT, "unsupported epilogue for the sparse pair kernel");
    }
    if (bn == 240) bn = 0;
    if (mode == 0 && dense_mn && !packed && sparse_pair_left_wanted(R, Cn, dev, bn, false))
        return sparse_pair_left(epi, false, S_comp, meta_tiled, Dn, out, R, Cn, K, ld, tensor_scale, dev,
                                static_cast<cudaStream_t>(stream_v));
    if (bn == 224) bn = 0;

    if (bn == 0) {
        if (mode == 1) {
            // tokens on the accumulator columns: the narrowest tile that holds them, up to 128
            bn = 16;
            while (bn < 128 && bn < Cn) bn <<= 1;
            if (Cn > 128 && tiles_r * ceil_div(Cn, 256) >= dev->sm_count) bn = 256;
        } else {
            // 128 columns at most: a 256-column sparse tile leaves room for 2 ring stages and one
            // accumulator only and was measured 20 % slower (4096^3: 72.6 vs 60.9 us; 8192 x 8192 x 4096:
            // 279 vs 241 us)
            const int min_bn = dense_mn ? 128 : 64;
            bn = min_bn;
            for (int cand = 128; cand >= min_bn; cand >>= 1)
                if (tiles_r * ceil_div(Cn, cand) >= dev->sm_count || cand == min_bn) { bn = cand; break; }
        }
    }
    if (dense_mn && bn < 128) bn = 128;
    if (mode == 0 && bn < 64) bn = 64;

    CUtensorMap map_s, map_d;
    if (packed) memset(&map_s, 0, sizeof(map_s));
    else if (int rc = make_tensor_map_u8(&map_s, S_comp, K / 2, R, K / 2, 128, kBM, true)) return rc;
    if (dense_mn) {
        if (int rc = make_tensor_map_u8(&map_d, Dn, Cn, K, Cn, 128, kSpKLogical, true)) return rc;
    } else {
        if (int rc = make_tensor_map_u8(&map_d, Dn, K, Cn, K, 128, bn, true)) return rc;
    }

    SparseParams p{};
    p.epi.out = out;
    p.epi.ld = ld;
    p.epi.rows = out_rows;
    p.epi.cols = out_cols;
    p.epi.tensor_scale = tensor_scale;
    p.epi.row_scale = row_scale;
    p.epi.col_scale = col_scale;
    p.epi.col_zero = nullptr;
    p.epi.vec_ok = aligned16(out) && (static_cast<size_t>(ld) * out_elem_size(epi)) % 16 == 0;
    p.meta_tiled = meta_tiled;
    p.tiles_r = tiles_r;
    p.tiles_c = ceil_div(Cn, bn);
    p.k_blocks = ceil_div(K, kSpKLogical);
    p.status = dev->status;
    const int num_tiles = p.tiles_r * p.tiles_c;
    const int resident = dev->sm_count * (bn <= 64 ? 2 : 1);      // narrow tiles run two CTAs per SM
    int grid = num_tiles < resident ? num_tiles : resident;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    // (Dealing out (tile, K block) units instead of whole tiles — stream-K, partial sums parked in global
    // memory and finished by the last arrival — was measured slower on every decode shape and is not built:
    // N = 28672, K = 8192: 34.8 vs 26.5 us at 1 token, 45.5 vs 30.1 us at 64.  The parked sums put a dependent
    // chain — park, fence, count, re-read every part — at the very end of the launch, where nothing hides it.)
    p.sparse_rows = R;

    // Row-balanced tiles for the decode shapes (packed weights, all tokens in one column tile): whole
    // 128-row tiles would give some SMs two tiles and others one (224 tiles on 148 SMs); dealing the
    // rows out in multiples of 8 keeps every SM streaming the same number of bytes.  Option
    // "row_balanced" = 0 switches it off.
    if (mode == 1 && packed && p.tiles_c == 1 && num_tiles % resident != 0 && R >= 8 * resident &&
        opt(OPT_ROW_BALANCED) != 0) {
        p.row_balanced = 1;
        grid = resident;
    }
    // Few rows per CTA (the slab of an N-split layer: 3584 channels on 296 CTA slots are 8-16 rows each): ring
    // stages sized for 32 or 64 rows instead of 128, so up to 12 K blocks are in flight per CTA instead of 4 —
    // a CTA walks ALL K blocks of its rows one after the other, and with a 4-deep ring that walk is 8 memory
    // round trips long however few bytes it moves.  Option "decode_tile_rows" = 128 keeps the full stages.
    int tile_rows = 128;
    if (p.row_balanced && bn <= 64) {
        const int per_cta = ceil_div(ceil_div(R, 8), grid) * 8;
        tile_rows = per_cta <= 32 ? 32 : per_cta <= 64 ? 64 : 128;
        const int forced = opt(OPT_DECODE_TILE_ROWS);
        if (forced == 32 || forced == 64 || forced == 128) tile_rows = forced;
    }

#define BM_SP(BNV, MN, TR, E) return launch_sparse_inst<BNV, MN, TR, E>(map_s, map_d, p, grid, stream)
    if (mode == 0) {
        if (epi == EPI_I32) {
            if (dense_mn) { if (bn == 256) BM_SP(256, true, false, EPI_I32); if (bn == 128) BM_SP(128, true, false, EPI_I32); }
            else { if (bn == 256) BM_SP(256, false, false, EPI_I32); if (bn == 128) BM_SP(128, false, false, EPI_I32);
                   if (bn == 64) BM_SP(64, false, false, EPI_I32); }
        } else if (epi == EPI_F32_TENSOR) {
            if (dense_mn) { if (bn == 256) BM_SP(256, true, false, EPI_F32_TENSOR); if (bn == 128) BM_SP(128, true, false, EPI_F32_TENSOR); }
            else { if (bn == 256) BM_SP(256, false, false, EPI_F32_TENSOR); if (bn == 128) BM_SP(128, false, false, EPI_F32_TENSOR);
                   if (bn == 64) BM_SP(64, false, false, EPI_F32_TENSOR); }
        }
    } else if (!dense_mn && packed) {
#define BM_SPP(BNV, E) return launch_sparse_inst<BNV, false, true, E, true>(map_s, map_d, p, grid, stream)
#define BM_SPR(BNV, E, R_) if (bn == BNV && tile_rows == R_) return launch_sparse_inst<BNV, false, true, E, true, R_>(map_s, map_d, p, grid, stream)
        if (epi == EPI_I32) {
            BM_SPR(64, EPI_I32, 32); BM_SPR(64, EPI_I32, 64); BM_SPR(32, EPI_I32, 32); BM_SPR(32, EPI_I32, 64);
            BM_SPR(16, EPI_I32, 32); BM_SPR(16, EPI_I32, 64);
        } else if (epi == EPI_F16_ROWCOL) {
            BM_SPR(64, EPI_F16_ROWCOL, 32); BM_SPR(64, EPI_F16_ROWCOL, 64); BM_SPR(32, EPI_F16_ROWCOL, 32);
            BM_SPR(32, EPI_F16_ROWCOL, 64); BM_SPR(16, EPI_F16_ROWCOL, 32); BM_SPR(16, EPI_F16_ROWCOL, 64);
        }
#undef BM_SPR
        if (epi == EPI_I32) {
            if (bn == 256) BM_SPP(256, EPI_I32); if (bn == 128) BM_SPP(128, EPI_I32); if (bn == 64) BM_SPP(64, EPI_I32);
            if (bn == 32) BM_SPP(32, EPI_I32);   if (bn == 16) BM_SPP(16, EPI_I32);
        } else if (epi == EPI_F16_ROWCOL) {
            if (bn == 256) BM_SPP(256, EPI_F16_ROWCOL); if (bn == 128) BM_SPP(128, EPI_F16_ROWCOL);
            if (bn == 64) BM_SPP(64, EPI_F16_ROWCOL);   if (bn == 32) BM_SPP(32, EPI_F16_ROWCOL);
            if (bn == 16) BM_SPP(16, EPI_F16_ROWCOL);
        }
#undef BM_SPP
    } else if (!dense_mn) {
        if (epi == EPI_I32) {
            if (bn == 256) BM_SP(256, false, true, EPI_I32); if (bn == 128) BM_SP(128, false, true, EPI_I32);
            if (bn == 64) BM_SP(64, false, true, EPI_I32);   if (bn == 32) BM_SP(32, false, true, EPI_I32);
            if (bn == 16) BM_SP(16, false, true, EPI_I32);
        } else if (epi == EPI_F16_ROWCOL) {
            if (bn == 256) BM_SP(256, false, true, EPI_F16_ROWCOL); if (bn == 128) BM_SP(128, false, true, EPI_F16_ROWCOL);
            if (bn == 64) BM_SP(64, false, true, EPI_F16_ROWCOL);   if (bn == 32) BM_SP(32, false, true, EPI_F16_ROWCOL);
            if (bn == 16) BM_SP(16, false, true, EPI_F16_ROWCOL);
        }
    }
#undef BM_SP
    return fail_msg(BM_ERR_SHAPE, "unsupported sparse GEMM configuration");
}

// A wait that nothing will ever satisfy, with a short limit: the give-up path of the pipeline
// waits, exercised without hanging or faulting anything.
__global__ void selftest_bounded_wait_kernel(int* status, unsigned long long limit_ns, int* returned) {
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

// =========================================================================================
// C ABI
// =========================================================================================
using namespace bm;

// FP16 2:4 GEMM (kernels/gemm/hgemm_sparse): the sparse kernel in its fp16 form, one CTA per tile
template <int BN>
static int launch_hsparse(const CUtensorMap& ms, const CUtensorMap& md, const SparseParams& p, int grid,
                          cudaStream_t stream) {
    using Cfg = SparseCfg<BN>;
    auto kern = igemm_sparse_kernel<BN, true, false, EPI_I32, false, true>;
    static ConfiguredFlags flags;
    if (int rc = ensure_smem_limit(flags, kern, Cfg::SMEM_BYTES)) return rc;
    BM_CUDA_TRY(launch_pdl(kern, dim3(grid), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, stream, 1, ms, md, p));
    return BM_OK;
}

extern "C" {

int bm_igemm_i8_i32(const int8_t* A, const int8_t* B, int32_t* C, int M, int N, int K, int64_t ldc, int b_layout,
                    void* stream) {
    return dense_gemm(EPI_I32, A, B, C, M, N, K, ldc, b_layout, 1.f, nullptr, nullptr, nullptr, stream);
}

int bm_igemm_i8_f32(const int8_t* A, const int8_t* B, float* C, int M, int N, int K, float scale_a, float scale_b,
                    int64_t ldc, int b_layout, void* stream) {
    // the reference multiplies the two scales first (igemm.cu:104), in fp32
    volatile float dequant = scale_a * scale_b;
    return dense_gemm(EPI_F32_TENSOR, A, B, C, M, N, K, ldc, b_layout, dequant, nullptr, nullptr, nullptr, stream);
}

int bm_igemm_i8_f32_perchannel(const int8_t* A, const int8_t* B, float* C, int M, int N, int K, const float* scale_n,
                               const int32_t* zero_point_n, int64_t ldc, int b_layout, void* stream) {
    return dense_gemm(EPI_F32_CHANNEL, A, B, C, M, N, K, ldc, b_layout, 1.f, nullptr, scale_n, zero_point_n, stream);
}

int bm_w8a8_f16(const int8_t* X, const int8_t* W, uint16_t* D, const float* sa_m, const float* sw_n, int M, int N,
                int K, int64_t ldd, int w_layout, void* stream) {
    return dense_gemm(EPI_F16_ROWCOL, X, W, D, M, N, K, ldd, w_layout, 1.f, sa_m, sw_n, nullptr, stream);
}

int bm_w8a8_f16_gather(const int8_t* X, const int8_t* W, uint16_t* const* D_peers, int n_peers, int self_index,
                       const float* sa_m, const float* sw_n, int M, int N, int K, int64_t ldd, int w_layout,
                       void* stream) {
    if (!D_peers || n_peers <= 0) return fail_msg(BM_ERR_NULL, "no gather destinations given");
    if (self_index < -1 || self_index >= n_peers) return fail_msg(BM_ERR_SHAPE, "self_index must be -1 or an index into D_peers");
    return dense_gemm(EPI_F16_ROWCOL, X, W, D_peers[self_index < 0 ? 0 : self_index], M, N, K, ldd, w_layout, 1.f, sa_m,
                      sw_n, nullptr, stream, reinterpret_cast<void* const*>(D_peers), n_peers, self_index);
}

int bm_gather_slab_f16(uint16_t* const* D_peers, int n_peers, int self_index, int M, int n_len, int64_t ldd, void* stream) {
    if (!D_peers || n_peers <= 0 || n_peers > kGatherMaxPeers) return fail_msg(BM_ERR_NULL, "1 to 8 gather destinations are needed");
    if (self_index < 0 || self_index >= n_peers) return fail_msg(BM_ERR_SHAPE, "self_index must be an index into D_peers");
    if (M <= 0 || n_len <= 0 || ldd < n_len) return fail_msg(BM_ERR_SHAPE, "M, n_len must be positive and ldd >= n_len");
    if (n_len % 8 != 0 || ldd % 8 != 0) return fail_msg(BM_ERR_ALIGN, "slab width and pitch must be multiples of 8 elements (16 bytes)");
    GatherDests dests{};
    for (int d = 0; d < n_peers; ++d) {
        if (!D_peers[d] || !aligned16(D_peers[d])) return fail_msg(BM_ERR_ALIGN, "gather destinations must be 16-byte aligned");
        dests.ptr[d] = D_peers[d];
    }
    if (n_peers == 1) return BM_OK;
    DeviceState* dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;
    const int row_bytes = n_len * 2;
    const long long tiles = static_cast<long long>((M + 31) / 32) * ((row_bytes + 511) / 512);
    const long long cap = static_cast<long long>(dev->sm_count) * 8;
    const int gbs = opt(OPT_GATHER_GBS);
    const unsigned cost = gbs > 0 ? static_cast<unsigned>((4096.0 * 16.0) / gbs + 0.5) : 0u;
    gather_slab_kernel<<<static_cast<unsigned>(tiles < cap ? tiles : cap), kGatherThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        dests, n_peers, self_index, M, row_bytes, static_cast<long long>(ldd) * 2, dev->link_clock, cost);
    BM_CUDA_TRY(cudaGetLastError());
    return BM_OK;
}

int bm_peer_barrier(uint32_t* const* flag_arrays, int n_peers, int self_index, void* stream) {
    if (!flag_arrays || n_peers <= 0 || n_peers > kGatherMaxPeers) return fail_msg(BM_ERR_NULL, "1 to 8 flag arrays are needed");
    if (self_index < 0 || self_index >= n_peers) return fail_msg(BM_ERR_SHAPE, "self_index must be an index into flag_arrays");
    BarrierFlags flags{};
    for (int d = 0; d < n_peers; ++d) {
        if (!flag_arrays[d] || (reinterpret_cast<uintptr_t>(flag_arrays[d]) & 3u)) return fail_msg(BM_ERR_ALIGN, "flag arrays must be 4-byte aligned");
        flags.ptr[d] = flag_arrays[d];
    }
    DeviceState* dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;
    BM_CUDA_TRY(launch_pdl(peer_barrier_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), 1, flags, n_peers,
                           self_index, dev->status));
    return BM_OK;
}

int bm_quantize_rows_f16(const uint16_t* X_f16, int8_t* X_q, float* scale_m, int M, int K, void* stream) {
    if (!X_f16 || !X_q || !scale_m) return fail_msg(BM_ERR_NULL, "pointer is NULL");
    if (M <= 0 || K <= 0 || K % 16 != 0) return fail_msg(BM_ERR_SHAPE, "K must be a positive multiple of 16");
    if (!aligned16(X_f16) || !aligned16(X_q)) return fail_msg(BM_ERR_ALIGN, "buffers must be 16-byte aligned");
    quantize_rows_f16_kernel<<<(M + kQuantThreads / 32 - 1) / (kQuantThreads / 32), kQuantThreads, 0,
                               static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const __half*>(X_f16), X_q, scale_m, M, K);
    BM_CUDA_TRY(cudaGetLastError());
    return BM_OK;
}

size_t bm_online_quant_workspace_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
    return up(static_cast<size_t>(M) * K) + up(static_cast<size_t>(K) * N) + up(sizeof(float) * M) + up(sizeof(float) * N);
}

int bm_online_quant_gemm_f32(const uint16_t* A_f16, const uint16_t* B_f16, float* C, int M, int N, int K,
                             int col_block, void* workspace, size_t workspace_bytes, void* stream) {
    if (!A_f16 || !B_f16 || !C || !workspace) return fail_msg(BM_ERR_NULL, "pointer is NULL");
    if (M <= 0 || N <= 0 || K <= 0) return fail_msg(BM_ERR_SHAPE, "M, N, K must be positive");
    if (K % 16 != 0 || N % 16 != 0) return fail_msg(BM_ERR_SHAPE, "K and N must be multiples of 16");
    if (col_block != 128 && col_block != 256) return fail_msg(BM_ERR_SHAPE, "column block must be 128 or 256");
    if (!aligned16(A_f16) || !aligned16(B_f16) || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        return fail_msg(BM_ERR_ALIGN, "operands must be 16-byte aligned, the workspace 256-byte aligned");
    if (workspace_bytes < bm_online_quant_workspace_bytes(M, N, K))
        return fail_msg(BM_ERR_TOO_LARGE, "workspace is smaller than bm_online_quant_workspace_bytes()");
    DeviceState* dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;
    auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    int8_t* Aq = reinterpret_cast<int8_t*>(ws);                 ws += up(static_cast<size_t>(M) * K);
    int8_t* Bq = reinterpret_cast<int8_t*>(ws);                 ws += up(static_cast<size_t>(K) * N);
    float* row_scale = reinterpret_cast<float*>(ws);            ws += up(sizeof(float) * M);
    float* col_scale = reinterpret_cast<float*>(ws);            ws += up(sizeof(float) * N);
    const int blocks_a = ceil_div(M, kOqRowBlock), blocks_b = ceil_div(N, col_block);
    const int a_per = ceil_div(K, 256), b_per = ceil_div(K, kOqChunkElems / col_block);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    oq_quantize_kernel<<<blocks_a * a_per + blocks_b * b_per, kOqThreads, 0, st>>>(
        reinterpret_cast<const __half*>(A_f16), reinterpret_cast<const __half*>(B_f16), Aq, Bq, row_scale, col_scale, M,
        N, K, col_block, blocks_a * a_per, a_per, b_per);
    BM_CUDA_TRY(cudaGetLastError());
    return dense_gemm(EPI_F32_ROWCOL, Aq, Bq, C, M, N, K, N, BM_B_KN, 1.f, row_scale, col_scale, nullptr, stream);
}

int bm_prune_2_4_i8(const int8_t* W, int8_t* W_comp, uint8_t* W_meta_rows, int R, int K, void* stream) {
    if (!W || !W_comp || !W_meta_rows) return fail_msg(BM_ERR_NULL, "pointer is NULL");
    if (R <= 0 || K <= 0 || K % 32 != 0) return fail_msg(BM_ERR_SHAPE, "K must be a positive multiple of 32");
    if (!aligned16(W) || !aligned16(W_comp) || reinterpret_cast<uintptr_t>(W_meta_rows) % 4 != 0)
        return fail_msg(BM_ERR_ALIGN, "W and W_comp must be 16-byte aligned, the metadata 4-byte aligned");
    DeviceState* dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;
    const size_t units = static_cast<size_t>(R) * K / 32;
    const size_t want = (units + 255) / 256, cap = static_cast<size_t>(dev->sm_count) * 16;
    prune_2_4_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        W, W_comp, W_meta_rows, units);
    BM_CUDA_TRY(cudaGetLastError());
    return BM_OK;
}

int bm_pack_b_kn_to_nk(const int8_t* B_kn, int8_t* W_nk, int K, int N, void* stream) {
    if (!B_kn || !W_nk) return fail_msg(BM_ERR_NULL, "pointer is NULL");
    if (K <= 0 || N <= 0) return fail_msg(BM_ERR_SHAPE, "K and N must be positive");
    dim3 grid((N + 63) / 64, (K + 63) / 64), block(64, 8);
    transpose_kn_to_nk_kernel<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(B_kn, W_nk, K, N);
    BM_CUDA_TRY(cudaGetLastError());
    return BM_OK;
}

size_t bm_sp_meta_tiled_bytes(int R, int K) {
    if (R <= 0 || K <= 0) return 0;
    return meta_tiled_bytes(R, K);
}

int bm_sp_pack_meta(const void* meta_in, int meta_format, void* meta_tiled, int R, int K, void* stream) {
    return pack_meta(meta_in, meta_format, meta_tiled, R, K, static_cast<cudaStream_t>(stream));
}

// metadata in a caller format is re-tiled into library scratch first (same stream, so ordered)
static int resolve_meta(const void* meta, int fmt, int R, int K, void* stream, const uint8_t** tiled) {
    if (fmt == BM_META_TILED) {
        *tiled = static_cast<const uint8_t*>(meta);
        return BM_OK;
    }
    DeviceState* dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;
    if (int rc = ensure_scratch(dev, meta_tiled_bytes(R, K))) return rc;
    if (int rc = pack_meta(meta, fmt, dev->scratch, R, K, static_cast<cudaStream_t>(stream))) return rc;
    *tiled = static_cast<const uint8_t*>(dev->scratch);
    return BM_OK;
}

int bm_igemm_sparse_f32(const int8_t* A_comp, const int8_t* B, float* C, const uint32_t* meta, int M, int N, int K,
                        float scale_a, float scale_b, void* stream) {
    if (!meta) return fail_msg(BM_ERR_NULL, "metadata pointer is NULL");
    if (M <= 0 || M % 16 != 0) return fail_msg(BM_ERR_SHAPE, "M must be a positive multiple of 16");
    if (K <= 0 || K % 32 != 0) return fail_msg(BM_ERR_SHAPE, "K must be a positive multiple of 32");
    const uint8_t* tiled = nullptr;
    if (int rc = resolve_meta(meta, BM_META_REF, M, K, stream, &tiled)) return rc;
    volatile float dequant = scale_a * scale_b;       // igemm_sparse_tiled.cu:365
    return sparse_gemm(0, EPI_F32_TENSOR, A_comp, tiled, B, C, M, N, K, N, BM_B_KN, dequant, nullptr, nullptr, stream);
}

int bm_hgemm_sparse_f32(const uint16_t* A_comp, const uint16_t* B, float* C, const void* meta, int meta_format,
                        int M, int N, int K, int64_t ldc, void* stream_v) {
    if (!A_comp || !B || !C || !meta) return fail_msg(BM_ERR_NULL, "pointer is NULL");
    if (M <= 0 || N <= 0 || K <= 0) return fail_msg(BM_ERR_SHAPE, "dimensions must be positive");
    if (K % 16 != 0 || N % 16 != 0) return fail_msg(BM_ERR_SHAPE, "K and N must be multiples of 16");
    if (ldc < N) return fail_msg(BM_ERR_SHAPE, "output pitch is smaller than the row length");
    if (!aligned16(A_comp) || !aligned16(B)) return fail_msg(BM_ERR_ALIGN, "operands must be 16-byte aligned");
    if (meta_format == BM_META_REF) return fail_msg(BM_ERR_LAYOUT, "the int8 reference metadata format does not describe fp16 operands");
    if (meta_format == BM_META_ROWS) meta_format = BM_META_ROWS_F16;      // per-row bytes, tiled in the fp16 lane order
    const uint8_t* tiled = nullptr;
    if (int rc = resolve_meta(meta, meta_format, M, K, stream_v, &tiled)) return rc;
    DeviceState* dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;
    const int tiles_r = ceil_div(M, kBM);
    int bn = forced_bn();
    if (sparse_pair_left_wanted(M, N, dev, bn, true))
        return sparse_pair_left(EPI_I32, true, A_comp, tiled, B, C, M, N, K, ldc, 1.f, dev, static_cast<cudaStream_t>(stream_v));
    // 128-column tiles: 4 stages and two accumulators fit; 256-column tiles leave room for 2 stages and
    // one accumulator only and were measured slower (4096^3: 122 vs 99 us; 8192^3: 904 vs 801 us)
    if (bn != 128 && bn != 256) bn = 128;
    CUtensorMap map_s, map_d;        // byte maps: compressed A is [M x K bytes], B is [K x 2N bytes]
    if (int rc = make_tensor_map_u8(&map_s, A_comp, K, M, K, 128, kBM, true)) return rc;
    if (int rc = make_tensor_map_u8(&map_d, B, 2 * static_cast<size_t>(N), K, 2 * static_cast<size_t>(N), 128, 128, true))
        return rc;
    SparseParams p{};
    p.epi.out = C;                   // fp32 accumulator bits are stored as they are (EPI_I32)
    p.epi.ld = ldc;
    p.epi.rows = M;
    p.epi.cols = N;
    p.epi.vec_ok = aligned16(C) && (static_cast<size_t>(ldc) * 4) % 16 == 0;
    p.meta_tiled = tiled;
    p.tiles_r = tiles_r;
    p.tiles_c = ceil_div(N, bn);
    p.k_blocks = ceil_div(K, 128);
    p.status = dev->status;
    p.sparse_rows = M;
    const int num_tiles = p.tiles_r * p.tiles_c;
    const int grid = num_tiles < dev->sm_count ? num_tiles : dev->sm_count;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    return bn == 256 ? launch_hsparse<256>(map_s, map_d, p, grid, stream) : launch_hsparse<128>(map_s, map_d, p, grid, stream);
}

int bm_igemm_sparse_i32(const int8_t* A_comp, const void* meta, int meta_format, const int8_t* B, int32_t* C, int M,
                        int N, int K, int64_t ldc, int b_layout, void* stream) {
    if (!meta) return fail_msg(BM_ERR_NULL, "metadata pointer is NULL");
    if (M <= 0 || K <= 0 || K % 32 != 0) return fail_msg(BM_ERR_SHAPE, "K must be a positive multiple of 32");
    if (b_layout != BM_B_KN && b_layout != BM_B_NK) return fail_msg(BM_ERR_LAYOUT, "unknown B layout tag");
    const uint8_t* tiled = nullptr;
    if (int rc = resolve_meta(meta, meta_format, M, K, stream, &tiled)) return rc;
    return sparse_gemm(0, EPI_I32, A_comp, tiled, B, C, M, N, K, ldc, b_layout, 1.f, nullptr, nullptr, stream);
}

int bm_w8a8_sparse_i32(const int8_t* X, const int8_t* W_comp, const void* W_meta_tiled, int32_t* C, int M, int N, int K,
                       int64_t ldc, void* stream) {
    return sparse_gemm(1, EPI_I32, W_comp, static_cast<const uint8_t*>(W_meta_tiled), X, C, N, M, K, ldc, BM_B_NK, 1.f,
                       nullptr, nullptr, stream);
}

int bm_w8a8_sparse_f16(const int8_t* X, const int8_t* W_comp, const void* W_meta_tiled, uint16_t* D, const float* sa_m,
                       const float* sw_n, int M, int N, int K, int64_t ldd, void* stream) {
    return sparse_gemm(1, EPI_F16_ROWCOL, W_comp, static_cast<const uint8_t*>(W_meta_tiled), X, D, N, M, K, ldd,
                       BM_B_NK, 1.f, sa_m, sw_n, stream);
}

size_t bm_sp_packed_weight_bytes(int N, int K) {
    if (N <= 0 || K <= 0) return 0;
    return static_cast<size_t>(ceil_div(N, 128)) * 128 * ceil_div(K, kSpKLogical) * kSpPackedRowBytes;
}

int bm_sp_pack_weights(const int8_t* W_comp, const void* W_meta, int meta_format, void* W_packed, int N, int K,
                       void* stream_v) {
    if (!W_comp || !W_meta || !W_packed) return fail_msg(BM_ERR_NULL, "pointer is NULL");
    if (N <= 0 || K <= 0 || K % 32 != 0) return fail_msg(BM_ERR_SHAPE, "K must be a positive multiple of 32");
    if (!aligned16(W_comp) || !aligned16(W_packed)) return fail_msg(BM_ERR_ALIGN, "buffers must be 16-byte aligned");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int k_blocks = ceil_div(K, kSpKLogical);
    const size_t chunks = static_cast<size_t>(ceil_div(N, 128)) * k_blocks * 1024;
    pack_comp_blocks_kernel<<<static_cast<unsigned>((chunks + 255) / 256), 256, 0, stream>>>(
        W_comp, static_cast<uint8_t*>(W_packed), N, K, k_blocks, chunks, ceil_div(N, 128) * 128);
    BM_CUDA_TRY(cudaGetLastError());
    return pack_meta(W_meta, meta_format, W_packed, N, K, stream, true);
}

int bm_w8a8_sparse_i32_packed(const int8_t* X, const void* W_packed, int32_t* C, int M, int N, int K, int64_t ldc,
                              void* stream) {
    return sparse_gemm(1, EPI_I32, nullptr, static_cast<const uint8_t*>(W_packed), X, C, N, M, K, ldc, BM_B_NK, 1.f,
                       nullptr, nullptr, stream, true);
}

int bm_w8a8_sparse_f16_packed(const int8_t* X, const void* W_packed, uint16_t* D, const float* sa_m, const float* sw_n,
                              int M, int N, int K, int64_t ldd, void* stream) {
    return sparse_gemm(1, EPI_F16_ROWCOL, nullptr, static_cast<const uint8_t*>(W_packed), X, D, N, M, K, ldd, BM_B_NK,
                       1.f, sa_m, sw_n, stream, true);
}

int bm_last_device_status(int* code) {
    if (!code) return fail_msg(BM_ERR_NULL, "code pointer is NULL");
    DeviceState* dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;
    BM_CUDA_TRY(cudaDeviceSynchronize());
    BM_CUDA_TRY(cudaMemcpy(code, dev->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (*code != 0) BM_CUDA_TRY(cudaMemset(dev->status, 0, sizeof(int)));
    // launches of the no-alloc entry point record their give-ups in a word of their own
    int fixed = 0;
    if (int rc = noalloc_read_status(&fixed)) return rc;
    if (*code == 0) *code = fixed;
    return BM_OK;
}

int bm_set_option(const char* name, int value) {
    if (!name) return fail_msg(BM_ERR_NULL, "option name is NULL");
    for (int i = 0; i < OPT_COUNT; ++i)
        if (strcmp(name, option_specs()[i].name) == 0) {
            option_values()[i].store(value, std::memory_order_relaxed);
            return BM_OK;
        }
    return fail_msg(BM_ERR_LAYOUT, "unknown option name");
}

int bm_get_option(const char* name, int* value) {
    if (!name || !value) return fail_msg(BM_ERR_NULL, "pointer is NULL");
    for (int i = 0; i < OPT_COUNT; ++i)
        if (strcmp(name, option_specs()[i].name) == 0) {
            *value = opt(i);
            return BM_OK;
        }
    return fail_msg(BM_ERR_LAYOUT, "unknown option name");
}

int bm_tensor_map_cache_stats(uint64_t* hits, uint64_t* misses, uint64_t* entries) {
    MapCache& c = map_cache();
    std::lock_guard<std::mutex> lock(c.mutex);
    if (hits) *hits = c.hits.load();
    if (misses) *misses = c.misses.load();
    if (entries) *entries = c.maps.size();
    return BM_OK;
}

int bm_selftest_bounded_wait(unsigned limit_us, int* outcome) {
    if (!outcome) return fail_msg(BM_ERR_NULL, "outcome pointer is NULL");
    if (limit_us == 0 || limit_us > 2000000u) return fail_msg(BM_ERR_SHAPE, "limit must be 1 us .. 2 s");
    DeviceState* dev = nullptr;
    if (int rc = current_device_state(&dev)) return rc;
    int* d_ret = nullptr;
    BM_CUDA_TRY(cudaMalloc(&d_ret, sizeof(int)));
    BM_CUDA_TRY(cudaMemset(d_ret, 0, sizeof(int)));
    selftest_bounded_wait_kernel<<<1, 32>>>(dev->status, static_cast<unsigned long long>(limit_us) * 1000ull, d_ret);
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(outcome, d_ret, sizeof(int), cudaMemcpyDeviceToHost);
    cudaFree(d_ret);
    if (e != cudaSuccess) return fail_cuda(e, "bounded-wait self-test");
    return BM_OK;
}

const char* bm_last_error_string(void) { return error_buffer(); }

void bm_shutdown(void) {
    {
        MapCache& c = map_cache();
        std::lock_guard<std::mutex> lock(c.mutex);
        c.maps.clear();
    }
    std::lock_guard<std::mutex> lock(state_mutex());
    for (int d = 0; d < kMaxDevices; ++d) {
        DeviceState& s = device_states()[d];
        if (!s.ready) continue;
        int prev = 0;
        if (cudaGetDevice(&prev) != cudaSuccess) continue;
        if (cudaSetDevice(d) == cudaSuccess) {
            cudaFree(s.status);
            cudaFree(s.scratch);
        }
        cudaSetDevice(prev);
        s = DeviceState{};
    }
}

const char* bm_version(void) { return "0.1"; }

}  // extern "C"
