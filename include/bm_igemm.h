/*
 * bm_igemm.h — C ABI of the B200-native INT8 GEMM hot path (libbm_igemm.so).
 *
 * This is the drop-in boundary for the quantized-GEMM kernels of pjt222/bare-metal
 * (kernels/gemm/igemm/).  The reference exposes each kernel as an `extern "C" __global__`
 * symbol that a C++ host program loads with cuModuleGetFunction and launches with
 * cuLaunchKernel (kernels/gemm/igemm/bench.cu:85-92,375-378).  Every launcher below takes the
 * SAME operand pointers, dimensions and scale arguments as the kernel symbol it replaces, in
 * the same order and with the same meaning, and adds only a trailing layout tag / stream.
 * Launch geometry, shared memory and tensor maps are the library's business.
 *
 * Conventions
 *   - all matrix pointers are DEVICE pointers owned by the caller; the library never frees
 *     or reallocates them.  Operand base addresses must be 16-byte aligned.
 *   - launches are asynchronous on `stream` (a cudaStream_t / CUstream passed as void*;
 *     NULL = the legacy default stream, as the reference benches use).
 *   - return value: 0 = launched; negative = argument rejected, nothing was launched
 *     (the reference kernels have no error channel and silently skip edge tiles,
 *     igemm_tiled.cu:98-99,162 — here every element of C is written and bad arguments are
 *     reported); the kernels never abort the process (the reference's CHECK_CU does,
 *     kernels/_common/bench.h:21-31).
 *   - plain C types only; no CUDA or torch headers are needed to bind this file.
 */
#ifndef BM_IGEMM_H
#define BM_IGEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------- */
#define BM_OK                 0
#define BM_ERR_NULL          (-1)  /* a required pointer is NULL                          */
#define BM_ERR_SHAPE         (-2)  /* non-positive or unsupported M / N / K               */
#define BM_ERR_ALIGN         (-3)  /* pointer or leading dimension not 16-byte aligned    */
#define BM_ERR_LAYOUT        (-4)  /* unknown layout / format tag                         */
#define BM_ERR_CUDA          (-5)  /* a CUDA call failed; see bm_last_error_string()      */
#define BM_ERR_TOO_LARGE     (-6)  /* exceeds a documented capacity                       */

/* ---- layout of the right-hand operand (weights) ------------------------------------- */
#define BM_B_KN 0   /* B[K x N] row-major, N contiguous — the reference ABI (igemm.cu:54)  */
#define BM_B_NK 1   /* W[N x K] row-major, K contiguous — pre-packed weights               */

/* =======================================================================================
 * Dense INT8 GEMM, int32 accumulate.  A[M x K] int8 row-major.
 * Constraints: K % 16 == 0; with BM_B_KN also N % 16 == 0 (16-byte row pitch for TMA).
 * `ldc` is the row pitch of C in ELEMENTS (>= N), so a rank can write its column slab of a
 * wider output in place; pass N for a dense C.
 * ===================================================================================== */

/* Raw accumulators: C[m][n] = sum_k A[m][k] * B[k][n] (int32).  The integer core of every
 * reference kernel (igemm.cu:52-117); the reference never stores it, the B200 workloads do. */
int bm_igemm_i8_i32(const int8_t *A, const int8_t *B, int32_t *C, int M, int N, int K,
                    int64_t ldc, int b_layout, void *stream);

/* Replaces igemm_wmma / igemm_tiled / igemm_register_blocked / igemm_pipelined /
 * igemm_pipelined_cpasync(_bk64) / igemm_8warp(_256,_256x256,_tribuf) / igemm_persistent
 * (igemm.cu:52-59 and same-signature siblings; igemm_persistent.cu:60-69 minus its tile
 * counter): C[m][n] = (float)acc * (scale_a * scale_b). */
int bm_igemm_i8_f32(const int8_t *A, const int8_t *B, float *C, int M, int N, int K,
                    float scale_a, float scale_b, int64_t ldc, int b_layout, void *stream);

/* Replaces igemm_pipelined_cpasync_perchannel (igemm_pipelined_cpasync_perchannel.cu:48-56):
 * C[m][n] = ((float)acc - (float)zero_point[n]) * scale[n]. */
int bm_igemm_i8_f32_perchannel(const int8_t *A, const int8_t *B, float *C, int M, int N, int K,
                               const float *scale_n, const int32_t *zero_point_n,
                               int64_t ldc, int b_layout, void *stream);

/* W8A8 linear of the B200 workloads (no reference counterpart; same integer core):
 * D[m][n] = half_rn((float)acc * (sa[m] * sw[n])), D is IEEE binary16 (uint16_t bits). */
int bm_w8a8_f16(const int8_t *X, const int8_t *W, uint16_t *D, const float *sa_m, const float *sw_n,
                int M, int N, int K, int64_t ldd, int w_layout, void *stream);

/* N-split W8A8 linear fused with the all-gather of its output (no reference counterpart; the
 * reference is single-GPU).  The rank computes its column slab D[:, slab] exactly as bm_w8a8_f16
 * and the epilogue stores every finished box to the `n_peers` (<= 8) destinations in `D_peers`:
 * HOST array of DEVICE pointers, each already pointing at the slab's first column inside that
 * GPU's [M x N_total] output (peer-mapped memory for the other GPUs, e.g. symmetric memory).
 * `self_index` names the entry that is this GPU's own buffer (-1: none — every destination is
 * treated as remote).  Stores to the other entries cross NVLink and are paced to the rate of
 * option "gather_gbs" (GB/s this GPU may send; 0 = unpaced): peer stores offered faster than the
 * link drains them stall the operand loads of the whole GPU.  `ldd` = N_total.  Plain TMA stores,
 * no multicast.  The caller orders the kernel against its peers (a barrier across the group after
 * the launch) before anyone reads D. */
int bm_w8a8_f16_gather(const int8_t *X, const int8_t *W, uint16_t *const *D_peers, int n_peers,
                       int self_index, const float *sa_m, const float *sw_n, int M, int N, int K,
                       int64_t ldd, int w_layout, void *stream);

/* All-gather of an fp16 column slab by plain peer stores (no reference counterpart), for N-split
 * layers whose GEMM does not gather by itself (the 2:4-sparse entry points).  The rank's slab
 * [M x n_len] already sits in its own [M x N_total] output at D_peers[self_index]; it is copied to
 * the same place in the other `n_peers - 1` outputs (peer-mapped pointers).  Local 16-byte loads,
 * paced 16-byte peer stores ("gather_gbs"); no peer loads, no multicast.  n_len % 8 == 0,
 * ldd % 8 == 0.  The caller orders it against its peers (group barrier) before anyone reads. */
int bm_gather_slab_f16(uint16_t *const *D_peers, int n_peers, int self_index, int M, int n_len,
                       int64_t ldd, void *stream);

/* Group barrier for the step after a peer-store gather (no reference counterpart).  flag_arrays[d] is GPU d's
 * array of 64 32-bit words in peer-mapped memory, all zero before the first round: words [0, n_peers) are written
 * by the peers, word 32 is GPU d's own round counter.  Every call is one round: this GPU advances its counter on
 * the device, writes the round number into word `self_index` of every other array and waits until the other GPUs
 * have written theirs here — so every GPU of the group must make the same number of calls, and a call recorded in
 * a CUDA graph stays correct when the graph is replayed.  One tiny kernel on `stream`, ordered behind the kernels
 * already enqueued there (their stores to the peers are complete and visible before the flag goes out); its wait
 * is bounded (1 s), a timeout is reported by bm_last_device_status as code 7. */
int bm_peer_barrier(uint32_t *const *flag_arrays, int n_peers, int self_index, void *stream);

/* Per-token dynamic quantisation fp16 -> int8, the step before the W8A8 GEMM.  B200 form of the
 * reference's online-quant kernels (igemm_online_quant.cu:144-150 take fp16 and quantise per K tile
 * with scale = max|x|/127); here one scale per row, arithmetic of the reference's host quantiser
 * (bench.cu:28-51): scale[m] = max|x[m][:]|/127 (1 if zero), q = clamp(roundf(x * (1/scale)), -128, 127).
 * X_f16 is IEEE binary16 bits, row-major [M x K], K % 16 == 0. */
int bm_quantize_rows_f16(const uint16_t *X_f16, int8_t *X_q, float *scale_m, int M, int K, void *stream);

/* Replaces igemm_online_quant (igemm_online_quant.cu:144-150) and its variants with the same
 * arithmetic — igemm_online_quant_inplace, igemm_online_quant_bankfree, igemm_warp_specialized
 * (col_block = 128) and igemm_online_quant_bf_128x256 (col_block = 256): FP16 operands A[M x K] and
 * B[K x N] (IEEE binary16 bits, row-major), fp32 C[M x N] = sum over K of int8-quantised products.
 * As in the reference each 128-row block of A and each col_block-column block of B gets ONE factor,
 * taken from its first 32 columns / rows of K (inv = 127 / max|x|, 1 if max is 0) and applied to all
 * of K: q = clamp(rint(x * inv), -128, 127); C = sum * ((max_a / 127) * (max_b / 127)).  The int32
 * sums are kept exactly over all of K and scaled once, where the reference adds one fp32 product per
 * 32-wide K tile (igemm_online_quant.cu:340-347): results agree to fp32 summation rounding.
 * The int8 copies and the scales live in caller-owned `workspace`
 * (>= bm_online_quant_workspace_bytes(M, N, K), 256-byte aligned).  K % 16 == 0, N % 16 == 0. */
size_t bm_online_quant_workspace_bytes(int M, int N, int K);
int bm_online_quant_gemm_f32(const uint16_t *A_f16, const uint16_t *B_f16, float *C, int M, int N, int K,
                             int col_block, void *workspace, size_t workspace_bytes, void *stream);

/* One-time weight repack B[K x N] -> W[N x K] (excluded from GEMM timing). */
int bm_pack_b_kn_to_nk(const int8_t *B_kn, int8_t *W_nk, int K, int N, void *stream);

/* =======================================================================================
 * 2:4 structured-sparse INT8 GEMM.
 *
 * The sparse operand S has R rows and logical depth K; it is stored as
 *   comp [R x K/2] int8 row-major : the two kept values of every aligned group of 4,
 *                                   lower position first (sparse_meta_int8.h:141-164);
 *   meta                          : the 2-bit positions, 4 bits per group (idx1 << 2) | idx0,
 *                                   in one of the formats below.
 * Constraints: R % 16 == 0 for the reference format; K % 32 == 0.
 * ===================================================================================== */
#define BM_META_REF   0  /* uint32 words [(R/16)(K/32)8], rows r and r+8 of a 16-row tile share
                            one word (sparse_meta_int8.h:13-31,166-175)                      */
#define BM_META_ROWS  1  /* bytes [R x K/8]: per row, byte j = groups 2j (low nibble), 2j+1  */
#define BM_META_TILED 2  /* the kernel's own order, produced by bm_sp_pack_meta             */
#define BM_META_REF_F16 3 /* FP16 sibling: uint32 words [(R/16)(K/16)8], 4 nibbles in bits 15:0
                            (kernels/gemm/hgemm_sparse/sparse_meta.h:10-30); K % 16 == 0    */
#define BM_META_ROWS_F16 4 /* BM_META_ROWS bytes, to be tiled for the FP16 kernel: tcgen05's
                            kind::f16 keeps the metadata of rows i and i+8 interleaved across
                            two lanes, so its tiled order differs from the int8 one; a tiled
                            buffer made from format 3 or 4 serves bm_hgemm_sparse_f32 only     */

/* bytes of a BM_META_TILED buffer for an R x K sparse operand */
size_t bm_sp_meta_tiled_bytes(int R, int K);

/* one-time metadata repack (device -> device) into the kernel's tiled order */
int bm_sp_pack_meta(const void *meta_in, int meta_format, void *meta_tiled, int R, int K, void *stream);

/* Replaces hgemm_sparse_tiled (kernels/gemm/hgemm_sparse/hgemm_sparse_tiled.cu:122-129) and, with
 * all-0x44444444 metadata, hgemm_sparse_naive (hgemm_sparse_naive.cu; fixed positions {0,1}):
 * FP16 2:4 GEMM, C[M x N] fp32 = A_sparse[M x K] * B[K x N], A stored as A_comp[M x K/2] fp16 (kept
 * values, lower position first) + metadata, B fp16 row-major, fp32 accumulation on
 * tcgen05.mma.sp.kind::f16.  `meta_format`: BM_META_REF_F16 (the reference's array, re-tiled into
 * library scratch on every call), BM_META_ROWS / BM_META_ROWS_F16 (K % 32 == 0), or BM_META_TILED made
 * by bm_sp_pack_meta from one of those two fp16 formats.  Operands are IEEE
 * binary16 bits.  M % 16 == 0 for the reference format, K % 16 == 0, N % 16 == 0. */
int bm_hgemm_sparse_f32(const uint16_t *A_comp, const uint16_t *B, float *C, const void *meta, int meta_format,
                        int M, int N, int K, int64_t ldc, void *stream);

/* Weight tooling: magnitude-prune a dense int8 matrix W[R x K] to 2:4 along K and compress it in one
 * pass.  Of every aligned group of 4 the two entries of largest |w| stay (ties: lower position),
 * written lower position first to W_comp[R x K/2]; positions go to W_meta_rows[R x K/8] in the
 * BM_META_ROWS format.  For a matrix that is already 2:4 without stored zeros this is exactly what
 * compress_2_4_int8 produces (sparse_meta_int8.h:116-178), which finds the kept entries by
 * "value != 0"; the reference has no pruner.  K % 32 == 0. */
int bm_prune_2_4_i8(const int8_t *W, int8_t *W_comp, uint8_t *W_meta_rows, int R, int K, void *stream);

/* Replaces igemm_sparse_tiled (igemm_sparse_tiled.cu:88-96; also the _ldsm, _ldsm_fused and
 * _persistent variants minus the tile counter): sparse operand on the LEFT,
 * C[M x N] = (float)(A_sparse[M x K] * B[K x N]) * (scale_a * scale_b), metadata in the
 * reference format.  The metadata is re-tiled into library-owned scratch on every call. */
int bm_igemm_sparse_f32(const int8_t *A_comp, const int8_t *B, float *C, const uint32_t *meta,
                        int M, int N, int K, float scale_a, float scale_b, void *stream);

/* No counterpart in the reference.  Same arguments and result as bm_igemm_sparse_f32, for callers
 * that must not allocate device memory (a serving loop with a fixed memory footprint, a process
 * whose pool owns the whole device, start-up-only allocation policies): the re-tiled metadata
 * lives in a fixed 2 MiB array inside the library instead of cudaMalloc'ed scratch, and the call
 * makes no CUDA allocation or free.  Limits: ceil(M/128) * ceil(K/256) * 4096 bytes <= 2 MiB
 * (M = K = 4096 fits), otherwise BM_ERR_TOO_LARGE and nothing is launched; N % 16 == 0.  All
 * calls on a device share the array: calls that overlap on the GPU race, so keep them on one
 * stream or order them.
 * First call on a device: it resolves the array's device address, and — under the CUDA runtime's
 * default lazy module loading — it is also the moment the runtime loads this library's device
 * image there, which reserves the 2 MiB array and the kernel code.  Make that call with the device
 * current, outside stream capture, and BEFORE a pool claims the rest of the device's memory (or
 * run with CUDA_MODULE_LOADING=EAGER, which moves the reservation to context creation).
 * A bounded wait that gives up inside one of its launches is recorded in a status word of its
 * own: read it with bm_noalloc_last_device_status. */
int bm_igemm_sparse_f32_noalloc(const int8_t *A_comp, const int8_t *B, float *C, const uint32_t *meta,
                                int M, int N, int K, float scale_a, float scale_b, void *stream);
/* No counterpart in the reference.  Reads (and clears) the status word of the no-alloc entry
 * point on the current device without allocating anything: *code 0 = no launch gave up, or the
 * entry point has not been used on this device.  Synchronises the device.
 * bm_last_device_status reports the same word, but its first use creates the library's regular
 * per-device state with a 4-byte cudaMalloc — callers that may not allocate use this one. */
int bm_noalloc_last_device_status(int *code);
/* Failure-detection self-test of that status channel (no allocation): a one-CTA kernel waits, with
 * a limit of `limit_us`, on a barrier nothing signals and records the give-up in the no-alloc
 * status word.  *outcome = 2 when the wait gave up cleanly; bm_noalloc_last_device_status then
 * returns code 5 once.  The device context stays usable. */
int bm_noalloc_selftest_bounded_wait(unsigned limit_us, int *outcome);

/* Sparse-left, int32 out, any metadata format, either layout of the dense operand. */
int bm_igemm_sparse_i32(const int8_t *A_comp, const void *meta, int meta_format, const int8_t *B,
                        int32_t *C, int M, int N, int K, int64_t ldc, int b_layout, void *stream);

/* Sparse WEIGHTS (the B200 workloads): W_sparse[N x K] compressed along K, X[M x K] dense.
 * C[m][n] = sum_k X[m][k] * W[n][k].  Metadata must be BM_META_TILED. */
int bm_w8a8_sparse_i32(const int8_t *X, const int8_t *W_comp, const void *W_meta_tiled, int32_t *C,
                       int M, int N, int K, int64_t ldc, void *stream);
int bm_w8a8_sparse_f16(const int8_t *X, const int8_t *W_comp, const void *W_meta_tiled, uint16_t *D,
                       const float *sa_m, const float *sw_n, int M, int N, int K, int64_t ldd,
                       void *stream);

/* Packed sparse weights: per 256-wide K block one slice of (N padded to 128) x 160 bytes — the kept
 * values of every row (128 B per row, already in the shared-memory order of the kernel), then the
 * metadata of every row in 8-row groups — so a decode-shaped GEMM fetches ANY range of rows that
 * starts on a multiple of 8 with two linear copies per K block (values, metadata).  An opaque
 * library format: only bm_sp_pack_weights writes it, only the _packed entry points read it.
 * One-time repack (no reference counterpart; the reference only compresses, sparse_meta_int8.h:116). */
size_t bm_sp_packed_weight_bytes(int N, int K);
int bm_sp_pack_weights(const int8_t *W_comp, const void *W_meta, int meta_format, void *W_packed,
                       int N, int K, void *stream);
int bm_w8a8_sparse_i32_packed(const int8_t *X, const void *W_packed, int32_t *C, int M, int N, int K,
                              int64_t ldc, void *stream);
int bm_w8a8_sparse_f16_packed(const int8_t *X, const void *W_packed, uint16_t *D, const float *sa_m,
                              const float *sw_n, int M, int N, int K, int64_t ldd, void *stream);

/* =======================================================================================
 * Library state
 * ===================================================================================== */
/* Reads (and clears) the device status word that a bounded in-kernel wait sets when it gives
 * up: *code 0 = none.  Synchronises the whole device (every stream), so call it at checkpoints,
 * not per launch.  Also reports a give-up recorded by the no-alloc entry point. */
int bm_last_device_status(int *code);
/* Launcher options (tuning / testing switches; no reference counterpart — the reference fixes
 * launch geometry in its bench drivers, bench.cu:375-636).  Names: "force_bn" (pin the tile width;
 * 0 = choose), "dense_pair", "sparse_pair" (0 = single-CTA kernels only), "row_balanced"
 * (0 = whole 128-row tiles on the decode shapes), "tma_store" (0 = direct-store epilogue),
 * "dense_group_m", "sparse_col_first" (-1 automatic), "tail_narrow", "pdl", "gather_gbs",
 * "decode_tile_rows" (row-balanced decode tiles on packed weights: 0 = choose the ring-stage height
 * from the rows a CTA is dealt, 32 / 64 / 128 pins it).
 * Each starts from the environment variable BM_<NAME> read once at first use, else its default;
 * launchers never read the environment on the launch path.  Process-wide; set them while no
 * other thread is launching.  Unknown names return BM_ERR_LAYOUT. */
int bm_set_option(const char *name, int value);
int bm_get_option(const char *name, int *value);
/* TMA descriptors are cached by (address, shape, pitch, box): counts of lookups served from the
 * cache, descriptors encoded, and entries held.  Any pointer may be NULL. */
int bm_tensor_map_cache_stats(uint64_t *hits, uint64_t *misses, uint64_t *entries);
/* Failure-detection self-test (no reference counterpart; the reference's persistent kernels have
 * no watchdog): runs a one-CTA kernel that waits, with a limit of `limit_us`, on a barrier nothing
 * signals.  *outcome = 2 when the wait gave up cleanly; bm_last_device_status then reports the
 * recorded code (5).  The device context stays usable. */
int bm_selftest_bounded_wait(unsigned limit_us, int *outcome);
/* Text of the last host-side CUDA error seen by a launcher on this thread. */
const char *bm_last_error_string(void);
/* Frees library-owned scratch (metadata staging, split-K partial sums, status word) and empties
 * the descriptor cache. */
void bm_shutdown(void);
/* "major.minor" of this ABI. */
const char *bm_version(void);

#ifdef __cplusplus
}
#endif
#endif /* BM_IGEMM_H */
