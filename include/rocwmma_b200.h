/*
 * rocwmma_b200 - C ABI of the B200-native GEMM / DLRM / GEMV hot path.
 *
 * rocWMMA itself is a header-only device library: its "host entry points" are the kernel
 * signatures its samples and test harness launch.  Each entry point below replaces one of
 * those launches; the comment above it cites the reference kernel / host driver it stands in
 * for (paths relative to the rocWMMA project root).
 *
 * Conventions
 *   - Every function returns a b200wmma_status (0 = success) and never exits the process.
 *   - Unless the name ends in `_host`, all data pointers are DEVICE pointers on the CUDA
 *     device that is current in the calling thread; the caller owns every buffer.
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream).  Device-pointer
 *     entry points only enqueue work; they do not synchronise.
 *   - `_host` entry points take HOST pointers, copy through device buffers held by a
 *     b200wmma_ctx, run the same kernel and copy the result back, synchronously.
 *   - Leading dimensions are in elements.  Layout flags: 0 = row major, 1 = column major
 *     (the order of rocwmma::layout_t, library/include/rocwmma/rocwmma.hpp:104-108).
 *   - Kernels that wait on hardware barriers do so with a bounded spin; if a wait gives up
 *     the kernel records B200WMMA_ERR_DEVICE_TIMEOUT in a per-device status word that
 *     b200wmma_device_status() returns.
 */
#ifndef ROCWMMA_B200_H
#define ROCWMMA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum b200wmma_status
{
    B200WMMA_OK                 = 0,
    B200WMMA_ERR_INVALID_ARG    = 1, /* null pointer, zero/overflowing size, bad enum        */
    B200WMMA_ERR_UNSUPPORTED    = 2, /* legal request this build has no kernel for           */
    B200WMMA_ERR_ALIGNMENT      = 3, /* pointer / leading dimension breaks a 16-byte rule    */
    B200WMMA_ERR_CUDA           = 4, /* a CUDA runtime / driver call failed                  */
    B200WMMA_ERR_DEVICE_TIMEOUT = 5, /* a bounded device-side wait gave up                   */
    B200WMMA_ERR_NO_DEVICE      = 6  /* no sm_100 device is current                          */
} b200wmma_status;

enum { B200WMMA_ROW_MAJOR = 0, B200WMMA_COL_MAJOR = 1 };
enum { B200WMMA_OUT_F16 = 0, B200WMMA_OUT_F32 = 1, B200WMMA_OUT_BF16 = 2 };
enum { B200WMMA_FP8_E4M3 = 0, B200WMMA_FP8_E5M2 = 1 }; /* OCP 8-bit float formats (finite-only e4m3, IEEE-like e5m2) */

/* Human-readable text for the last error raised on the calling thread. */
const char* b200wmma_last_error_string(void);
/* Library version as major*10000 + minor*100 + patch. */
int b200wmma_version(void);

/* Overrides of the library's own kernel selection, process wide; for A/B measurements and for tests that have to reach
 * every kernel.  value 0 restores the built-in choice.  Keys:
 *   "gemm_tile_variant"  dense tcgen05 GEMM tile shape: 1 = 128x256 per SM, 2 = 256x256 per SM pair, 3 = 512x256 per pair
 *   "gemm_group_m"       rasterisation band height of that GEMM, in row tiles
 *   "sp24_force_expand"  1: b200wmma_gemm_i8_sp24 always densifies A into the workspace and runs the dense kernel
 *   "gemm_split_tail"    512x256 kernel given a workspace (b200wmma_gemm_*_ws, the host drivers): 2 = never split the last
 *                        round along K
 *   "gemm_split_fixup"   cost of that split's exchange as the planner counts it, in K slabs (0 = built-in estimate); the
 *                        split is used when slabs per pair + this < slabs of a whole tile
 *   "gemm_mma_order"     512x256 kernel, MMAs of a tile's first and last K slabs: 1 = accumulator by accumulator (so each
 *                        accumulator's drain overlaps the other's MMAs), 2 = slab by slab
 *   "dlrm_bwd_stages"    one-warp-per-sample DLRM backward kernel: depth of each warp's sample ring, 2 or 3
 *   "dlrm_bwd_warps"     ... and warps per CTA, 1..12 (clipped to what fits in shared memory)
 *   "dlrm_fwd_stages", "dlrm_fwd_warps"   the same two for the forward kernel
 *   "gemm_f64_kernel"    b200wmma_gemm_f64: 1 = the cp.async-fed kernel (the one ragged shapes always get), 2 = the TMA-fed
 *                        kernel, B200WMMA_ERR_UNSUPPORTED where it cannot run (a contiguous extent that is no multiple of 4)
 *   "gemv_rows"          row-major GEMV: 4 = four rows of A per CTA with two loads per thread in flight (the default is
 *                        one row per CTA with eight)
 *   "gemv_col_vn"        column-major GEMV: 2 or 4 = that many consecutive rows per lane (default 1)
 *   "frag_perf_slab_k"   b200wmma_perf_hgemm_fragment: K depth of one shared-memory slab, 16 (the default), 32 or 64
 *                        (used when it divides k)
 * Unknown keys and out-of-range values return B200WMMA_ERR_INVALID_ARG.  The library reads no environment variable
 * except B200WMMA_NCCL_LIBRARY (see the multi-GPU section). */
int b200wmma_set_tuning(const char* key, int value);

/* Synchronises `stream`, then reads and clears the current device's status word.
 * *out_status is B200WMMA_OK or B200WMMA_ERR_DEVICE_TIMEOUT; *out_detail (may be NULL)
 * identifies the wait that gave up (role << 24 | block index). */
int b200wmma_device_status(void* stream, int* out_status, unsigned* out_detail);

/* ------------------------------------------------------------------------------------------
 * GEMM: D = alpha * (A x B) + beta * C
 *
 * Replaces the launch of gemm_rocwmma_d (samples/perf_hgemm.cpp:515-711, launched at
 * :820-842) and of the test harness kernel type KernelFunc
 *   void(*)(m,n,k, a,b,c,d, lda,ldb,ldc,ldd, alpha,beta)
 * (test/gemm/gemm_kernel_base.hpp:102-114; gemm_PGR1_LB2_MP0_MB_CP,
 *  test/gemm/gemm_PGR1_LB2_MP0_MB_CP/device/kernel_device_func.hpp:70-283).
 * Same argument meaning; the compile-time layout / type parameters of the reference become
 * the trailing flags.  A is m x k, B is k x n, C and D are m x n.  `c` may be NULL when
 * beta == 0 (it is then not read); `c == d` is allowed.
 *
 * f16: fp16 inputs, fp32 accumulate, D/C fp16 or fp32 (out_type).  tcgen05 tensor cores.
 * i8 : int8 inputs, int32 accumulate / scalars / outputs (wrap-around arithmetic).
 * f64: fp64 everywhere (DMMA).
 * bf16 / fp8: bfloat16 resp. OCP fp8 (both operands of one format) inputs, fp32 accumulate, C/D fp32 -
 *   the reference's bfloat16_t and float8 / bfloat8 input types (docs/api-reference-guide.rst:84-143).
 * f16 / i8 / bf16 / fp8 / f64 accept every combination of row / column major A, B and C/D (C and D share one layout),
 * as the reference's NN / NT / TN / TT sweeps do.
 * A and B base pointers and leading dimensions (in bytes) must be multiples of 16 (TMA / 16-byte async copies; for
 * f64 also k even when an operand is stored with K contiguous); C / D may be unaligned (slower element-wise epilogue).
 * ------------------------------------------------------------------------------------------ */
int b200wmma_gemm_f16(uint32_t m, uint32_t n, uint32_t k,
                      const void* a, const void* b, const void* c, void* d,
                      uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                      float alpha, float beta,
                      int layout_a, int layout_b, int layout_cd, int out_type, void* stream);

int b200wmma_gemm_i8(uint32_t m, uint32_t n, uint32_t k,
                     const int8_t* a, const int8_t* b, const int32_t* c, int32_t* d,
                     uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                     int32_t alpha, int32_t beta,
                     int layout_a, int layout_b, int layout_cd, void* stream);
/* The same two GEMMs with an optional caller-owned scratch buffer of b200wmma_gemm_split_workspace_bytes() bytes (for the
 * current device; 16-byte aligned).  The kernels are persistent: a problem whose tiles do not fill a whole number of
 * rounds over the SM pairs leaves pairs idle in the last round (64 tiles on 74 pairs, say, when a GEMM is sharded over
 * 8 GPUs).  With the scratch the tiles of that last round are cut along K into equal ranges, one per pair; the partial
 * accumulators (fp32 / int32) meet in the scratch and the pair that holds a tile's last K range applies alpha / beta.
 * int8 stays bit-exact (integer addition is associative); fp16 results differ from the unsplit ones by fp32
 * summation order only.  workspace == NULL, a buffer that is too small, unaligned C / D rows, or a problem for which
 * the split would not pay give the unsplit schedule.  The library allocates nothing; calls that may overlap on
 * the GPU must not share one workspace.  No counterpart in the reference (its kernels are not persistent). */
size_t b200wmma_gemm_split_workspace_bytes(void);
int b200wmma_gemm_f16_ws(uint32_t m, uint32_t n, uint32_t k,
                         const void* a, const void* b, const void* c, void* d,
                         uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                         float alpha, float beta,
                         int layout_a, int layout_b, int layout_cd, int out_type,
                         void* workspace, size_t workspace_bytes, void* stream);
int b200wmma_gemm_i8_ws(uint32_t m, uint32_t n, uint32_t k,
                        const int8_t* a, const int8_t* b, const int32_t* c, int32_t* d,
                        uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                        int32_t alpha, int32_t beta,
                        int layout_a, int layout_b, int layout_cd,
                        void* workspace, size_t workspace_bytes, void* stream);
/* fp32 inputs and outputs with fp32-class accuracy on the tensor cores (each operand split into two TF32
 * terms, three products accumulated in fp32): the reference's fp32 GEMM samples sgemm_rocwmma_d
 * (samples/simple_sgemm.cpp) and gemm_rocwmma_d of samples/perf_sgemm.cpp.  Every combination of row / column major
 * A, B and C/D; k a multiple of 4; the rows of an operand stored with K contiguous 16-byte aligned.  `workspace`:
 * caller-owned device scratch of b200wmma_gemm_f32_workspace_bytes() bytes (the split copies of A and B, always
 * written K-contiguous, which is where the other layouts are absorbed). */
size_t b200wmma_gemm_f32_workspace_bytes(uint32_t m, uint32_t n, uint32_t k);
int b200wmma_gemm_f32(uint32_t m, uint32_t n, uint32_t k,
                      const float* a, const float* b, const float* c, float* d,
                      uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                      float alpha, float beta,
                      int layout_a, int layout_b, int layout_cd,
                      void* workspace, size_t workspace_bytes, void* stream);
int b200wmma_gemm_bf16(uint32_t m, uint32_t n, uint32_t k,
                       const void* a, const void* b, const float* c, float* d,
                       uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                       float alpha, float beta,
                       int layout_a, int layout_b, int layout_cd, void* stream);
/* The other (InputT, OutputT, ComputeT) sets of the reference's GEMM sweep (test/gemm/gemm_common_test_params.hpp:51-147):
 * bfloat16 inputs with bfloat16 C / D and fp32 compute (out_type B200WMMA_OUT_BF16; B200WMMA_OUT_F32 is
 * b200wmma_gemm_bf16), and int8 inputs with int8 C / D and int32 compute: d = int8(alpha * acc + beta * int32(c)), the
 * int32 value cast as the reference's static_cast<OutputT> does (test/reference_impl.hpp:77-78: the low 8 bits).
 * All layout combinations.  The int8-output form drains 32 or 16 bytes per access where the C / D rows are aligned
 * accordingly, byte by byte otherwise. */
int b200wmma_gemm_bf16_out(uint32_t m, uint32_t n, uint32_t k,
                           const void* a, const void* b, const void* c, void* d,
                           uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                           float alpha, float beta,
                           int layout_a, int layout_b, int layout_cd, int out_type, void* stream);
int b200wmma_gemm_i8_i8(uint32_t m, uint32_t n, uint32_t k,
                        const int8_t* a, const int8_t* b, const int8_t* c, int8_t* d,
                        uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                        int32_t alpha, int32_t beta,
                        int layout_a, int layout_b, int layout_cd, void* stream);
int b200wmma_gemm_fp8(uint32_t m, uint32_t n, uint32_t k,
                      const void* a, const void* b, const float* c, float* d,
                      uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                      float alpha, float beta,
                      int layout_a, int layout_b, int layout_cd, int fp8_format, void* stream);

/* Replaces gemm_rocwmma_d of samples/perf_dgemm.cpp:461 (same 13-argument signature). */
int b200wmma_gemm_f64(uint32_t m, uint32_t n, uint32_t k,
                      const double* a, const double* b, const double* c, double* d,
                      uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                      double alpha, double beta,
                      int layout_a, int layout_b, int layout_cd, void* stream);

/* ------------------------------------------------------------------------------------------
 * Structured-sparse and packed-int4 integer GEMM.  rocWMMA v1.6.0 has no counterpart of
 * these two (no sparse or int4 code in the project); the semantics are those of
 * b200wmma_gemm_i8 applied to the densified / sign-extended operands.
 *
 * sp24: A is 2:4 sparse along K.  a_vals is m x k/2 int8, row major (lda_vals elements per
 *   row): for each aligned group of 4 K-positions the two kept values in ascending position
 *   order.  a_meta is m x k/8 bytes, row major (ld_meta bytes per row): one nibble per group,
 *   idx0 | (idx1 << 2) with idx0 < idx1 the kept positions, two groups per byte, low nibble =
 *   even group.  B column major int8, C/D row major int32.
 * i4: A (row major, m x k) and B (column major, k x n) hold int4 values in [-8,7], two per
 *   byte along K, low nibble = even k.  lda / ldb are in BYTES per row / column; k a multiple of 32, packed rows
 *   16-byte aligned.  The nibbles are sign-extended to int8 inside the kernel (TMA brings the packed bytes to shared
 *   memory, converter warps rewrite them as the int8 tile the tensor core reads): no int8 copy of the operands ever
 *   exists in device memory, so `workspace` is not used - NULL / 0 are accepted, and
 *   b200wmma_gemm_i4_workspace_bytes() returns 0.
 * `workspace` is caller-owned device scratch of at least b200wmma_gemm_*_workspace_bytes().
 *   sp24 with k a multiple of 128 and 16-byte aligned rows (a_vals, a_meta, b and their pitches) runs
 *   on the sparse tensor cores straight from the compressed operands; the workspace is then optional
 *   (NULL / 0 allowed) and only buys a faster metadata fetch.  Every other sp24 shape needs it.
 * ------------------------------------------------------------------------------------------ */
size_t b200wmma_gemm_i8_sp24_workspace_bytes(uint32_t m, uint32_t n, uint32_t k);
int b200wmma_gemm_i8_sp24(uint32_t m, uint32_t n, uint32_t k,
                          const int8_t* a_vals, const uint8_t* a_meta,
                          const int8_t* b, const int32_t* c, int32_t* d,
                          uint32_t lda_vals, uint32_t ld_meta, uint32_t ldb,
                          uint32_t ldc, uint32_t ldd,
                          int32_t alpha, int32_t beta,
                          void* workspace, size_t workspace_bytes, void* stream);

/* The sparse tensor-core kernel fetches A's metadata fastest from a re-tiled copy (8 KiB blocks of 256 rows x
 * 256 K).  b200wmma_gemm_i8_sp24 makes that copy in its workspace on every call; when A is reused (weights),
 * make it once with b200wmma_sp24_repack_meta into a buffer of b200wmma_sp24_packed_meta_bytes(m, k) bytes and
 * call b200wmma_gemm_i8_sp24_packed, which takes that buffer instead of a_meta and needs no workspace.
 * k must be a multiple of 128; a_vals, b rows and `packed` 16-byte aligned. */
size_t b200wmma_sp24_packed_meta_bytes(uint32_t m, uint32_t k);
int b200wmma_sp24_repack_meta(uint32_t m, uint32_t k, const uint8_t* a_meta, uint32_t ld_meta,
                              void* packed, size_t packed_bytes, void* stream);
int b200wmma_gemm_i8_sp24_packed(uint32_t m, uint32_t n, uint32_t k,
                                 const int8_t* a_vals, const void* a_meta_packed,
                                 const int8_t* b, const int32_t* c, int32_t* d,
                                 uint32_t lda_vals, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                                 int32_t alpha, int32_t beta, void* stream);

/* No counterpart in the reference.  Same computation and arguments as b200wmma_gemm_i8_sp24 minus the
 * workspace: for callers that cannot provide scratch memory - code that launches through the plain
 * 13-argument GEMM kernel signature (which has no slot for a workspace), or that runs in a process whose
 * device memory is entirely owned by an arena set up elsewhere, so that neither it nor this library may
 * call the CUDA allocator.  The expanded copy of A is kept in an array of
 * B200WMMA_SP24_STATIC_SCRATCH_BYTES bytes built into the library (each GPU that loads the library holds
 * it until the process ends); the call allocates nothing.
 *   - Problems with m * k above B200WMMA_SP24_STATIC_SCRATCH_BYTES are refused with
 *     B200WMMA_ERR_UNSUPPORTED; use b200wmma_gemm_i8_sp24 for those.
 *   - The first call on each device looks up the array's device address (once, cached afterwards);
 *     make that first call before starting any stream capture (a first call on a capturing stream is
 *     refused with B200WMMA_ERR_INVALID_ARG).
 *   - The array of the device that is current in the calling thread is used; `stream` must belong to
 *     that device (checked).
 *   - All calls on a device use the same array.  Calls whose GPU work can overlap (different streams,
 *     or different host threads without ordering between them) overwrite each other's data: keep
 *     them ordered on one stream or separate them with events.  Nothing has to be cleared between
 *     calls; each call rewrites every byte it reads. */
#define B200WMMA_SP24_STATIC_SCRATCH_BYTES (16u << 20)
int b200wmma_gemm_i8_sp24_static(uint32_t m, uint32_t n, uint32_t k,
                                 const int8_t* a_vals, const uint8_t* a_meta,
                                 const int8_t* b, const int32_t* c, int32_t* d,
                                 uint32_t lda_vals, uint32_t ld_meta, uint32_t ldb,
                                 uint32_t ldc, uint32_t ldd,
                                 int32_t alpha, int32_t beta, void* stream);

size_t b200wmma_gemm_i4_workspace_bytes(uint32_t m, uint32_t n, uint32_t k);
int b200wmma_gemm_i4(uint32_t m, uint32_t n, uint32_t k,
                     const uint8_t* a_packed, const uint8_t* b_packed,
                     const int32_t* c, int32_t* d,
                     uint32_t lda_bytes, uint32_t ldb_bytes, uint32_t ldc, uint32_t ldd,
                     int32_t alpha, int32_t beta,
                     void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------
 * Naive fragment-API GEMM: one 16x16 block per warp, written against this repository's
 * <rocwmma/rocwmma.hpp>.  Replaces the launch of hgemm_rocwmma_d
 * (samples/simple_hgemm.cpp:81-139, launched at :192-230): A row major, B column major,
 * C/D row major; out_type selects fp16 (the sample's own) or fp32 C/D.
 * m, n, k must be multiples of 16.
 * ------------------------------------------------------------------------------------------ */
int b200wmma_simple_hgemm(uint32_t m, uint32_t n, uint32_t k,
                          const void* a, const void* b, const void* c, void* d,
                          uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                          float alpha, float beta, int out_type, void* stream);

/* The same naive kernel with the types of sgemm_rocwmma_d (samples/simple_sgemm.cpp:81-139: fp32 fragments,
 * computed as three TF32 mma.sync products per fp32 product) and dgemm_rocwmma_d (samples/simple_dgemm.cpp:81-139:
 * fp64 fragments, DMMA).  A row major, B column major, C/D row major; m, n, k multiples of 16. */
int b200wmma_simple_sgemm(uint32_t m, uint32_t n, uint32_t k,
                          const float* a, const float* b, const float* c, float* d,
                          uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                          float alpha, float beta, void* stream);
int b200wmma_simple_dgemm(uint32_t m, uint32_t n, uint32_t k,
                          const double* a, const double* b, const double* c, double* d,
                          uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                          double alpha, double beta, void* stream);

/* perf_hgemm's kernel source pattern (cooperative global reads, shared-memory double buffer,
 * fragment transforms; samples/perf_hgemm.cpp:515-711) compiled against this repository's
 * fragment headers: 128x128 macro tile, A column major, B row major, C/D row major fp16 -
 * the layouts the sample ships with (:264-271).  m, n multiples of 128, k of 16. */
int b200wmma_perf_hgemm_fragment(uint32_t m, uint32_t n, uint32_t k,
                                 const void* a, const void* b, const void* c, void* d,
                                 uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                                 float alpha, float beta, void* stream);

/* Measures, on the current device, the rate at which the SMs issue the warp-level tensor-core instruction the
 * fragment API's 16-bit multiplies (kind 0: mma.sync m16n8k16, fp16 inputs, fp32 accumulate) or the fp64 GEMM
 * (kind 1: mma.sync m16n8k8, fp64) are built on: every SM runs 16 warps that issue it back to back from registers.
 * *tflops receives the rate; it is the denominator for those kernels' throughput.  Synchronises `stream`; allocates
 * and frees a small device buffer.  No reference counterpart (a measurement aid). */
int b200wmma_measure_mma_sync_rate(int kind, double* tflops, void* stream);

/* ------------------------------------------------------------------------------------------
 * DLRM dot interaction.
 *
 * Forward replaces dlrmDotFwd (samples/simple_dlrm.cpp:184-284, launched :503-530;
 * test/dlrm/device/dlrm_dot_fwd.hpp:37-136):
 *   output[b] = [ input[b,0,0:k] , { Z[i][j] : 0 <= j < i < m, row-major order } ],
 *   Z = X X^T with fp32 accumulation, stored as fp16.
 * input  : batch x m_stride x k fp16 (row i of sample b at (b*m_stride + i)*k; rows m..m_stride-1
 *          are padding and are not read).
 * output : batch x out_stride fp16, out_stride >= k + m(m-1)/2; columns past the packed
 *          triangle are written as zero.
 * The reference's fp32 scratch `acc` is not needed and has no parameter.
 * Requires k a multiple of 16 and out_stride % 8 == 0.  m <= 32 with k <= 256 (the DLRM benchmark shapes)
 * runs on kernels tuned for them; anything larger (the reference test sweep's m = 128 and m = k = 1024
 * among them) on general block-tiled kernels, which need m_stride >= m rounded up to 16 (they read, and
 * discard, the padding rows of the last 16-row block) and batch <= 65535.
 *
 * Backward replaces trilReconstruct + dlrmDotBwd (samples/simple_dlrm.cpp:290-331, :349-441,
 * launched :535-584; test/dlrm/device/dlrm_dot_bwd.hpp:35-172):
 *   bottom_mlp_grad[b,:] = upstream[b,0:k]            (skipped when the pointer is NULL)
 *   T = symmetric m x m matrix rebuilt from upstream[b,k:], zero diagonal
 *   grad[b] = T x X[b]   (fp32 accumulate, stored fp16), rows 0..m-1 only.
 * With fuse_mlp_into_row0 != 0, upstream[b,0:k] is added to grad[b,0,:] in fp32 before the
 * fp16 conversion (the bottom-MLP row receives its pass-through gradient in the same pass).
 * ------------------------------------------------------------------------------------------ */
int b200wmma_dlrm_fwd(const void* input, void* output,
                      uint32_t m, uint32_t m_stride, uint32_t k, uint32_t batch,
                      uint32_t out_stride, void* stream);

int b200wmma_dlrm_bwd(const void* input, const void* upstream, void* grad, void* bottom_mlp_grad,
                      uint32_t m, uint32_t m_stride, uint32_t k, uint32_t batch,
                      uint32_t upstream_stride, int fuse_mlp_into_row0, void* stream);
/* fp32 data (the reference sweep's other data type): same contracts with 4-byte elements; always the general
 * block-tiled kernels (m_stride >= m rounded up to 16, batch <= 65535, k a multiple of 16). */
int b200wmma_dlrm_fwd_f32(const float* input, float* output, uint32_t m, uint32_t m_stride, uint32_t k,
                          uint32_t batch, uint32_t out_stride, void* stream);
int b200wmma_dlrm_bwd_f32(const float* input, const float* upstream, float* grad, float* bottom_mlp_grad,
                          uint32_t m, uint32_t m_stride, uint32_t k, uint32_t batch, uint32_t upstream_stride,
                          int fuse_mlp_into_row0, void* stream);

/* ------------------------------------------------------------------------------------------
 * GEMV: y = alpha * A x + beta * y  (in place on y), A is m x n.
 * Replaces sgemv_rocwmma_d / dgemv_rocwmma_d (samples/simple_sgemv.cpp:103-155 launched
 * :198-227, samples/simple_dgemv.cpp:103) as a true matrix-vector product: x has n elements,
 * y has m elements, nothing outside them is touched.  layout_a row major (lda >= n) or
 * column major (lda >= m, the sample's own storage).
 * ------------------------------------------------------------------------------------------ */
int b200wmma_gemv_f32(uint32_t m, uint32_t n, const float* a, uint32_t lda, int layout_a,
                      const float* x, float* y, float alpha, float beta, void* stream);
int b200wmma_gemv_f64(uint32_t m, uint32_t n, const double* a, uint32_t lda, int layout_a,
                      const double* x, double* y, double alpha, double beta, void* stream);

/* ------------------------------------------------------------------------------------------
 * Host-buffer drivers.  These stand in for the reference samples' host functions
 * gemm_test (samples/perf_hgemm.cpp:713-941), dlrm_test (samples/simple_dlrm.cpp:443-710)
 * and sgemv_test (samples/simple_sgemv.cpp:157-273): allocate-or-reuse device buffers,
 * copy the inputs host -> device, launch, copy the result device -> host, synchronise.
 * A b200wmma_ctx caches the device buffers (grown on demand) and one stream, so repeated
 * calls do not allocate.  All pointers in *_host calls are host pointers; pinned host
 * memory gives the fastest copies but pageable memory works.
 * The GEMM drivers take every layout combination: with a row-major A, C and D (either layout of B) the copies and the
 * kernels are pipelined over chunks of rows; with a column-major A or C / D, whose row chunks are not contiguous, the
 * whole matrices go up, one GEMM runs and D comes back.
 * ------------------------------------------------------------------------------------------ */
typedef struct b200wmma_ctx b200wmma_ctx;
int b200wmma_ctx_create(b200wmma_ctx** out_ctx);
int b200wmma_ctx_destroy(b200wmma_ctx* ctx);
/* Device times (ms, CUDA events) of the stages of the last successful b200wmma_gemm_*_host / _host_mg call on `ctx`:
 * out_ms5[0] span of the host -> device copies, [1] exchange of A between the GPUs (sum over chunks; 0 on one GPU),
 * [2] GEMM kernels (sum), [3] device -> host copies (sum), [4] first copy in to last copy out.  The stages overlap,
 * so [0..3] do not add up to [4].  The GEMM host drivers check every argument before they queue any work; should a
 * CUDA call fail later, they drain their streams before returning, so the caller's buffers are never in use after
 * the call returns. */
int b200wmma_ctx_last_stage_ms(b200wmma_ctx* ctx, float* out_ms5);

int b200wmma_gemm_f16_host(b200wmma_ctx* ctx, uint32_t m, uint32_t n, uint32_t k,
                           const void* a, const void* b, const void* c, void* d,
                           uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                           float alpha, float beta,
                           int layout_a, int layout_b, int layout_cd, int out_type);
int b200wmma_gemm_i8_host(b200wmma_ctx* ctx, uint32_t m, uint32_t n, uint32_t k,
                          const int8_t* a, const int8_t* b, const int32_t* c, int32_t* d,
                          uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                          int32_t alpha, int32_t beta,
                          int layout_a, int layout_b, int layout_cd);
int b200wmma_dlrm_fwd_host(b200wmma_ctx* ctx, const void* input, void* output,
                           uint32_t m, uint32_t m_stride, uint32_t k, uint32_t batch,
                           uint32_t out_stride);
int b200wmma_dlrm_bwd_host(b200wmma_ctx* ctx, const void* input, const void* upstream,
                           void* grad, void* bottom_mlp_grad,
                           uint32_t m, uint32_t m_stride, uint32_t k, uint32_t batch,
                           uint32_t upstream_stride, int fuse_mlp_into_row0);
int b200wmma_gemv_f32_host(b200wmma_ctx* ctx, uint32_t m, uint32_t n, const float* a,
                           uint32_t lda, int layout_a, const float* x, float* y,
                           float alpha, float beta);
int b200wmma_gemv_f64_host(b200wmma_ctx* ctx, uint32_t m, uint32_t n, const double* a,
                           uint32_t lda, int layout_a, const double* x, double* y,
                           double alpha, double beta);

/* ------------------------------------------------------------------------------------------
 * Multi-GPU plumbing: one process per GPU.  The reference is single-GPU; its paths shard with no
 * exchange after the kernel - GEMM by blocks of N columns (B column-major and C / D are split, A is
 * needed whole by every rank), DLRM by batch, GEMV by rows of A (x is needed whole) - so the only
 * communication is one broadcast before the kernels, done here with NCCL.
 *
 * Rank 0 calls b200wmma_mg_unique_id and ships the B200WMMA_MG_ID_BYTES bytes to the other ranks by any
 * means (a file, MPI, a socket); every rank then calls b200wmma_mg_create with the device it will use
 * current.  b200wmma_mg_broadcast works in place on device memory, asynchronously on `stream`.
 * NCCL is opened at run time (the copy already loaded in the process, else libnccl.so.2; the environment variable
 * B200WMMA_NCCL_LIBRARY, read at the first of these calls, names another file).  When it cannot be opened, lacks a
 * needed symbol, or ncclGetUniqueId / ncclCommInitRank fails, these calls return B200WMMA_ERR_UNSUPPORTED with the
 * reason in b200wmma_last_error_string(); nothing else in the library depends on NCCL.  b200wmma_mg_create is
 * collective and runs one small broadcast and all-gather, so that NCCL's channel set-up is not left for the first
 * timed call.  b200wmma_mg_allgather works in place: rank r contributes the bytes_per_rank bytes at
 * buf + r * bytes_per_rank and afterwards every rank holds all nranks pieces.
 * b200wmma_shard_range gives rank `index` of `parts` its contiguous share of `total` units, which
 * must split into whole granules (e.g. 16 columns, one sample, one row).
 * ------------------------------------------------------------------------------------------ */
#define B200WMMA_MG_ID_BYTES 128
typedef struct b200wmma_mg b200wmma_mg;
int b200wmma_mg_unique_id(void* id_out);
int b200wmma_mg_create(b200wmma_mg** out_mg, const void* id, int rank, int nranks);
int b200wmma_mg_broadcast(b200wmma_mg* mg, void* buf, size_t bytes, int root, void* stream);
int b200wmma_mg_allgather(b200wmma_mg* mg, void* buf, size_t bytes_per_rank, void* stream);
int b200wmma_mg_destroy(b200wmma_mg* mg);
int b200wmma_mg_rank(const b200wmma_mg* mg); /* -1 for a null handle */
int b200wmma_mg_size(const b200wmma_mg* mg); /*  0 for a null handle */
/* b200wmma_gemm_f16_host for a column-sharded GEMM (A row-major, B column-major, C / D row-major): n, b, c, d are this
 * rank's block of columns; A is needed whole by every rank.  root >= 0: only rank `root` reads its host copy `a`
 * (ignored elsewhere) and each chunk of rows is broadcast over NCCL inside the copy / compute pipeline.  root = -1:
 * every rank holds A on the host; the rows are cut into up to four chunks, of each chunk every rank uploads one
 * equal slice, and one all-gather per chunk assembles it on every GPU (a rank moves A / nranks over PCIe).
 * Collective: every rank of `mg` makes the call with the same m, k, lda, root, on the device `mg` was created on.
 * If the call fails on one rank only, the others may be left inside a collective: destroy the handle on every rank. */
int b200wmma_gemm_f16_host_mg(b200wmma_ctx* ctx, b200wmma_mg* mg, int root, uint32_t m, uint32_t n, uint32_t k,
                              const void* a, const void* b, const void* c, void* d,
                              uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                              float alpha, float beta, int out_type);
/* the same for b200wmma_gemm_i8_host */
int b200wmma_gemm_i8_host_mg(b200wmma_ctx* ctx, b200wmma_mg* mg, int root, uint32_t m, uint32_t n, uint32_t k,
                             const int8_t* a, const int8_t* b, const int32_t* c, int32_t* d,
                             uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                             int32_t alpha, int32_t beta);
int b200wmma_shard_range(uint64_t total, uint32_t parts, uint32_t index, uint32_t granule,
                         uint64_t* begin, uint64_t* count);

#ifdef __cplusplus
}
#endif
#endif /* ROCWMMA_B200_H */
