// fp64 GEMM D = alpha * (A x B) + beta * C on the double-precision tensor-core path (DMMA).
//
// Stands in for gemm_rocwmma_d of samples/perf_dgemm.cpp:461 (the perf_hgemm pipeline with
// 16x16x16 fp64 blocks).  tcgen05 has no fp64 kind, so the math is warp-level mma.sync.m16n8k8.f64:
//   CTA tile 128x128, K slab 32, 16 math warps as 4 (M) x 4 (N), warp tile 32x32.
// Two kernels feed it:
//   * gemm_f64_tma_kernel (the usual case): a 17th warp brings the slabs in with TMA into a 3-stage ring guarded by
//     full / empty mbarriers; the math warps issue no load instructions and never meet at a CTA-wide barrier, so one
//     warp's stall is covered by the others.  The operand is described to TMA as a 3-D tensor whose innermost
//     dimension is four doubles (32 bytes), so that a slab lands as [K chunk][row][4] (K-contiguous operand) or
//     [row chunk][k][4] (M / N-contiguous operand): rows of 32 bytes, which the 8-byte fragment reads of a half-warp
//     (4 rows x 4 k positions) hit without bank conflicts - a 128-byte swizzle leaves them two-way conflicted.
//   * gemm_f64_kernel (ragged cases: a K-contiguous operand with k % 4 != 0 or an M / N-contiguous one with
//     m resp. n % 4 != 0, which the 3-D view cannot describe): every warp loads with cp.async into padded tiles and
//     the CTA synchronises once per slab.
// Native layouts: A row major (K contiguous), B column major (K contiguous), C / D row major.  A column-major A or a
// row-major B (M / N contiguous, the reference's other NN / NT / TN / TT cases,
// docs/api-reference/api-reference-guide.rst:169-187) is read from a slab stored the other way round, into the same
// fragments; column-major C / D is the transposed problem D^T = alpha * B^T A^T + beta * C^T with the operands
// swapped on the host.
// Measured at 4096^3 (1.96 GHz, no throttling; the DMMA pipe's own rate, from a register-only loop of the same
// instruction, is 37.1 TFLOP/s): the cp.async kernel 31.2 TFLOP/s; the same kernel with its loads removed 34.5, with
// its CTA barrier removed 34.5, with both removed 35.9 - which is what moving the loads to TMA and the
// synchronisation to per-stage mbarriers recovers.
#include "common.cuh"
#include "gemm_tc05_common.cuh" // tensor-map encoder entry point
#include "ptx_sm100.cuh"
#include "tuning.cuh"

namespace b200wmma
{
    namespace f64
    {
        constexpr int BM = 128, BN = 128;
        template <int BK, int STAGES>
        struct Cfg
        {
            static constexpr int PITCH       = BK + 4; // doubles per shared row: pad -> conflict-free 8-byte reads
            static constexpr int PITCH_MN    = BM + 4; // the transposed tile of an M / N-contiguous operand: [k][m]
            // a tile holds 128 x BK values either as 128 rows of PITCH or as BK rows of PITCH_MN
            static constexpr int TILE_ELEMS  = (BM * PITCH > BK * PITCH_MN) ? BM * PITCH : BK * PITCH_MN;
            static constexpr int STAGE_ELEMS = 2 * TILE_ELEMS;
            static constexpr size_t SMEM_BYTES = static_cast<size_t>(STAGES) * STAGE_ELEMS * sizeof(double);
        };

        // 16-byte async copy of which the first `bytes` (16, 8 or 0) come from src; the rest is zero-filled
        __device__ __forceinline__ void cp_async16_zfill(double* dst, const double* src, int bytes)
        {
            const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes)
                         : "memory");
        }
        __device__ __forceinline__ void cp_async_commit()
        {
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        template <int N>
        __device__ __forceinline__ void cp_async_wait()
        {
            asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
        }
        // D(16x8) += A(16x8) x B(8x8): a[2c + h] = A[g + 8h][4c + t], b[c] = B[4c + t][g]
        __device__ __forceinline__ void dmma_1688(double (&c)[4], const double (&a)[4], const double (&b)[2])
        {
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 "
                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+d"(c[0]), "+d"(c[1]), "+d"(c[2]), "+d"(c[3])
                         : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(b[0]), "d"(b[1]));
        }
        // Loads one 128 x 16 K-major slab (rows `row0..row0+127` of a matrix with `rows` rows and
        // pitch ld, K columns k0..k0+15) into shared memory; out-of-range chunks become zeros.
        template <int BK, int THREADS>
        __device__ __forceinline__ void load_slab(double* dst, const double* src, size_t ld, uint32_t rows,
                                                  uint32_t kdim, uint32_t row0, uint32_t k0)
        {
            constexpr int PITCH = BK + 4, CH = BK / 2; // chunks of 2 doubles per row
            // 128 rows x CH chunks / 256 threads
#pragma unroll
            for(int i = 0; i < 128 * CH / THREADS; ++i)
            {
                const uint32_t idx = threadIdx.x + i * THREADS;
                const uint32_t r = idx / CH, ch = idx % CH;
                const uint32_t gr = row0 + r, gk = k0 + ch * 2;
                const bool     ok = gr < rows && gk < kdim; // kdim is even: a chunk is all in or out
                const double*  s  = ok ? src + static_cast<size_t>(gr) * ld + gk : src;
                cp_async16_zfill(dst + r * PITCH + ch * 2, s, ok ? 16 : 0);
            }
        }
        // The same slab of an operand whose M / N index is the contiguous one (element (row, kk) at src[kk * ld + row]):
        // chunks of two consecutive rows at one K position land in the transposed tile dst[kk][row].
        template <int BK, int THREADS>
        __device__ __forceinline__ void load_slab_mn(double* dst, const double* src, size_t ld, uint32_t rows,
                                                     uint32_t kdim, uint32_t row0, uint32_t k0)
        {
            constexpr int PITCH_MN = BM + 4, CH = BM / 2; // chunks of 2 rows per K position
#pragma unroll
            for(int i = 0; i < BK * CH / THREADS; ++i)
            {
                const uint32_t idx = threadIdx.x + i * THREADS;
                const uint32_t kk = idx / CH, ch = idx % CH;
                const uint32_t gk = k0 + kk, gr = row0 + ch * 2;
                const int      bytes = (gk < kdim && gr < rows) ? (gr + 1 < rows ? 16 : 8) : 0;
                const double*  s     = bytes ? src + static_cast<size_t>(gk) * ld + gr : src;
                cp_async16_zfill(dst + kk * PITCH_MN + ch * 2, s, bytes);
            }
        }

        template <int BK, int STAGES, int WARPS_M, int WARPS_N, bool A_MN, bool B_MN>
        __global__ void __launch_bounds__(32 * WARPS_M * WARPS_N, 1)
            gemm_f64_kernel(uint32_t m, uint32_t n, uint32_t k, const double* __restrict__ a,
                            const double* __restrict__ b, const double* __restrict__ c,
                            double* __restrict__ d, size_t lda, size_t ldb, size_t ldc, size_t ldd,
                            double alpha, double beta, int vec_ok)
        {
            constexpr int THREADS = 32 * WARPS_M * WARPS_N, WM = BM / WARPS_M, WN = BN / WARPS_N, MI = WM / 16, NJ = WN / 8;
            constexpr int PITCH = Cfg<BK, STAGES>::PITCH, PITCH_MN = Cfg<BK, STAGES>::PITCH_MN,
                          TILE_ELEMS = Cfg<BK, STAGES>::TILE_ELEMS, STAGE_ELEMS = Cfg<BK, STAGES>::STAGE_ELEMS;
            extern __shared__ __align__(16) uint8_t smem_raw[];
            double*        smem = reinterpret_cast<double*>(smem_raw);
            const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            const uint32_t g = lane >> 2, t = lane & 3;
            const uint32_t wm = warp / WARPS_N, wn = warp % WARPS_N;
            const uint32_t row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
            const uint32_t num_kb = (k + BK - 1) / BK;
            const auto     row0_of = [](uint32_t block) { return block * static_cast<uint32_t>(BM); }; // BM == BN
            const auto load_a = [&](double* dst, uint32_t k0) {
                if constexpr(A_MN)
                    load_slab_mn<BK, THREADS>(dst, a, lda, m, k, row0_of(blockIdx.y), k0);
                else
                    load_slab<BK, THREADS>(dst, a, lda, m, k, row0_of(blockIdx.y), k0);
            };
            const auto load_b = [&](double* dst, uint32_t k0) {
                if constexpr(B_MN)
                    load_slab_mn<BK, THREADS>(dst, b, ldb, n, k, row0_of(blockIdx.x), k0);
                else
                    load_slab<BK, THREADS>(dst, b, ldb, n, k, row0_of(blockIdx.x), k0);
            };

            double acc[MI][NJ][4]; // [m16 tile][n8 tile][c0..c3]
#pragma unroll
            for(int i = 0; i < MI; ++i)
#pragma unroll
                for(int j = 0; j < NJ; ++j)
#pragma unroll
                    for(int e = 0; e < 4; ++e)
                        acc[i][j][e] = 0.0;

            // prologue: STAGES-1 slabs in flight
#pragma unroll
            for(int s = 0; s < STAGES - 1; ++s)
            {
                if(static_cast<uint32_t>(s) < num_kb)
                {
                    load_a(smem + s * STAGE_ELEMS, s * BK);
                    load_b(smem + s * STAGE_ELEMS + TILE_ELEMS, s * BK);
                }
                cp_async_commit();
            }

            for(uint32_t kb = 0; kb < num_kb; ++kb)
            {
                cp_async_wait<STAGES - 2>();
                __syncthreads(); // slab kb visible to all; slab kb-1's buffer is free again
                {
                    const uint32_t nxt = kb + STAGES - 1;
                    if(nxt < num_kb)
                    {
                        double* st = smem + (nxt % STAGES) * STAGE_ELEMS;
                        load_a(st, nxt * BK);
                        load_b(st + TILE_ELEMS, nxt * BK);
                    }
                    cp_async_commit();
                }
                // element (r, kk) of the warp's part of the tile: K-major tile[r][kk], transposed tile[kk][r]
                const double* as = smem + (kb % STAGES) * STAGE_ELEMS + (A_MN ? wm * WM : (wm * WM) * PITCH);
                const double* bs = smem + (kb % STAGES) * STAGE_ELEMS + TILE_ELEMS + (B_MN ? wn * WN : (wn * WN) * PITCH);
                const auto a_at = [&](int r, int kk) { return A_MN ? as[kk * PITCH_MN + r] : as[r * PITCH + kk]; };
                const auto b_at = [&](int r, int kk) { return B_MN ? bs[kk * PITCH_MN + r] : bs[r * PITCH + kk]; };
                {
#pragma unroll
                    for(int ks = 0; ks < BK; ks += 8)
                    {
                        double af[MI][4], bf[NJ][2];
#pragma unroll
                        for(int i = 0; i < MI; ++i)
#pragma unroll
                            for(int q = 0; q < 4; ++q)
                                af[i][q] = a_at(i * 16 + g + 8 * (q & 1), ks + 4 * (q >> 1) + t);
#pragma unroll
                        for(int j = 0; j < NJ; ++j)
#pragma unroll
                            for(int q = 0; q < 2; ++q)
                                bf[j][q] = b_at(j * 8 + g, ks + 4 * q + t);
#pragma unroll
                        for(int i = 0; i < MI; ++i)
#pragma unroll
                            for(int j = 0; j < NJ; ++j)
                                dmma_1688(acc[i][j], af[i], bf[j]);
                    }
                }
            }
            cp_async_wait<0>();

            const bool read_c = (beta != 0.0) && c != nullptr;
#pragma unroll
            for(int i = 0; i < MI; ++i)
#pragma unroll
                for(int h = 0; h < 2; ++h)
                {
                    const uint32_t row = row0 + wm * WM + i * 16 + g + 8 * h;
                    if(row >= m)
                        continue;
#pragma unroll
                    for(int j = 0; j < NJ; ++j)
                    {
                        const uint32_t col = col0 + wn * WN + j * 8 + 2 * t;
                        if(col >= n)
                            continue;
                        const double v0 = acc[i][j][2 * h], v1 = acc[i][j][2 * h + 1];
                        double*       dp = d + static_cast<size_t>(row) * ldd + col;
                        const double* cp = c + static_cast<size_t>(row) * ldc + col;
                        if(vec_ok && col + 1 < n)
                        {
                            double2 cv = make_double2(0.0, 0.0);
                            if(read_c)
                                cv = *reinterpret_cast<const double2*>(cp);
                            *reinterpret_cast<double2*>(dp)
                                = make_double2(alpha * v0 + beta * cv.x, alpha * v1 + beta * cv.y);
                        }
                        else
                        {
                            dp[0] = alpha * v0 + beta * (read_c ? cp[0] : 0.0);
                            if(col + 1 < n)
                                dp[1] = alpha * v1 + beta * (read_c ? cp[1] : 0.0);
                        }
                    }
                }
        }

        // ---------------------------------- TMA-fed kernel ---------------------------------------
        constexpr int      T_BK = 32, T_STAGES = 3, T_MATH_WARPS = 16, T_THREADS = 32 * (T_MATH_WARPS + 1);
        constexpr uint32_t T_TILE_BYTES  = BM * T_BK * sizeof(double); // 32 KiB per operand per stage
        constexpr uint32_t T_STAGE_BYTES = 2 * T_TILE_BYTES;
        constexpr uint32_t T_SMEM_BYTES  = 128 + T_STAGES * T_STAGE_BYTES + 64;
        constexpr uint64_t T_WAIT_NS     = 2000000000ull;

        // Offset (in doubles) of element (r, kk) of a 128 x 32 slab: K-contiguous operand [kk / 4][r][kk % 4],
        // M / N-contiguous operand [r / 4][kk][r % 4].
        template <bool MN>
        __device__ __forceinline__ uint32_t slab_off(uint32_t r, uint32_t kk)
        {
            return MN ? (((r >> 2) * T_BK + kk) << 2) + (r & 3u) : ((((kk >> 2) * BM) + r) << 2) + (kk & 3u);
        }

        template <bool A_MN, bool B_MN>
        __global__ void __launch_bounds__(T_THREADS, 1)
            gemm_f64_tma_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                uint32_t m, uint32_t n, uint32_t k, const double* __restrict__ c, double* __restrict__ d,
                                size_t ldc, size_t ldd, double alpha, double beta, int vec_ok, unsigned* status)
        {
            constexpr int WARPS_N = 4, WM = 32, WN = 32, MI = WM / 16, NJ = WN / 8;
            extern __shared__ uint8_t smem_raw[];
            const uint32_t raw  = ptx::smem_u32(smem_raw);
            const uint32_t base = (raw + 127u) & ~127u;
            uint8_t*       smem = smem_raw + (base - raw);
            const uint32_t bar_off = T_STAGES * T_STAGE_BYTES; // full[s] at +8s, empty[s] at +32+8s, abort flag at +56
            volatile uint32_t* cta_abort = reinterpret_cast<volatile uint32_t*>(smem + bar_off + 56);
            const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            const uint32_t row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
            const uint32_t num_kb = (k + T_BK - 1) / T_BK;

            if(threadIdx.x == 0)
            {
                *cta_abort = 0u;
                for(uint32_t s = 0; s < T_STAGES; ++s)
                {
                    ptx::mbar_init(base + bar_off + 8u * s, 1);
                    ptx::mbar_init(base + bar_off + 32u + 8u * s, T_MATH_WARPS);
                }
                ptx::fence_barrier_init();
            }
            __syncthreads();

            if(warp == T_MATH_WARPS)
            {
                // ---- loader: one lane, one TMA box per operand per slab ----
                if(lane == 0)
                {
                    for(uint32_t kb = 0; kb < num_kb; ++kb)
                    {
                        const uint32_t s = kb % T_STAGES;
                        if(kb >= T_STAGES
                           && !ptx::mbar_wait_bounded(base + bar_off + 32u + 8u * s, ((kb / T_STAGES) - 1u) & 1u, cta_abort,
                                                      status, (5u << 28) | blockIdx.x, T_WAIT_NS))
                            break;
                        const uint32_t full = base + bar_off + 8u * s;
                        ptx::mbar_arrive_expect_tx(full, T_STAGE_BYTES);
                        const uint32_t dst = base + s * T_STAGE_BYTES;
                        if constexpr(A_MN)
                            ptx::tma_load_3d(dst, &tmap_a, 0, static_cast<int32_t>(kb * T_BK), static_cast<int32_t>(row0 >> 2), full);
                        else
                            ptx::tma_load_3d(dst, &tmap_a, 0, static_cast<int32_t>(row0), static_cast<int32_t>(kb * (T_BK / 4)), full);
                        if constexpr(B_MN)
                            ptx::tma_load_3d(dst + T_TILE_BYTES, &tmap_b, 0, static_cast<int32_t>(kb * T_BK),
                                             static_cast<int32_t>(col0 >> 2), full);
                        else
                            ptx::tma_load_3d(dst + T_TILE_BYTES, &tmap_b, 0, static_cast<int32_t>(col0),
                                             static_cast<int32_t>(kb * (T_BK / 4)), full);
                    }
                }
            }
            else
            {
                // ---- math warps ----
                const uint32_t g = lane >> 2, t = lane & 3;
                const uint32_t wm = warp / WARPS_N, wn = warp % WARPS_N;
                double         acc[MI][NJ][4];
#pragma unroll
                for(int i = 0; i < MI; ++i)
#pragma unroll
                    for(int j = 0; j < NJ; ++j)
#pragma unroll
                        for(int e = 0; e < 4; ++e)
                            acc[i][j][e] = 0.0;
                bool alive = true;
                for(uint32_t kb = 0; kb < num_kb; ++kb)
                {
                    const uint32_t s = kb % T_STAGES;
                    const bool     ok = ptx::mbar_wait_bounded(base + bar_off + 8u * s, (kb / T_STAGES) & 1u, cta_abort, status,
                                                               (6u << 28) | blockIdx.x, T_WAIT_NS);
                    if(!__all_sync(0xFFFFFFFFu, ok))
                    {
                        alive = false;
                        break;
                    }
                    const double* as = reinterpret_cast<const double*>(smem + s * T_STAGE_BYTES);
                    const double* bs = reinterpret_cast<const double*>(smem + s * T_STAGE_BYTES + T_TILE_BYTES);
#pragma unroll
                    for(int ks = 0; ks < T_BK; ks += 8)
                    {
                        double af[MI][4], bf[NJ][2];
#pragma unroll
                        for(int i = 0; i < MI; ++i)
#pragma unroll
                            for(int q = 0; q < 4; ++q)
                                af[i][q] = as[slab_off<A_MN>(wm * WM + i * 16 + g + 8 * (q & 1), ks + 4 * (q >> 1) + t)];
#pragma unroll
                        for(int j = 0; j < NJ; ++j)
#pragma unroll
                            for(int q = 0; q < 2; ++q)
                                bf[j][q] = bs[slab_off<B_MN>(wn * WN + j * 8 + g, ks + 4 * q + t)];
#pragma unroll
                        for(int i = 0; i < MI; ++i)
#pragma unroll
                            for(int j = 0; j < NJ; ++j)
                                dmma_1688(acc[i][j], af[i], bf[j]);
                    }
                    __syncwarp(); // every lane has read the stage
                    if(lane == 0)
                        ptx::mbar_arrive(base + bar_off + 32u + 8u * s);
                }
                if(alive)
                {
                    const bool read_c = (beta != 0.0) && c != nullptr;
#pragma unroll
                    for(int i = 0; i < MI; ++i)
#pragma unroll
                        for(int h = 0; h < 2; ++h)
                        {
                            const uint32_t row = row0 + wm * WM + i * 16 + g + 8 * h;
                            if(row >= m)
                                continue;
#pragma unroll
                            for(int j = 0; j < NJ; ++j)
                            {
                                const uint32_t col = col0 + wn * WN + j * 8 + 2 * t;
                                if(col >= n)
                                    continue;
                                const double  v0 = acc[i][j][2 * h], v1 = acc[i][j][2 * h + 1];
                                double*       dp = d + static_cast<size_t>(row) * ldd + col;
                                const double* cp = c + static_cast<size_t>(row) * ldc + col;
                                if(vec_ok && col + 1 < n)
                                {
                                    double2 cv = make_double2(0.0, 0.0);
                                    if(read_c)
                                        cv = *reinterpret_cast<const double2*>(cp);
                                    *reinterpret_cast<double2*>(dp)
                                        = make_double2(alpha * v0 + beta * cv.x, alpha * v1 + beta * cv.y);
                                }
                                else
                                {
                                    dp[0] = alpha * v0 + beta * (read_c ? cp[0] : 0.0);
                                    if(col + 1 < n)
                                        dp[1] = alpha * v1 + beta * (read_c ? cp[1] : 0.0);
                                }
                            }
                        }
                }
            }
            __syncthreads();
            if(*cta_abort)
            {
                // a wait was abandoned: give copies still in flight a bounded time to land before this CTA's shared
                // memory is released
                const uint64_t t0 = ptx::globaltimer_ns();
                while(ptx::globaltimer_ns() - t0 < 2000000ull)
                    __nanosleep(1000);
            }
        }
    } // namespace f64
} // namespace b200wmma

namespace b200wmma
{
    namespace f64
    {
        // 3-D view of an operand (rows x k, pitch ld) for the TMA-fed kernel, innermost dimension four doubles:
        // K contiguous:      {4, rows, k / 4},  strides {ld, 4} doubles,  box {4, 128, 8}  -> slab [k chunk][row][4]
        // M / N contiguous:  {4, k, rows / 4},  strides {ld, 4} doubles,  box {4, 32, 32}  -> slab [row chunk][k][4]
        // Out-of-range rows, K positions and chunks read as zeros.  False when the encoder refuses the view.
        static bool operand_tmap(CUtensorMap* out, const double* ptr, uint32_t rows, uint32_t k, uint32_t ld, bool mn)
        {
            tc05::EncodeTiledFn fn = tc05::get_encode_fn();
            if(fn == nullptr)
                return false;
            cuuint64_t gdim[3]    = {4, mn ? k : rows, (mn ? rows : k) / 4};
            cuuint64_t gstride[2] = {static_cast<cuuint64_t>(ld) * sizeof(double), 4 * sizeof(double)};
            cuuint32_t box[3]     = {4, mn ? static_cast<cuuint32_t>(T_BK) : static_cast<cuuint32_t>(BM),
                                 mn ? static_cast<cuuint32_t>(BM / 4) : static_cast<cuuint32_t>(T_BK / 4)};
            cuuint32_t estr[3]    = {1, 1, 1};
            return fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 3, const_cast<double*>(ptr), gdim, gstride, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                   == CUDA_SUCCESS;
        }

        // A is m x k with element (i, h) at a[i * lda + h] (a_mn false) or a[h * lda + i] (a_mn true); B likewise as
        // n x k; C / D row major.
        static int launch(uint32_t m, uint32_t n, uint32_t k, const double* a, const double* b, const double* c, double* d,
                          uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, double alpha, double beta, bool a_mn,
                          bool b_mn, cudaStream_t stream)
        {
            B200_REQUIRE(lda >= (a_mn ? m : k) && ldb >= (b_mn ? n : k) && ldd >= n && (!c || ldc >= n),
                         B200WMMA_ERR_INVALID_ARG, "gemm_f64: leading dimension smaller than the row/column it strides");
            B200_REQUIRE(lda % 2 == 0 && ldb % 2 == 0 && aligned16(a) && aligned16(b) && (a_mn || k % 2 == 0)
                             && (b_mn || k % 2 == 0),
                         B200WMMA_ERR_ALIGNMENT,
                         "gemm_f64: lda, ldb (and k, for an operand stored with K contiguous) must be even and A, B 16-byte "
                         "aligned (16-byte async copies)");
            if(int e = require_sm100())
                return e;
            const int vec_ok = aligned16(d) && ldd % 2 == 0 && (!c || (aligned16(c) && ldc % 2 == 0));
            dim3      grid(ceil_div(n, BN), ceil_div(m, BM));
            // The TMA-fed kernel needs the operands' 3-D views: whole groups of four along the contiguous index.
            const int which = tuning::get(tuning::GEMM_F64_KERNEL);
            if(which != 1 && (a_mn ? m % 4 == 0 : k % 4 == 0) && (b_mn ? n % 4 == 0 : k % 4 == 0))
            {
                CUtensorMap tm_a, tm_b;
                if(operand_tmap(&tm_a, a, m, k, lda, a_mn) && operand_tmap(&tm_b, b, n, k, ldb, b_mn))
                {
                    unsigned* status = nullptr;
                    if(int e = status_word_ptr(&status))
                        return e;
                    using KernT = decltype(&gemm_f64_tma_kernel<false, false>);
                    const KernT kerns[4] = {gemm_f64_tma_kernel<false, false>, gemm_f64_tma_kernel<false, true>,
                                            gemm_f64_tma_kernel<true, false>, gemm_f64_tma_kernel<true, true>};
                    const int   id       = (a_mn ? 2 : 0) + (b_mn ? 1 : 0);
                    static bool attr_ok_dev[4][MAX_DEVICES];
                    bool&       attr_ok = attr_ok_dev[id][current_device_slot()];
                    if(!attr_ok)
                    {
                        B200_CHECK_CUDA(cudaFuncSetAttribute(kerns[id], cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                             static_cast<int>(T_SMEM_BYTES)));
                        attr_ok = true;
                    }
                    kerns[id]<<<grid, T_THREADS, T_SMEM_BYTES, stream>>>(tm_a, tm_b, m, n, k, c, d, ldc, ldd, alpha, beta, vec_ok,
                                                                         status);
                    B200_CHECK_CUDA(cudaGetLastError());
                    return B200WMMA_OK;
                }
            }
            B200_REQUIRE(which != 2, B200WMMA_ERR_UNSUPPORTED,
                         "gemm_f64: the TMA-fed kernel was asked for, but these operands have no 3-D view (contiguous extent "
                         "not a multiple of 4, or the tensor-map encoder refused it)");
            constexpr int BK = 32, STAGES = 3, WARPS_M = 4, WARPS_N = 4;
            using KernT = decltype(&gemm_f64_kernel<BK, STAGES, WARPS_M, WARPS_N, false, false>);
            const KernT kerns[4] = {gemm_f64_kernel<BK, STAGES, WARPS_M, WARPS_N, false, false>,
                                    gemm_f64_kernel<BK, STAGES, WARPS_M, WARPS_N, false, true>,
                                    gemm_f64_kernel<BK, STAGES, WARPS_M, WARPS_N, true, false>,
                                    gemm_f64_kernel<BK, STAGES, WARPS_M, WARPS_N, true, true>};
            const int   id   = (a_mn ? 2 : 0) + (b_mn ? 1 : 0);
            KernT       kern = kerns[id];
            static bool attr_ok_dev[4][MAX_DEVICES];
            bool&       attr_ok = attr_ok_dev[id][current_device_slot()];
            if(!attr_ok)
            {
                B200_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     static_cast<int>(Cfg<BK, STAGES>::SMEM_BYTES)));
                attr_ok = true;
            }
            kern<<<grid, 32 * WARPS_M * WARPS_N, Cfg<BK, STAGES>::SMEM_BYTES, stream>>>(m, n, k, a, b, c, d, lda, ldb, ldc, ldd,
                                                                                      alpha, beta, vec_ok);
            B200_CHECK_CUDA(cudaGetLastError());
            return B200WMMA_OK;
        }
    } // namespace f64
} // namespace b200wmma

extern "C" int b200wmma_gemm_f64(uint32_t m, uint32_t n, uint32_t k, const double* a, const double* b,
                                 const double* c, double* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                                 uint32_t ldd, double alpha, double beta, int layout_a, int layout_b,
                                 int layout_cd, void* stream)
{
    using namespace b200wmma;
    clear_error();
    B200_REQUIRE((layout_a == 0 || layout_a == 1) && (layout_b == 0 || layout_b == 1)
                     && (layout_cd == 0 || layout_cd == 1),
                 B200WMMA_ERR_INVALID_ARG, "gemm_f64: layout flags must be 0 (row) or 1 (col)");
    B200_REQUIRE(m && n && k, B200WMMA_ERR_INVALID_ARG, "gemm_f64: m, n, k must be non-zero");
    B200_REQUIRE(a && b && d, B200WMMA_ERR_INVALID_ARG, "gemm_f64: a, b, d must be non-null");
    B200_REQUIRE(c || beta == 0.0, B200WMMA_ERR_INVALID_ARG, "gemm_f64: c may be null only when beta == 0");
    const bool a_mn = layout_a == B200WMMA_COL_MAJOR, b_mn = layout_b == B200WMMA_ROW_MAJOR;
    if(layout_cd == B200WMMA_ROW_MAJOR)
        return f64::launch(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, a_mn, b_mn, as_stream(stream));
    // column-major C / D: the transposed problem; B^T (n x k) takes A's role and is K-contiguous exactly when B was
    return f64::launch(n, m, k, b, a, c, d, ldb, lda, ldc, ldd, alpha, beta, b_mn, a_mn, as_stream(stream));
}
