// Dense GEMM D = alpha * (A x B) + beta * C on the 5th-generation tensor cores (tcgen05).
//
// Stands in for rocWMMA's perf_hgemm kernel gemm_rocwmma_d (samples/perf_hgemm.cpp:515-711)
// and the test-suite kernel gemm_PGR1_LB2_MP0_MB_CP
// (test/gemm/gemm_PGR1_LB2_MP0_MB_CP/device/kernel_device_func.hpp:70-283): where the
// reference prefetches one 16-wide K step through two LDS buffers and feeds per-wave MFMA
// blocks, this kernel runs a 4-stage TMA -> shared-memory ring of 128-byte-wide K slabs into
// 128x256 tcgen05.mma tiles that accumulate in tensor memory, and applies
// alpha * acc + beta * C while draining tensor memory (the reference's uniformFma, :493-513).
//
// Operand layout: A row major (m x k, K contiguous), B column major (k x n, K contiguous),
// C / D row major.  fp16 -> fp32 accumulate (C/D fp16 or fp32) and int8 -> int32.
//
// Kernel structure (persistent, one CTA per SM, 192 threads):
//   warp 0  : TMA producer (one lane)  - waits empty[s], arms full[s], issues 2 box loads
//   warp 1  : owns tensor memory; one lane issues tcgen05.mma and commits to empty[s] /
//             tmem_full[buf]
//   warp 2-5: epilogue - tcgen05.ld their 32-lane quadrant, alpha/beta, store D
// Two 256-column accumulator buffers let the epilogue of tile i overlap the MMAs of tile i+1.
// Every barrier wait is bounded (see ptx::mbar_wait_bounded).
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace b200wmma
{
    namespace tc05
    {
        constexpr uint32_t BLOCK_M       = 128;
        constexpr uint32_t BLOCK_N       = 256;
        constexpr uint32_t BLOCK_K_BYTES = 128; // one 128-byte swizzle row: 64 fp16 / 128 int8
        constexpr uint32_t STAGES        = 4;
        constexpr uint32_t A_STAGE_BYTES = BLOCK_M * BLOCK_K_BYTES; // 16 KiB
        constexpr uint32_t B_STAGE_BYTES = BLOCK_N * BLOCK_K_BYTES; // 32 KiB
        constexpr uint32_t STAGE_BYTES   = A_STAGE_BYTES + B_STAGE_BYTES;
        constexpr uint32_t NUM_THREADS   = 192;
        constexpr uint32_t TMEM_COLS     = 512; // 2 accumulator buffers x 256 fp32/int32 columns
        constexpr uint32_t GROUP_M       = 16; // tile rasterisation: 16 row tiles share B slabs
        constexpr uint32_t SMEM_BYTES    = 1024 /*alignment slack*/ + STAGES * STAGE_BYTES + 256;
        constexpr uint64_t WAIT_TIMEOUT_NS = 2000000000ull; // 2 s: far beyond any healthy wait

        enum Kind : int
        {
            KIND_F16 = 0,
            KIND_I8  = 1
        };
        enum Role : uint32_t
        {
            ROLE_PRODUCER = 1,
            ROLE_MMA      = 2,
            ROLE_EPILOGUE = 3
        };

        // tcgen05 instruction descriptor (32-bit): D format bits [4,6), A format [7,10),
        // B format [10,13), A/B major bits 15/16 (0 = K-major), N>>3 at [17,23), M>>4 at [24,29).
        template <int KIND>
        __host__ __device__ constexpr uint32_t make_idesc()
        {
            uint32_t d = 0;
            if(KIND == KIND_F16)
            {
                d |= 1u << 4; // D = F32;  A = B = F16 (format 0)
            }
            else
            {
                d |= 2u << 4; // D = S32
                d |= 1u << 7; // A = signed 8-bit
                d |= 1u << 10; // B = signed 8-bit
            }
            d |= (BLOCK_N >> 3) << 17;
            d |= (BLOCK_M >> 4) << 24;
            return d;
        }

        __device__ __forceinline__ void tile_coords(uint32_t  tile,
                                                    uint32_t  tiles_m,
                                                    uint32_t  tiles_n,
                                                    uint32_t& m_idx,
                                                    uint32_t& n_idx)
        {
            const uint32_t group_size = GROUP_M * tiles_n;
            const uint32_t group      = tile / group_size;
            const uint32_t first_m    = group * GROUP_M;
            const uint32_t gm         = min(tiles_m - first_m, GROUP_M);
            const uint32_t within     = tile - group * group_size;
            m_idx                     = first_m + within % gm;
            n_idx                     = within / gm;
        }

        // ---- epilogue element helpers -----------------------------------------------------
        __device__ __forceinline__ float epi(float acc, float c, float alpha, float beta)
        {
            return alpha * acc + beta * c;
        }
        __device__ __forceinline__ int32_t epi(int32_t acc, int32_t c, int32_t alpha, int32_t beta)
        {
            // wrap-around int32 arithmetic, as the reference's int32 ComputeT does
            return static_cast<int32_t>(static_cast<uint32_t>(alpha) * static_cast<uint32_t>(acc)
                                        + static_cast<uint32_t>(beta) * static_cast<uint32_t>(c));
        }

        // One thread's 32 consecutive output columns of one row.
        // OutT = __half: acc is fp32 bits.  OutT = float: fp32.  OutT = int32_t: int32.
        template <typename OutT, typename ScalarT>
        __device__ __forceinline__ void epilogue_row_chunk(const uint32_t (&v)[32],
                                                           const OutT* __restrict__ c_row,
                                                           OutT* __restrict__ d_row,
                                                           uint32_t ncols, // valid columns (<= 32)
                                                           ScalarT  alpha,
                                                           ScalarT  beta,
                                                           bool     read_c,
                                                           bool     vec_ok)
        {
            if(ncols == 32 && vec_ok)
            {
                if constexpr(sizeof(OutT) == 2)
                {
                    // 32 halfs = 4 x 16 bytes
#pragma unroll
                    for(int q = 0; q < 4; ++q)
                    {
                        uint4 cv = make_uint4(0, 0, 0, 0);
                        if(read_c)
                            cv = *reinterpret_cast<const uint4*>(c_row + q * 8);
                        const __half2* ch = reinterpret_cast<const __half2*>(&cv);
                        uint4          ov;
                        __half2*       oh = reinterpret_cast<__half2*>(&ov);
#pragma unroll
                        for(int j = 0; j < 4; ++j)
                        {
                            const float2 cf = __half22float2(ch[j]);
                            const float  x0
                                = epi(__uint_as_float(v[q * 8 + 2 * j]), cf.x, alpha, beta);
                            const float x1
                                = epi(__uint_as_float(v[q * 8 + 2 * j + 1]), cf.y, alpha, beta);
                            oh[j] = __floats2half2_rn(x0, x1);
                        }
                        *reinterpret_cast<uint4*>(d_row + q * 8) = ov;
                    }
                }
                else
                {
                    // 32 x 4-byte = 8 x 16 bytes
#pragma unroll
                    for(int q = 0; q < 8; ++q)
                    {
                        uint4 cv = make_uint4(0, 0, 0, 0);
                        if(read_c)
                            cv = *reinterpret_cast<const uint4*>(c_row + q * 4);
                        const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
                        uint32_t       ow[4];
#pragma unroll
                        for(int j = 0; j < 4; ++j)
                        {
                            if constexpr(std::is_same<OutT, float>::value)
                                ow[j] = __float_as_uint(epi(__uint_as_float(v[q * 4 + j]),
                                                            __uint_as_float(cw[j]),
                                                            alpha,
                                                            beta));
                            else
                                ow[j] = static_cast<uint32_t>(epi(static_cast<int32_t>(v[q * 4 + j]),
                                                                  static_cast<int32_t>(cw[j]),
                                                                  alpha,
                                                                  beta));
                        }
                        *reinterpret_cast<uint4*>(d_row + q * 4)
                            = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                    }
                }
            }
            else
            {
#pragma unroll
                for(int j = 0; j < 32; ++j)
                {
                    if(static_cast<uint32_t>(j) < ncols)
                    {
                        if constexpr(std::is_same<OutT, int32_t>::value)
                        {
                            const int32_t cvv = read_c ? c_row[j] : 0;
                            d_row[j] = epi(static_cast<int32_t>(v[j]), cvv, alpha, beta);
                        }
                        else
                        {
                            const float cvv = read_c ? static_cast<float>(c_row[j]) : 0.0f;
                            d_row[j]
                                = static_cast<OutT>(epi(__uint_as_float(v[j]), cvv, alpha, beta));
                        }
                    }
                }
            }
        }

        template <int KIND, typename OutT, typename ScalarT>
        __global__ void __launch_bounds__(NUM_THREADS, 1)
            gemm_tc05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                             const __grid_constant__ CUtensorMap tmap_b,
                             const OutT* __restrict__ c,
                             OutT* __restrict__ d,
                             uint32_t  m,
                             uint32_t  n,
                             uint32_t  k_bytes, // K extent in bytes of the input type
                             uint32_t  ldc,
                             uint32_t  ldd,
                             ScalarT   alpha,
                             ScalarT   beta,
                             uint32_t  tiles_m,
                             uint32_t  tiles_n,
                             int       vec_ok, // C/D rows 16-byte aligned -> vector epilogue
                             unsigned* status)
        {
            extern __shared__ uint8_t smem_raw[];
            const uint32_t            raw_addr = ptx::smem_u32(smem_raw);
            const uint32_t            base     = (raw_addr + 1023u) & ~1023u;
            uint8_t*                  smem     = smem_raw + (base - raw_addr);

            // [A stages][B stages][barriers][tmem slot][abort flag]
            const uint32_t     smem_a    = base;
            const uint32_t     smem_b    = base + STAGES * A_STAGE_BYTES;
            const uint32_t     bar_base  = base + STAGES * STAGE_BYTES;
            const uint32_t     full_bar  = bar_base; // STAGES x 8 bytes
            const uint32_t     empty_bar = bar_base + 8 * STAGES;
            const uint32_t     tfull_bar = bar_base + 16 * STAGES; // 2 x 8
            const uint32_t     tempty_bar = tfull_bar + 16; // 2 x 8
            uint32_t*          tmem_slot
                = reinterpret_cast<uint32_t*>(smem + STAGES * STAGE_BYTES + 16 * STAGES + 32);
            volatile uint32_t* cta_abort = tmem_slot + 1;

            const uint32_t warp      = threadIdx.x >> 5;
            const uint32_t lane      = threadIdx.x & 31u;
            const uint32_t num_tiles = tiles_m * tiles_n;
            const uint32_t num_kb    = (k_bytes + BLOCK_K_BYTES - 1) / BLOCK_K_BYTES;

            if(threadIdx.x == 0)
            {
                ptx::prefetch_tensormap(&tmap_a);
                ptx::prefetch_tensormap(&tmap_b);
                for(uint32_t s = 0; s < STAGES; ++s)
                {
                    ptx::mbar_init(full_bar + 8 * s, 1);
                    ptx::mbar_init(empty_bar + 8 * s, 1);
                }
                for(uint32_t s = 0; s < 2; ++s)
                {
                    ptx::mbar_init(tfull_bar + 8 * s, 1);
                    ptx::mbar_init(tempty_bar + 8 * s, 128);
                }
                *cta_abort = 0u;
                ptx::fence_barrier_init();
                ptx::fence_proxy_async_smem();
            }
            if(warp == 1)
            {
                ptx::tmem_alloc(ptx::smem_u32(tmem_slot), TMEM_COLS);
                ptx::tmem_relinquish();
            }
            ptx::tc_fence_before_sync();
            __syncthreads();
            ptx::tc_fence_after_sync();
            const uint32_t tmem_base = *tmem_slot;

            if(warp == 0)
            {
                // ------------------------------ TMA producer ------------------------------
                if(lane == 0)
                {
                    uint32_t stage = 0, phase = 0;
                    bool     ok = true;
                    for(uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x)
                    {
                        uint32_t m_idx, n_idx;
                        tile_coords(tile, tiles_m, tiles_n, m_idx, n_idx);
                        const int32_t row_a = static_cast<int32_t>(m_idx * BLOCK_M);
                        const int32_t row_b = static_cast<int32_t>(n_idx * BLOCK_N);
                        for(uint32_t kb = 0; kb < num_kb; ++kb)
                        {
                            ok = ptx::mbar_wait_bounded(empty_bar + 8 * stage,
                                                        phase ^ 1u,
                                                        cta_abort,
                                                        status,
                                                        (ROLE_PRODUCER << 24) | blockIdx.x,
                                                        WAIT_TIMEOUT_NS);
                            if(!ok)
                                break;
                            const uint32_t fb = full_bar + 8 * stage;
                            ptx::mbar_arrive_expect_tx(fb, STAGE_BYTES);
                            // inner coordinate in elements: fp16 -> 64 per slab, int8 -> 128
                            const int32_t kc = static_cast<int32_t>(
                                kb * (KIND == KIND_F16 ? BLOCK_K_BYTES / 2 : BLOCK_K_BYTES));
                            ptx::tma_load_2d(smem_a + stage * A_STAGE_BYTES, &tmap_a, kc, row_a, fb);
                            ptx::tma_load_2d(smem_b + stage * B_STAGE_BYTES, &tmap_b, kc, row_b, fb);
                            if(++stage == STAGES)
                            {
                                stage = 0;
                                phase ^= 1u;
                            }
                        }
                    }
                }
                __syncwarp();
            }
            else if(warp == 1)
            {
                // ------------------------------- MMA issuer -------------------------------
                if(lane == 0)
                {
                    constexpr uint32_t idesc = make_idesc<KIND>();
                    uint32_t           stage = 0, phase = 0;
                    uint32_t           iter = 0;
                    bool               ok   = true;
                    for(uint32_t tile = blockIdx.x; ok && tile < num_tiles;
                        tile += gridDim.x, ++iter)
                    {
                        const uint32_t buf    = iter & 1u;
                        const uint32_t bphase = (iter >> 1) & 1u;
                        ok = ptx::mbar_wait_bounded(tempty_bar + 8 * buf,
                                                    bphase ^ 1u,
                                                    cta_abort,
                                                    status,
                                                    (ROLE_MMA << 24) | blockIdx.x,
                                                    WAIT_TIMEOUT_NS);
                        if(!ok)
                            break;
                        ptx::tc_fence_after_sync();
                        const uint32_t d_tmem = tmem_base + buf * BLOCK_N;
                        for(uint32_t kb = 0; kb < num_kb; ++kb)
                        {
                            ok = ptx::mbar_wait_bounded(full_bar + 8 * stage,
                                                        phase,
                                                        cta_abort,
                                                        status,
                                                        (ROLE_MMA << 24) | (1u << 20) | blockIdx.x,
                                                        WAIT_TIMEOUT_NS);
                            if(!ok)
                                break;
                            ptx::tc_fence_after_sync();
                            const uint64_t a_desc
                                = ptx::make_kmajor_sw128_desc(smem_a + stage * A_STAGE_BYTES);
                            const uint64_t b_desc
                                = ptx::make_kmajor_sw128_desc(smem_b + stage * B_STAGE_BYTES);
#pragma unroll
                            for(uint32_t ks = 0; ks < BLOCK_K_BYTES / 32; ++ks)
                            {
                                // each MMA consumes 32 bytes of K (16 fp16 / 32 int8):
                                // +32 bytes = +2 in the descriptor's 16-byte address units
                                const uint32_t acc = (kb | ks) != 0u ? 1u : 0u;
                                if constexpr(KIND == KIND_F16)
                                    ptx::mma_f16_ss(d_tmem, a_desc + 2 * ks, b_desc + 2 * ks, idesc, acc);
                                else
                                    ptx::mma_i8_ss(d_tmem, a_desc + 2 * ks, b_desc + 2 * ks, idesc, acc);
                            }
                            ptx::tc_commit(empty_bar + 8 * stage); // slot reusable once MMAs retire
                            if(++stage == STAGES)
                            {
                                stage = 0;
                                phase ^= 1u;
                            }
                        }
                        if(ok)
                            ptx::tc_commit(tfull_bar + 8 * buf); // accumulator complete
                    }
                }
                __syncwarp();
            }
            else
            {
                // -------------------------------- epilogue --------------------------------
                const uint32_t quad   = warp & 3u; // tensor-memory lane quadrant of this warp
                const bool     read_c = (beta != ScalarT(0)) && (c != nullptr);
                uint32_t       iter   = 0;
                bool           ok     = true;
                for(uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++iter)
                {
                    const uint32_t buf    = iter & 1u;
                    const uint32_t bphase = (iter >> 1) & 1u;
                    uint32_t       m_idx, n_idx;
                    tile_coords(tile, tiles_m, tiles_n, m_idx, n_idx);
                    ok = ptx::mbar_wait_bounded(tfull_bar + 8 * buf,
                                                bphase,
                                                cta_abort,
                                                status,
                                                (ROLE_EPILOGUE << 24) | blockIdx.x,
                                                WAIT_TIMEOUT_NS);
                    // the warp must stay converged for the .sync.aligned tcgen05.ld below
                    ok = __all_sync(0xFFFFFFFFu, ok);
                    if(!ok)
                        break;
                    ptx::tc_fence_after_sync();
                    const uint32_t row     = m_idx * BLOCK_M + quad * 32u + lane;
                    const bool     row_ok  = row < m;
                    const uint32_t col_base = n_idx * BLOCK_N;
                    const OutT*    c_row   = c + static_cast<size_t>(row) * ldc + col_base;
                    OutT*          d_row   = d + static_cast<size_t>(row) * ldd + col_base;
#pragma unroll 1
                    for(uint32_t ch = 0; ch < BLOCK_N / 32; ++ch)
                    {
                        uint32_t v[32];
                        ptx::tmem_ld_32x32b_x32(
                            tmem_base + ((quad * 32u) << 16) + buf * BLOCK_N + ch * 32u, v);
                        ptx::tmem_ld_wait();
                        const uint32_t col0 = col_base + ch * 32u;
                        if(row_ok && col0 < n)
                        {
                            const uint32_t ncols = min(32u, n - col0);
                            epilogue_row_chunk<OutT, ScalarT>(v,
                                                              c_row + ch * 32u,
                                                              d_row + ch * 32u,
                                                              ncols,
                                                              alpha,
                                                              beta,
                                                              read_c,
                                                              vec_ok != 0);
                        }
                    }
                    ptx::tc_fence_before_sync();
                    ptx::mbar_arrive(tempty_bar + 8 * buf);
                }
            }

            // ---------------------------------- teardown ----------------------------------
            ptx::tc_fence_before_sync();
            __syncthreads();
            if(*cta_abort)
            {
                // A wait was abandoned: TMA copies or MMAs of this CTA may still be in flight.
                // Give them a bounded grace period before shared and tensor memory are released.
                const uint64_t t0 = ptx::globaltimer_ns();
                while(ptx::globaltimer_ns() - t0 < 2000000ull)
                    __nanosleep(1000);
                __syncthreads();
            }
            if(warp == 1)
            {
                ptx::tc_fence_after_sync();
                ptx::tmem_dealloc(tmem_base, TMEM_COLS);
            }
        }

        // ---- host side ------------------------------------------------------------------
        typedef CUresult (*EncodeTiledFn)(CUtensorMap*,
                                          CUtensorMapDataType,
                                          cuuint32_t,
                                          void*,
                                          const cuuint64_t*,
                                          const cuuint64_t*,
                                          const cuuint32_t*,
                                          const cuuint32_t*,
                                          CUtensorMapInterleave,
                                          CUtensorMapSwizzle,
                                          CUtensorMapL2promotion,
                                          CUtensorMapFloatOOBfill);

        static EncodeTiledFn get_encode_fn()
        {
            static EncodeTiledFn fn = []() -> EncodeTiledFn {
                void*                           p = nullptr;
                cudaDriverEntryPointQueryResult q;
                if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q)
                       != cudaSuccess
                   || q != cudaDriverEntryPointSuccess)
                    return nullptr;
                return reinterpret_cast<EncodeTiledFn>(p);
            }();
            return fn;
        }

        // K-major operand: `rows` rows of `k_elems` contiguous elements, row pitch ld elements.
        // Box = one 128-byte K slab x box_rows rows, 128-byte swizzle, zero fill out of bounds.
        static int make_kmajor_tmap(CUtensorMap*        out,
                                    CUtensorMapDataType dtype,
                                    uint32_t            elem_bytes,
                                    const void*         ptr,
                                    uint32_t            rows,
                                    uint32_t            k_elems,
                                    uint32_t            ld,
                                    uint32_t            box_rows)
        {
            EncodeTiledFn fn = get_encode_fn();
            B200_REQUIRE(fn != nullptr, B200WMMA_ERR_CUDA, "cuTensorMapEncodeTiled not available");
            cuuint64_t gdim[2]    = {k_elems, rows};
            cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
            cuuint32_t box[2]     = {BLOCK_K_BYTES / elem_bytes, box_rows};
            cuuint32_t estr[2]    = {1, 1};
            CUresult   r          = fn(out,
                            dtype,
                            2,
                            const_cast<void*>(ptr),
                            gdim,
                            gstride,
                            box,
                            estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            B200_REQUIRE(r == CUDA_SUCCESS,
                         B200WMMA_ERR_CUDA,
                         "cuTensorMapEncodeTiled failed with CUresult %d",
                         static_cast<int>(r));
            return B200WMMA_OK;
        }

        template <int KIND, typename OutT, typename ScalarT>
        static int launch(uint32_t     m,
                          uint32_t     n,
                          uint32_t     k,
                          const void*  a,
                          const void*  b,
                          const OutT*  c,
                          OutT*        d,
                          uint32_t     lda,
                          uint32_t     ldb,
                          uint32_t     ldc,
                          uint32_t     ldd,
                          ScalarT      alpha,
                          ScalarT      beta,
                          cudaStream_t stream)
        {
            constexpr uint32_t EB = (KIND == KIND_F16) ? 2u : 1u;
            B200_REQUIRE(m && n && k, B200WMMA_ERR_INVALID_ARG, "gemm: m, n, k must be non-zero");
            B200_REQUIRE(a && b && d, B200WMMA_ERR_INVALID_ARG, "gemm: a, b, d must be non-null");
            B200_REQUIRE(c || beta == ScalarT(0),
                         B200WMMA_ERR_INVALID_ARG,
                         "gemm: c may be null only when beta == 0");
            B200_REQUIRE(lda >= k && ldb >= k && ldd >= n && (!c || ldc >= n),
                         B200WMMA_ERR_INVALID_ARG,
                         "gemm: leading dimension smaller than the row/column it strides");
            B200_REQUIRE(aligned16(a) && aligned16(b) && (static_cast<uint64_t>(lda) * EB) % 16 == 0
                             && (static_cast<uint64_t>(ldb) * EB) % 16 == 0,
                         B200WMMA_ERR_ALIGNMENT,
                         "gemm: A/B base pointers and row pitches must be multiples of 16 bytes "
                         "(TMA requirement)");
            if(int e = require_sm100())
                return e;
            unsigned* status = nullptr;
            if(int e = status_word_ptr(&status))
                return e;

            CUtensorMap               tm_a, tm_b;
            const CUtensorMapDataType dt
                = (KIND == KIND_F16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
            if(int e = make_kmajor_tmap(&tm_a, dt, EB, a, m, k, lda, BLOCK_M))
                return e;
            if(int e = make_kmajor_tmap(&tm_b, dt, EB, b, n, k, ldb, BLOCK_N))
                return e;

            const bool vec_ok = aligned16(d) && (static_cast<uint64_t>(ldd) * sizeof(OutT)) % 16 == 0
                                && (!c
                                    || (aligned16(c)
                                        && (static_cast<uint64_t>(ldc) * sizeof(OutT)) % 16 == 0));

            auto        kern    = gemm_tc05_kernel<KIND, OutT, ScalarT>;
            static bool attr_ok = false; // one flag per template instantiation
            if(!attr_ok)
            {
                B200_CHECK_CUDA(cudaFuncSetAttribute(
                    kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
                attr_ok = true;
            }
            int dev = 0, sms = 0;
            B200_CHECK_CUDA(cudaGetDevice(&dev));
            B200_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
            const uint32_t tiles_m = ceil_div(m, BLOCK_M), tiles_n = ceil_div(n, BLOCK_N);
            const uint32_t grid = min(tiles_m * tiles_n, static_cast<uint32_t>(sms));
            kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tm_a,
                                                             tm_b,
                                                             c,
                                                             d,
                                                             m,
                                                             n,
                                                             k * EB,
                                                             ldc,
                                                             ldd,
                                                             alpha,
                                                             beta,
                                                             tiles_m,
                                                             tiles_n,
                                                             vec_ok ? 1 : 0,
                                                             status);
            B200_CHECK_CUDA(cudaGetLastError());
            return B200WMMA_OK;
        }
    } // namespace tc05

    int launch_gemm_tc05_f16(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b,
                             const void* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                             uint32_t ldd, float alpha, float beta, int out_type,
                             cudaStream_t stream)
    {
        if(out_type == B200WMMA_OUT_F16)
            return tc05::launch<tc05::KIND_F16, __half, float>(m, n, k, a, b,
                                                               static_cast<const __half*>(c),
                                                               static_cast<__half*>(d),
                                                               lda, ldb, ldc, ldd, alpha, beta, stream);
        if(out_type == B200WMMA_OUT_F32)
            return tc05::launch<tc05::KIND_F16, float, float>(m, n, k, a, b,
                                                              static_cast<const float*>(c),
                                                              static_cast<float*>(d),
                                                              lda, ldb, ldc, ldd, alpha, beta, stream);
        return set_error(B200WMMA_ERR_INVALID_ARG, "gemm_f16: out_type must be 0 (f16) or 1 (f32)");
    }

    int launch_gemm_tc05_i8(uint32_t m, uint32_t n, uint32_t k, const int8_t* a,
                            const int8_t* b, const int32_t* c, int32_t* d, uint32_t lda,
                            uint32_t ldb, uint32_t ldc, uint32_t ldd, int32_t alpha,
                            int32_t beta, cudaStream_t stream)
    {
        return tc05::launch<tc05::KIND_I8, int32_t, int32_t>(m, n, k, a, b, c, d, lda, ldb, ldc, ldd,
                                                             alpha, beta, stream);
    }
} // namespace b200wmma
