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
#include "gemm_tc05_common.cuh"
#include "gemm_tc05_pair.cuh"
#include "gemm_tc05_pair512.cuh"
#include "tuning.cuh"

namespace b200wmma
{
    namespace tc05
    {
        constexpr uint32_t BLOCK_M       = 128;
        constexpr uint32_t BLOCK_N       = 256;
        constexpr uint32_t STAGES        = 4;
        constexpr uint32_t A_STAGE_BYTES = BLOCK_M * BLOCK_K_BYTES; // 16 KiB
        constexpr uint32_t B_STAGE_BYTES = BLOCK_N * BLOCK_K_BYTES; // 32 KiB
        constexpr uint32_t STAGE_BYTES   = A_STAGE_BYTES + B_STAGE_BYTES;
        constexpr uint32_t NUM_THREADS   = 192;
        constexpr uint32_t TMEM_COLS     = 512; // 2 accumulator buffers x 256 fp32/int32 columns
        constexpr uint32_t GROUP_M       = 16; // tile rasterisation: 16 row tiles share B slabs
        constexpr uint32_t SMEM_BYTES    = 1024 /*alignment slack*/ + STAGES * STAGE_BYTES + 256;

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
                             int       vec_ok, // widest aligned epilogue access: 0 / 1 (16 B) / 2 (32 B)
                             uint32_t  group_m, // rasterisation band height in row tiles
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
                        tile_coords(tile, tiles_m, tiles_n, group_m, m_idx, n_idx);
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
                    constexpr uint32_t idesc = make_idesc<KIND, BLOCK_M, BLOCK_N>();
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
                    tile_coords(tile, tiles_m, tiles_n, group_m, m_idx, n_idx);
                    ok = ptx::mbar_wait_bounded_warp(tfull_bar + 8 * buf, bphase, cta_abort, status,
                                                     (ROLE_EPILOGUE << 24) | blockIdx.x, WAIT_TIMEOUT_NS, lane);
                    if(!ok)
                        break;
                    ptx::tc_fence_after_sync();
                    drain_accumulator<OutT, ScalarT, BLOCK_N>(tmem_base + buf * BLOCK_N, quad, lane,
                                                              m_idx * BLOCK_M, n_idx * BLOCK_N, m, n, c, d, ldc, ldd,
                                                              alpha, beta, read_c, vec_ok);
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

        // Tuning overrides set through b200wmma_set_tuning (0 = built-in choice): see tuning.cuh.
        static uint32_t group_override(uint32_t dflt)
        {
            const int v = tuning::get(tuning::GEMM_GROUP_M);
            return v > 0 ? static_cast<uint32_t>(v) : dflt;
        }
        // 0 = automatic, 1 = one-CTA tiles, 2 = two-CTA 256x256 pair tiles, 3 = two-CTA 512x256 pair tiles
        static int forced_variant()
        {
            const int v = tuning::get(tuning::GEMM_TILE_VARIANT);
            return (v >= 1 && v <= 3) ? v : 0;
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
                          bool         a_mn, // A column-major (M contiguous) instead of row-major
                          bool         b_mn, // B row-major (N contiguous) instead of column-major
                          cudaStream_t stream,
                          void*        split_ws       = nullptr, // optional scratch for the split-K tail (512 x 256 kernel)
                          size_t       split_ws_bytes = 0)
        {
            constexpr uint32_t EB = elem_bytes<KIND>();
            // bf16 and fp8 inputs run on the 512 x 256 pair kernel only
            // ... and so do the extra output types (bf16 outputs, int8 outputs of the int8 GEMM)
            constexpr bool ONLY_Q = (KIND != KIND_F16 && KIND != KIND_I8) || sizeof(OutT) == 1;
            B200_REQUIRE(m && n && k, B200WMMA_ERR_INVALID_ARG, "gemm: m, n, k must be non-zero");
            B200_REQUIRE(a && b && d, B200WMMA_ERR_INVALID_ARG, "gemm: a, b, d must be non-null");
            B200_REQUIRE(c || beta == ScalarT(0),
                         B200WMMA_ERR_INVALID_ARG,
                         "gemm: c may be null only when beta == 0");
            B200_REQUIRE(lda >= (a_mn ? m : k) && ldb >= (b_mn ? n : k) && ldd >= n && (!c || ldc >= n),
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

            const CUtensorMapDataType dt
                = (KIND == KIND_F16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                     : (KIND == KIND_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
            // widest epilogue access every C / D row start allows: 32 bytes, 16 bytes, or element-wise
            auto row_align = [](const void* p, uint32_t ld, size_t es, uint64_t bytes) {
                return (reinterpret_cast<uintptr_t>(p) % bytes) == 0 && (static_cast<uint64_t>(ld) * es) % bytes == 0;
            };
            int vec_ok = 0;
            if(sizeof(OutT) == 1)
                vec_ok = 0; // one-byte outputs: element-wise drain
            else if(row_align(d, ldd, sizeof(OutT), 32) && (!c || row_align(c, ldc, sizeof(OutT), 32)))
                vec_ok = 2;
            else if(row_align(d, ldd, sizeof(OutT), 16) && (!c || row_align(c, ldc, sizeof(OutT), 16)))
                vec_ok = 1;
            int dev = 0, sms = 0;
            B200_CHECK_CUDA(cudaGetDevice(&dev));
            B200_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));

            // Tile shape.  Three kernels exist: 512 x 256 per SM pair (least operand traffic, fastest per
            // flop), 256 x 256 per pair and 128 x 256 per SM.  All are persistent, so a problem costs
            // ceil(tiles / slots) rounds of one tile each; pick the shape with the smallest estimated
            // time = rounds x outputs per SM per tile / relative speed (measured at 8192^3: 1, 0.955, 0.91).
            // b200wmma_set_tuning("gemm_tile_variant", 1 | 2 | 3) forces one, for comparison.
            const int forced = (a_mn || b_mn || ONLY_Q) ? 3 : forced_variant(); // MN-major operands: 512 x 256 kernel only
            int       pick   = forced;
            if(pick == 0)
            {
                const uint64_t slots1 = static_cast<uint64_t>(sms), slots2 = static_cast<uint64_t>(sms / 2);
                auto rounds = [](uint64_t tiles, uint64_t slots) { return (tiles + slots - 1) / slots; };
                const double t512 = rounds(static_cast<uint64_t>(ceil_div(m, 512)) * ceil_div(n, 256), slots2) * 65536.0;
                const double t256 = rounds(static_cast<uint64_t>(ceil_div(m, 256)) * ceil_div(n, 256), slots2) * 32768.0 / 0.955;
                const double t128 = rounds(static_cast<uint64_t>(ceil_div(m, 128)) * ceil_div(n, 256), slots1) * 32768.0 / 0.91;
                pick              = (t512 <= t256 && t512 <= t128) ? 3 : (t256 <= t128 ? 2 : 1);
                if(split_ws != nullptr && m > tc05p::PAIR_M)
                    pick = 3; // with a split-K tail the 512 x 256 kernel has no partial round to lose
                if(m <= BLOCK_M)
                    pick = 1; // a single 128-row band: pairing would multiply zeros
                else if(m <= tc05p::PAIR_M && pick == 3)
                    pick = 2;
            }
            const bool use_q    = pick == 3;
            const bool use_pair = pick == 2;
            CUtensorMap tm_a, tm_b;
            if(int e = a_mn ? make_mnmajor_tmap(&tm_a, dt, EB, a, m, k, lda)
                            : make_kmajor_tmap(&tm_a, dt, EB, a, m, k, lda, use_q ? tc05q::CTA_M : BLOCK_M))
                return e;
            if(int e = b_mn ? make_mnmajor_tmap(&tm_b, dt, EB, b, n, k, ldb)
                            : make_kmajor_tmap(&tm_b, dt, EB, b, n, k, ldb, (use_pair || use_q) ? tc05p::HALF_N : BLOCK_N))
                return e;

            if(use_q)
            {
                using KernT = decltype(&tc05q::gemm_tc05_pair512_kernel<KIND, OutT, ScalarT, false, false, false>);
                const KernT kerns[8] = {tc05q::gemm_tc05_pair512_kernel<KIND, OutT, ScalarT, false, false, false>,
                                        tc05q::gemm_tc05_pair512_kernel<KIND, OutT, ScalarT, false, true, false>,
                                        tc05q::gemm_tc05_pair512_kernel<KIND, OutT, ScalarT, true, false, false>,
                                        tc05q::gemm_tc05_pair512_kernel<KIND, OutT, ScalarT, true, true, false>,
                                        tc05q::gemm_tc05_pair512_kernel<KIND, OutT, ScalarT, false, false, true>,
                                        tc05q::gemm_tc05_pair512_kernel<KIND, OutT, ScalarT, false, true, true>,
                                        tc05q::gemm_tc05_pair512_kernel<KIND, OutT, ScalarT, true, false, true>,
                                        tc05q::gemm_tc05_pair512_kernel<KIND, OutT, ScalarT, true, true, true>};
                // MMA order of a tile's first and last slabs: by accumulator (1, default) or by slab (2)
                const bool  split     = tuning::get(tuning::GEMM_MMA_ORDER) != 2;
                const int   layout_id = (a_mn ? 2 : 0) + (b_mn ? 1 : 0) + (split ? 4 : 0);
                KernT       kern      = kerns[layout_id];
                static int  max_clusters_dev[8][MAX_DEVICES]; // per template instantiation, layout and device
                int&        max_clusters = max_clusters_dev[layout_id][current_device_slot()];
                const uint32_t tiles_m = ceil_div(m, tc05q::PAIR_M), tiles_n = ceil_div(n, tc05q::TILE_N);
                cudaLaunchConfig_t  cfg = {};
                cudaLaunchAttribute attr[1];
                attr[0].id               = cudaLaunchAttributeClusterDimension;
                attr[0].val.clusterDim.x = 2;
                attr[0].val.clusterDim.y = 1;
                attr[0].val.clusterDim.z = 1;
                cfg.blockDim         = dim3(tc05q::NUM_THREADS);
                cfg.dynamicSmemBytes = tc05q::SMEM_BYTES;
                cfg.stream           = stream;
                cfg.attrs            = attr;
                cfg.numAttrs         = 1;
                if(max_clusters == 0)
                {
                    B200_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                         tc05q::SMEM_BYTES));
                    cfg.gridDim = dim3(static_cast<unsigned>(sms) & ~1u);
                    int nc      = 0;
                    B200_CHECK_CUDA(cudaOccupancyMaxActiveClusters(&nc, kern, &cfg));
                    B200_REQUIRE(nc > 0, B200WMMA_ERR_CUDA, "no two-CTA cluster of the GEMM kernel fits on this device");
                    max_clusters = nc;
                }
                uint32_t pairs = min(tiles_m * tiles_n, static_cast<uint32_t>(max_clusters));
                // Split-K tail: when the tiles do not fill a whole number of rounds, the tiles of the last, partial round
                // are cut along K into equal slab ranges, one per SM pair, so that every pair works to the end; the
                // partial accumulators meet in the caller's workspace.  Worth it when the slabs saved exceed the cost of
                // the exchange (about FIXUP_SLABS slabs' worth of time); needs the TMA epilogue.
                tc05q::SplitPlan plan = {0u, 0u, 0u};
                if(split_ws != nullptr && vec_ok != 0 && tuning::get(tuning::GEMM_SPLIT_TAIL) != 2)
                {
                    // The exchange costs a pair about as much time as FIXUP_SLABS K slabs.  Measured (fp16, 64-wide slabs, 74
                    // pairs): writing a partial 6 k + 2 k cycles (stores, fence), adding one 8.5 k on top of the 6 k drain, a
                    // second pipeline ramp and the flag reset; in all 33 slabs' worth at 8192 x 1024 x 8192 (two pieces per
                    // tile) and about 75 at 8192 x 4096 x 8192 (three pieces per tile after three whole rounds).  With 80
                    // the split is taken where a few left-over tiles would otherwise cost a whole round.
                    constexpr uint32_t MIN_SLABS   = 16;
                    const uint32_t     fix_tuned   = static_cast<uint32_t>(tuning::get(tuning::GEMM_SPLIT_FIXUP));
                    const uint32_t     FIXUP_SLABS = fix_tuned ? fix_tuned : 80u;
                    const uint32_t pmax = static_cast<uint32_t>(max_clusters), tiles = tiles_m * tiles_n;
                    const uint32_t num_kb = ceil_div(k * EB, BLOCK_K_BYTES);
                    const uint32_t full = tiles / pmax, rem = tiles % pmax;
                    const uint64_t slabs = static_cast<uint64_t>(rem) * num_kb;
                    uint32_t       sk_pairs = static_cast<uint32_t>(slabs / MIN_SLABS < pmax ? slabs / MIN_SLABS : pmax);
                    const uint32_t used = full > 0 ? pmax : sk_pairs;
                    const size_t   need = static_cast<size_t>(used) * (tc05q::SLOT_WORDS * 4u + 4u);
                    if(rem > 0 && sk_pairs > rem && slabs < (1ull << 31) && split_ws_bytes >= need && aligned16(split_ws))
                    {
                        const uint64_t per_pair = (slabs + sk_pairs - 1) / sk_pairs;
                        if(per_pair + FIXUP_SLABS < num_kb)
                        {
                            plan.dp_rounds = full, plan.sk_tiles = rem, plan.sk_pairs = sk_pairs;
                            pairs = used;
                            uint32_t* flags = static_cast<uint32_t*>(split_ws) + static_cast<size_t>(pairs) * tc05q::SLOT_WORDS;
#ifndef B200WMMA_SK_NO_MEMSET // (timing experiments only: results are wrong without the reset)
                            B200_CHECK_CUDA(cudaMemsetAsync(flags, 0, sizeof(uint32_t) * pairs, stream));
#endif
                        }
                    }
                }
                cfg.gridDim = dim3(2 * pairs);
                // C / D staging boxes for the TMA epilogue (used when the rows are 16-byte aligned)
                CUtensorMap tm_c = tm_a, tm_d = tm_a; // placeholders, never dereferenced when vec_ok == 0
                if(vec_ok != 0)
                {
                    if(int e = make_rowbox_tmap(&tm_d, sizeof(OutT), d, m, n, ldd))
                        return e;
                    tm_c = tm_d;
                    if(c)
                        if(int e = make_rowbox_tmap(&tm_c, sizeof(OutT), c, m, n, ldc))
                            return e;
                }
                B200_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, tm_a, tm_b, tm_c, tm_d, c, d, m, n, k * EB, ldc, ldd, alpha,
                                                   beta, tiles_m, tiles_n, vec_ok, group_override(tc05q::GROUP_M), status, plan,
                                                   static_cast<uint32_t*>(split_ws)));
                return B200WMMA_OK;
            }

            if constexpr(!ONLY_Q)
            {
            if(use_pair)
            {
                auto        kern    = tc05p::gemm_tc05_pair_kernel<KIND, OutT, ScalarT>;
                static int max_clusters_dev[MAX_DEVICES]; // per template instantiation and device
                int&       max_clusters = max_clusters_dev[current_device_slot()];
                const uint32_t tiles_m = ceil_div(m, tc05p::PAIR_M), tiles_n = ceil_div(n, tc05p::TILE_N);
                cudaLaunchConfig_t  cfg = {};
                cudaLaunchAttribute attr[1];
                attr[0].id               = cudaLaunchAttributeClusterDimension;
                attr[0].val.clusterDim.x = 2;
                attr[0].val.clusterDim.y = 1;
                attr[0].val.clusterDim.z = 1;
                cfg.blockDim         = dim3(tc05p::NUM_THREADS);
                cfg.dynamicSmemBytes = tc05p::SMEM_BYTES;
                cfg.stream           = stream;
                cfg.attrs            = attr;
                cfg.numAttrs         = 1;
                if(max_clusters == 0)
                {
                    B200_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                         tc05p::SMEM_BYTES));
                    cfg.gridDim = dim3(static_cast<unsigned>(sms) & ~1u);
                    int nc      = 0;
                    B200_CHECK_CUDA(cudaOccupancyMaxActiveClusters(&nc, kern, &cfg));
                    B200_REQUIRE(nc > 0, B200WMMA_ERR_CUDA, "no two-CTA cluster of the GEMM kernel fits on this device");
                    max_clusters = nc;
                }
                const uint32_t pairs = min(tiles_m * tiles_n, static_cast<uint32_t>(max_clusters));
                cfg.gridDim          = dim3(2 * pairs);
                B200_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, tm_a, tm_b, c, d, m, n, k * EB, ldc, ldd, alpha, beta,
                                                   tiles_m, tiles_n, vec_ok, group_override(tc05p::GROUP_M), status));
                return B200WMMA_OK;
            }

            auto        kern    = gemm_tc05_kernel<KIND, OutT, ScalarT>;
            static bool attr_ok_dev[MAX_DEVICES]; // per template instantiation and device
            bool&       attr_ok = attr_ok_dev[current_device_slot()];
            if(!attr_ok)
            {
                B200_CHECK_CUDA(cudaFuncSetAttribute(
                    kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
                attr_ok = true;
            }
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
                                                             vec_ok,
                                                             group_override(GROUP_M),
                                                             status);
            B200_CHECK_CUDA(cudaGetLastError());
            return B200WMMA_OK;
            }
            else
                return set_error(B200WMMA_ERR_UNSUPPORTED, "gemm: no kernel for this input type and shape");
        }
    } // namespace tc05

    // Layout handling shared by both element types.  An operand is "MN-major" when its M / N index
    // is the contiguous one (column-major A, row-major B).  Column-major C / D is the row-major
    // transposed problem D^T = alpha * B^T A^T + beta * C^T: swap the operands and m <-> n.
    template <int KIND, typename OutT, typename ScalarT>
    static int launch_any_layout(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b, const OutT* c,
                                 OutT* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, ScalarT alpha,
                                 ScalarT beta, int layout_a, int layout_b, int layout_cd, cudaStream_t stream,
                                 void* split_ws = nullptr, size_t split_ws_bytes = 0)
    {
        const bool a_mn = layout_a == B200WMMA_COL_MAJOR, b_mn = layout_b == B200WMMA_ROW_MAJOR;
        if(layout_cd == B200WMMA_ROW_MAJOR)
            return tc05::launch<KIND, OutT, ScalarT>(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, a_mn, b_mn,
                                                     stream, split_ws, split_ws_bytes);
        // B^T (n x k) takes the role of A: it is K-major exactly when B was; likewise A^T for B
        return tc05::launch<KIND, OutT, ScalarT>(n, m, k, b, a, c, d, ldb, lda, ldc, ldd, alpha, beta, b_mn, a_mn, stream,
                                                 split_ws, split_ws_bytes);
    }

    size_t gemm_split_workspace_bytes()
    {
        int dev = 0, sms = 0;
        if(cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return 0;
        return static_cast<size_t>(sms / 2) * (tc05q::SLOT_WORDS * 4u + 4u);
    }

    int launch_gemm_tc05_f16(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b,
                             const void* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                             uint32_t ldd, float alpha, float beta, int layout_a, int layout_b, int layout_cd,
                             int out_type, cudaStream_t stream, void* split_ws, size_t split_ws_bytes)
    {
        if(out_type == B200WMMA_OUT_F16)
            return launch_any_layout<tc05::KIND_F16, __half, float>(m, n, k, a, b, static_cast<const __half*>(c),
                                                                    static_cast<__half*>(d), lda, ldb, ldc, ldd, alpha,
                                                                    beta, layout_a, layout_b, layout_cd, stream, split_ws,
                                                                    split_ws_bytes);
        if(out_type == B200WMMA_OUT_F32)
            return launch_any_layout<tc05::KIND_F16, float, float>(m, n, k, a, b, static_cast<const float*>(c),
                                                                   static_cast<float*>(d), lda, ldb, ldc, ldd, alpha, beta,
                                                                   layout_a, layout_b, layout_cd, stream, split_ws,
                                                                   split_ws_bytes);
        return set_error(B200WMMA_ERR_INVALID_ARG, "gemm_f16: out_type must be 0 (f16) or 1 (f32)");
    }

    int launch_gemm_tc05_bf16(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b, const void* c, void* d,
                              uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, float alpha, float beta, int layout_a,
                              int layout_b, int layout_cd, int out_type, cudaStream_t stream)
    {
        if(out_type == B200WMMA_OUT_F32)
            return launch_any_layout<tc05::KIND_BF16, float, float>(m, n, k, a, b, static_cast<const float*>(c),
                                                                    static_cast<float*>(d), lda, ldb, ldc, ldd, alpha, beta,
                                                                    layout_a, layout_b, layout_cd, stream);
        if(out_type == B200WMMA_OUT_BF16)
            return launch_any_layout<tc05::KIND_BF16, __nv_bfloat16, float>(m, n, k, a, b, static_cast<const __nv_bfloat16*>(c),
                                                                            static_cast<__nv_bfloat16*>(d), lda, ldb, ldc, ldd,
                                                                            alpha, beta, layout_a, layout_b, layout_cd, stream);
        return set_error(B200WMMA_ERR_INVALID_ARG, "gemm_bf16: out_type must be B200WMMA_OUT_F32 or B200WMMA_OUT_BF16");
    }

    int launch_gemm_tc05_i8_i8(uint32_t m, uint32_t n, uint32_t k, const int8_t* a, const int8_t* b, const int8_t* c, int8_t* d,
                               uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, int32_t alpha, int32_t beta, int layout_a,
                               int layout_b, int layout_cd, cudaStream_t stream)
    {
        return launch_any_layout<tc05::KIND_I8, int8_t, int32_t>(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, layout_a,
                                                                 layout_b, layout_cd, stream);
    }

    int launch_gemm_tc05_fp8(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b, const float* c, float* d,
                             uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, float alpha, float beta, int layout_a,
                             int layout_b, int layout_cd, int fp8_format, cudaStream_t stream)
    {
        if(fp8_format == B200WMMA_FP8_E4M3)
            return launch_any_layout<tc05::KIND_E4M3, float, float>(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta,
                                                                    layout_a, layout_b, layout_cd, stream);
        if(fp8_format == B200WMMA_FP8_E5M2)
            return launch_any_layout<tc05::KIND_E5M2, float, float>(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta,
                                                                    layout_a, layout_b, layout_cd, stream);
        return set_error(B200WMMA_ERR_INVALID_ARG, "gemm_fp8: fp8_format must be 0 (e4m3) or 1 (e5m2)");
    }

    int launch_gemm_tc05_i8(uint32_t m, uint32_t n, uint32_t k, const int8_t* a,
                            const int8_t* b, const int32_t* c, int32_t* d, uint32_t lda,
                            uint32_t ldb, uint32_t ldc, uint32_t ldd, int32_t alpha,
                            int32_t beta, int layout_a, int layout_b, int layout_cd, cudaStream_t stream, void* split_ws,
                            size_t split_ws_bytes)
    {
        return launch_any_layout<tc05::KIND_I8, int32_t, int32_t>(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta,
                                                                  layout_a, layout_b, layout_cd, stream, split_ws,
                                                                  split_ws_bytes);
    }
} // namespace b200wmma
