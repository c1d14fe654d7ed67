// fp32 GEMM D = alpha * (A x B) + beta * C on the tensor cores with fp32-class accuracy (3 x TF32).
//
// Stands in for rocWMMA's fp32 GEMM samples - sgemm_rocwmma_d (samples/simple_sgemm.cpp) and
// gemm_rocwmma_d of samples/perf_sgemm.cpp - whose MFMA path multiplies fp32 inputs exactly.  The
// sm_100 tensor cores have no fp32 input kind: kind::tf32 keeps 10 mantissa bits of each input.  Each
// operand is therefore split once into hi = tf32(x) and lo = tf32(x - hi) (a streaming pre-pass into the
// caller's workspace) and the kernel accumulates hi*hi + hi*lo + lo*hi in fp32; the dropped lo*lo term
// is below 2^-21 of a product, the same order as fp32 rounding of the sum.
//
// Kernel: the 512 x 256 pair tile, roles and barrier protocol of gemm_tc05_pair512.cuh.  A stage holds
// four operand tiles of one 32-wide K slab (A hi / lo: 256 rows x 128 B each, B hi / lo: 128 rows x 128 B
// each per CTA) = 96 KiB, two stages; per slab the MMA thread issues 4 K steps x 2 accumulators x 3
// products = 24 MMAs (M = 256, N = 256, K = 8), 3072 clocks of tensor work, which hides the reload of
// the other stage.  Operands K-major only: A row major, B column major, C / D row major.
#include "gemm_tc05_common.cuh"
#include "gemm_tc05_pair512.cuh"

namespace b200wmma
{
    namespace tc05t
    {
        using namespace tc05;

        constexpr uint32_t SUB_M         = 128;
        constexpr uint32_t CTA_M         = 256;
        constexpr uint32_t PAIR_M        = 512;
        constexpr uint32_t TILE_N        = 256;
        constexpr uint32_t HALF_N        = 128;
        constexpr uint32_t SLAB_K        = 32; // fp32 elements per 128-byte row
        constexpr uint32_t STAGES        = 2;
        constexpr uint32_t A_TILE_BYTES  = CTA_M * BLOCK_K_BYTES; // 32 KiB (hi or lo)
        constexpr uint32_t B_TILE_BYTES  = HALF_N * BLOCK_K_BYTES; // 16 KiB
        constexpr uint32_t STAGE_BYTES   = 2 * A_TILE_BYTES + 2 * B_TILE_BYTES; // 96 KiB
        constexpr uint32_t EPI_WARPS     = 8;
        constexpr uint32_t NUM_THREADS   = 64 + EPI_WARPS * 32;
        constexpr uint32_t TMEM_COLS     = 512;
        constexpr uint32_t GROUP_M       = 8;
        constexpr uint32_t EPI_BUF_BYTES = tc05q::EPI_BUF_BYTES;
        constexpr uint32_t EPI_BYTES     = EPI_WARPS * 2 * EPI_BUF_BYTES;
        constexpr uint32_t MISC_BYTES    = 512;
        constexpr uint32_t SMEM_BYTES    = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + MISC_BYTES;
        static_assert(SMEM_BYTES <= 232448, "shared memory budget");

        // D = F32, A = B = TF32 (format 2 of kind::tf32), K-major operands
        constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((TILE_N >> 3) << 17) | ((2 * SUB_M >> 4) << 24);

        __device__ __forceinline__ void mma_tf32_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate)
        {
            asm volatile("{\n"
                         ".reg .pred p;\n"
                         "setp.ne.b32 p, %4, 0;\n"
                         "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n"
                         "}" ::"r"(d_tmem),
                         "l"(a_desc), "l"(b_desc), "r"(IDESC), "r"(accumulate)
                         : "memory");
        }

        __global__ void __launch_bounds__(NUM_THREADS, 1)
            gemm_tc05_f32x3_kernel(const __grid_constant__ CUtensorMap tmap_ahi, const __grid_constant__ CUtensorMap tmap_alo,
                                   const __grid_constant__ CUtensorMap tmap_bhi, const __grid_constant__ CUtensorMap tmap_blo,
                                   const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_d,
                                   const float* __restrict__ c, float* __restrict__ d, uint32_t m, uint32_t n, uint32_t k,
                                   uint32_t ldc, uint32_t ldd, float alpha, float beta, uint32_t tiles_m, uint32_t tiles_n,
                                   int vec_ok, uint32_t group_m, unsigned* status)
        {
            extern __shared__ uint8_t smem_raw[];
            const uint32_t            raw_addr = ptx::smem_u32(smem_raw);
            const uint32_t            base     = (raw_addr + 1023u) & ~1023u;
            uint8_t*                  smem     = smem_raw + (base - raw_addr);

            // per stage: [A hi][A lo][B hi][B lo]; then the epilogue staging tiles and the barriers
            const uint32_t     epi_off    = STAGES * STAGE_BYTES;
            const uint32_t     misc_off   = epi_off + EPI_BYTES;
            const uint32_t     bar_base   = base + misc_off;
            const uint32_t     full_bar   = bar_base;
            const uint32_t     empty_bar  = bar_base + 32;
            const uint32_t     tfull_bar  = bar_base + 64;
            const uint32_t     tempty_bar = bar_base + 72;
            const uint32_t     cbar_base  = bar_base + 96;
            uint32_t*          tmem_slot  = reinterpret_cast<uint32_t*>(smem + misc_off + 96 + EPI_WARPS * 16);
            volatile uint32_t* cta_abort  = tmem_slot + 1;

            const uint32_t warp      = threadIdx.x >> 5;
            const uint32_t lane      = threadIdx.x & 31u;
            const uint32_t rank      = ptx::cluster_ctarank();
            const uint32_t pair      = blockIdx.x >> 1;
            const uint32_t num_pairs = gridDim.x >> 1;
            const uint32_t num_tiles = tiles_m * tiles_n;
            const uint32_t num_kb    = (k + SLAB_K - 1) / SLAB_K;

            if(threadIdx.x == 0)
            {
                ptx::prefetch_tensormap(&tmap_ahi);
                ptx::prefetch_tensormap(&tmap_alo);
                ptx::prefetch_tensormap(&tmap_bhi);
                ptx::prefetch_tensormap(&tmap_blo);
                ptx::prefetch_tensormap(&tmap_c);
                ptx::prefetch_tensormap(&tmap_d);
                for(uint32_t s = 0; s < STAGES; ++s)
                {
                    ptx::mbar_init(full_bar + 8 * s, 1);
                    ptx::mbar_init(empty_bar + 8 * s, 1);
                }
                ptx::mbar_init(tfull_bar, 1);
                ptx::mbar_init(tempty_bar, 8);
                ptx::mbar_init(tempty_bar + 8, 8);
                for(uint32_t i = 0; i < EPI_WARPS * 2; ++i)
                    ptx::mbar_init(cbar_base + 8 * i, 1);
                *cta_abort = 0u;
                ptx::fence_barrier_init();
                ptx::fence_proxy_async_smem();
            }
            if(warp == 1)
            {
                ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), TMEM_COLS);
                ptx::tmem_relinquish_pair();
            }
            ptx::tc_fence_before_sync();
            ptx::cluster_sync();
            ptx::tc_fence_after_sync();
            const uint32_t tmem_base = *tmem_slot;

            if(warp == 0)
            {
                // ------------------------------ TMA producer (both CTAs) ------------------------------
                if(lane == 0)
                {
                    uint32_t stage = 0, phase = 0;
                    bool     ok = true;
                    for(uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs)
                    {
                        uint32_t m_idx, n_idx;
                        tile_coords(tile, tiles_m, tiles_n, group_m, m_idx, n_idx);
                        const int32_t row_a = static_cast<int32_t>(m_idx * PAIR_M + rank * CTA_M);
                        const int32_t row_b = static_cast<int32_t>(n_idx * TILE_N + rank * HALF_N);
                        for(uint32_t kb = 0; kb < num_kb; ++kb)
                        {
                            ok = ptx::mbar_wait_bounded(empty_bar + 8 * stage, phase ^ 1u, cta_abort, status,
                                                        (ROLE_PRODUCER << 24) | blockIdx.x, WAIT_TIMEOUT_NS);
                            if(!ok)
                                break;
                            if(rank == 0)
                                ptx::mbar_arrive_expect_tx(full_bar + 8 * stage, 2u * STAGE_BYTES);
                            const uint32_t leader_full = ptx::mapa(full_bar + 8 * stage, 0u);
                            const uint32_t st          = base + stage * STAGE_BYTES;
                            const int32_t  kc          = static_cast<int32_t>(kb * SLAB_K); // 32 elements = 128 bytes
                            ptx::tma_load_2d_pair(st, &tmap_ahi, kc, row_a, leader_full);
                            ptx::tma_load_2d_pair(st + 2 * A_TILE_BYTES, &tmap_bhi, kc, row_b, leader_full);
                            ptx::tma_load_2d_pair(st + A_TILE_BYTES, &tmap_alo, kc, row_a, leader_full);
                            ptx::tma_load_2d_pair(st + 2 * A_TILE_BYTES + B_TILE_BYTES, &tmap_blo, kc, row_b, leader_full);
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
                // ------------------------------- MMA issuer (leader only) -------------------------------
                if(lane == 0 && rank == 0)
                {
                    uint32_t stage = 0, phase = 0, iter = 0;
                    bool     ok = true;
                    for(uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs, ++iter)
                    {
                        const uint32_t tphase = iter & 1u;
                        for(uint32_t kb = 0; kb < num_kb && ok; ++kb)
                        {
                            ok = ptx::mbar_wait_bounded(full_bar + 8 * stage, phase, cta_abort, status,
                                                        (ROLE_MMA << 24) | (1u << 20) | blockIdx.x, WAIT_TIMEOUT_NS);
                            if(!ok)
                                break;
                            ptx::tc_fence_after_sync();
                            const uint32_t st   = base + stage * STAGE_BYTES;
                            const uint64_t b_hi = ptx::make_kmajor_sw128_desc(st + 2 * A_TILE_BYTES);
                            const uint64_t b_lo = ptx::make_kmajor_sw128_desc(st + 2 * A_TILE_BYTES + B_TILE_BYTES);
#pragma unroll
                            for(uint32_t j = 0; j < 2; ++j)
                            {
                                if(kb == 0)
                                {
                                    ok = ptx::mbar_wait_bounded(tempty_bar + 8 * j, tphase ^ 1u, cta_abort, status,
                                                                (ROLE_MMA << 24) | blockIdx.x, WAIT_TIMEOUT_NS);
                                    if(!ok)
                                        break;
                                    ptx::tc_fence_after_sync();
                                }
                                const uint64_t a_hi = ptx::make_kmajor_sw128_desc(st + j * (SUB_M * BLOCK_K_BYTES));
                                const uint64_t a_lo = ptx::make_kmajor_sw128_desc(st + A_TILE_BYTES + j * (SUB_M * BLOCK_K_BYTES));
                                const uint32_t acc  = tmem_base + j * TILE_N;
#pragma unroll
                                for(uint32_t ks = 0; ks < BLOCK_K_BYTES / 32; ++ks)
                                {
                                    // 8 fp32 (32 bytes) of K per MMA; the two small products first
                                    mma_tf32_ss_pair(acc, a_lo + 2 * ks, b_hi + 2 * ks, (kb | ks) != 0u ? 1u : 0u);
                                    mma_tf32_ss_pair(acc, a_hi + 2 * ks, b_lo + 2 * ks, 1u);
                                    mma_tf32_ss_pair(acc, a_hi + 2 * ks, b_hi + 2 * ks, 1u);
                                }
                            }
                            if(!ok)
                                break;
                            ptx::tc_commit_pair(empty_bar + 8 * stage, 0x3);
                            if(++stage == STAGES)
                            {
                                stage = 0;
                                phase ^= 1u;
                            }
                        }
                        if(ok)
                            ptx::tc_commit_pair(tfull_bar, 0x3);
                    }
                }
                __syncwarp();
            }
            else
            {
                // -------------------------------- epilogue (both CTAs) --------------------------------
                const uint32_t e       = warp - 2u;
                const uint32_t quad    = warp & 3u;
                const uint32_t j       = e >> 2;
                const bool     read_c  = (beta != 0.0f) && (c != nullptr);
                const uint32_t buf_off = epi_off + e * 2u * EPI_BUF_BYTES;
                const uint32_t buf0    = base + buf_off;
                const uint32_t cbar0   = cbar_base + e * 16u;
                using Drain            = tc05q::StagedDrain<float, float, TILE_N>;
                uint32_t iter = 0, cpar = 0;
                bool     ok   = true;
                for(uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs, ++iter)
                {
                    uint32_t m_idx, n_idx;
                    tile_coords(tile, tiles_m, tiles_n, group_m, m_idx, n_idx);
                    const uint32_t row_base = m_idx * PAIR_M + rank * CTA_M + j * SUB_M;
                    const uint32_t row0     = row_base + quad * 32u;
                    const uint32_t col_base = n_idx * TILE_N;
                    const bool     staged   = vec_ok != 0 && row0 < m && col_base < n;
                    if(staged && read_c && lane == 0)
                        Drain::prefetch_c(&tmap_c, buf0, cbar0, col_base, row0, n);
                    ok = ptx::mbar_wait_bounded_warp(tfull_bar, iter & 1u, cta_abort, status,
                                                     (ROLE_EPILOGUE << 24) | blockIdx.x, WAIT_TIMEOUT_NS, lane);
                    if(!ok)
                        break;
                    ptx::tc_fence_after_sync();
                    const uint32_t tmem_acc = tmem_base + j * TILE_N;
                    if(staged)
                        ok = Drain::run(tmem_acc, quad, lane, smem, buf_off, buf0, cbar0, &tmap_c, &tmap_d, col_base, row0, n,
                                        alpha, beta, read_c, cpar, cta_abort, status,
                                        (ROLE_EPILOGUE << 24) | (1u << 20) | blockIdx.x);
                    else if(vec_ok == 0)
                        drain_accumulator<float, float, TILE_N>(tmem_acc, quad, lane, row_base, col_base, m, n, c, d, ldc, ldd,
                                                                alpha, beta, read_c, 0);
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if(lane == 0)
                        ptx::mbar_arrive_cluster(ptx::mapa(tempty_bar + 8 * j, 0u));
                }
                if(lane == 0)
                    ptx::bulk_wait_group<0>();
                __syncwarp();
            }

            // ---------------------------------- teardown ----------------------------------
            ptx::tc_fence_before_sync();
            ptx::cluster_sync();
            {
                const uint32_t peer_abort = ptx::ld_shared_cluster_u32(
                    ptx::mapa(ptx::smem_u32(const_cast<uint32_t*>(cta_abort)), rank ^ 1u));
                if(*cta_abort || peer_abort)
                {
                    const uint64_t t0 = ptx::globaltimer_ns();
                    while(ptx::globaltimer_ns() - t0 < 2000000ull)
                        __nanosleep(1000);
                }
            }
            ptx::cluster_sync();
            if(warp == 1)
            {
                ptx::tc_fence_after_sync();
                ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
            }
        }

        // hi = tf32(x) (round to nearest), lo = tf32(x - hi); 4 elements per thread, compact outputs (pitch k)
        __global__ void __launch_bounds__(256)
            split_tf32_kernel(const float* __restrict__ src, float* __restrict__ hi, float* __restrict__ lo, uint32_t rows,
                              uint32_t k, size_t ld)
        {
            const uint32_t quads = k >> 2;
            const size_t   total = static_cast<size_t>(rows) * quads;
            for(size_t u = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; u < total; u += static_cast<size_t>(gridDim.x) * 256)
            {
                const size_t   row = u / quads;
                const uint32_t q   = static_cast<uint32_t>(u - row * quads);
                const float4   x   = __ldcs(reinterpret_cast<const float4*>(src + row * ld) + q);
                const float    xs[4] = {x.x, x.y, x.z, x.w};
                float          h[4], l[4];
#pragma unroll
                for(int i = 0; i < 4; ++i)
                {
                    uint32_t hb, lb;
                    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(xs[i]));
                    h[i] = __uint_as_float(hb);
                    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lb) : "f"(xs[i] - h[i]));
                    l[i] = __uint_as_float(lb);
                }
                reinterpret_cast<float4*>(hi + row * k)[q] = make_float4(h[0], h[1], h[2], h[3]);
                reinterpret_cast<float4*>(lo + row * k)[q] = make_float4(l[0], l[1], l[2], l[3]);
            }
        }

        // The same split for an operand whose M / N index is the contiguous one (element (row, kk) at src[kk * ld + row],
        // a column-major A or a row-major B): 32 x 32 tiles are transposed through shared memory, so that reads and
        // writes are both coalesced and the outputs are K-major like the other kernel's.
        __global__ void __launch_bounds__(256)
            split_tf32_transposed_kernel(const float* __restrict__ src, float* __restrict__ hi, float* __restrict__ lo, uint32_t rows,
                                         uint32_t k, size_t ld)
        {
            __shared__ float th[32][33], tl[32][33];
            const uint32_t   tx = threadIdx.x & 31u, ty = threadIdx.x >> 5; // 32 x 8
            const uint32_t   tiles_r = (rows + 31u) / 32u, tiles_k = (k + 31u) / 32u;
            for(uint32_t t = blockIdx.x; t < tiles_r * tiles_k; t += gridDim.x)
            {
                const uint32_t r0 = (t % tiles_r) * 32u, k0 = (t / tiles_r) * 32u;
#pragma unroll
                for(uint32_t i = 0; i < 4; ++i)
                {
                    const uint32_t kk = k0 + ty + 8u * i, r = r0 + tx;
                    float          x  = 0.0f;
                    if(kk < k && r < rows)
                        x = __ldcs(src + static_cast<size_t>(kk) * ld + r);
                    uint32_t hb, lb;
                    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(x));
                    const float h = __uint_as_float(hb);
                    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lb) : "f"(x - h));
                    th[ty + 8u * i][tx] = h;
                    tl[ty + 8u * i][tx] = __uint_as_float(lb);
                }
                __syncthreads();
#pragma unroll
                for(uint32_t i = 0; i < 4; ++i)
                {
                    const uint32_t r = r0 + ty + 8u * i, kk = k0 + tx;
                    if(r < rows && kk < k)
                    {
                        hi[static_cast<size_t>(r) * k + kk] = th[tx][ty + 8u * i];
                        lo[static_cast<size_t>(r) * k + kk] = tl[tx][ty + 8u * i];
                    }
                }
                __syncthreads();
            }
        }

        static size_t round256(size_t x)
        {
            return (x + 255) & ~static_cast<size_t>(255);
        }
    } // namespace tc05t

    size_t gemm_f32_workspace_bytes(uint32_t m, uint32_t n, uint32_t k)
    {
        return 2 * tc05t::round256(static_cast<size_t>(m) * k * 4) + 2 * tc05t::round256(static_cast<size_t>(n) * k * 4);
    }

    int launch_gemm_tc05_f32(uint32_t m, uint32_t n, uint32_t k, const float* a, const float* b, const float* c, float* d,
                             uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, float alpha, float beta, void* workspace,
                             size_t workspace_bytes, cudaStream_t stream, bool a_mn, bool b_mn)
    {
        // a_mn: A is column-major (element (i, h) at a[h * lda + i]); b_mn: B is row-major (element (h, j) at b[h * ldb + j]).
        // Either way the split pre-pass leaves K-major hi / lo copies, so the GEMM kernel itself knows one layout only.
        using namespace tc05t;
        B200_REQUIRE(m && n && k, B200WMMA_ERR_INVALID_ARG, "gemm_f32: m, n, k must be non-zero");
        B200_REQUIRE(a && b && d && workspace, B200WMMA_ERR_INVALID_ARG, "gemm_f32: a, b, d, workspace must be non-null");
        B200_REQUIRE(c || beta == 0.0f, B200WMMA_ERR_INVALID_ARG, "gemm_f32: c may be null only when beta == 0");
        B200_REQUIRE(lda >= (a_mn ? m : k) && ldb >= (b_mn ? n : k) && ldd >= n && (!c || ldc >= n), B200WMMA_ERR_INVALID_ARG,
                     "gemm_f32: leading dimension smaller than the row / column it strides");
        B200_REQUIRE(k % 4 == 0, B200WMMA_ERR_UNSUPPORTED, "gemm_f32: k must be a multiple of 4");
        B200_REQUIRE((a_mn || (aligned16(a) && lda % 4 == 0)) && (b_mn || (aligned16(b) && ldb % 4 == 0)) && aligned16(workspace),
                     B200WMMA_ERR_ALIGNMENT,
                     "gemm_f32: the rows of an operand stored with K contiguous, and the workspace, must be 16-byte aligned");
        B200_REQUIRE(workspace_bytes >= gemm_f32_workspace_bytes(m, n, k), B200WMMA_ERR_INVALID_ARG,
                     "gemm_f32: workspace too small (%zu < %zu bytes)", workspace_bytes, gemm_f32_workspace_bytes(m, n, k));
        if(int e = require_sm100())
            return e;
        unsigned* status = nullptr;
        if(int e = status_word_ptr(&status))
            return e;

        uint8_t* ws   = static_cast<uint8_t*>(workspace);
        float*   a_hi = reinterpret_cast<float*>(ws);
        float*   a_lo = reinterpret_cast<float*>(ws + round256(static_cast<size_t>(m) * k * 4));
        float*   b_hi = reinterpret_cast<float*>(ws + 2 * round256(static_cast<size_t>(m) * k * 4));
        float*   b_lo = reinterpret_cast<float*>(ws + 2 * round256(static_cast<size_t>(m) * k * 4)
                                               + round256(static_cast<size_t>(n) * k * 4));
        auto grid_for = [](size_t units) {
            const size_t want = (units + 255) / 256;
            return static_cast<uint32_t>(want < 148u * 16u ? (want ? want : 1) : 148u * 16u);
        };
        const auto tiles32 = [](uint32_t rows, uint32_t kk) { return static_cast<size_t>((rows + 31) / 32) * ((kk + 31) / 32) * 256; };
        if(a_mn)
            split_tf32_transposed_kernel<<<grid_for(tiles32(m, k)), 256, 0, stream>>>(a, a_hi, a_lo, m, k, lda);
        else
            split_tf32_kernel<<<grid_for(static_cast<size_t>(m) * (k / 4)), 256, 0, stream>>>(a, a_hi, a_lo, m, k, lda);
        if(b_mn)
            split_tf32_transposed_kernel<<<grid_for(tiles32(n, k)), 256, 0, stream>>>(b, b_hi, b_lo, n, k, ldb);
        else
            split_tf32_kernel<<<grid_for(static_cast<size_t>(n) * (k / 4)), 256, 0, stream>>>(b, b_hi, b_lo, n, k, ldb);
        B200_CHECK_CUDA(cudaGetLastError());

        auto row_align = [](const void* p, uint32_t ld) {
            return (reinterpret_cast<uintptr_t>(p) % 16) == 0 && (static_cast<uint64_t>(ld) * 4) % 16 == 0;
        };
        const int   vec_ok = (row_align(d, ldd) && (!c || row_align(c, ldc))) ? 1 : 0;
        CUtensorMap tm_ahi, tm_alo, tm_bhi, tm_blo;
        const auto  dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
        if(int e = make_kmajor_tmap(&tm_ahi, dt, 4, a_hi, m, k, k, CTA_M))
            return e;
        if(int e = make_kmajor_tmap(&tm_alo, dt, 4, a_lo, m, k, k, CTA_M))
            return e;
        if(int e = make_kmajor_tmap(&tm_bhi, dt, 4, b_hi, n, k, k, HALF_N))
            return e;
        if(int e = make_kmajor_tmap(&tm_blo, dt, 4, b_lo, n, k, k, HALF_N))
            return e;
        CUtensorMap tm_c = tm_ahi, tm_d = tm_ahi; // placeholders, never dereferenced when vec_ok == 0
        if(vec_ok != 0)
        {
            if(int e = make_rowbox_tmap(&tm_d, 4, d, m, n, ldd))
                return e;
            tm_c = tm_d;
            if(c)
                if(int e = make_rowbox_tmap(&tm_c, 4, c, m, n, ldc))
                    return e;
        }
        int dev = 0, sms = 0;
        B200_CHECK_CUDA(cudaGetDevice(&dev));
        B200_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        static int     max_clusters_dev[MAX_DEVICES];
        int&           max_clusters = max_clusters_dev[current_device_slot()];
        const uint32_t tiles_m = ceil_div(m, PAIR_M), tiles_n = ceil_div(n, TILE_N);
        cudaLaunchConfig_t  cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id               = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.blockDim         = dim3(NUM_THREADS);
        cfg.dynamicSmemBytes = SMEM_BYTES;
        cfg.stream           = stream;
        cfg.attrs            = attr;
        cfg.numAttrs         = 1;
        if(max_clusters == 0)
        {
            B200_CHECK_CUDA(cudaFuncSetAttribute(gemm_tc05_f32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
            cfg.gridDim = dim3(static_cast<unsigned>(sms) & ~1u);
            int nc      = 0;
            B200_CHECK_CUDA(cudaOccupancyMaxActiveClusters(&nc, gemm_tc05_f32x3_kernel, &cfg));
            B200_REQUIRE(nc > 0, B200WMMA_ERR_CUDA, "no two-CTA cluster of the fp32 GEMM kernel fits on this device");
            max_clusters = nc;
        }
        const uint32_t pairs = min(tiles_m * tiles_n, static_cast<uint32_t>(max_clusters));
        cfg.gridDim          = dim3(2 * pairs);
        B200_CHECK_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc05_f32x3_kernel, tm_ahi, tm_alo, tm_bhi, tm_blo, tm_c, tm_d, c, d, m, n, k,
                                           ldc, ldd, alpha, beta, tiles_m, tiles_n, vec_ok, static_cast<uint32_t>(GROUP_M), status));
        return B200WMMA_OK;
    }
} // namespace b200wmma
