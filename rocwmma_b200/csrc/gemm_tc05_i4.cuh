// int4 x int4 -> int32 GEMM with both operands unpacked to int8 in the load path (no pass over HBM, no workspace).
//
// The sm_100 tensor cores have no 4-bit integer kind, so the packed operands (two values per byte along K, low
// nibble = even k) have to become int8 before tcgen05.mma.kind::i8 reads them.  Here that happens inside the
// kernel, between the TMA load and the MMA:
//
//   TMA (packed bytes, 64 B of K per row)  ->  raw ring, 2 stages of 24 KiB, unswizzled
//   16 worker warps turn nibbles into bytes ->  int8 ring, 3 stages of 48 KiB in the K-major SWIZZLE_128B layout the
//                                               MMA descriptors of the dense int8 kernel expect
//   fence.proxy.async + mbarrier            ->  tcgen05.mma.cta_group::2.kind::i8, accumulators in tensor memory
//
// Tile shape, pairing, tensor-memory use and the epilogue are those of the 512 x 256 pair kernel
// (gemm_tc05_pair512.cuh): 256 rows of A and half of the B slab per CTA, two 128 x 256 int32 accumulators, D (and
// C) staged through swizzled shared-memory tiles and moved by TMA.  The sixteen worker warps convert while a
// tile is being multiplied and drain the accumulators when it is complete, so the kernel needs no more threads than
// the dense one.  HBM traffic is the packed operands plus C / D: nothing is written back in int8.
//
// The conversion is on the critical path (an int8 stage has to be rewritten within one stage's worth of MMA time), so
// its instruction count matters.  SCALED = true moves every nibble into the HIGH half of its byte, which yields the
// int8 value 16 * v without any sign extension (and the values are not interleaved back into K order, see unpack8: 3
// instead of 9 instructions per 8 values); the accumulators are then
// 256 times the true sums and the drain shifts them right by 8, which is exact.  That holds while 256 * |sum| fits
// int32: k * 128 * 128 < 2^31, i.e. k < 131072; longer K runs the sign-extending form (SCALED = false).
//
// Roles (576 threads): warp 0 TMA producer (one lane, both CTAs, each CTA fills its own raw ring), warp 1
// tensor-memory owner / MMA issuer (one lane, leader CTA), warps 2-17 workers.
// Barriers: raw_full / raw_empty per raw stage (local to each CTA); conv_full per int8 stage in the leader CTA,
// counting the worker warps of BOTH CTAs (the MMA reads both CTAs' shared memory); conv_empty per int8 stage in each
// CTA, signalled by the MMA issuer's commits; tmem_full per tile, tmem_empty per accumulator; drain_done per CTA:
// every worker warp has finished with the staging tiles that alias the second int8 stage.
#pragma once
#include "gemm_tc05_pair512.cuh"

namespace b200wmma
{
    namespace tc05i4
    {
        using namespace tc05;

        constexpr uint32_t SUB_M           = 128;
        constexpr uint32_t CTA_M           = 256;
        constexpr uint32_t PAIR_M          = 512;
        constexpr uint32_t TILE_N          = 256;
        constexpr uint32_t HALF_N          = 128;
        // Two raw stages cover the TMA latency; three int8 stages let the unpacking run two slabs ahead of the MMAs
        // instead of one (with 4 + 2 in the same shared memory the two were coupled slab by slab: 2935 against 2989 TOP/s
        // sustained).
        constexpr uint32_t RAW_STAGES      = 2;
        constexpr uint32_t CONV_STAGES     = 3;
        static_assert(RAW_STAGES <= 4 && CONV_STAGES <= 4, "barrier layout below holds four of each");
        constexpr uint32_t RAW_ROW_BYTES   = BLOCK_K_BYTES / 2; // 64 packed bytes = 128 int4 = one K slab
        constexpr uint32_t RAW_A_BYTES     = CTA_M * RAW_ROW_BYTES; // 16 KiB
        constexpr uint32_t RAW_B_BYTES     = HALF_N * RAW_ROW_BYTES; // 8 KiB
        constexpr uint32_t RAW_STAGE_BYTES = RAW_A_BYTES + RAW_B_BYTES;
        constexpr uint32_t A_STAGE_BYTES   = CTA_M * BLOCK_K_BYTES; // 32 KiB
        constexpr uint32_t B_STAGE_BYTES   = HALF_N * BLOCK_K_BYTES; // 16 KiB
        constexpr uint32_t WORK_WARPS      = 16;
        constexpr uint32_t NUM_THREADS     = 64 + WORK_WARPS * 32;
        constexpr uint32_t TMEM_COLS       = 512;
        constexpr uint32_t GROUP_M         = 8;
        constexpr uint32_t EPI_BUF_BYTES   = 2048; // 32 rows x 64 bytes
        constexpr uint32_t EPI_BYTES       = WORK_WARPS * EPI_BUF_BYTES;
        constexpr uint32_t MISC_BYTES      = 512;
        constexpr uint32_t SMEM_BYTES      = 1024 + CONV_STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + RAW_STAGES * RAW_STAGE_BYTES
                                        + EPI_BYTES + MISC_BYTES;
        constexpr uint32_t CHUNKS_A        = RAW_A_BYTES / 16; // 16-byte packed chunks per stage
        constexpr uint32_t CHUNKS_B        = RAW_B_BYTES / 16;
        constexpr uint32_t CHUNKS_PER_PASS = WORK_WARPS * 32;
        static_assert(CHUNKS_A % CHUNKS_PER_PASS == 0 && CHUNKS_B % CHUNKS_PER_PASS == 0, "whole passes over A and B");
        static_assert(WORK_WARPS * EPI_BUF_BYTES <= A_STAGE_BYTES, "aliased staging tiles fit the A region of an int8 stage");

        // 4 packed bytes (8 int4, low nibble = even k) -> 8 int8, even K positions first (see the end of the function).
        // A nibble v in a byte of its own sign-extends to v + 0xF0 when bit 3 is set: (v & 8) * 0x1E == 0xF0, and the
        // sum cannot carry into the next byte.
        template <bool SCALED>
        __device__ __forceinline__ void unpack8(uint32_t x, uint32_t& out0, uint32_t& out1)
        {
            uint32_t los, his;
            if constexpr(SCALED)
            {
                los = (x << 4) & 0xF0F0F0F0u; // 16 * low nibble as a signed byte
                his = x & 0xF0F0F0F0u; // 16 * high nibble
            }
            else
            {
                const uint32_t lo = x & 0x0F0F0F0Fu, hi = (x >> 4) & 0x0F0F0F0Fu;
                los = lo + (lo & 0x08080808u) * 0x1Eu;
                his = hi + (hi & 0x08080808u) * 0x1Eu;
            }
            // The even-k values and the odd-k values stay in words of their own: A and B are unpacked by this same
            // function, so both see the same permutation of the eight K positions, and a sum over K does not care about
            // their order (interleaving them back would cost two more instructions per word).
            out0 = los; // k = 0, 2, 4, 6 of the eight
            out1 = his; // k = 1, 3, 5, 7
        }

        // One 16-byte packed chunk (32 values) of row `row`, chunk j (0..3) of the slab -> 32 bytes = 16-byte cells
        // 2j and 2j+1 of that row in a K-major SWIZZLE_128B tile at `tile` (row r at r * 128 bytes, cell index XOR r % 8).
        template <bool SCALED>
        __device__ __forceinline__ void convert_chunk(const uint8_t* raw_chunk, uint8_t* tile, uint32_t row, uint32_t j)
        {
            const uint4 p = *reinterpret_cast<const uint4*>(raw_chunk);
            uint32_t    o[8];
            unpack8<SCALED>(p.x, o[0], o[1]);
            unpack8<SCALED>(p.y, o[2], o[3]);
            unpack8<SCALED>(p.z, o[4], o[5]);
            unpack8<SCALED>(p.w, o[6], o[7]);
            uint8_t*       rowp = tile + row * BLOCK_K_BYTES;
            const uint32_t sw   = row & 7u;
            *reinterpret_cast<uint4*>(rowp + (((2u * j) ^ sw) << 4))      = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(rowp + (((2u * j + 1u) ^ sw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
        }

        template <bool SCALED>
        __global__ void __launch_bounds__(NUM_THREADS, 1)
            gemm_tc05_i4_kernel(const __grid_constant__ CUtensorMap tmap_a, // packed A: 64-byte x 256-row boxes, unswizzled
                                const __grid_constant__ CUtensorMap tmap_b, // packed B: 64-byte x 128-row boxes
                                const __grid_constant__ CUtensorMap tmap_c, // 32-row x 64-byte boxes of C
                                const __grid_constant__ CUtensorMap tmap_d, // ... and of D (both unused if vec_ok == 0)
                                const int32_t* __restrict__ c,
                                int32_t* __restrict__ d,
                                uint32_t  m,
                                uint32_t  n,
                                uint32_t  k_packed_bytes, // k / 2
                                uint32_t  ldc,
                                uint32_t  ldd,
                                int32_t   alpha,
                                int32_t   beta,
                                uint32_t  tiles_m,
                                uint32_t  tiles_n,
                                int       vec_ok,
                                uint32_t  group_m,
                                unsigned* status)
        {
            extern __shared__ uint8_t smem_raw[];
            const uint32_t            raw_addr = ptx::smem_u32(smem_raw);
            const uint32_t            base     = (raw_addr + 1023u) & ~1023u;
            uint8_t*                  smem     = smem_raw + (base - raw_addr);

            // [int8 A stages][int8 B stages][raw stages: A then B each][epilogue staging tiles][barriers ...]
            const uint32_t     conv_a_off = 0;
            const uint32_t     conv_b_off = CONV_STAGES * A_STAGE_BYTES;
            const uint32_t     raw_off    = CONV_STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
            const uint32_t     epi_off    = raw_off + RAW_STAGES * RAW_STAGE_BYTES;
            const uint32_t     misc_off   = epi_off + EPI_BYTES;
            const uint32_t     bar_base   = base + misc_off;
            const uint32_t     raw_full   = bar_base; // RAW_STAGES x 8
            const uint32_t     raw_empty  = bar_base + 32;
            const uint32_t     conv_full  = bar_base + 64; // CONV_STAGES x 8 (leader's copy in use)
            const uint32_t     conv_empty = bar_base + 96;
            const uint32_t     tfull_bar  = bar_base + 128;
            const uint32_t     tempty_bar = bar_base + 136; // 2 x 8 (leader's copy in use)
            const uint32_t     drain_bar  = bar_base + 152;
            const uint32_t     cbar_base  = bar_base + 160; // WORK_WARPS x 2 x 8
            uint32_t*          tmem_slot  = reinterpret_cast<uint32_t*>(smem + misc_off + 160 + WORK_WARPS * 16);
            volatile uint32_t* cta_abort  = tmem_slot + 1;
            const uint32_t     alias_off  = conv_a_off + (CONV_STAGES - 1) * A_STAGE_BYTES; // A region of the last int8 stage

            const uint32_t warp      = threadIdx.x >> 5;
            const uint32_t lane      = threadIdx.x & 31u;
            const uint32_t rank      = ptx::cluster_ctarank();
            const uint32_t pair      = blockIdx.x >> 1;
            const uint32_t num_pairs = gridDim.x >> 1;
            const uint32_t num_tiles = tiles_m * tiles_n;
            const uint32_t num_kb    = (k_packed_bytes + RAW_ROW_BYTES - 1) / RAW_ROW_BYTES;

            if(threadIdx.x == 0)
            {
                ptx::prefetch_tensormap(&tmap_a);
                ptx::prefetch_tensormap(&tmap_b);
                ptx::prefetch_tensormap(&tmap_c);
                ptx::prefetch_tensormap(&tmap_d);
                for(uint32_t s = 0; s < RAW_STAGES; ++s)
                {
                    ptx::mbar_init(raw_full + 8 * s, 1);
                    ptx::mbar_init(raw_empty + 8 * s, WORK_WARPS);
                }
                for(uint32_t s = 0; s < CONV_STAGES; ++s)
                {
                    ptx::mbar_init(conv_full + 8 * s, 2 * WORK_WARPS); // the worker warps of both CTAs
                    ptx::mbar_init(conv_empty + 8 * s, 1);
                }
                ptx::mbar_init(tfull_bar, 1);
                ptx::mbar_init(tempty_bar, 16); // accumulator 0: 8 warps x 2 CTAs
                ptx::mbar_init(tempty_bar + 8, 16);
                ptx::mbar_init(drain_bar, WORK_WARPS);
                for(uint32_t i = 0; i < WORK_WARPS * 2; ++i)
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
                // ------------------------------ TMA producer (both CTAs, own raw ring) ------------------------------
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
                            ok = ptx::mbar_wait_bounded(raw_empty + 8 * stage, phase ^ 1u, cta_abort, status,
                                                        (ROLE_PRODUCER << 24) | blockIdx.x, WAIT_TIMEOUT_NS);
                            if(!ok)
                                break;
                            const uint32_t fb  = raw_full + 8 * stage;
                            const uint32_t dst = base + raw_off + stage * RAW_STAGE_BYTES;
                            ptx::mbar_arrive_expect_tx(fb, RAW_STAGE_BYTES);
                            const int32_t kc = static_cast<int32_t>(kb * RAW_ROW_BYTES); // byte column of the packed rows
                            ptx::tma_load_2d(dst, &tmap_a, kc, row_a, fb);
                            ptx::tma_load_2d(dst + RAW_A_BYTES, &tmap_b, kc, row_b, fb);
                            if(++stage == RAW_STAGES)
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
                    constexpr uint32_t idesc = make_idesc<KIND_I8, 2 * SUB_M, TILE_N>();
                    uint32_t           stage = 0, phase = 0, iter = 0;
                    bool               ok = true;
                    for(uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs, ++iter)
                    {
                        const uint32_t tphase = iter & 1u;
                        for(uint32_t kb = 0; kb < num_kb && ok; ++kb)
                        {
                            ok = ptx::mbar_wait_bounded(conv_full + 8 * stage, phase, cta_abort, status,
                                                        (ROLE_MMA << 24) | (1u << 20) | blockIdx.x, WAIT_TIMEOUT_NS);
                            if(!ok)
                                break;
                            ptx::tc_fence_after_sync();
                            const uint64_t b_desc = ptx::make_kmajor_sw128_desc(base + conv_b_off + stage * B_STAGE_BYTES);
#pragma unroll
                            for(uint32_t j = 0; j < 2; ++j)
                            {
                                if(kb == 0)
                                {
                                    // accumulator j of the previous tile must have been drained by both CTAs
                                    ok = ptx::mbar_wait_bounded(tempty_bar + 8 * j, tphase ^ 1u, cta_abort, status,
                                                                (ROLE_MMA << 24) | blockIdx.x, WAIT_TIMEOUT_NS);
                                    if(!ok)
                                        break;
                                    ptx::tc_fence_after_sync();
                                }
                                const uint64_t a_desc = ptx::make_kmajor_sw128_desc(base + conv_a_off + stage * A_STAGE_BYTES
                                                                                    + j * (SUB_M * BLOCK_K_BYTES));
#pragma unroll
                                for(uint32_t ks = 0; ks < BLOCK_K_BYTES / 32; ++ks)
                                    ptx::mma_i8_ss_pair(tmem_base + j * TILE_N, a_desc + 2u * ks, b_desc + 2u * ks, idesc,
                                                        (kb | ks) != 0u ? 1u : 0u);
                            }
                            if(!ok)
                                break;
                            ptx::tc_commit_pair(conv_empty + 8 * stage, 0x3);
                            if(++stage == CONV_STAGES)
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
                // ---------------- workers (both CTAs): unpack while the tile is multiplied, then drain it ----------------
                const uint32_t e      = warp - 2u; // 0..15
                const uint32_t quad   = warp & 3u; // tensor-memory lane quadrant this warp may read
                const uint32_t j      = (e >> 2) & 1u; // accumulator this warp drains
                const uint32_t first  = e >> 3; // 0: even 64-byte column steps, 1: odd steps
                const bool     read_c = (beta != 0) && (c != nullptr);
                const uint32_t buf_off  = epi_off + e * EPI_BUF_BYTES; // first staging tile: dedicated
                const uint32_t buf0     = base + buf_off;
                const uint32_t buf1_off = alias_off + e * EPI_BUF_BYTES; // second: inside the last int8 stage
                const uint32_t buf1     = base + buf1_off;
                const uint32_t cbar0    = cbar_base + e * 16u;
                const uint32_t conv_full_leader = ptx::mapa(conv_full, 0u);
                constexpr int ACC_SHIFT = SCALED ? 8 : 0; // both operands carry a factor 16
                using Drain             = tc05q::StagedDrain<int32_t, int32_t, TILE_N, 2, 64, ACC_SHIFT>;
                uint32_t rstage = 0, rphase = 0, cstage = 0, cphase = 0, iter = 0, cpar = 0;
                bool     ok = true;
                for(uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs, ++iter)
                {
                    uint32_t m_idx, n_idx;
                    tile_coords(tile, tiles_m, tiles_n, group_m, m_idx, n_idx);
                    const uint32_t row_base = m_idx * PAIR_M + rank * CTA_M + j * SUB_M;
                    const uint32_t row0     = row_base + quad * 32u;
                    const uint32_t col_base = n_idx * TILE_N;
                    const bool     staged   = vec_ok != 0 && row0 < m && col_base < n;
                    if(iter != 0u)
                    {
                        // the last int8 stage held staging tiles of the previous tile's drain: every worker warp's TMA
                        // stores must have read them before anyone unpacks into that stage again
                        ok = ptx::mbar_wait_bounded_warp(drain_bar, (iter - 1u) & 1u, cta_abort, status,
                                                         (ROLE_EPILOGUE << 24) | (3u << 20) | blockIdx.x, WAIT_TIMEOUT_NS, lane);
                        if(!ok)
                            break;
                    }
                    // C does not depend on the accumulators: the tile of the warp's first step is requested now
                    if(staged && read_c && lane == 0)
                        Drain::prefetch_c(&tmap_c, buf0, cbar0, col_base, row0, n, first, 0, 1, buf1);
                    for(uint32_t kb = 0; kb < num_kb; ++kb)
                    {
                        // per-slab waits: every lane polls (one warp instruction per poll), which reacts within tens of
                        // cycles; the long per-tile waits below park one lane instead
                        ok = ptx::mbar_wait_bounded(raw_full + 8 * rstage, rphase, cta_abort, status,
                                                    (ROLE_EPILOGUE << 24) | (4u << 20) | blockIdx.x, WAIT_TIMEOUT_NS);
                        if(ok)
                            ok = ptx::mbar_wait_bounded(conv_empty + 8 * cstage, cphase ^ 1u, cta_abort, status,
                                                        (ROLE_EPILOGUE << 24) | (5u << 20) | blockIdx.x, WAIT_TIMEOUT_NS);
                        ok = __all_sync(0xFFFFFFFFu, ok);
                        if(!ok)
                            break;
                        ptx::tc_fence_after_sync(); // the MMAs that read this int8 stage have completed (commit -> conv_empty)
                        const uint8_t* raw    = smem + raw_off + rstage * RAW_STAGE_BYTES;
                        uint8_t*       tile_a = smem + conv_a_off + cstage * A_STAGE_BYTES;
                        uint8_t*       tile_b = smem + conv_b_off + cstage * B_STAGE_BYTES;
#pragma unroll
                        for(uint32_t pass = 0; pass < CHUNKS_A / CHUNKS_PER_PASS; ++pass)
                        {
                            const uint32_t g = pass * CHUNKS_PER_PASS + e * 32u + lane; // consecutive lanes: consecutive chunks
                            convert_chunk<SCALED>(raw + g * 16u, tile_a, g >> 2, g & 3u);
                        }
#pragma unroll
                        for(uint32_t pass = 0; pass < CHUNKS_B / CHUNKS_PER_PASS; ++pass)
                        {
                            const uint32_t g = pass * CHUNKS_PER_PASS + e * 32u + lane;
                            convert_chunk<SCALED>(raw + RAW_A_BYTES + g * 16u, tile_b, g >> 2, g & 3u);
                        }
                        ptx::fence_proxy_async_smem(); // the int8 tile written above -> visible to the tensor core
                        __syncwarp();
                        if(lane == 0)
                        {
                            ptx::mbar_arrive_cluster(conv_full_leader + 8 * cstage);
                            ptx::mbar_arrive(raw_empty + 8 * rstage);
                        }
                        if(++rstage == RAW_STAGES)
                        {
                            rstage = 0;
                            rphase ^= 1u;
                        }
                        if(++cstage == CONV_STAGES)
                        {
                            cstage = 0;
                            cphase ^= 1u;
                        }
                    }
                    if(!ok)
                        break;
                    ok = ptx::mbar_wait_bounded_warp(tfull_bar, iter & 1u, cta_abort, status,
                                                     (ROLE_EPILOGUE << 24) | blockIdx.x, WAIT_TIMEOUT_NS, lane);
                    if(!ok)
                        break;
                    ptx::tc_fence_after_sync();
                    // every MMA of the tile has retired: the aliased staging tiles may be written now
                    if(staged && read_c && lane == 0)
                        Drain::prefetch_c(&tmap_c, buf0, cbar0, col_base, row0, n, first, 1, 2, buf1);
                    const uint32_t tmem_acc = tmem_base + j * TILE_N;
                    if(staged)
                        ok = Drain::run(tmem_acc, quad, lane, smem, buf_off, buf0, cbar0, &tmap_c, &tmap_d, col_base, row0, n,
                                        alpha, beta, read_c, cpar, cta_abort, status,
                                        (ROLE_EPILOGUE << 24) | (1u << 20) | blockIdx.x, first, buf1_off, buf1);
                    else if(vec_ok == 0 && first == 0u)
                        drain_accumulator<int32_t, int32_t, TILE_N, ACC_SHIFT>(tmem_acc, quad, lane, row_base, col_base, m, n, c, d, ldc,
                                                                    ldd, alpha, beta, read_c, 0);
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if(lane == 0)
                    {
                        ptx::mbar_arrive_cluster(ptx::mapa(tempty_bar + 8 * j, 0u));
                        ptx::bulk_wait_group_read<0>(); // this warp's stores have read its staging tiles
                        ptx::mbar_arrive(drain_bar);
                    }
                }
                if(lane == 0)
                    ptx::bulk_wait_group<0>(); // the staging tiles must outlive the stores that read them
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
    } // namespace tc05i4
} // namespace b200wmma
