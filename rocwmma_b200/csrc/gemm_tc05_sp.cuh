// 2:4 structured-sparse int8 GEMM on the sparse tensor-core path (tcgen05.mma.sp, kind::i8).
//
// rocWMMA v1.6.0 has no sparse GEMM; the semantics are the dense int8 GEMM of
// gemm_rocwmma_d (samples/perf_hgemm.cpp:515-711 with the int8 / int32 types of
// test/gemm/gemm_common_test_params.hpp:51-147) applied to the densified A, bit-exact in int32.
//
// A never exists in dense form on the device.  The kernel streams the compressed values
// (m x k/2 bytes) and the position metadata (m x k/8 bytes) as they are, 256 logical K per slab:
//   * values: one TMA box of 128 bytes x 256 rows, 128-byte swizzle;
//   * metadata: two TMA boxes of 16 bytes x 256 rows (one per 128 K), unswizzled (row r at r * 16
//     bytes).  A tcgen05.cp per box moves both 128-row sub-tiles (4 KiB) into 8 tensor-memory
//     columns, 4 per sub-tile, where the MMAs read them (2 columns = 64 logical K each).  The byte
//     format of the C interface - one nibble idx0 | idx1 << 2 per group of four K positions, low
//     nibble = even group - is the hardware's own, so no repacking pass is needed;
//   * B: two TMA boxes of 128 bytes x 112 rows, 128-byte swizzle (each CTA of the pair loads half of N).
// One tcgen05.mma.sp consumes 32 bytes per row of compressed A and 64 bytes per row of B: twice the
// logical K of a dense int8 MMA per instruction, in the same 112 clocks (measured, N = 224, pair).
//
// Tile: 512 x 224 per SM pair.  Each CTA owns 256 rows (two 128-lane accumulators of 224 columns =
// 448 tensor-memory columns); the metadata needs 16 columns per pipeline stage (3 stages = 48),
// which is why N is 224 and not 256: 2 x 256 accumulator columns would leave no room for it.  The
// tall tile keeps the L2 -> shared-memory traffic at ~78 bytes per clock per SM at full sparse rate.
//
// Why 256 K per slab: the eight MMAs of a slab run for 896 clocks, and ONE thread issues them,
// waits for the slab, copies its metadata and commits.  With 128 K per slab that thread needed
// ~620 clocks of its own instruction latency per 448 clocks of tensor work and the tensor pipe
// idled a quarter of the time; with 256 K the per-slab overhead is paid half as often.
//
// Shared memory: 3 stages x 68 KiB leave no room for the epilogue's staging tiles (eight warps x two tiles
// of 32 rows x 128 bytes), so those alias the A and B regions of the last stage (the last warp's second tile
// has 4 KiB of its own).  While a tile is drained that stage is not refilled:
// the producer waits for a counter the epilogue warps bump once their TMA stores have read the
// tiles (two stages = 136 KiB of the next tile are prefetched meanwhile).
//
// Roles and barrier protocol are those of gemm_tc05_pair512.cuh: warp 0 TMA producer (one lane,
// both CTAs, loads counted on the leader's full[s]), warp 1 tensor-memory owner and MMA issuer (one
// lane, leader only; commits signal both CTAs), warps 2-9 epilogue through TMA-staged C / D tiles.
// Every wait is bounded.
#pragma once
#include "gemm_tc05_common.cuh"
#include "gemm_tc05_pair512.cuh"

namespace b200wmma
{
    namespace tc05s
    {
        using namespace tc05;

        constexpr uint32_t SUB_M         = 128; // rows per MMA per CTA
        constexpr uint32_t CTA_M         = 256; // rows of A / D per CTA (two accumulators)
        constexpr uint32_t PAIR_M        = 512;
        constexpr uint32_t TILE_N        = 224;
        constexpr uint32_t HALF_N        = 112;
        constexpr uint32_t SLAB_K        = 256; // logical K per pipeline stage
        constexpr uint32_t HALF_K        = 128; // logical K per metadata / B box
        constexpr uint32_t STAGES        = 3;
        constexpr uint32_t A_ROW_BYTES   = SLAB_K / 2; // 128: compressed values
        constexpr uint32_t E_ROW_BYTES   = HALF_K / 8; // 16: metadata of 128 K
        constexpr uint32_t A_STAGE_BYTES = CTA_M * A_ROW_BYTES; // 32 KiB
        constexpr uint32_t E_BOX_BYTES   = CTA_M * E_ROW_BYTES; // 4 KiB per 128 K
        constexpr uint32_t E_STAGE_BYTES = 2 * E_BOX_BYTES; // 8 KiB
        constexpr uint32_t B_BOX_BYTES   = HALF_N * HALF_K; // 14 KiB per 128 K
        constexpr uint32_t B_STAGE_BYTES = 2 * B_BOX_BYTES; // 28 KiB
        constexpr uint32_t STAGE_BYTES   = A_STAGE_BYTES + E_STAGE_BYTES + B_STAGE_BYTES; // 68 KiB
        constexpr uint32_t EPI_WARPS     = 8;
        constexpr uint32_t NUM_THREADS   = 64 + EPI_WARPS * 32;
        constexpr uint32_t TMEM_COLS     = 512;
        constexpr uint32_t E_COL0        = 2 * TILE_N; // metadata columns: E_COL0 + 16 * stage + 8 * K half + 4 * sub-tile
        constexpr uint32_t GROUP_M       = 8;
        constexpr uint32_t EPI_ROW_BYTES = 128; // staging tiles: 32 rows x 128 bytes, TMA SWIZZLE_128B
        constexpr uint32_t EPI_BUF_BYTES = 32 * EPI_ROW_BYTES;
        constexpr uint32_t EPI_BYTES     = EPI_WARPS * EPI_BUF_BYTES; // first staging tiles: alias the A region of the last stage
        constexpr uint32_t EPI_IN_B      = B_STAGE_BYTES / EPI_BUF_BYTES; // second staging tiles that fit in its B region
        constexpr uint32_t EPI_EXTRA     = (EPI_WARPS - EPI_IN_B) * EPI_BUF_BYTES; // the rest have memory of their own
        constexpr uint32_t EPI_STAGE     = STAGES - 1;
        constexpr uint32_t E_PACKED_ROWS = E_STAGE_BYTES / 128; // 128-byte rows of one re-tiled metadata block
        constexpr uint32_t MISC_BYTES    = 1024;
        constexpr uint32_t SMEM_BYTES    = 1024 + STAGES * STAGE_BYTES + MISC_BYTES + EPI_EXTRA;
        static_assert(E_COL0 + 16 * STAGES <= TMEM_COLS, "metadata does not fit beside the accumulators");
        static_assert(EPI_BYTES <= A_STAGE_BYTES && EPI_IN_B <= EPI_WARPS, "staging tiles must fit in one A stage");
        static_assert(SMEM_BYTES <= 232448, "shared memory budget");

        // E_PACKED: the metadata comes from a re-tiled copy (repack_meta_kernel) instead of the caller's
        // row-major array: one box of 64 x 128 bytes per slab instead of two boxes of 256 x 16 bytes.
        template <bool E_PACKED>
        __global__ void __launch_bounds__(NUM_THREADS, 1)
            gemm_tc05_sp_kernel(const __grid_constant__ CUtensorMap tmap_a, // compressed values, 128 B x 256 rows, SW128
                                const __grid_constant__ CUtensorMap tmap_e, // metadata: 16 B x 256 rows, or 128 B x 64 rows of the re-tiled copy
                                const __grid_constant__ CUtensorMap tmap_b, // B^T rows, 128 B x 112 rows, SW128
                                const __grid_constant__ CUtensorMap tmap_c,
                                const __grid_constant__ CUtensorMap tmap_d,
                                const int32_t* __restrict__ c,
                                int32_t* __restrict__ d,
                                uint32_t  m,
                                uint32_t  n,
                                uint32_t  k, // logical K, a multiple of HALF_K
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

            // [A stages][B stages][E stages][barriers, tensor-memory slot, abort flag, epilogue counter];
            // the epilogue staging tiles alias A stage EPI_STAGE
            const uint32_t     smem_a     = base;
            const uint32_t     smem_b     = smem_a + STAGES * A_STAGE_BYTES;
            const uint32_t     smem_e     = smem_b + STAGES * B_STAGE_BYTES;
            const uint32_t     epi_off    = EPI_STAGE * A_STAGE_BYTES;
            const uint32_t     epi_b_off  = STAGES * A_STAGE_BYTES + EPI_STAGE * B_STAGE_BYTES; // B region of the same stage
            const uint32_t     epi_x_off  = STAGES * STAGE_BYTES + MISC_BYTES; // staging tiles that alias nothing
            const uint32_t     misc_off   = STAGES * STAGE_BYTES;
            const uint32_t     bar_base   = base + misc_off;
            const uint32_t     full_bar   = bar_base; // STAGES x 8 (leader's copy in use)
            const uint32_t     empty_bar  = bar_base + 64;
            const uint32_t     tfull_bar  = bar_base + 128;
            const uint32_t     tempty_bar = bar_base + 136; // 2 x 8, one per accumulator (leader's copy in use)
            const uint32_t     cbar_base  = bar_base + 160; // EPI_WARPS x 2 x 8
            uint32_t*          tmem_slot  = reinterpret_cast<uint32_t*>(smem + misc_off + 160 + EPI_WARPS * 16);
            volatile uint32_t* cta_abort  = tmem_slot + 1;
            uint32_t*          epi_count  = tmem_slot + 2; // epilogue warps x tiles whose staging tiles are free again

            const uint32_t warp      = threadIdx.x >> 5;
            const uint32_t lane      = threadIdx.x & 31u;
            const uint32_t rank      = ptx::cluster_ctarank();
            const uint32_t pair      = blockIdx.x >> 1;
            const uint32_t num_pairs = gridDim.x >> 1;
            const uint32_t num_tiles = tiles_m * tiles_n;
            const uint32_t num_kb    = (k + SLAB_K - 1) / SLAB_K; // the last slab may hold only 128 K
            const bool     half_tail = (k % SLAB_K) != 0u;

            if(threadIdx.x == 0)
            {
                ptx::prefetch_tensormap(&tmap_a);
                ptx::prefetch_tensormap(&tmap_e);
                ptx::prefetch_tensormap(&tmap_b);
                ptx::prefetch_tensormap(&tmap_c);
                ptx::prefetch_tensormap(&tmap_d);
                for(uint32_t s = 0; s < STAGES; ++s)
                {
                    ptx::mbar_init(full_bar + 8 * s, 1);
                    ptx::mbar_init(empty_bar + 8 * s, 1);
                }
                ptx::mbar_init(tfull_bar, 1);
                ptx::mbar_init(tempty_bar, 8); // accumulator 0: 4 warps x 2 CTAs
                ptx::mbar_init(tempty_bar + 8, 8); // accumulator 1
                for(uint32_t i = 0; i < EPI_WARPS * 2; ++i)
                    ptx::mbar_init(cbar_base + 8 * i, 1);
                *cta_abort = 0u;
                *epi_count = 0u;
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
                    const uint32_t leader_full0 = ptx::mapa(full_bar, 0u);
                    uint32_t       stage = 0, phase = 0, iter = 0;
                    bool           ok = true;
                    for(uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs, ++iter)
                    {
                        uint32_t m_idx, n_idx;
                        tile_coords(tile, tiles_m, tiles_n, group_m, m_idx, n_idx);
                        const int32_t row_a = static_cast<int32_t>(m_idx * PAIR_M + rank * CTA_M);
                        const int32_t row_b = static_cast<int32_t>(n_idx * TILE_N + rank * HALF_N);
                        // inner coordinates are byte offsets into the value / metadata / B rows: 128, 2 x 16 and
                        // 2 x 128 bytes per slab, all multiples of 16
                        int32_t ka = 0, ke = 0, kbb = 0;
                        const uint32_t e_blk0 = (m_idx * 2u + rank) * num_kb; // first re-tiled metadata block of this CTA's rows
                        for(uint32_t kb = 0; kb < num_kb; ++kb)
                        {
                            ok = ptx::mbar_wait_bounded(empty_bar + 8 * stage, phase ^ 1u, cta_abort, status,
                                                        (ROLE_PRODUCER << 24) | blockIdx.x, WAIT_TIMEOUT_NS);
                            if(!ok)
                                break;
                            if(stage == EPI_STAGE && iter != 0u)
                            {
                                // this stage's A and B regions double as the epilogue's staging tiles: every epilogue
                                // warp must have finished with them for all earlier tiles (bounded wait)
                                const uint64_t t0 = ptx::globaltimer_ns();
                                uint32_t       spins = 0;
                                while(ptx::ld_acquire_shared_u32(epi_count) < EPI_WARPS * iter)
                                {
                                    if((++spins & 0xFFu) == 0u)
                                    {
                                        if(*cta_abort)
                                        {
                                            ok = false;
                                            break;
                                        }
                                        if(ptx::globaltimer_ns() - t0 > WAIT_TIMEOUT_NS)
                                        {
                                            *cta_abort = 1u;
                                            if(atomicCAS(status, 0u, ptx::STATUS_TIMEOUT_CODE) == 0u)
                                                status[1] = (ROLE_PRODUCER << 24) | (2u << 20) | blockIdx.x;
                                            ok = false;
                                            break;
                                        }
                                    }
                                }
                                if(!ok)
                                    break;
                                ptx::fence_proxy_async_smem(); // generic writes of the staging tiles before the TMA overwrite
                            }
                            const uint32_t fb = full_bar + 8 * stage, lf = leader_full0 + 8 * stage;
                            if(rank == 0)
                                ptx::mbar_arrive_expect_tx(fb, 2u * STAGE_BYTES);
                            const uint32_t sb = smem_b + stage * B_STAGE_BYTES, se = smem_e + stage * E_STAGE_BYTES;
                            ptx::tma_load_2d_pair(sb, &tmap_b, kbb, row_b, lf);
                            ptx::tma_load_2d_pair(smem_a + stage * A_STAGE_BYTES, &tmap_a, ka, row_a, lf);
                            if constexpr(E_PACKED)
                                ptx::tma_load_2d_pair(se, &tmap_e, 0, static_cast<int32_t>((e_blk0 + kb) * E_PACKED_ROWS), lf);
                            else
                                ptx::tma_load_2d_pair(se, &tmap_e, ke, row_a, lf);
                            ptx::tma_load_2d_pair(sb + B_BOX_BYTES, &tmap_b, kbb + static_cast<int32_t>(HALF_K), row_b, lf);
                            if constexpr(!E_PACKED)
                                ptx::tma_load_2d_pair(se + E_BOX_BYTES, &tmap_e, ke + static_cast<int32_t>(E_ROW_BYTES), row_a, lf);
                            ka += static_cast<int32_t>(A_ROW_BYTES), ke += static_cast<int32_t>(2 * E_ROW_BYTES),
                                kbb += static_cast<int32_t>(SLAB_K);
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
                    // One thread feeds the tensor cores of both SMs; what it executes per slab besides the MMAs
                    // (wait, fence, two metadata copies, commit) has to hide behind 896 clocks of tensor work.
                    // The ring is walked by an unrolled loop over the stages, so that every descriptor,
                    // metadata column and barrier address is a loop-invariant value plus a compile-time offset.
                    // dense int8 descriptor with the sparsity flag (bit 2); metadata format id 0
                    constexpr uint32_t idesc  = make_idesc<KIND_I8, 2 * SUB_M, TILE_N>() | (1u << 2);
                    constexpr uint64_t A_STEP = A_STAGE_BYTES >> 4, B_STEP = B_STAGE_BYTES >> 4, E_STEP = E_STAGE_BYTES >> 4;
                    constexpr uint64_t A_SUB  = (SUB_M * A_ROW_BYTES) >> 4; // second 128-row sub-tile
                    constexpr uint64_t B_H1   = B_BOX_BYTES >> 4, E_H1 = E_BOX_BYTES >> 4; // second 128 K of the slab
                    const uint64_t     a_desc0 = ptx::make_kmajor_sw128_desc(smem_a);
                    const uint64_t     b_desc0 = ptx::make_kmajor_sw128_desc(smem_b);
                    // metadata source of one 128-K box: its two 128-row blocks (2 KiB apart) are the two 16-byte
                    // column blocks of a 128 x 32-byte tile; one copy fills 8 columns (4 per sub-tile)
                    const uint64_t e_desc0 = ptx::make_rows16_desc(smem_e, SUB_M * E_ROW_BYTES);
                    const uint32_t e_tmem0 = tmem_base + E_COL0;
                    const uint32_t acc0 = tmem_base, acc1 = tmem_base + TILE_N;
                    const uint32_t my_tiles = pair < num_tiles ? (num_tiles - pair + num_pairs - 1) / num_pairs : 0u;
                    uint32_t       left     = my_tiles * num_kb; // slabs this pair still has to multiply
                    uint32_t       phase = 0, kb = 0, tphase = 0;
                    bool           ok = true;
                    while(ok && left != 0u)
                    {
#pragma unroll
                        for(uint32_t st = 0; st < STAGES; ++st)
                        {
                            if(left == 0u)
                                break;
                            ok = ptx::mbar_wait_bounded(full_bar + 8 * st, phase, cta_abort, status,
                                                        (ROLE_MMA << 24) | (1u << 20) | blockIdx.x, WAIT_TIMEOUT_NS);
                            if(!ok)
                                break;
                            ptx::tc_fence_after_sync();
                            const uint32_t e_t = e_tmem0 + 16u * st;
                            const uint64_t a_d = a_desc0 + st * A_STEP, b_d = b_desc0 + st * B_STEP;
                            // a slab that ends the K range with only 128 K (k % 256 == 128) runs its first half only
                            const bool full_slab = !(half_tail && kb + 1u == num_kb);
                            ptx::tmem_cp_128x256b_pair(e_t, e_desc0 + st * E_STEP);
                            if(full_slab)
                                ptx::tmem_cp_128x256b_pair(e_t + 8u, e_desc0 + st * E_STEP + E_H1);
                            const uint32_t acc = kb != 0u ? 1u : 0u; // first slab of a tile overwrites
                            if(kb == 0u)
                            {
                                // accumulator 0 of the previous tile must have been drained by both CTAs
                                ok = ptx::mbar_wait_bounded(tempty_bar, tphase ^ 1u, cta_abort, status,
                                                            (ROLE_MMA << 24) | blockIdx.x, WAIT_TIMEOUT_NS);
                                if(!ok)
                                    break;
                                ptx::tc_fence_after_sync();
                            }
                            // 64 logical K per MMA = 32 bytes of compressed A (+2), 64 bytes of B (+4), 2 metadata columns
                            ptx::mma_i8_sp_ss_pair(acc0, a_d, b_d, e_t, idesc, acc);
                            ptx::mma_i8_sp_ss_pair(acc0, a_d + 2, b_d + 4, e_t + 2, idesc, 1u);
                            if(full_slab)
                            {
                                ptx::mma_i8_sp_ss_pair(acc0, a_d + 4, b_d + B_H1, e_t + 8, idesc, 1u);
                                ptx::mma_i8_sp_ss_pair(acc0, a_d + 6, b_d + B_H1 + 4, e_t + 10, idesc, 1u);
                            }
                            if(kb == 0u)
                            {
                                ok = ptx::mbar_wait_bounded(tempty_bar + 8, tphase ^ 1u, cta_abort, status,
                                                            (ROLE_MMA << 24) | blockIdx.x, WAIT_TIMEOUT_NS);
                                if(!ok)
                                    break;
                                ptx::tc_fence_after_sync();
                            }
                            ptx::mma_i8_sp_ss_pair(acc1, a_d + A_SUB, b_d, e_t + 4, idesc, acc);
                            ptx::mma_i8_sp_ss_pair(acc1, a_d + A_SUB + 2, b_d + 4, e_t + 6, idesc, 1u);
                            if(full_slab)
                            {
                                ptx::mma_i8_sp_ss_pair(acc1, a_d + A_SUB + 4, b_d + B_H1, e_t + 12, idesc, 1u);
                                ptx::mma_i8_sp_ss_pair(acc1, a_d + A_SUB + 6, b_d + B_H1 + 4, e_t + 14, idesc, 1u);
                            }
                            ptx::tc_commit_pair(empty_bar + 8 * st, 0x3); // the slot is free in both CTAs once these MMAs retire
                            --left;
                            if(++kb == num_kb)
                            {
                                kb = 0;
                                tphase ^= 1u;
                                ptx::tc_commit_pair(tfull_bar, 0x3); // accumulators complete
                            }
                        }
                        phase ^= 1u;
                    }
                }
                __syncwarp();
            }
            else
            {
                // -------------------------------- epilogue (both CTAs) --------------------------------
                const uint32_t e       = warp - 2u; // 0..7
                const uint32_t quad    = warp & 3u; // lane quadrant this warp may read
                const uint32_t j       = e >> 2; // accumulator: warps 2-5 -> 0, warps 6-9 -> 1
                const bool     read_c  = (beta != 0) && (c != nullptr);
                const uint32_t buf_off = epi_off + e * EPI_BUF_BYTES; // first tile: in the A region of the last stage
                const uint32_t buf0    = base + buf_off;
                // second tile: in the B region of that stage, or (the last warp) in memory of its own
                const uint32_t buf1_off
                    = e < EPI_IN_B ? epi_b_off + e * EPI_BUF_BYTES : epi_x_off + (e - EPI_IN_B) * EPI_BUF_BYTES;
                const uint32_t buf1    = base + buf1_off;
                const uint32_t cbar0   = cbar_base + e * 16u;
                using Drain            = tc05q::StagedDrain<int32_t, int32_t, TILE_N, 1, EPI_ROW_BYTES>;
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
                    ok = ptx::mbar_wait_bounded_warp(tfull_bar, iter & 1u, cta_abort, status,
                                                     (ROLE_EPILOGUE << 24) | blockIdx.x, WAIT_TIMEOUT_NS, lane);
                    if(!ok)
                        break;
                    ptx::tc_fence_after_sync();
                    // the staging tiles share memory with an operand stage: only now, with every MMA of the
                    // tile retired, may anything (the first C tiles included) be written there
                    if(staged && read_c && lane == 0)
                        Drain::prefetch_c(&tmap_c, buf0, cbar0, col_base, row0, n, 0, 0, 2, buf1);
                    const uint32_t tmem_acc = tmem_base + j * TILE_N;
                    if(staged)
                        ok = Drain::run(tmem_acc, quad, lane, smem, buf_off, buf0, cbar0, &tmap_c, &tmap_d, col_base, row0, n,
                                        alpha, beta, read_c, cpar, cta_abort, status,
                                        (ROLE_EPILOGUE << 24) | (1u << 20) | blockIdx.x, 0, buf1_off, buf1);
                    else if(vec_ok == 0)
                        drain_accumulator<int32_t, int32_t, TILE_N>(tmem_acc, quad, lane, row_base, col_base, m, n, c, d, ldc,
                                                                    ldd, alpha, beta, read_c, 0);
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if(lane == 0)
                    {
                        ptx::mbar_arrive_cluster(ptx::mapa(tempty_bar + 8 * j, 0u));
                        // hand the staging tiles back to the producer once this warp's stores have read them
                        ptx::bulk_wait_group_read<0>();
                        ptx::red_release_shared_add_u32(epi_count, 1u);
                    }
                }
                if(lane == 0)
                    ptx::bulk_wait_group<0>(); // the stores must have completed before the CTA exits
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

        // Re-tiles the metadata for gemm_tc05_sp_kernel<true>: for every block of 256 rows x 256 K the 8 KiB
        // image the kernel wants in shared memory - [K half][128-row sub-tile][row][16 bytes] - stored
        // contiguously, blocks ordered (row block, slab).  The caller's array is read in full 32-byte
        // sectors (both K halves of a row at once); rows >= m and bytes >= k/8 become zero (their products
        // are never stored / never issued).  One thread per row of a block.
        __global__ void __launch_bounds__(256)
            repack_meta_kernel(const uint8_t* __restrict__ meta, uint8_t* __restrict__ packed, uint32_t m, uint32_t k,
                               size_t ld_meta, uint32_t num_kb)
        {
            const uint32_t r      = threadIdx.x; // row inside the 256-row block
            const uint32_t kb     = blockIdx.x;
            const uint32_t rb     = blockIdx.y;
            const uint32_t row    = rb * CTA_M + r;
            const uint32_t col    = kb * (SLAB_K / 8); // byte offset in the metadata row
            const uint32_t rowlen = k / 8;
            uint4          h0 = make_uint4(0, 0, 0, 0), h1 = make_uint4(0, 0, 0, 0);
            if(row < m)
            {
                const uint8_t* src = meta + static_cast<size_t>(row) * ld_meta + col;
                if(col < rowlen)
                    h0 = __ldcs(reinterpret_cast<const uint4*>(src));
                if(col + 16u < rowlen)
                    h1 = __ldcs(reinterpret_cast<const uint4*>(src + 16));
            }
            uint8_t* blk = packed + (static_cast<size_t>(rb) * num_kb + kb) * E_STAGE_BYTES;
            const uint32_t sub = r >> 7, rr = r & 127u;
            *reinterpret_cast<uint4*>(blk + sub * (SUB_M * E_ROW_BYTES) + rr * E_ROW_BYTES)               = h0;
            *reinterpret_cast<uint4*>(blk + E_BOX_BYTES + sub * (SUB_M * E_ROW_BYTES) + rr * E_ROW_BYTES) = h1;
        }
    } // namespace tc05s
} // namespace b200wmma
