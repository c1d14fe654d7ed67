// Two-CTA variant of the tcgen05 GEMM: a cluster of two CTAs (two SMs) owns one 256 x 256 output
// tile and runs `tcgen05.mma.cta_group::2` on it.
//
// Why: with one CTA per 128 x 256 tile every SM pulls 48 KiB of operands per 64-wide K slab through
// its 128 B/clk L2 port (75 % of the port at full tensor rate).  In a pair each CTA loads its own 128
// rows of A and only HALF of the 256-wide B slab (the tensor core reads the other half from the
// peer's shared memory), i.e. 32 KiB per slab per SM, and the freed shared memory deepens the ring
// from 4 to 6 stages.
//
// Protocol (rank 0 of the pair = leader):
//   producer (warp 0, one lane, BOTH CTAs): wait own empty[s]; the leader arms its full[s] with the
//       byte count of both CTAs; each CTA issues its two box loads with `.cta_group::2`, whose
//       completion bytes are counted on the LEADER's full[s] (address via mapa).  No multicast.
//   MMA issuer (warp 1, one lane, leader only): wait full[s]; 4 x tcgen05.mma.cta_group::2 (M = 256,
//       N = 256, 32 bytes of K each); tcgen05.commit arrives on empty[s] of BOTH CTAs (barrier signal
//       to both ranks);
//       after the last slab commit to tmem_full[buf] of both CTAs.
//   epilogue (warps 2-5, both CTAs): wait own tmem_full[buf]; drain own 128 lanes x 256 columns;
//       one lane per warp arrives on the LEADER's tmem_empty[buf] (8 arrivals per phase).
// Tensor memory is allocated / freed with the cta_group::2 forms by warp 1 of each CTA.
// Every wait is bounded; set-up and tear-down use cluster barriers, which both CTAs always reach.
#pragma once
#include "gemm_tc05_common.cuh"

namespace b200wmma
{
    namespace tc05p
    {
        using namespace tc05;

        constexpr uint32_t CTA_M         = 128; // rows of A / D per CTA
        constexpr uint32_t PAIR_M        = 256;
        constexpr uint32_t TILE_N        = 256;
        constexpr uint32_t HALF_N        = 128; // rows of B^T (columns of B) each CTA loads
        constexpr uint32_t STAGES        = 6;
        constexpr uint32_t A_STAGE_BYTES = CTA_M * BLOCK_K_BYTES; // 16 KiB
        constexpr uint32_t B_STAGE_BYTES = HALF_N * BLOCK_K_BYTES; // 16 KiB
        constexpr uint32_t STAGE_BYTES   = A_STAGE_BYTES + B_STAGE_BYTES; // per CTA
        constexpr uint32_t NUM_THREADS   = 192;
        constexpr uint32_t TMEM_COLS     = 512;
        constexpr uint32_t GROUP_M       = 8; // rasterisation: 8 pair-row tiles (2048 rows) share B slabs
        constexpr uint32_t SMEM_BYTES    = 1024 + STAGES * STAGE_BYTES + 256;

        template <int KIND, typename OutT, typename ScalarT>
        __global__ void __launch_bounds__(NUM_THREADS, 1)
            gemm_tc05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                  const __grid_constant__ CUtensorMap tmap_b,
                                  const OutT* __restrict__ c,
                                  OutT* __restrict__ d,
                                  uint32_t  m,
                                  uint32_t  n,
                                  uint32_t  k_bytes,
                                  uint32_t  ldc,
                                  uint32_t  ldd,
                                  ScalarT   alpha,
                                  ScalarT   beta,
                                  uint32_t  tiles_m, // pair tiles along M (256 rows each)
                                  uint32_t  tiles_n,
                                  int       vec_ok,
                                  uint32_t  group_m,
                                  unsigned* status)
        {
            extern __shared__ uint8_t smem_raw[];
            const uint32_t            raw_addr = ptx::smem_u32(smem_raw);
            const uint32_t            base     = (raw_addr + 1023u) & ~1023u;
            uint8_t*                  smem     = smem_raw + (base - raw_addr);

            // identical layout in both CTAs: [A stages][B stages][barriers][tmem slot][abort flag]
            const uint32_t     smem_a     = base;
            const uint32_t     smem_b     = base + STAGES * A_STAGE_BYTES;
            const uint32_t     bar_base   = base + STAGES * STAGE_BYTES;
            const uint32_t     full_bar   = bar_base;
            const uint32_t     empty_bar  = bar_base + 8 * STAGES;
            const uint32_t     tfull_bar  = bar_base + 16 * STAGES;
            const uint32_t     tempty_bar = tfull_bar + 16;
            uint32_t*          tmem_slot
                = reinterpret_cast<uint32_t*>(smem + STAGES * STAGE_BYTES + 16 * STAGES + 32);
            volatile uint32_t* cta_abort = tmem_slot + 1;

            const uint32_t warp      = threadIdx.x >> 5;
            const uint32_t lane      = threadIdx.x & 31u;
            const uint32_t rank      = ptx::cluster_ctarank(); // 0 = leader, 1 = peer
            const uint32_t pair      = blockIdx.x >> 1;
            const uint32_t num_pairs = gridDim.x >> 1;
            const uint32_t num_tiles = tiles_m * tiles_n;
            const uint32_t num_kb    = (k_bytes + BLOCK_K_BYTES - 1) / BLOCK_K_BYTES;

            if(threadIdx.x == 0)
            {
                ptx::prefetch_tensormap(&tmap_a);
                ptx::prefetch_tensormap(&tmap_b);
                for(uint32_t s = 0; s < STAGES; ++s)
                {
                    ptx::mbar_init(full_bar + 8 * s, 1); // leader's copy is the one in use
                    ptx::mbar_init(empty_bar + 8 * s, 1);
                }
                for(uint32_t s = 0; s < 2; ++s)
                {
                    ptx::mbar_init(tfull_bar + 8 * s, 1);
                    ptx::mbar_init(tempty_bar + 8 * s, 8); // 4 epilogue warps x 2 CTAs (leader's copy in use)
                }
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
            ptx::cluster_sync(); // barrier inits and the allocation are visible to both CTAs
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
                            const int32_t  kc          = static_cast<int32_t>(
                                kb * (KIND == KIND_F16 ? BLOCK_K_BYTES / 2 : BLOCK_K_BYTES));
                            ptx::tma_load_2d_pair(smem_a + stage * A_STAGE_BYTES, &tmap_a, kc, row_a, leader_full);
                            ptx::tma_load_2d_pair(smem_b + stage * B_STAGE_BYTES, &tmap_b, kc, row_b, leader_full);
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
                    constexpr uint32_t idesc = make_idesc<KIND, PAIR_M, TILE_N>();
                    uint32_t           stage = 0, phase = 0, iter = 0;
                    bool               ok = true;
                    for(uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs, ++iter)
                    {
                        const uint32_t buf    = iter & 1u;
                        const uint32_t bphase = (iter >> 1) & 1u;
                        ok = ptx::mbar_wait_bounded(tempty_bar + 8 * buf, bphase ^ 1u, cta_abort, status,
                                                    (ROLE_MMA << 24) | blockIdx.x, WAIT_TIMEOUT_NS);
                        if(!ok)
                            break;
                        ptx::tc_fence_after_sync();
                        const uint32_t d_tmem = tmem_base + buf * TILE_N;
                        for(uint32_t kb = 0; kb < num_kb; ++kb)
                        {
                            ok = ptx::mbar_wait_bounded(full_bar + 8 * stage, phase, cta_abort, status,
                                                        (ROLE_MMA << 24) | (1u << 20) | blockIdx.x, WAIT_TIMEOUT_NS);
                            if(!ok)
                                break;
                            ptx::tc_fence_after_sync();
                            const uint64_t a_desc = ptx::make_kmajor_sw128_desc(smem_a + stage * A_STAGE_BYTES);
                            const uint64_t b_desc = ptx::make_kmajor_sw128_desc(smem_b + stage * B_STAGE_BYTES);
#pragma unroll
                            for(uint32_t ks = 0; ks < BLOCK_K_BYTES / 32; ++ks)
                            {
                                const uint32_t acc = (kb | ks) != 0u ? 1u : 0u;
                                if constexpr(KIND == KIND_F16)
                                    ptx::mma_f16_ss_pair(d_tmem, a_desc + 2 * ks, b_desc + 2 * ks, idesc, acc);
                                else
                                    ptx::mma_i8_ss_pair(d_tmem, a_desc + 2 * ks, b_desc + 2 * ks, idesc, acc);
                            }
                            // the slot is free in BOTH CTAs once these MMAs retire
                            ptx::tc_commit_pair(empty_bar + 8 * stage, 0x3);
                            if(++stage == STAGES)
                            {
                                stage = 0;
                                phase ^= 1u;
                            }
                        }
                        if(ok)
                        {
                            ptx::tc_commit_pair(tfull_bar + 8 * buf, 0x3);
                        }
                    }
                }
                __syncwarp();
            }
            else
            {
                // -------------------------------- epilogue (both CTAs) --------------------------------
                const uint32_t quad   = warp & 3u;
                const bool     read_c = (beta != ScalarT(0)) && (c != nullptr);
                uint32_t       iter   = 0;
                bool           ok     = true;
                for(uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs, ++iter)
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
                    drain_accumulator<OutT, ScalarT, TILE_N>(tmem_base + buf * TILE_N, quad, lane,
                                                             m_idx * PAIR_M + rank * CTA_M, n_idx * TILE_N, m, n, c, d,
                                                             ldc, ldd, alpha, beta, read_c, vec_ok);
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if(lane == 0)
                        ptx::mbar_arrive_cluster(ptx::mapa(tempty_bar + 8 * buf, 0u));
                }
            }

            // ---------------------------------- teardown ----------------------------------
            ptx::tc_fence_before_sync();
            ptx::cluster_sync(); // neither CTA issues anything that touches the other from here on
            {
                const uint32_t peer_abort = ptx::ld_shared_cluster_u32(
                    ptx::mapa(ptx::smem_u32(const_cast<uint32_t*>(cta_abort)), rank ^ 1u));
                if(*cta_abort || peer_abort)
                {
                    // A wait was abandoned somewhere in the pair: copies or MMAs may still be in
                    // flight.  Bounded grace period before shared and tensor memory are released.
                    const uint64_t t0 = ptx::globaltimer_ns();
                    while(ptx::globaltimer_ns() - t0 < 2000000ull)
                        __nanosleep(1000);
                }
            }
            ptx::cluster_sync(); // the peer has finished reading this CTA's abort flag
            if(warp == 1)
            {
                ptx::tc_fence_after_sync();
                ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
            }
        }
    } // namespace tc05p
} // namespace b200wmma
