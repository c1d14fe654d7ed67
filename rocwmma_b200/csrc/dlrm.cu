// DLRM dot-interaction forward and backward, one warp per sample, everything fused, all global
// traffic moved by the TMA engine.
//
// Forward stands in for dlrmDotFwd (samples/simple_dlrm.cpp:184-284;
// test/dlrm/device/dlrm_dot_fwd.hpp:37-136).  The reference computes each 16x16 tile of
// Z = X X^T in its own wave, stores it to a global fp32 scratch, re-reads the scratch and
// writes the strict lower triangle element by element.  Here each warp owns a small ring of
// shared-memory sample tiles: one lane asks the TMA unit for the sample's m x k rows (64-column
// boxes, 128-byte swizzle, so ldmatrix reads are conflict-free), the warp runs the lower-triangle
// tiles on mma.sync with fp32 accumulators, packs [X row 0 | tril(Z)] into a shared-memory row
// and one lane hands that row back to the TMA unit as a bulk store.  X is read once, the output
// written once, no scratch, and no thread computes a global address per element.
//
// Backward stands in for trilReconstruct + dlrmDotBwd (samples/simple_dlrm.cpp:290-331,
// :349-441; test/dlrm/device/dlrm_dot_bwd.hpp:35-172), which rebuild the symmetric matrix in
// global memory in one kernel, synchronise on the host, and multiply in a second kernel.
// Here the packed upstream row arrives by bulk copy, is expanded to the symmetric m x m fp16
// matrix in shared memory, multiplied with X on mma.sync; the product overwrites the X tile in
// place (16-column slabs) and leaves through TMA tile stores that cover rows 0..m-1 only,
// optionally with the bottom-MLP pass-through gradient added to row 0.
//
// Both are HBM-bound: the arithmetic is 2*m*m*k flop per sample against ~8-15 KB of traffic.
#include <algorithm>

#include "gemm_tc05_common.cuh" // make_kmajor_tmap: 64-column, 128-byte-swizzled box maps
#include "ptx_sm100.cuh"
#include "tuning.cuh"

namespace b200wmma
{
    namespace dlrm
    {
        constexpr int      MAX_M       = 32;
        constexpr int      MAX_K       = 256;
        constexpr int      FWD_MAX_WARPS = 12; // both kernels take their warp count from the launch
        constexpr int      BWD_MAX_WARPS = 12; // the backward kernel takes its warp count from the launch
        constexpr int      BWD_BATCH     = 4; // 16-column slabs of dX in flight per warp
        constexpr int      TPITCH      = 40; // halfs per row of the 32x32 symmetric matrix (+8 pad)
        constexpr uint32_t BOX_BYTES   = MAX_M * 128; // one 64-column box: 32 rows of 128 bytes
        constexpr uint64_t WAIT_NS     = 2000000000ull;

        __device__ __forceinline__ void
            ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr)
        {
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                         : "r"(addr));
        }
        __device__ __forceinline__ void
            ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr)
        {
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                         : "r"(addr));
        }
        // D(16x8, fp32) += A(16x16, fp16, row) x B(16x8, fp16, col)
        __device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                  uint32_t b1)
        {
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
        }

        // Byte offset, inside a sample tile, of the 16-byte chunk holding columns c..c+7 of row r.
        // The tile is a sequence of 64-column boxes (BOX_BYTES each, rows of 128 bytes) as written by
        // TMA with the 128-byte swizzle: chunk index XOR (row mod 8).
        __device__ __forceinline__ uint32_t tile_off(uint32_t r, uint32_t c)
        {
            return (c >> 6) * BOX_BYTES + r * 128u + ((((c >> 3) & 7u) ^ (r & 7u)) << 4);
        }

        // ---------------------------------- forward ----------------------------------------
        // Shared memory per warp: FWD_STAGES sample tiles, two output rows (double-buffered bulk
        // stores), FWD_STAGES mbarriers.  Warps per CTA = blockDim.x / 32, chosen by the launch.
        template <int FWD_STAGES>
        __global__ void __launch_bounds__(FWD_MAX_WARPS * 32)
            dlrm_fwd_kernel(const __grid_constant__ CUtensorMap tmap_x, __half* __restrict__ output,
                            uint32_t m, uint32_t m_stride, uint32_t k, uint32_t batch,
                            uint32_t out_stride, unsigned* status)
        {
            extern __shared__ uint8_t smem_raw[];
            const uint32_t raw   = ptx::smem_u32(smem_raw);
            const uint32_t base  = (raw + 1023u) & ~1023u;
            uint8_t*       smem  = smem_raw + (base - raw);
            const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            const uint32_t WARPS     = blockDim.x >> 5;
            const uint32_t nbox      = (k + 63u) >> 6;
            const uint32_t tile_b    = nbox * BOX_BYTES;
            const uint32_t orow_b    = out_stride * 2u; // multiple of 16
            const uint32_t tiles_off = warp * FWD_STAGES * tile_b;
            const uint32_t orow_off  = WARPS * FWD_STAGES * tile_b + warp * 2u * orow_b;
            const uint32_t bar_off   = WARPS * FWD_STAGES * tile_b + WARPS * 2u * orow_b + warp * FWD_STAGES * 8u;
            const uint32_t flag_off  = WARPS * FWD_STAGES * tile_b + WARPS * 2u * orow_b + WARPS * FWD_STAGES * 8u;
            volatile uint32_t* cta_abort = reinterpret_cast<volatile uint32_t*>(smem + flag_off);
            const uint32_t g = lane >> 2, t = lane & 3;
            const uint32_t tri_end = k + m * (m - 1) / 2;
            const uint32_t tx_bytes = nbox * m * 128u; // bytes one sample's boxes deliver

            // rows m..31 take part in the MMA tiles as zeros; TMA never writes them
            for(uint32_t s = 0; s < FWD_STAGES; ++s)
                for(uint32_t bx = 0; bx < nbox; ++bx)
                    for(uint32_t i = m * 128u + lane * 16u; i < BOX_BYTES; i += 512u)
                        *reinterpret_cast<uint4*>(smem + tiles_off + s * tile_b + bx * BOX_BYTES + i) = make_uint4(0, 0, 0, 0);
            // columns past the packed triangle are written as zero for every sample
            for(uint32_t ob = 0; ob < 2; ++ob)
                for(uint32_t i = tri_end + lane; i < out_stride; i += 32)
                    reinterpret_cast<__half*>(smem + orow_off + ob * orow_b)[i] = __float2half(0.0f);
            if(threadIdx.x == 0)
                *cta_abort = 0u;
            if(lane == 0)
            {
                for(uint32_t s = 0; s < FWD_STAGES; ++s)
                    ptx::mbar_init(base + bar_off + 8u * s, 1);
                ptx::fence_barrier_init();
            }
            ptx::fence_proxy_async_smem(); // the zero fills above precede any TMA write to the same tiles
            __syncthreads();
            // Everything above touched shared memory only and may have run while the previous kernel of the stream
            // was finishing (programmatic dependent launch); global memory is touched from here on.  This grid is
            // fully resident, so the next kernel's CTAs may take over each SM as soon as this grid's CTAs leave it.
            ptx::grid_dep_launch_dependents();
            ptx::grid_dep_wait();

            const uint32_t stride = gridDim.x * WARPS;
            const uint32_t first  = blockIdx.x * WARPS + warp;
            auto issue_load = [&](uint32_t sample, uint32_t stage) {
                const uint32_t bar = base + bar_off + 8u * stage;
                ptx::mbar_arrive_expect_tx(bar, tx_bytes);
                for(uint32_t bx = 0; bx < nbox; ++bx)
                    ptx::tma_load_2d(base + tiles_off + stage * tile_b + bx * BOX_BYTES, &tmap_x,
                                     static_cast<int32_t>(bx * 64u), static_cast<int32_t>(sample * m_stride), bar);
            };
            if(lane == 0)
                for(uint32_t s = 0; s < FWD_STAGES; ++s)
                    if(first + s * stride < batch)
                        issue_load(first + s * stride, s);

            uint32_t it = 0;
            for(uint32_t b = first; b < batch; b += stride, ++it)
            {
                const uint32_t stage = it % FWD_STAGES, phase = (it / FWD_STAGES) & 1u;
                bool ok = ptx::mbar_wait_bounded(base + bar_off + 8u * stage, phase, cta_abort, status,
                                                 (1u << 28) | blockIdx.x, WAIT_NS);
                if(!__all_sync(0xFFFFFFFFu, ok))
                    break;
                const uint32_t xs = base + tiles_off + stage * tile_b;

                // acc0: rows 0-15 x cols 0-15 ; acc1: rows 16-31 x cols 0-31
                float acc0[2][4] = {}, acc1[4][4] = {};
                const bool two_blocks = m > 16;
                for(uint32_t ks = 0; ks < k; ks += 16)
                {
                    uint32_t a0[4], a1[4], bf[8];
                    const uint32_t acol = ks + (lane >> 4) * 8;
                    ldmatrix_x4(a0[0], a0[1], a0[2], a0[3], xs + tile_off(lane & 15, acol));
                    // B = X^T: n index = row of X.  One x4 load covers two 8-wide n tiles.
                    const uint32_t brow = (lane & 7) + (lane >> 4) * 8, bcol = ks + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(bf[0], bf[1], bf[2], bf[3], xs + tile_off(brow, bcol));
                    mma_16816(acc0[0], a0, bf[0], bf[1]);
                    mma_16816(acc0[1], a0, bf[2], bf[3]);
                    if(two_blocks)
                    {
                        ldmatrix_x4(a1[0], a1[1], a1[2], a1[3], xs + tile_off(16 + (lane & 15), acol));
                        ldmatrix_x4(bf[4], bf[5], bf[6], bf[7], xs + tile_off(16 + brow, bcol));
                        mma_16816(acc1[0], a1, bf[0], bf[1]);
                        mma_16816(acc1[1], a1, bf[2], bf[3]);
                        mma_16816(acc1[2], a1, bf[4], bf[5]);
                        mma_16816(acc1[3], a1, bf[6], bf[7]);
                    }
                }

                // the output row used two samples ago must have been read by its bulk store
                const uint32_t ob = it & 1u;
                if(lane == 0)
                    ptx::bulk_wait_group_read<1>();
                __syncwarp();
                __half* orow = reinterpret_cast<__half*>(smem + orow_off + ob * orow_b);
                // pass-through: X row 0 (row 0 is not permuted by the swizzle)
                if(lane < (k >> 3))
                    reinterpret_cast<uint4*>(orow)[lane]
                        = *reinterpret_cast<const uint4*>(smem + tiles_off + stage * tile_b + (lane >> 3) * BOX_BYTES + (lane & 7u) * 16u);
                __syncwarp(); // every lane is done with this sample tile: refill it
                if(lane == 0 && b + FWD_STAGES * stride < batch)
                    issue_load(b + FWD_STAGES * stride, stage);
#pragma unroll
                for(int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for(int i = 0; i < 4; ++i)
                    {
                        const uint32_t r = g + 8 * (i >> 1), c = 8 * nt + 2 * t + (i & 1);
                        if(c < r && r < m)
                            orow[k + r * (r - 1) / 2 + c] = __float2half_rn(acc0[nt][i]);
                    }
                if(two_blocks)
                {
#pragma unroll
                    for(int nt = 0; nt < 4; ++nt)
#pragma unroll
                        for(int i = 0; i < 4; ++i)
                        {
                            const uint32_t r = 16 + g + 8 * (i >> 1), c = 8 * nt + 2 * t + (i & 1);
                            if(c < r && r < m)
                                orow[k + r * (r - 1) / 2 + c] = __float2half_rn(acc1[nt][i]);
                        }
                }
                ptx::fence_proxy_async_smem(); // generic writes of orow -> visible to the bulk store
                __syncwarp();
                if(lane == 0)
                {
                    ptx::bulk_store_1d(output + static_cast<size_t>(b) * out_stride, base + orow_off + ob * orow_b, orow_b);
                    ptx::bulk_commit_group();
                }
            }
            if(lane == 0)
                ptx::bulk_wait_group<0>(); // shared memory must outlive the stores that read it
            __syncwarp();
            if(*cta_abort)
            {
                // a wait was abandoned: give copies still in flight a bounded time to land before
                // this CTA's shared memory is released
                const uint64_t t0 = ptx::globaltimer_ns();
                while(ptx::globaltimer_ns() - t0 < 2000000ull)
                    __nanosleep(1000);
            }
        }

        // ---------------------------------- backward ---------------------------------------
        // Shared memory per warp: BWD_STAGES x (sample tile + upstream row), the symmetric matrix,
        // BWD_STAGES mbarriers.  The launch picks the warp count (blockDim.x / 32): as many as shared memory holds
        // with two stages each.  Measured at B = 16384, k = 128 on one B200, per launch: 6 / 8 / 10 / 11 warps per SM
        // with two stages 66.5 / 55.3 / 48.9 / 46.4 us (a device copy of the same bytes: 44.3 us); three stages (the
        // previous sample's stage is handed back to the loader after this sample's stores were issued, so no warp
        // waits for its own stores to be read) fit 7 warps and take 58.7 us.  A warp works through its samples one
        // after the other, so the number of warps, not the depth of each warp's ring, hides the latencies.
        template <int BWD_STAGES>
        __global__ void __launch_bounds__(BWD_MAX_WARPS * 32)
            dlrm_bwd_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_g,
                            const __half* __restrict__ upstream, __half* __restrict__ bottom_mlp_grad,
                            uint32_t m, uint32_t m_stride, uint32_t k, uint32_t batch, uint32_t up_stride,
                            int fuse_mlp, unsigned* status)
        {
            extern __shared__ uint8_t smem_raw[];
            const uint32_t raw   = ptx::smem_u32(smem_raw);
            const uint32_t base  = (raw + 1023u) & ~1023u;
            uint8_t*       smem  = smem_raw + (base - raw);
            const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            const uint32_t WARPS    = blockDim.x >> 5;
            const uint32_t nbox     = (k + 63u) >> 6;
            const uint32_t tile_b   = nbox * BOX_BYTES;
            const uint32_t up_b     = up_stride * 2u; // multiple of 16
            const uint32_t up_slot  = (up_b + 127u) & ~127u;
            const uint32_t tiles_off = warp * BWD_STAGES * tile_b;
            const uint32_t up_off    = WARPS * BWD_STAGES * tile_b + warp * BWD_STAGES * up_slot;
            const uint32_t t_off     = WARPS * BWD_STAGES * (tile_b + up_slot) + warp * (MAX_M * TPITCH * 2u);
            const uint32_t bar_off   = WARPS * BWD_STAGES * (tile_b + up_slot) + WARPS * (MAX_M * TPITCH * 2u) + warp * BWD_STAGES * 8u;
            const uint32_t flag_off  = WARPS * BWD_STAGES * (tile_b + up_slot) + WARPS * (MAX_M * TPITCH * 2u) + WARPS * BWD_STAGES * 8u;
            volatile uint32_t* cta_abort = reinterpret_cast<volatile uint32_t*>(smem + flag_off);
            __half*        ts = reinterpret_cast<__half*>(smem + t_off);
            const uint32_t g = lane >> 2, t = lane & 3;
            const uint32_t tx_bytes = nbox * m * 128u + up_b;

            if(threadIdx.x == 0)
                *cta_abort = 0u;
            if(lane == 0)
            {
                for(uint32_t s = 0; s < BWD_STAGES; ++s)
                    ptx::mbar_init(base + bar_off + 8u * s, 1);
                ptx::fence_barrier_init();
            }
            __syncthreads();

            const uint32_t stride = gridDim.x * WARPS;
            const uint32_t first  = blockIdx.x * WARPS + warp;
            // rows m..31 of a tile must be zero for the MMA; TMA never writes them
            auto clear_pad_rows = [&](uint32_t stage) {
                for(uint32_t bx = 0; bx < nbox; ++bx)
                    for(uint32_t i = m * 128u + lane * 16u; i < BOX_BYTES; i += 512u)
                        *reinterpret_cast<uint4*>(smem + tiles_off + stage * tile_b + bx * BOX_BYTES + i) = make_uint4(0, 0, 0, 0);
            };
            auto issue_load = [&](uint32_t sample, uint32_t stage) {
                const uint32_t bar = base + bar_off + 8u * stage;
                ptx::mbar_arrive_expect_tx(bar, tx_bytes);
                for(uint32_t bx = 0; bx < nbox; ++bx)
                    ptx::tma_load_2d(base + tiles_off + stage * tile_b + bx * BOX_BYTES, &tmap_x,
                                     static_cast<int32_t>(bx * 64u), static_cast<int32_t>(sample * m_stride), bar);
                ptx::bulk_load_1d(base + up_off + stage * up_slot, upstream + static_cast<size_t>(sample) * up_stride, up_b, bar);
            };
            for(uint32_t s = 0; s < BWD_STAGES; ++s)
                clear_pad_rows(s);
            ptx::fence_proxy_async_smem();
            __syncwarp();
            // shared memory only up to here (see the forward kernel): global memory is touched from here on
            ptx::grid_dep_launch_dependents();
            ptx::grid_dep_wait();
            if(lane == 0)
                for(uint32_t s = 0; s < BWD_STAGES; ++s)
                    if(first + s * stride < batch)
                        issue_load(first + s * stride, s);

            uint32_t it = 0;
            for(uint32_t b = first; b < batch; b += stride, ++it)
            {
                const uint32_t stage = it % BWD_STAGES, phase = (it / BWD_STAGES) & 1u;
                bool ok = ptx::mbar_wait_bounded(base + bar_off + 8u * stage, phase, cta_abort, status,
                                                 (2u << 28) | blockIdx.x, WAIT_NS);
                if(!__all_sync(0xFFFFFFFFu, ok))
                    break;
                const uint32_t xs_off = tiles_off + stage * tile_b;
                const uint32_t xs     = base + xs_off;
                const __half*  gs     = reinterpret_cast<const __half*>(smem + up_off + stage * up_slot);

                // symmetric matrix with zero diagonal; lane = column index
                for(uint32_t i = 0; i < MAX_M; ++i)
                {
                    const uint32_t j = lane;
                    __half         v = __float2half(0.0f);
                    if(i < m && j < m && i != j)
                    {
                        const uint32_t hi = max(i, j), lo = min(i, j);
                        v = gs[k + hi * (hi - 1) / 2 + lo];
                    }
                    ts[i * TPITCH + j] = v;
                }
                __syncwarp();

                // A fragments of the symmetric matrix: [row block][k step]
                uint32_t af[2][2][4];
                const uint32_t ts_addr = base + t_off;
#pragma unroll
                for(int rb = 0; rb < 2; ++rb)
#pragma unroll
                    for(int ks = 0; ks < 2; ++ks)
                        ldmatrix_x4(af[rb][ks][0], af[rb][ks][1], af[rb][ks][2], af[rb][ks][3],
                                    ts_addr + ((16 * rb + (lane & 15)) * TPITCH + 16 * ks + (lane >> 4) * 8) * 2u);

                // dX[:, n0:n0+16] depends only on X[:, n0:n0+16]: compute 16-column slabs, then overwrite those
                // columns of the shared tile with the result.  BWD_BATCH slabs go through together so that their
                // loads, MMAs and stores overlap (one warp has nothing else to hide their latencies with).
                for(uint32_t n0 = 0; n0 < k; n0 += 16u * BWD_BATCH)
                {
                    float    acc[BWD_BATCH][2][2][4] = {};
                    uint32_t bf[BWD_BATCH][2][4];
#pragma unroll
                    for(int s = 0; s < BWD_BATCH; ++s)
                        if(n0 + 16u * s < k)
                        {
#pragma unroll
                            for(int ks = 0; ks < 2; ++ks)
                                ldmatrix_x4_trans(bf[s][ks][0], bf[s][ks][1], bf[s][ks][2], bf[s][ks][3],
                                                  xs + tile_off(16 * ks + (lane & 7) + ((lane >> 3) & 1) * 8,
                                                                n0 + 16u * s + (lane >> 4) * 8));
                        }
#pragma unroll
                    for(int s = 0; s < BWD_BATCH; ++s)
                        if(n0 + 16u * s < k)
                        {
#pragma unroll
                            for(int rb = 0; rb < 2; ++rb)
#pragma unroll
                                for(int ks = 0; ks < 2; ++ks)
                                {
                                    mma_16816(acc[s][rb][0], af[rb][ks], bf[s][ks][0], bf[s][ks][1]);
                                    mma_16816(acc[s][rb][1], af[rb][ks], bf[s][ks][2], bf[s][ks][3]);
                                }
                        }
                    __syncwarp(); // every lane has read these slabs of X
#pragma unroll
                    for(int s = 0; s < BWD_BATCH; ++s)
                        if(n0 + 16u * s < k)
                        {
#pragma unroll
                            for(int rb = 0; rb < 2; ++rb)
#pragma unroll
                                for(int nt = 0; nt < 2; ++nt)
#pragma unroll
                                    for(int h = 0; h < 2; ++h)
                                    {
                                        const uint32_t r = 16 * rb + g + 8 * h, c = n0 + 16u * s + 8 * nt + 2 * t;
                                        float          v0 = acc[s][rb][nt][2 * h], v1 = acc[s][rb][nt][2 * h + 1];
                                        if(fuse_mlp && r == 0)
                                        {
                                            v0 += __half2float(gs[c]);
                                            v1 += __half2float(gs[c + 1]);
                                        }
                                        *reinterpret_cast<__half2*>(smem + xs_off + tile_off(r, c) + (c & 7u) * 2u)
                                            = __floats2half2_rn(v0, v1);
                                    }
                        }
                }
                ptx::fence_proxy_async_smem(); // generic writes of dX -> visible to the TMA stores
                __syncwarp();
                if(lane == 0)
                {
                    for(uint32_t bx = 0; bx < nbox; ++bx)
                        ptx::tma_store_2d(&tmap_g, static_cast<int32_t>(bx * 64u), static_cast<int32_t>(b * m_stride),
                                          xs + bx * BOX_BYTES);
                    if(bottom_mlp_grad)
                        ptx::bulk_store_1d(bottom_mlp_grad + static_cast<size_t>(b) * k, base + up_off + stage * up_slot, k * 2u);
                    ptx::bulk_commit_group();
                    // Rows m..31 of a tile still hold zeros after a pass: the product of the zero rows of the
                    // symmetric matrix was written over them.
                    if constexpr(BWD_STAGES >= 3)
                    {
                        // hand the PREVIOUS sample's stage to the loader: its stores have been read by now or
                        // nearly so, and this sample's stores stay in flight
                        ptx::bulk_wait_group_read<1>();
                        if(it > 0 && b + (BWD_STAGES - 1) * stride < batch)
                            issue_load(b + (BWD_STAGES - 1) * stride, (it - 1) % BWD_STAGES);
                    }
                    else
                    {
                        ptx::bulk_wait_group_read<0>();
                        if(b + BWD_STAGES * stride < batch)
                            issue_load(b + BWD_STAGES * stride, stage);
                    }
                }
                __syncwarp();
            }
            if(lane == 0)
                ptx::bulk_wait_group<0>();
            __syncwarp();
            if(*cta_abort)
            {
                const uint64_t t0 = ptx::globaltimer_ns();
                while(ptx::globaltimer_ns() - t0 < 2000000ull)
                    __nanosleep(1000);
            }
        }

        // Shapes beyond the one-warp-per-sample kernels (m <= 32, k <= 256, packed rows of at most 2048 values)
        // go to the block-tiled kernels of dlrm_general.cu.
        static bool needs_general(uint32_t m, uint32_t k, uint32_t packed_stride)
        {
            return m > static_cast<uint32_t>(MAX_M) || k > static_cast<uint32_t>(MAX_K) || packed_stride > 2048u;
        }

        static int check_common(const void* input, uint32_t m, uint32_t m_stride, uint32_t k,
                                uint32_t batch, bool general)
        {
            B200_REQUIRE(input, B200WMMA_ERR_INVALID_ARG, "dlrm: input must be non-null");
            B200_REQUIRE(m >= 1 && batch >= 1 && k >= 1, B200WMMA_ERR_INVALID_ARG,
                         "dlrm: m, k, batch must be non-zero");
            B200_REQUIRE(m_stride >= m, B200WMMA_ERR_INVALID_ARG, "dlrm: m_stride must be >= m");
            B200_REQUIRE(k % 16 == 0, B200WMMA_ERR_UNSUPPORTED, "dlrm: k = %u not supported (multiple of 16)", k);
            B200_REQUIRE(general || (m <= MAX_M && k <= MAX_K), B200WMMA_ERR_UNSUPPORTED, "dlrm: internal dispatch error");
            if(general)
            {
                // the block-tiled kernels read whole 16-row blocks and index the batch with a grid dimension
                B200_REQUIRE(m_stride >= ((m + 15u) & ~15u), B200WMMA_ERR_UNSUPPORTED,
                             "dlrm: beyond m = 32 / k = 256 the row stride must cover m rounded up to 16 (%u < %u)", m_stride,
                             (m + 15u) & ~15u);
                B200_REQUIRE(batch <= 65535u && m <= 65535u * 16u, B200WMMA_ERR_UNSUPPORTED,
                             "dlrm: batch above 65535 is not supported beyond m = 32 / k = 256");
            }
            B200_REQUIRE(static_cast<uint64_t>(batch) * m_stride < (1ull << 31), B200WMMA_ERR_UNSUPPORTED,
                         "dlrm: batch * m_stride must stay below 2^31 rows");
            B200_REQUIRE(aligned16(input), B200WMMA_ERR_ALIGNMENT, "dlrm: input must be 16-byte aligned");
            return B200WMMA_OK;
        }

        // Warps per CTA: as many as fit (`fit`), but no more than spreads a small batch over every SM.
        static uint32_t warps_for(uint32_t batch, size_t fit, int max_warps, int forced)
        {
            int dev = 0, sms = 148;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            uint32_t warps = static_cast<uint32_t>(std::min<size_t>(max_warps, fit));
            if(forced > 0)
                return std::min<uint32_t>(static_cast<uint32_t>(forced), warps);
            return std::min<uint32_t>(warps, std::max<uint32_t>(4u, ceil_div(batch, static_cast<uint32_t>(sms))));
        }

        static uint32_t grid_for(uint32_t batch, const void* kernel, size_t smem_bytes, uint32_t warps)
        {
            int dev = 0, sms = 148, per_sm = 1;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, warps * 32, smem_bytes);
            if(per_sm < 1)
                per_sm = 1;
            const uint32_t want = ceil_div(batch, warps);
            const uint32_t cap  = static_cast<uint32_t>(sms) * per_sm;
            return want < cap ? want : cap;
        }

        // Launch with programmatic stream serialization: the kernel's prologue (barrier set-up, pad rows) may overlap
        // the tail of the preceding kernel in the stream; the kernel itself waits for that kernel's completion
        // (grid_dep_wait) before it touches global memory, so stream order is kept.
        static cudaLaunchConfig_t pdl_config(cudaLaunchAttribute (&attr)[1], uint32_t grid, size_t smem, cudaStream_t stream,
                                             uint32_t warps)
        {
            attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cudaLaunchConfig_t cfg                             = {};
            cfg.gridDim                                        = dim3(grid);
            cfg.blockDim                                       = dim3(warps * 32);
            cfg.dynamicSmemBytes                               = smem;
            cfg.stream                                         = stream;
            cfg.attrs                                          = attr;
            cfg.numAttrs                                       = 1;
            return cfg;
        }

        // 2-D view [(batch-1)*m_stride + m rows, k columns] of a sample buffer: only real rows are covered.
        static int sample_tmap(CUtensorMap* out, const void* ptr, uint32_t m, uint32_t m_stride, uint32_t k,
                               uint32_t batch)
        {
            return tc05::make_kmajor_tmap(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, ptr, (batch - 1) * m_stride + m, k, k, m);
        }
    } // namespace dlrm
} // namespace b200wmma

extern "C" int b200wmma_dlrm_fwd(const void* input, void* output, uint32_t m, uint32_t m_stride,
                                 uint32_t k, uint32_t batch, uint32_t out_stride, void* stream)
{
    using namespace b200wmma;
    using namespace b200wmma::dlrm;
    clear_error();
    const bool general = needs_general(m, k, out_stride);
    if(int e = check_common(input, m, m_stride, k, batch, general))
        return e;
    B200_REQUIRE(output, B200WMMA_ERR_INVALID_ARG, "dlrm_fwd: output must be non-null");
    B200_REQUIRE(out_stride >= k + m * (m - 1) / 2, B200WMMA_ERR_INVALID_ARG,
                 "dlrm_fwd: out_stride %u smaller than k + m(m-1)/2 = %u", out_stride,
                 k + m * (m - 1) / 2);
    B200_REQUIRE(out_stride % 8 == 0 && aligned16(output), B200WMMA_ERR_ALIGNMENT,
                 "dlrm_fwd: output rows must be 16-byte aligned (out_stride %% 8 == 0)");
    if(int e = require_sm100())
        return e;
    if(general)
        return launch_dlrm_fwd_general(input, output, m, m_stride, k, batch, out_stride, false, as_stream(stream));
    unsigned* status = nullptr;
    if(int e = status_word_ptr(&status))
        return e;
    CUtensorMap tm_x;
    if(int e = sample_tmap(&tm_x, input, m, m_stride, k, batch))
        return e;
    const uint32_t nbox = (k + 63) / 64;
    auto per_warp = [&](uint32_t stages) -> size_t {
        return static_cast<size_t>(stages) * nbox * BOX_BYTES + 2 * out_stride * 2 + stages * 8;
    };
    // A warp's samples go through one after the other, so what keeps the memory system busy is the number of warps
    // per SM: two stages per warp and as many warps as shared memory holds.
    const size_t budget = 227 * 1024 - 1024 - 16;
    uint32_t     stages = 2;
    if(const int forced = tuning::get(tuning::DLRM_FWD_STAGES); forced == 2 || forced == 3)
        stages = static_cast<uint32_t>(forced);
    const uint32_t warps = warps_for(batch, budget / per_warp(stages), FWD_MAX_WARPS, tuning::get(tuning::DLRM_FWD_WARPS));
    B200_REQUIRE(warps >= 1, B200WMMA_ERR_INVALID_ARG, "dlrm_fwd: one sample's tiles do not fit in shared memory");
    auto* const  dlrm_fwd_kernel = stages == 3 ? dlrm::dlrm_fwd_kernel<3> : dlrm::dlrm_fwd_kernel<2>;
    const size_t smem            = 1024 + warps * per_warp(stages) + 16;
    static size_t attr_set_dev[MAX_DEVICES][2];
    size_t&       attr_set = attr_set_dev[current_device_slot()][stages - 2];
    if(smem > 48 * 1024 && smem > attr_set)
    {
        B200_CHECK_CUDA(cudaFuncSetAttribute(dlrm_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem)));
        attr_set = smem;
    }
    const uint32_t grid = grid_for(batch, reinterpret_cast<const void*>(dlrm_fwd_kernel), smem, warps);
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t  cfg = pdl_config(attr, grid, smem, as_stream(stream), warps);
    B200_CHECK_CUDA(cudaLaunchKernelEx(&cfg, dlrm_fwd_kernel, tm_x, static_cast<__half*>(output), m, m_stride, k, batch,
                                       out_stride, status));
    return B200WMMA_OK;
}

extern "C" int b200wmma_dlrm_bwd(const void* input, const void* upstream, void* grad,
                                 void* bottom_mlp_grad, uint32_t m, uint32_t m_stride, uint32_t k,
                                 uint32_t batch, uint32_t upstream_stride, int fuse_mlp_into_row0,
                                 void* stream)
{
    using namespace b200wmma;
    using namespace b200wmma::dlrm;
    clear_error();
    const bool general = needs_general(m, k, upstream_stride);
    if(int e = check_common(input, m, m_stride, k, batch, general))
        return e;
    B200_REQUIRE(upstream && grad, B200WMMA_ERR_INVALID_ARG, "dlrm_bwd: upstream and grad must be non-null");
    B200_REQUIRE(upstream_stride >= k + m * (m - 1) / 2, B200WMMA_ERR_INVALID_ARG,
                 "dlrm_bwd: upstream_stride %u smaller than k + m(m-1)/2 = %u", upstream_stride,
                 k + m * (m - 1) / 2);
    B200_REQUIRE(upstream_stride % 8 == 0 && aligned16(upstream) && aligned16(grad)
                     && (!bottom_mlp_grad || aligned16(bottom_mlp_grad)),
                 B200WMMA_ERR_ALIGNMENT,
                 "dlrm_bwd: buffers must be 16-byte aligned and upstream_stride %% 8 == 0");
    if(int e = require_sm100())
        return e;
    if(general)
        return launch_dlrm_bwd_general(input, upstream, grad, bottom_mlp_grad, m, m_stride, k, batch, upstream_stride,
                                       fuse_mlp_into_row0, false, as_stream(stream));
    unsigned* status = nullptr;
    if(int e = status_word_ptr(&status))
        return e;
    CUtensorMap tm_x, tm_g;
    if(int e = sample_tmap(&tm_x, input, m, m_stride, k, batch))
        return e;
    if(int e = sample_tmap(&tm_g, grad, m, m_stride, k, batch))
        return e;
    const uint32_t nbox    = (k + 63) / 64;
    const uint32_t up_slot = (upstream_stride * 2 + 127) & ~127u;
    auto per_warp = [&](uint32_t stages) -> size_t {
        return static_cast<size_t>(stages) * (nbox * BOX_BYTES + up_slot) + MAX_M * TPITCH * 2 + stages * 8;
    };
    // warps per CTA from what one SM's shared memory holds (see the kernel's header comment)
    const size_t budget = 227 * 1024 - 1024 - 16;
    uint32_t     stages = 2;
    if(const int forced = tuning::get(tuning::DLRM_BWD_STAGES); forced == 2 || forced == 3)
        stages = static_cast<uint32_t>(forced);
    const uint32_t warps = warps_for(batch, budget / per_warp(stages), BWD_MAX_WARPS, tuning::get(tuning::DLRM_BWD_WARPS));
    B200_REQUIRE(warps >= 1, B200WMMA_ERR_INVALID_ARG, "dlrm_bwd: one sample's tiles do not fit in shared memory");
    auto* const  kernel = stages == 3 ? dlrm_bwd_kernel<3> : dlrm_bwd_kernel<2>;
    const size_t smem   = 1024 + warps * per_warp(stages) + 16;
    static size_t attr_set_dev[MAX_DEVICES][2];
    size_t&       attr_set = attr_set_dev[current_device_slot()][stages - 2];
    if(smem > 48 * 1024 && smem > attr_set)
    {
        B200_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attr_set = smem;
    }
    const uint32_t grid = grid_for(batch, reinterpret_cast<const void*>(kernel), smem, warps);
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t  cfg = pdl_config(attr, grid, smem, as_stream(stream), warps);
    B200_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kernel, tm_x, tm_g, static_cast<const __half*>(upstream),
                                       static_cast<__half*>(bottom_mlp_grad), m, m_stride, k, batch, upstream_stride,
                                       fuse_mlp_into_row0, status));
    return B200WMMA_OK;
}

// fp32 data (the second data type of the reference's DLRM sweep, test/dlrm/test/dlrm_test_params.hpp:51): always on the
// block-tiled kernels of dlrm_general.cu.
extern "C" int b200wmma_dlrm_fwd_f32(const float* input, float* output, uint32_t m, uint32_t m_stride, uint32_t k,
                                     uint32_t batch, uint32_t out_stride, void* stream)
{
    using namespace b200wmma;
    using namespace b200wmma::dlrm;
    clear_error();
    if(int e = check_common(input, m, m_stride, k, batch, true))
        return e;
    B200_REQUIRE(output, B200WMMA_ERR_INVALID_ARG, "dlrm_fwd_f32: output must be non-null");
    B200_REQUIRE(out_stride >= k + m * (m - 1) / 2, B200WMMA_ERR_INVALID_ARG,
                 "dlrm_fwd_f32: out_stride %u smaller than k + m(m-1)/2 = %u", out_stride, k + m * (m - 1) / 2);
    if(int e = require_sm100())
        return e;
    return launch_dlrm_fwd_general(input, output, m, m_stride, k, batch, out_stride, true, as_stream(stream));
}

extern "C" int b200wmma_dlrm_bwd_f32(const float* input, const float* upstream, float* grad, float* bottom_mlp_grad, uint32_t m,
                                     uint32_t m_stride, uint32_t k, uint32_t batch, uint32_t upstream_stride,
                                     int fuse_mlp_into_row0, void* stream)
{
    using namespace b200wmma;
    using namespace b200wmma::dlrm;
    clear_error();
    if(int e = check_common(input, m, m_stride, k, batch, true))
        return e;
    B200_REQUIRE(upstream && grad, B200WMMA_ERR_INVALID_ARG, "dlrm_bwd_f32: upstream and grad must be non-null");
    B200_REQUIRE(upstream_stride >= k + m * (m - 1) / 2, B200WMMA_ERR_INVALID_ARG,
                 "dlrm_bwd_f32: upstream_stride %u smaller than k + m(m-1)/2 = %u", upstream_stride, k + m * (m - 1) / 2);
    B200_REQUIRE(aligned16(grad), B200WMMA_ERR_ALIGNMENT, "dlrm_bwd_f32: grad must be 16-byte aligned");
    if(int e = require_sm100())
        return e;
    return launch_dlrm_bwd_general(input, upstream, grad, bottom_mlp_grad, m, m_stride, k, batch, upstream_stride,
                                   fuse_mlp_into_row0, true, as_stream(stream));
}
