// DLRM dot-interaction forward and backward, one warp per sample, everything fused.
//
// Forward stands in for dlrmDotFwd (samples/simple_dlrm.cpp:184-284;
// test/dlrm/device/dlrm_dot_fwd.hpp:37-136).  The reference computes each 16x16 tile of
// Z = X X^T in its own wave, stores it to a global fp32 scratch, re-reads the scratch and
// writes the strict lower triangle element by element.  Here a warp brings the sample's
// X (m x k fp16) into shared memory once, runs the lower-triangle tiles on mma.sync with
// fp32 accumulators, packs [X row 0 | tril(Z)] into a shared-memory row and writes it with
// 16-byte coalesced stores: X is read once, the output written once, no scratch.
//
// Backward stands in for trilReconstruct + dlrmDotBwd (samples/simple_dlrm.cpp:290-331,
// :349-441; test/dlrm/device/dlrm_dot_bwd.hpp:35-172), which rebuild the symmetric matrix in
// global memory in one kernel, synchronise on the host, and multiply in a second kernel.
// Here the packed upstream row is expanded to the symmetric m x m fp16 matrix in shared
// memory, multiplied with X on mma.sync and written back in the same pass, optionally with
// the bottom-MLP pass-through gradient added to row 0.
//
// Both are HBM-bound: the arithmetic is 2*m*m*k flop per sample against ~8-15 KB of traffic.
#include "common.cuh"

namespace b200wmma
{
    namespace dlrm
    {
        constexpr int WARPS  = 4;
        constexpr int MAX_M  = 32;
        constexpr int MAX_K  = 256;
        constexpr int TPITCH = 40; // halfs per row of the 32x32 symmetric matrix (+8 pad)

        __device__ __forceinline__ uint32_t smem_u32(const void* p)
        {
            return static_cast<uint32_t>(__cvta_generic_to_shared(p));
        }
        __device__ __forceinline__ void cp_async16(void* dst_smem, const void* src)
        {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)),
                         "l"(src)
                         : "memory");
        }
        __device__ __forceinline__ void cp_async_wait_all()
        {
            asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
        }
        __device__ __forceinline__ void
            ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p)
        {
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                         : "r"(smem_u32(p)));
        }
        __device__ __forceinline__ void
            ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p)
        {
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                         : "r"(smem_u32(p)));
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

        // Copies rows 0..m-1 of one sample (k halfs each, contiguous in global memory) into the
        // padded shared-memory tile with 16-byte async copies.  Whole warp participates.
        __device__ __forceinline__ void load_sample(__half* xs, uint32_t xpitch, const __half* src,
                                                    uint32_t m, uint32_t k, uint32_t lane)
        {
            const uint32_t chunks_per_row = k >> 3;
            const uint32_t total          = m * chunks_per_row;
            for(uint32_t i = lane; i < total; i += 32)
            {
                const uint32_t r = i / chunks_per_row, ch = i - r * chunks_per_row;
                cp_async16(xs + r * xpitch + ch * 8, src + static_cast<size_t>(r) * k + ch * 8);
            }
        }

        // ---------------------------------- forward ----------------------------------------
        __global__ void __launch_bounds__(WARPS * 32)
            dlrm_fwd_kernel(const __half* __restrict__ input, __half* __restrict__ output,
                            uint32_t m, uint32_t m_stride, uint32_t k, uint32_t batch,
                            uint32_t out_stride)
        {
            extern __shared__ __align__(16) uint8_t smem[];
            const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            const uint32_t xpitch   = k + 8;
            const uint32_t per_warp = MAX_M * xpitch + out_stride; // halfs
            __half*        xs       = reinterpret_cast<__half*>(smem) + warp * per_warp;
            __half*        orow     = xs + MAX_M * xpitch;
            const uint32_t g = lane >> 2, t = lane & 3;
            const uint32_t tri_end = k + m * (m - 1) / 2;

            // rows m..31 take part in the MMA tiles as zeros; they are never overwritten
            for(uint32_t i = m * xpitch + lane; i < MAX_M * xpitch; i += 32)
                xs[i] = __float2half(0.0f);
            // columns past the packed triangle are written as zero for every sample
            for(uint32_t i = tri_end + lane; i < out_stride; i += 32)
                orow[i] = __float2half(0.0f);

            for(uint32_t b = blockIdx.x * WARPS + warp; b < batch; b += gridDim.x * WARPS)
            {
                load_sample(xs, xpitch, input + static_cast<size_t>(b) * m_stride * k, m, k, lane);
                cp_async_wait_all();
                __syncwarp();

                // acc0: rows 0-15 x cols 0-15 ; acc1: rows 16-31 x cols 0-31
                float acc0[2][4] = {}, acc1[4][4] = {};
                const bool two_blocks = m > 16;
                for(uint32_t ks = 0; ks < k; ks += 16)
                {
                    uint32_t a0[4], a1[4], bf[8];
                    ldmatrix_x4(a0[0], a0[1], a0[2], a0[3],
                                xs + (lane & 15) * xpitch + ks + (lane >> 4) * 8);
                    // B = X^T: n index = row of X.  One x4 load covers two 8-wide n tiles.
                    const uint32_t brow = (lane & 7) + (lane >> 4) * 8, bcol = ks + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(bf[0], bf[1], bf[2], bf[3], xs + brow * xpitch + bcol);
                    mma_16816(acc0[0], a0, bf[0], bf[1]);
                    mma_16816(acc0[1], a0, bf[2], bf[3]);
                    if(two_blocks)
                    {
                        ldmatrix_x4(a1[0], a1[1], a1[2], a1[3],
                                    xs + (16 + (lane & 15)) * xpitch + ks + (lane >> 4) * 8);
                        ldmatrix_x4(bf[4], bf[5], bf[6], bf[7], xs + (16 + brow) * xpitch + bcol);
                        mma_16816(acc1[0], a1, bf[0], bf[1]);
                        mma_16816(acc1[1], a1, bf[2], bf[3]);
                        mma_16816(acc1[2], a1, bf[4], bf[5]);
                        mma_16816(acc1[3], a1, bf[6], bf[7]);
                    }
                }

                // pack: [ X row 0 | strict lower triangle, row-major ]
                for(uint32_t i = lane; i < k; i += 32)
                    orow[i] = xs[i];
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
                __syncwarp();
                uint4*       dst = reinterpret_cast<uint4*>(output + static_cast<size_t>(b) * out_stride);
                const uint4* src = reinterpret_cast<const uint4*>(orow);
                for(uint32_t i = lane; i < (out_stride >> 3); i += 32)
                    __stcs(dst + i, src[i]);
                __syncwarp(); // xs / orow are rewritten by the next sample
            }
        }

        // ---------------------------------- backward ---------------------------------------
        __global__ void __launch_bounds__(WARPS * 32)
            dlrm_bwd_kernel(const __half* __restrict__ input, const __half* __restrict__ upstream,
                            __half* __restrict__ grad, __half* __restrict__ bottom_mlp_grad,
                            uint32_t m, uint32_t m_stride, uint32_t k, uint32_t batch,
                            uint32_t up_stride, int fuse_mlp)
        {
            extern __shared__ __align__(16) uint8_t smem[];
            const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            const uint32_t xpitch   = k + 8;
            const uint32_t per_warp = MAX_M * xpitch + up_stride + MAX_M * TPITCH; // halfs
            __half*        xs       = reinterpret_cast<__half*>(smem) + warp * per_warp;
            __half*        gs       = xs + MAX_M * xpitch; // packed upstream row
            __half*        ts       = gs + up_stride; // symmetric matrix, 32 x TPITCH
            const uint32_t g = lane >> 2, t = lane & 3;

            for(uint32_t b = blockIdx.x * WARPS + warp; b < batch; b += gridDim.x * WARPS)
            {
                // rows m..31 of X must be zero for the MMA; the tile is overwritten with dX
                // below, so they are cleared for every sample
                for(uint32_t i = m * xpitch + lane; i < MAX_M * xpitch; i += 32)
                    xs[i] = __float2half(0.0f);
                load_sample(xs, xpitch, input + static_cast<size_t>(b) * m_stride * k, m, k, lane);
                {
                    const __half* up = upstream + static_cast<size_t>(b) * up_stride;
                    for(uint32_t i = lane; i < (up_stride >> 3); i += 32)
                        cp_async16(gs + i * 8, up + i * 8);
                }
                cp_async_wait_all();
                __syncwarp();

                // symmetric matrix with zero diagonal; lane = column index
                for(uint32_t i = 0; i < MAX_M; ++i)
                {
                    const uint32_t j  = lane;
                    __half         v  = __float2half(0.0f);
                    if(i < m && j < m && i != j)
                    {
                        const uint32_t hi = max(i, j), lo = min(i, j);
                        v = gs[k + hi * (hi - 1) / 2 + lo];
                    }
                    ts[i * TPITCH + j] = v;
                }
                if(bottom_mlp_grad)
                {
                    uint4*       dst = reinterpret_cast<uint4*>(bottom_mlp_grad + static_cast<size_t>(b) * k);
                    const uint4* src = reinterpret_cast<const uint4*>(gs);
                    for(uint32_t i = lane; i < (k >> 3); i += 32)
                        __stcs(dst + i, src[i]);
                }
                __syncwarp();

                // A fragments of the symmetric matrix: [row block][k step]
                uint32_t af[2][2][4];
#pragma unroll
                for(int rb = 0; rb < 2; ++rb)
#pragma unroll
                    for(int ks = 0; ks < 2; ++ks)
                        ldmatrix_x4(af[rb][ks][0], af[rb][ks][1], af[rb][ks][2], af[rb][ks][3],
                                    ts + (16 * rb + (lane & 15)) * TPITCH + 16 * ks + (lane >> 4) * 8);

                // dX[:, n0:n0+16] depends only on X[:, n0:n0+16]: compute a 16-column slab,
                // then overwrite those columns of the shared tile with the result.
                for(uint32_t n0 = 0; n0 < k; n0 += 16)
                {
                    float    acc[2][2][4] = {};
                    uint32_t bf[2][4];
#pragma unroll
                    for(int ks = 0; ks < 2; ++ks)
                        ldmatrix_x4_trans(bf[ks][0], bf[ks][1], bf[ks][2], bf[ks][3],
                                          xs + (16 * ks + (lane & 7) + ((lane >> 3) & 1) * 8) * xpitch
                                              + n0 + (lane >> 4) * 8);
#pragma unroll
                    for(int rb = 0; rb < 2; ++rb)
#pragma unroll
                        for(int ks = 0; ks < 2; ++ks)
                        {
                            mma_16816(acc[rb][0], af[rb][ks], bf[ks][0], bf[ks][1]);
                            mma_16816(acc[rb][1], af[rb][ks], bf[ks][2], bf[ks][3]);
                        }
                    __syncwarp(); // every lane has read this slab of X
#pragma unroll
                    for(int rb = 0; rb < 2; ++rb)
#pragma unroll
                        for(int nt = 0; nt < 2; ++nt)
#pragma unroll
                            for(int h = 0; h < 2; ++h)
                            {
                                const uint32_t r = 16 * rb + g + 8 * h, c = n0 + 8 * nt + 2 * t;
                                float          v0 = acc[rb][nt][2 * h], v1 = acc[rb][nt][2 * h + 1];
                                if(fuse_mlp && r == 0)
                                {
                                    v0 += __half2float(gs[c]);
                                    v1 += __half2float(gs[c + 1]);
                                }
                                *reinterpret_cast<__half2*>(xs + r * xpitch + c)
                                    = __floats2half2_rn(v0, v1);
                            }
                }
                __syncwarp();
                {
                    __half*        dst            = grad + static_cast<size_t>(b) * m_stride * k;
                    const uint32_t chunks_per_row = k >> 3;
                    for(uint32_t i = lane; i < m * chunks_per_row; i += 32)
                    {
                        const uint32_t r = i / chunks_per_row, ch = i - r * chunks_per_row;
                        __stcs(reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * k + ch * 8),
                               *reinterpret_cast<const uint4*>(xs + r * xpitch + ch * 8));
                    }
                }
                __syncwarp();
            }
        }

        static int check_common(const void* input, uint32_t m, uint32_t m_stride, uint32_t k,
                                uint32_t batch)
        {
            B200_REQUIRE(input, B200WMMA_ERR_INVALID_ARG, "dlrm: input must be non-null");
            B200_REQUIRE(m >= 1 && batch >= 1 && k >= 1, B200WMMA_ERR_INVALID_ARG,
                         "dlrm: m, k, batch must be non-zero");
            B200_REQUIRE(m_stride >= m, B200WMMA_ERR_INVALID_ARG, "dlrm: m_stride must be >= m");
            B200_REQUIRE(m <= MAX_M, B200WMMA_ERR_UNSUPPORTED,
                         "dlrm: m = %u not supported (this kernel handles m <= %d)", m, MAX_M);
            B200_REQUIRE(k % 16 == 0 && k <= MAX_K, B200WMMA_ERR_UNSUPPORTED,
                         "dlrm: k = %u not supported (multiple of 16, <= %d)", k, MAX_K);
            B200_REQUIRE(aligned16(input), B200WMMA_ERR_ALIGNMENT, "dlrm: input must be 16-byte aligned");
            return B200WMMA_OK;
        }

        static uint32_t grid_for(uint32_t batch, const void* kernel, size_t smem_bytes)
        {
            int dev = 0, sms = 148, per_sm = 1;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, WARPS * 32, smem_bytes);
            if(per_sm < 1)
                per_sm = 1;
            const uint32_t want = ceil_div(batch, WARPS);
            const uint32_t cap  = static_cast<uint32_t>(sms) * per_sm;
            return want < cap ? want : cap;
        }
    } // namespace dlrm
} // namespace b200wmma

extern "C" int b200wmma_dlrm_fwd(const void* input, void* output, uint32_t m, uint32_t m_stride,
                                 uint32_t k, uint32_t batch, uint32_t out_stride, void* stream)
{
    using namespace b200wmma;
    using namespace b200wmma::dlrm;
    clear_error();
    if(int e = check_common(input, m, m_stride, k, batch))
        return e;
    B200_REQUIRE(output, B200WMMA_ERR_INVALID_ARG, "dlrm_fwd: output must be non-null");
    B200_REQUIRE(out_stride >= k + m * (m - 1) / 2, B200WMMA_ERR_INVALID_ARG,
                 "dlrm_fwd: out_stride %u smaller than k + m(m-1)/2 = %u", out_stride,
                 k + m * (m - 1) / 2);
    B200_REQUIRE(out_stride % 8 == 0 && aligned16(output), B200WMMA_ERR_ALIGNMENT,
                 "dlrm_fwd: output rows must be 16-byte aligned (out_stride %% 8 == 0)");
    B200_REQUIRE(out_stride <= 2048, B200WMMA_ERR_UNSUPPORTED, "dlrm_fwd: out_stride too large");
    if(int e = require_sm100())
        return e;
    const size_t smem = static_cast<size_t>(WARPS) * (MAX_M * (k + 8) + out_stride) * sizeof(__half);
    static size_t attr_set = 0;
    if(smem > 48 * 1024 && smem > attr_set)
    {
        B200_CHECK_CUDA(cudaFuncSetAttribute(dlrm_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem)));
        attr_set = smem;
    }
    const uint32_t grid = grid_for(batch, reinterpret_cast<const void*>(dlrm_fwd_kernel), smem);
    dlrm_fwd_kernel<<<grid, WARPS * 32, smem, as_stream(stream)>>>(
        static_cast<const __half*>(input), static_cast<__half*>(output), m, m_stride, k, batch, out_stride);
    B200_CHECK_CUDA(cudaGetLastError());
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
    if(int e = check_common(input, m, m_stride, k, batch))
        return e;
    B200_REQUIRE(upstream && grad, B200WMMA_ERR_INVALID_ARG, "dlrm_bwd: upstream and grad must be non-null");
    B200_REQUIRE(upstream_stride >= k + m * (m - 1) / 2, B200WMMA_ERR_INVALID_ARG,
                 "dlrm_bwd: upstream_stride %u smaller than k + m(m-1)/2 = %u", upstream_stride,
                 k + m * (m - 1) / 2);
    B200_REQUIRE(upstream_stride % 8 == 0 && aligned16(upstream) && aligned16(grad)
                     && (!bottom_mlp_grad || aligned16(bottom_mlp_grad)),
                 B200WMMA_ERR_ALIGNMENT,
                 "dlrm_bwd: buffers must be 16-byte aligned and upstream_stride %% 8 == 0");
    B200_REQUIRE(upstream_stride <= 2048, B200WMMA_ERR_UNSUPPORTED, "dlrm_bwd: upstream_stride too large");
    if(int e = require_sm100())
        return e;
    const size_t smem = static_cast<size_t>(WARPS) * (MAX_M * (k + 8) + upstream_stride + MAX_M * TPITCH)
                        * sizeof(__half);
    static size_t attr_set = 0;
    if(smem > 48 * 1024 && smem > attr_set)
    {
        B200_CHECK_CUDA(cudaFuncSetAttribute(dlrm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem)));
        attr_set = smem;
    }
    const uint32_t grid = grid_for(batch, reinterpret_cast<const void*>(dlrm_bwd_kernel), smem);
    dlrm_bwd_kernel<<<grid, WARPS * 32, smem, as_stream(stream)>>>(
        static_cast<const __half*>(input), static_cast<const __half*>(upstream), static_cast<__half*>(grad),
        static_cast<__half*>(bottom_mlp_grad), m, m_stride, k, batch, upstream_stride, fuse_mlp_into_row0);
    B200_CHECK_CUDA(cudaGetLastError());
    return B200WMMA_OK;
}
