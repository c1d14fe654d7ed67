// DLRM dot interaction for any number of feature rows: the sizes of the reference's own test sweep
// (m = 128 and 1024, test/dlrm/test/dlrm_test_params.hpp:55-58) that the one-warp-per-sample kernels of
// dlrm.cu (m <= 32, k <= 256) do not take.
//
// Written against this repository's rocWMMA-compatible fragment API, like the reference's kernels
// (test/dlrm/device/dlrm_dot_fwd.hpp:37-136, dlrm_dot_bwd.hpp:35-172), but without their global scratch:
//   forward : one 16x16 block of Z = X X^T per warp, lower-triangle blocks only; the accumulator goes through a
//             256-float shared tile and the elements with i > j are written straight to their place in the
//             packed row [X row 0 | strict lower triangle | zero pad].
//   backward: grad = T X with T the symmetric matrix rebuilt from the packed upstream row (zero diagonal).
//             A CTA owns 16 rows of grad and 8 x 16 columns of k; per 16-wide step over the inner dimension the
//             CTA gathers the 16x16 block of T once into shared memory (the reference's trilReconstruct pass,
//             samples/simple_dlrm.cpp:290-331, fused) and every warp multiplies it with its block of X.
#include "common.cuh"

#include <rocwmma/rocwmma.hpp>

namespace b200wmma
{
    namespace dlrmg
    {
        using namespace rocwmma;
        constexpr uint32_t T       = 16; // block size
        constexpr uint32_t WARPS   = 8;
        constexpr uint32_t THREADS = WARPS * 32;

        __device__ __forceinline__ size_t tri(size_t i, size_t j) // index of (i, j), i > j, in the row-major strict lower triangle
        {
            return i * (i - 1) / 2 + j;
        }

        // DataT: float16_t, or float32_t (the reference sweep's second data type; fp32 fragments multiply through
        // three TF32 products)
        template <typename DataT>
        __global__ void __launch_bounds__(THREADS)
            dlrm_fwd_general_kernel(const DataT* __restrict__ x, DataT* __restrict__ out, uint32_t m, uint32_t m_stride,
                                    uint32_t k, uint32_t out_stride, uint32_t nblk, uint32_t npairs)
        {
            __shared__ float tile[WARPS][T * T];
            const uint32_t   warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
            const uint32_t   b    = blockIdx.y;
            const uint32_t   p    = blockIdx.x * WARPS + warp; // index of the (bi, bj <= bi) block pair
            const DataT*     xb   = x + static_cast<size_t>(b) * m_stride * k;
            DataT*           ob   = out + static_cast<size_t>(b) * out_stride;
            if(p >= npairs)
                return;
            // p = bi (bi + 1) / 2 + bj
            uint32_t bi = static_cast<uint32_t>((sqrtf(8.0f * p + 1.0f) - 1.0f) * 0.5f);
            while(bi * (bi + 1) / 2 > p)
                --bi;
            while((bi + 1) * (bi + 2) / 2 <= p)
                ++bi;
            const uint32_t bj = p - bi * (bi + 1) / 2;
            (void)nblk;

            fragment<matrix_a, T, T, T, DataT, row_major> fa;
            fragment<matrix_b, T, T, T, DataT, col_major> fb; // B = X^T: B[h][j] = X[j][h], K contiguous
            fragment<accumulator, T, T, T, float32_t>     acc;
            fill_fragment(acc, 0.0f);
            const DataT* arow = xb + static_cast<size_t>(bi) * T * k;
            const DataT* brow = xb + static_cast<size_t>(bj) * T * k;
            for(uint32_t h = 0; h < k; h += T)
            {
                load_matrix_sync(fa, arow + h, k);
                load_matrix_sync(fb, brow + h, k);
                mma_sync(acc, fa, fb, acc);
            }
            store_matrix_sync(tile[warp], acc, T, mem_row_major);
            __syncwarp();
            for(uint32_t e = lane; e < T * T; e += 32)
            {
                const uint32_t i = bi * T + e / T, j = bj * T + e % T;
                if(i < m && j < i)
                    ob[k + tri(i, j)] = static_cast<DataT>(tile[warp][e]);
            }
            if(p == 0)
            {
                // row 0 of X in front, zeros behind the triangle
                for(uint32_t h = lane; h < k; h += 32)
                    ob[h] = xb[h];
                for(uint32_t h = k + m * (m - 1) / 2 + lane; h < out_stride; h += 32)
                    ob[h] = static_cast<DataT>(0.0f);
            }
        }

        template <typename DataT>
        __global__ void __launch_bounds__(THREADS)
            dlrm_bwd_general_kernel(const DataT* __restrict__ x, const DataT* __restrict__ up, DataT* __restrict__ grad,
                                    DataT* __restrict__ mlp, uint32_t m, uint32_t m_stride, uint32_t k, uint32_t up_stride,
                                    int fuse)
        {
            __shared__ __align__(16) DataT tblk[T * T];
            __shared__ float                   tile[WARPS][T * T];
            const uint32_t   warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
            const uint32_t   b    = blockIdx.z;
            const uint32_t   bi   = blockIdx.y; // 16 rows of grad
            const uint32_t   kc   = (blockIdx.x * WARPS + warp) * T; // this warp's 16 columns of k
            const bool       live = kc < k; // warps right of the matrix still help to build T and keep the barriers
            const DataT*     xb   = x + static_cast<size_t>(b) * m_stride * k;
            const DataT*     ub   = up + static_cast<size_t>(b) * up_stride;
            DataT*           gb   = grad + static_cast<size_t>(b) * m_stride * k;
            const uint32_t   nblk = (m + T - 1) / T;

            fragment<matrix_a, T, T, T, DataT, row_major> fa;
            fragment<matrix_b, T, T, T, DataT, row_major> fb; // B[j][h] = X[j][h], N contiguous
            fragment<accumulator, T, T, T, float32_t>         acc;
            fill_fragment(acc, 0.0f);
            for(uint32_t jb = 0; jb < nblk; ++jb)
            {
                // block (bi, jb) of the symmetric matrix, one element per thread
                {
                    const uint32_t e = threadIdx.x;
                    const uint32_t i = bi * T + e / T, j = jb * T + e % T;
                    DataT          v = static_cast<DataT>(0.0f);
                    if(i < m && j < m && i != j)
                        v = ub[k + (i > j ? tri(i, j) : tri(j, i))];
                    tblk[e] = v;
                }
                __syncthreads();
                if(live)
                {
                    load_matrix_sync(fa, tblk, T);
                    load_matrix_sync(fb, xb + static_cast<size_t>(jb) * T * k + kc, k);
                    mma_sync(acc, fa, fb, acc);
                }
                __syncthreads();
            }
            if(!live)
                return;
            store_matrix_sync(tile[warp], acc, T, mem_row_major);
            __syncwarp();
            for(uint32_t e = lane; e < T * T; e += 32)
            {
                const uint32_t i = bi * T + e / T, h = kc + e % T;
                if(i < m)
                {
                    float v = tile[warp][e];
                    if(fuse && i == 0)
                        v = static_cast<float>(static_cast<DataT>(v)) + static_cast<float>(ub[h]);
                    gb[static_cast<size_t>(i) * k + h] = static_cast<DataT>(v);
                }
            }
            if(bi == 0 && mlp != nullptr && lane < T)
                mlp[static_cast<size_t>(b) * k + kc + lane] = ub[kc + lane];
        }
    } // namespace dlrmg

    int launch_dlrm_fwd_general(const void* input, void* output, uint32_t m, uint32_t m_stride, uint32_t k, uint32_t batch,
                                uint32_t out_stride, bool f32, cudaStream_t stream)
    {
        using namespace dlrmg;
        const uint32_t nblk = ceil_div(m, T), npairs = nblk * (nblk + 1) / 2;
        B200_REQUIRE(k % T == 0, B200WMMA_ERR_UNSUPPORTED, "dlrm_fwd: k must be a multiple of 16");
        // (row stride and batch limits are checked by the caller before any device is touched)
        dim3 grid(ceil_div(npairs, WARPS), batch);
        if(f32)
            dlrm_fwd_general_kernel<float><<<grid, THREADS, 0, stream>>>(static_cast<const float*>(input),
                                                                         static_cast<float*>(output), m, m_stride, k,
                                                                         out_stride, nblk, npairs);
        else
            dlrm_fwd_general_kernel<rocwmma::float16_t><<<grid, THREADS, 0, stream>>>(
                static_cast<const rocwmma::float16_t*>(input), static_cast<rocwmma::float16_t*>(output), m, m_stride, k,
                out_stride, nblk, npairs);
        B200_CHECK_CUDA(cudaGetLastError());
        return B200WMMA_OK;
    }

    int launch_dlrm_bwd_general(const void* input, const void* upstream, void* grad, void* bottom_mlp_grad, uint32_t m,
                                uint32_t m_stride, uint32_t k, uint32_t batch, uint32_t upstream_stride, int fuse, bool f32,
                                cudaStream_t stream)
    {
        using namespace dlrmg;
        const uint32_t nblk = ceil_div(m, T);
        B200_REQUIRE(k % T == 0, B200WMMA_ERR_UNSUPPORTED, "dlrm_bwd: k must be a multiple of 16");
        // (row stride and batch limits are checked by the caller before any device is touched)
        dim3 grid(ceil_div(k, T * WARPS), nblk, batch);
        if(f32)
            dlrm_bwd_general_kernel<float><<<grid, THREADS, 0, stream>>>(
                static_cast<const float*>(input), static_cast<const float*>(upstream), static_cast<float*>(grad),
                static_cast<float*>(bottom_mlp_grad), m, m_stride, k, upstream_stride, fuse);
        else
            dlrm_bwd_general_kernel<rocwmma::float16_t><<<grid, THREADS, 0, stream>>>(
                static_cast<const rocwmma::float16_t*>(input), static_cast<const rocwmma::float16_t*>(upstream),
                static_cast<rocwmma::float16_t*>(grad), static_cast<rocwmma::float16_t*>(bottom_mlp_grad), m, m_stride, k,
                upstream_stride, fuse);
        B200_CHECK_CUDA(cudaGetLastError());
        return B200WMMA_OK;
    }
} // namespace b200wmma
