// Streaming GEMV  y = alpha * A x + beta * y  for fp32 and fp64.
//
// Stands in for sgemv_rocwmma_d / dgemv_rocwmma_d (samples/simple_sgemv.cpp:103-155,
// samples/simple_dgemv.cpp:103).  The reference pushes x through 16x16x16 MMA blocks as a
// 16-column "matrix"; a matrix-vector product has no data reuse for tensor cores to exploit,
// so this is a plain HBM-bound stream instead: every element of A is read exactly once with
// 16-byte loads that bypass L1 allocation, x (n elements, shared by all rows) comes through
// the read-only path, partial sums are reduced with warp shuffles and one shared-memory
// step, and alpha / beta are applied in the same pass.
#include "common.cuh"
#include "tuning.cuh"

namespace b200wmma
{
    namespace gemv
    {
        constexpr int THREADS = 256;

        template <typename T>
        struct Vec;
        template <>
        struct Vec<float>
        {
            using type = float4;
            static constexpr int N = 4;
            static __device__ __forceinline__ float dot(const float4& a, const float4& b, float acc)
            {
                acc = fmaf(a.x, b.x, acc);
                acc = fmaf(a.y, b.y, acc);
                acc = fmaf(a.z, b.z, acc);
                acc = fmaf(a.w, b.w, acc);
                return acc;
            }
        };
        template <>
        struct Vec<double>
        {
            using type = double2;
            static constexpr int N = 2;
            static __device__ __forceinline__ double dot(const double2& a, const double2& b, double acc)
            {
                acc = fma(a.x, b.x, acc);
                acc = fma(a.y, b.y, acc);
                return acc;
            }
        };

        template <typename T>
        __device__ __forceinline__ T warp_sum(T v)
        {
#pragma unroll
            for(int o = 16; o > 0; o >>= 1)
                v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            return v;
        }

        // Row-major A: one CTA owns ROWS consecutive rows (one, by default); its 256 threads stride over the
        // columns so that each warp-wide load instruction covers 512 contiguous bytes of a row.
        template <typename T, int ROWS, int UNROLL>
        __global__ void __launch_bounds__(THREADS)
            gemv_row_major_kernel(uint32_t m, uint32_t n, const T* __restrict__ a, size_t lda,
                                  const T* __restrict__ x, T* __restrict__ y, T alpha, T beta,
                                  int vec_ok)
        {
            using V          = typename Vec<T>::type;
            constexpr int VN = Vec<T>::N;
            const uint32_t row0 = blockIdx.x * ROWS;
            const T*       rows[ROWS];
#pragma unroll
            for(int r = 0; r < ROWS; ++r)
                rows[r] = a + static_cast<size_t>(min(row0 + r, m - 1)) * lda; // clamp: tail CTA
            T acc[ROWS];
#pragma unroll
            for(int r = 0; r < ROWS; ++r)
                acc[r] = T(0);

            uint32_t done = 0;
            if(vec_ok)
            {
                const uint32_t nvec = n / VN;
                const V*       xv   = reinterpret_cast<const V*>(x);
#pragma unroll UNROLL
                for(uint32_t v = threadIdx.x; v < nvec; v += THREADS)
                {
                    const V xx = __ldg(xv + v);
#pragma unroll
                    for(int r = 0; r < ROWS; ++r)
                    {
                        const V av = __ldcs(reinterpret_cast<const V*>(rows[r]) + v);
                        acc[r]     = Vec<T>::dot(av, xx, acc[r]);
                    }
                }
                done = nvec * VN;
            }
            for(uint32_t j = done + threadIdx.x; j < n; j += THREADS)
            {
                const T xx = __ldg(x + j);
#pragma unroll
                for(int r = 0; r < ROWS; ++r)
                    acc[r] += rows[r][j] * xx;
            }

            __shared__ T partial[ROWS][THREADS / 32];
            const int    warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
            for(int r = 0; r < ROWS; ++r)
            {
                const T s = warp_sum(acc[r]);
                if(lane == 0)
                    partial[r][warp] = s;
            }
            __syncthreads();
            if(threadIdx.x < ROWS)
            {
                const uint32_t row = row0 + threadIdx.x;
                if(row < m)
                {
                    T s = T(0);
#pragma unroll
                    for(int w = 0; w < THREADS / 32; ++w)
                        s += partial[threadIdx.x][w];
                    y[row] = alpha * s + beta * y[row];
                }
            }
        }

        // Column-major A (the reference sample's own storage, lda >= m): consecutive rows are contiguous, so each lane
        // owns VN consecutive rows (one 4- to 16-byte load per column) and the 8 warps of a CTA take interleaved columns;
        // the per-warp partial sums are combined in shared memory.  A CTA owns 32 * VN rows over ALL columns (no
        // reduction across CTAs), so VN also sets how many CTAs there are and how long each runs: the launch picks the
        // widest vector that still leaves several CTAs per SM.
        template <typename T, int VN>
        struct LaneVec;
        template <>
        struct LaneVec<float, 1> { using type = float; };
        template <>
        struct LaneVec<float, 2> { using type = float2; };
        template <>
        struct LaneVec<float, 4> { using type = float4; };
        template <>
        struct LaneVec<double, 1> { using type = double; };
        template <>
        struct LaneVec<double, 2> { using type = double2; };

        template <typename T, int VN, int UNROLL>
        __global__ void __launch_bounds__(THREADS)
            gemv_col_major_kernel(uint32_t m, uint32_t n, const T* __restrict__ a, size_t lda,
                                  const T* __restrict__ x, T* __restrict__ y, T alpha, T beta)
        {
            using V                 = typename LaneVec<T, VN>::type;
            constexpr int WARPS     = THREADS / 32;
            constexpr int CTA_ROWS  = 32 * VN;
            const int     warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            const uint32_t row = blockIdx.x * CTA_ROWS + lane * VN;
            T              acc[VN];
#pragma unroll
            for(int i = 0; i < VN; ++i)
                acc[i] = T(0);
            if(row + VN <= m)
            {
#pragma unroll UNROLL
                for(uint32_t h = warp; h < n; h += WARPS)
                {
                    const T  xx = __ldg(x + h);
                    const V  av = __ldcs(reinterpret_cast<const V*>(a + static_cast<size_t>(h) * lda + row));
                    const T* ap = reinterpret_cast<const T*>(&av);
#pragma unroll
                    for(int i = 0; i < VN; ++i)
                        acc[i] = fma(ap[i], xx, acc[i]);
                }
            }
            else
            {
                for(uint32_t h = warp; h < n; h += WARPS)
                {
                    const T xx = __ldg(x + h);
#pragma unroll
                    for(int i = 0; i < VN; ++i)
                        if(row + i < m)
                            acc[i] += a[static_cast<size_t>(h) * lda + row + i] * xx;
                }
            }
            __shared__ T partial[WARPS][CTA_ROWS];
#pragma unroll
            for(int i = 0; i < VN; ++i)
                partial[warp][lane * VN + i] = acc[i];
            __syncthreads();
            if(threadIdx.x < CTA_ROWS)
            {
                const uint32_t r = blockIdx.x * CTA_ROWS + threadIdx.x;
                if(r < m)
                {
                    T s = T(0);
#pragma unroll
                    for(int w = 0; w < WARPS; ++w)
                        s += partial[w][threadIdx.x];
                    y[r] = alpha * s + beta * y[r];
                }
            }
        }

        // Rows per lane: one, unless b200wmma_set_tuning("gemv_col_vn", 2 | 4) asks for a wider vector and its loads are
        // aligned (the wider forms measured slower, see the launch code; they are kept for that comparison).
        template <typename T>
        static int col_major_vn(uint32_t, const T* a, uint32_t lda, uint32_t)
        {
            const int forced = tuning::get(tuning::GEMV_COL_VN);
            for(int vn = Vec<T>::N; vn > 1; vn >>= 1)
                if(forced == vn && (reinterpret_cast<uintptr_t>(a) % (vn * sizeof(T))) == 0 && lda % vn == 0)
                    return vn;
            return 1;
        }

        template <typename T>
        static int launch(uint32_t m, uint32_t n, const T* a, uint32_t lda, int layout_a, const T* x,
                          T* y, T alpha, T beta, cudaStream_t stream)
        {
            B200_REQUIRE(m && n, B200WMMA_ERR_INVALID_ARG, "gemv: m and n must be non-zero");
            B200_REQUIRE(a && x && y, B200WMMA_ERR_INVALID_ARG, "gemv: a, x, y must be non-null");
            B200_REQUIRE(layout_a == B200WMMA_ROW_MAJOR || layout_a == B200WMMA_COL_MAJOR,
                         B200WMMA_ERR_INVALID_ARG, "gemv: layout_a must be 0 (row) or 1 (col)");
            B200_REQUIRE(lda >= (layout_a == B200WMMA_ROW_MAJOR ? n : m), B200WMMA_ERR_INVALID_ARG,
                         "gemv: lda smaller than the contiguous extent of A");
            if(int e = require_sm100())
                return e;
            const bool pitch_ok = (static_cast<uint64_t>(lda) * sizeof(T)) % 16 == 0 && aligned16(a);
            if(layout_a == B200WMMA_ROW_MAJOR)
            {
                const int vec_ok = pitch_ok && aligned16(x);
                // One row per CTA, eight 16-byte loads per thread in flight: the CTAs are short (128 KiB of A), so the
                // tail of the launch, when the last CTAs cannot fill the memory system, is short too.  Measured at
                // 32768 x 32768 on one B200: 1 row 7101-7131 GB/s (fp32) / 7212-7260 (fp64); 2 rows 6815-6910 / 7020-7220;
                // 4 rows with two loads in flight (the earlier choice, still selectable) 6590-6704 / 6804-6970;
                // 8 rows 6800 / 5200.
                if(tuning::get(tuning::GEMV_ROWS) == 4)
                    gemv_row_major_kernel<T, 4, 2><<<ceil_div(m, 4u), THREADS, 0, stream>>>(m, n, a, lda, x, y, alpha, beta, vec_ok);
                else
                    gemv_row_major_kernel<T, 1, 8><<<m, THREADS, 0, stream>>>(m, n, a, lda, x, y, alpha, beta, vec_ok);
            }
            else
            {
                int dev = 0, sms = 148;
                cudaGetDevice(&dev);
                cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
                // Measured at 32768 x 32768 on one B200 (GB/s, fp32 / fp64): one row per lane with 16 loads in flight
                // 6467 / 7122; with 8 in flight 6083 / 6888, with 32 (fp32) 6067; two rows per lane 5935 / 4056; four rows
                // per lane - 256 CTAs of 16 MiB on 148 SMs, the earlier shape - 3566 (fp32; fp64, two rows: 4307).
                const int vn = col_major_vn<T>(m, a, lda, 4u * static_cast<uint32_t>(sms));
                if constexpr(sizeof(T) == 4)
                {
                    if(vn == 4)
                        gemv_col_major_kernel<T, 4, 4><<<ceil_div(m, 128u), THREADS, 0, stream>>>(m, n, a, lda, x, y, alpha, beta);
                    else if(vn == 2)
                        gemv_col_major_kernel<T, 2, 8><<<ceil_div(m, 64u), THREADS, 0, stream>>>(m, n, a, lda, x, y, alpha, beta);
                    else
                        gemv_col_major_kernel<T, 1, 16><<<ceil_div(m, 32u), THREADS, 0, stream>>>(m, n, a, lda, x, y, alpha, beta);
                }
                else
                {
                    if(vn == 2)
                        gemv_col_major_kernel<T, 2, 4><<<ceil_div(m, 64u), THREADS, 0, stream>>>(m, n, a, lda, x, y, alpha, beta);
                    else
                        gemv_col_major_kernel<T, 1, 16><<<ceil_div(m, 32u), THREADS, 0, stream>>>(m, n, a, lda, x, y, alpha, beta);
                }
            }
            B200_CHECK_CUDA(cudaGetLastError());
            return B200WMMA_OK;
        }
    } // namespace gemv
} // namespace b200wmma

extern "C" int b200wmma_gemv_f32(uint32_t m, uint32_t n, const float* a, uint32_t lda, int layout_a,
                                 const float* x, float* y, float alpha, float beta, void* stream)
{
    b200wmma::clear_error();
    return b200wmma::gemv::launch<float>(m, n, a, lda, layout_a, x, y, alpha, beta,
                                         b200wmma::as_stream(stream));
}

extern "C" int b200wmma_gemv_f64(uint32_t m, uint32_t n, const double* a, uint32_t lda, int layout_a,
                                 const double* x, double* y, double alpha, double beta, void* stream)
{
    b200wmma::clear_error();
    return b200wmma::gemv::launch<double>(m, n, a, lda, layout_a, x, y, alpha, beta,
                                          b200wmma::as_stream(stream));
}
