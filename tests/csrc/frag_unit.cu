// Test kernels for the rocWMMA-compatible fragment API (include/rocwmma/*.hpp), built into
// tests/libfrag_unit.so.  They follow the shape of the reference's unit suites:
//   - load -> store round trip must reproduce the input (test/unit/load_store_matrix_sync_test),
//   - cooperative load -> store round trip with 1/2/4/8 waves (test/unit/load_store_matrix_coop_sync_test),
//   - fill_fragment (test/unit/fill_fragment_test),
//   - stores touch nothing outside the block (test/unit/contamination_test),
//   - naive one-block-per-wave GEMM for every supported type pair / layout (test/gemm/gemm_PGR0_LB0_MP0_SB_NC).
// Each kernel is selected by a small integer case id so the Python side can sweep them.
#include <cuda_runtime.h>
#include <cstdint>

#include <rocwmma/rocwmma.hpp>
#include <rocwmma/rocwmma_coop.hpp>
#include <rocwmma/rocwmma_transforms.hpp>

using namespace rocwmma;

namespace
{
    // Every wave copies block (waveRow, waveCol) of a matrix made of BH x BW blocks.
    template <typename Frag>
    __global__ void roundtrip_kernel(const typename Frag::element_type* src, typename Frag::element_type* dst,
                                     uint32_t rows, uint32_t cols, uint32_t ld_src, uint32_t ld_dst)
    {
        using T      = typename Frag::element_type;
        using Shape  = GetIOShape_t<Frag>;
        using Map    = MappingUtil<Shape::BlockHeight, Shape::BlockWidth, T,
                                typename detail::FragInfo<Frag>::Layout>;
        const auto mc = Map::matrixCoord();
        if(get<0>(mc) >= rows || get<1>(mc) >= cols)
            return;
        Frag f;
        load_matrix_sync(f, Map::dataCoord(src, mc, ld_src), ld_src);
        store_matrix_sync(Map::dataCoord(dst, mc, ld_dst), f, ld_dst);
    }

    // All waves of a thread block cooperatively copy ONE block; blockIdx.x selects the block column.
    template <typename Frag>
    __global__ void coop_roundtrip_kernel(const typename Frag::element_type* src, typename Frag::element_type* dst,
                                          uint32_t ld_src, uint32_t ld_dst, int use_default_args)
    {
        using T     = typename Frag::element_type;
        using Shape = GetIOShape_t<Frag>;
        using DS    = GetDataLayout_t<Frag>;
        const uint32_t off_src = DS::fromMatrixCoord(make_coord2d(0u, blockIdx.x * Shape::BlockWidth), ld_src);
        const uint32_t off_dst = DS::fromMatrixCoord(make_coord2d(0u, blockIdx.x * Shape::BlockWidth), ld_dst);
        Frag f;
        fill_fragment(f, static_cast<T>(0));
        if(use_default_args)
        {
            load_matrix_coop_sync(f, src + off_src, ld_src);
            store_matrix_coop_sync(dst + off_dst, f, ld_dst);
        }
        else
        {
            const uint32_t waveCount = (blockDim.x / Constants::AMDGCN_WAVE_SIZE) * blockDim.y;
            const uint32_t waveIndex = (threadIdx.x / Constants::AMDGCN_WAVE_SIZE) * blockDim.y + threadIdx.y;
            load_matrix_coop_sync(f, src + off_src, ld_src, waveIndex, waveCount);
            store_matrix_coop_sync(dst + off_dst, f, ld_dst, waveIndex, waveCount);
        }
    }

    template <typename Frag>
    __global__ void fill_kernel(typename Frag::element_type* dst, uint32_t ld, double value)
    {
        using T = typename Frag::element_type;
        Frag f;
        fill_fragment(f, static_cast<T>(static_cast<float>(value)));
        store_matrix_sync(dst, f, ld);
    }

    // Transposed view: load a matrix_a block (row major), reinterpret it as the matrix_b block of the
    // transposed matrix (column major) and store that: memory must come out identical.
    template <typename FragA>
    __global__ void transpose_kernel(const typename FragA::element_type* src, typename FragA::element_type* dst,
                                     uint32_t ld)
    {
        FragA f;
        load_matrix_sync(f, src, ld);
        store_matrix_sync(dst, applyTranspose(f), ld);
    }

    // One BM x BN output block per wave, K walked in BK steps; D = alpha * A B + beta * C.
    template <uint32_t BM, uint32_t BN, uint32_t BK, typename InT, typename CmpT, typename OutT, typename LA,
              typename LB>
    __global__ void naive_gemm_kernel(uint32_t m, uint32_t n, uint32_t k, const InT* a, const InT* b, const OutT* c,
                                      OutT* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, CmpT alpha,
                                      CmpT beta)
    {
        using MapA = MappingUtil<BM, BK, InT, LA>;
        using MapB = MappingUtil<BK, BN, InT, LB>;
        using MapC = MappingUtil<BM, BN, OutT, row_major>;
        fragment<matrix_a, BM, BN, BK, InT, LA>    fa;
        fragment<matrix_b, BM, BN, BK, InT, LB>    fb;
        fragment<accumulator, BM, BN, BK, CmpT>    acc;
        fragment<accumulator, BM, BN, BK, OutT>    fc;
        fill_fragment(acc, static_cast<CmpT>(0));
        const auto mc = MapC::matrixCoord();
        if(get<0>(mc) >= m || get<1>(mc) >= n)
            return;
        for(uint32_t kk = 0; kk < k; kk += BK)
        {
            load_matrix_sync(fa, MapA::dataCoord(a, make_coord2d(get<0>(mc), kk), lda), lda);
            load_matrix_sync(fb, MapB::dataCoord(b, make_coord2d(kk, get<1>(mc)), ldb), ldb);
            mma_sync(acc, fa, fb, acc);
        }
        load_matrix_sync(fc, MapC::dataCoord(c, mc, ldc), ldc, mem_row_major);
        for(uint32_t i = 0; i < fc.num_elements; ++i)
            fc.x[i] = static_cast<OutT>(alpha * static_cast<CmpT>(acc.x[i]) + beta * static_cast<CmpT>(fc.x[i]));
        store_matrix_sync(MapC::dataCoord(d, mc, ldd), fc, ldd, mem_row_major);
    }

    template <typename Frag>
    int run_roundtrip(const void* src, void* dst, uint32_t rows, uint32_t cols, uint32_t ld_src, uint32_t ld_dst,
                      uint32_t waves_x, uint32_t waves_y)
    {
        using T     = typename Frag::element_type;
        using Shape = GetIOShape_t<Frag>;
        dim3 block(waves_x * 32, waves_y);
        dim3 grid((rows / Shape::BlockHeight + waves_x - 1) / waves_x, (cols / Shape::BlockWidth + waves_y - 1) / waves_y);
        roundtrip_kernel<Frag><<<grid, block>>>(static_cast<const T*>(src), static_cast<T*>(dst), rows, cols, ld_src, ld_dst);
        return static_cast<int>(cudaDeviceSynchronize());
    }
    template <typename Frag>
    int run_coop(const void* src, void* dst, uint32_t ld_src, uint32_t ld_dst, uint32_t blocks, uint32_t waves_x,
                 uint32_t waves_y, int use_default)
    {
        using T = typename Frag::element_type;
        coop_roundtrip_kernel<Frag><<<blocks, dim3(waves_x * 32, waves_y)>>>(static_cast<const T*>(src),
                                                                              static_cast<T*>(dst), ld_src, ld_dst, use_default);
        return static_cast<int>(cudaDeviceSynchronize());
    }
}

#define FRAG(M, BM, BN, BK, T, L) fragment<M, BM, BN, BK, T, L>

// ---- case tables ----------------------------------------------------------------------------------
// round trip / coop cases: id -> fragment type.  Kept in sync with tests/test_gpu_fragment.py.
#define ROUNDTRIP_CASES(X)                                     \
    X(0, FRAG(matrix_a, 16, 16, 16, float16_t, row_major))      \
    X(1, FRAG(matrix_a, 16, 16, 16, float16_t, col_major))      \
    X(2, FRAG(matrix_b, 16, 16, 16, float16_t, row_major))      \
    X(3, FRAG(matrix_b, 16, 16, 16, float16_t, col_major))      \
    X(4, FRAG(accumulator, 16, 16, 16, float32_t, row_major))   \
    X(5, FRAG(accumulator, 16, 16, 16, float32_t, col_major))   \
    X(6, FRAG(matrix_a, 32, 32, 32, int8_t, row_major))         \
    X(7, FRAG(matrix_b, 32, 32, 32, int8_t, col_major))         \
    X(8, FRAG(matrix_a, 64, 16, 64, int8_t, col_major))         \
    X(9, FRAG(accumulator, 32, 32, 16, int32_t, row_major))     \
    X(10, FRAG(matrix_a, 16, 16, 4, float64_t, row_major))      \
    X(11, FRAG(matrix_b, 16, 16, 8, float64_t, row_major))      \
    X(12, FRAG(accumulator, 16, 16, 4, float64_t, col_major))   \
    X(13, FRAG(matrix_a, 32, 32, 8, float32_t, row_major))      \
    X(14, FRAG(matrix_b, 32, 32, 16, float32_t, col_major))     \
    X(15, FRAG(matrix_a, 128, 16, 16, float16_t, col_major))    \
    X(16, FRAG(matrix_b, 16, 128, 16, float16_t, row_major))    \
    X(17, FRAG(matrix_a, 256, 16, 32, float16_t, row_major))    \
    X(18, FRAG(matrix_b, 16, 64, 128, float16_t, col_major))    \
    X(19, FRAG(accumulator, 64, 32, 16, float16_t, row_major))  \
    X(20, FRAG(accumulator, 32, 32, 16, float16_t, col_major))  \
    X(21, FRAG(matrix_a, 64, 64, 256, int8_t, row_major))       \
    X(22, FRAG(matrix_a, 32, 16, 16, hfloat16_t, row_major))

extern "C" int frag_unit_block_shape(int case_id, uint32_t* bh, uint32_t* bw, uint32_t* elem_bytes, uint32_t* num_elements)
{
    switch(case_id)
    {
#define X(ID, F)                                   \
    case ID:                                       \
        *bh           = GetIOShape_t<F>::BlockHeight; \
        *bw           = GetIOShape_t<F>::BlockWidth;  \
        *elem_bytes   = sizeof(F::element_type);   \
        *num_elements = F::num_elements;           \
        return 0;
        ROUNDTRIP_CASES(X)
#undef X
    default:
        return -1;
    }
}

extern "C" int frag_unit_roundtrip(int case_id, const void* src, void* dst, uint32_t rows, uint32_t cols,
                                   uint32_t ld_src, uint32_t ld_dst, uint32_t waves_x, uint32_t waves_y)
{
    switch(case_id)
    {
#define X(ID, F) \
    case ID:     \
        return run_roundtrip<F>(src, dst, rows, cols, ld_src, ld_dst, waves_x, waves_y);
        ROUNDTRIP_CASES(X)
#undef X
    default:
        return -1;
    }
}

extern "C" int frag_unit_coop_roundtrip(int case_id, const void* src, void* dst, uint32_t ld_src, uint32_t ld_dst,
                                        uint32_t blocks, uint32_t waves_x, uint32_t waves_y, int use_default)
{
    switch(case_id)
    {
#define X(ID, F) \
    case ID:     \
        return run_coop<F>(src, dst, ld_src, ld_dst, blocks, waves_x, waves_y, use_default);
        ROUNDTRIP_CASES(X)
#undef X
    default:
        return -1;
    }
}

extern "C" int frag_unit_fill(int case_id, void* dst, uint32_t ld, double value)
{
    switch(case_id)
    {
#define X(ID, F)                                                                        \
    case ID:                                                                            \
        fill_kernel<F><<<1, 32>>>(static_cast<F::element_type*>(dst), ld, value);       \
        return static_cast<int>(cudaDeviceSynchronize());
        ROUNDTRIP_CASES(X)
#undef X
    default:
        return -1;
    }
}

// transpose: 0 = f16 16x16 (A row-major 16 x 16), 1 = i8 32 x 64, 2 = f64 16 x 8
extern "C" int frag_unit_transpose(int case_id, const void* src, void* dst, uint32_t ld)
{
    switch(case_id)
    {
    case 0:
        transpose_kernel<FRAG(matrix_a, 16, 16, 16, float16_t, row_major)><<<1, 32>>>(
            static_cast<const float16_t*>(src), static_cast<float16_t*>(dst), ld);
        break;
    case 1:
        transpose_kernel<FRAG(matrix_a, 32, 16, 64, int8_t, row_major)><<<1, 32>>>(
            static_cast<const int8_t*>(src), static_cast<int8_t*>(dst), ld);
        break;
    case 2:
        transpose_kernel<FRAG(matrix_a, 16, 16, 8, float64_t, row_major)><<<1, 32>>>(
            static_cast<const double*>(src), static_cast<double*>(dst), ld);
        break;
    default:
        return -1;
    }
    return static_cast<int>(cudaDeviceSynchronize());
}

// naive GEMM cases: (block shape, input, compute, output, layout A, layout B)
#define GEMM_CASES(X)                                                                         \
    X(0, 16, 16, 16, float16_t, float32_t, float32_t, row_major, col_major)                   \
    X(1, 32, 32, 16, float16_t, float32_t, float16_t, row_major, col_major)                   \
    X(2, 16, 16, 32, float16_t, float32_t, float32_t, col_major, row_major)                   \
    X(3, 32, 32, 16, float16_t, float32_t, float32_t, row_major, row_major)                   \
    X(4, 16, 16, 16, float16_t, float32_t, float32_t, col_major, col_major)                   \
    X(5, 16, 16, 16, float16_t, float16_t, float16_t, row_major, col_major)                   \
    X(6, 16, 16, 16, int8_t, int32_t, int32_t, row_major, col_major)                          \
    X(7, 32, 32, 32, int8_t, int32_t, int32_t, col_major, row_major)                          \
    X(8, 16, 16, 4, float64_t, float64_t, float64_t, row_major, col_major)                    \
    X(9, 16, 16, 16, float64_t, float64_t, float64_t, col_major, row_major)                   \
    X(10, 16, 16, 8, float32_t, float32_t, float32_t, row_major, col_major)                   \
    X(11, 32, 32, 16, float32_t, float32_t, float32_t, col_major, row_major)                  \
    X(12, 32, 16, 16, float16_t, float32_t, float32_t, row_major, col_major)                  \
    X(13, 16, 16, 16, hfloat16_t, float32_t, float32_t, row_major, col_major)                 \
    X(14, 32, 32, 8, float16_t, float32_t, float32_t, row_major, col_major)                   \
    X(15, 16, 16, 8, float16_t, float32_t, float16_t, col_major, row_major)                   \
    X(16, 16, 16, 4, float32_t, float32_t, float32_t, row_major, col_major)                   \
    X(17, 32, 32, 4, float32_t, float32_t, float32_t, col_major, row_major)                   \
    X(18, 16, 16, 16, bfloat16_t, float32_t, float32_t, row_major, col_major)                 \
    X(19, 32, 32, 8, bfloat16_t, float32_t, float32_t, col_major, row_major)                  \
    X(20, 16, 16, 16, bfloat16_t, bfloat16_t, float32_t, row_major, row_major)                \
    X(21, 32, 16, 24, float16_t, float32_t, float32_t, row_major, col_major)                  \
    X(22, 16, 16, 32, float8_t, float32_t, float32_t, row_major, col_major)                   \
    X(23, 32, 32, 16, bfloat8_t, float32_t, float32_t, col_major, row_major)                  \
    X(24, 16, 16, 8, xfloat32_t, float32_t, float32_t, row_major, col_major)                  \
    X(25, 32, 32, 4, xfloat32_t, float32_t, float32_t, col_major, row_major)                  \
    X(26, 32, 32, 8, int8_t, int32_t, int32_t, row_major, col_major)                          \
    X(27, 32, 32, 8, int8_t, int32_t, int32_t, col_major, row_major)                          \
    X(28, 32, 32, 2, float32_t, float32_t, float32_t, row_major, col_major)                   \
    X(29, 32, 32, 2, float32_t, float32_t, float32_t, col_major, row_major)                   \
    X(30, 32, 32, 2, xfloat32_t, float32_t, float32_t, row_major, row_major)                  \
    X(31, 16, 16, 24, int8_t, int32_t, int32_t, row_major, row_major)

extern "C" int frag_unit_gemm(int case_id, uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b,
                              const void* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                              double alpha, double beta, uint32_t waves_x, uint32_t waves_y)
{
    dim3 block(waves_x * 32, waves_y);
    switch(case_id)
    {
#define X(ID, BM, BN, BK, IN, CMP, OUT, LA, LB)                                                              \
    case ID:                                                                                                 \
    {                                                                                                        \
        dim3 grid((m / BM + waves_x - 1) / waves_x, (n / BN + waves_y - 1) / waves_y);                       \
        naive_gemm_kernel<BM, BN, BK, IN, CMP, OUT, LA, LB><<<grid, block>>>(                                \
            m, n, k, static_cast<const IN*>(a), static_cast<const IN*>(b), static_cast<const OUT*>(c),       \
            static_cast<OUT*>(d), lda, ldb, ldc, ldd, static_cast<CMP>(static_cast<float>(alpha)),           \
            static_cast<CMP>(static_cast<float>(beta)));                                                     \
        break;                                                                                               \
    }
        GEMM_CASES(X)
#undef X
    default:
        return -1;
    }
    return static_cast<int>(cudaDeviceSynchronize());
}

extern "C" int frag_unit_gemm_block(int case_id, uint32_t* bm, uint32_t* bn, uint32_t* bk)
{
    switch(case_id)
    {
#define X(ID, BM, BN, BK, IN, CMP, OUT, LA, LB) \
    case ID:                                    \
        *bm = BM;                               \
        *bn = BN;                               \
        *bk = BK;                               \
        return 0;
        GEMM_CASES(X)
#undef X
    default:
        return -1;
    }
}
