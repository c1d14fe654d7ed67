// Systematic sweep of fragment shapes for the load / store / cooperative / contamination checks, built into
// tests/libfrag_sweep.so.  It follows the parameter space of the reference's unit suites
// (test/unit/unit_test_params.hpp:86-141: BlockDim 16..256 x BlockK 8..64, and 128 / 256 of its extended set, x
// {i8, f16, f32, f64} x {row, col} major, for matrix_a, matrix_b and accumulator fragments), one template
// instantiation per point:
//   matrix_a    : fragment<matrix_a, BlockDim, 16, BlockK>       (BlockDim x BlockK in memory)
//   matrix_b    : fragment<matrix_b, 16, BlockDim, BlockK>       (BlockK x BlockDim in memory)
//   accumulator : fragment<accumulator, BlockDim, BlockK, 16>    (BlockDim x BlockK in memory)
// Points this implementation does not offer return -3: accumulator blocks narrower than 16, and blocks of more than
// 32 KB (1 KB = 256 registers per lane: a fragment lives in registers, and a thread has 255).
//
// The file is compiled once per (fragment kind, element type) with -DSWEEP_KIND=0..2 -DSWEEP_TYPE=0..3, so that the
// pieces build in parallel, and once without them for the dispatcher frag_sweep(); all objects are linked into one
// library.
#include <cuda_runtime.h>
#include <cstdint>
#include <tuple>

#include <rocwmma/rocwmma.hpp>
#include <rocwmma/rocwmma_coop.hpp>

using namespace rocwmma;

struct Args
{
    const void* src;
    void*       dst;
    uint32_t    rows, cols, ld_src, ld_dst, waves_x, waves_y, blocks;
    uint32_t*   shape; // out: block height, block width, element bytes, num_elements
};
#define SWEEP_PIECE_NAME2(K, T) frag_sweep_piece_##K##_##T
#define SWEEP_PIECE_NAME(K, T) SWEEP_PIECE_NAME2(K, T)

#if defined(SWEEP_KIND) && defined(SWEEP_TYPE)
namespace
{
    using SweepT = std::tuple_element_t<SWEEP_TYPE, std::tuple<int8_t, float16_t, float32_t, float64_t>>;
    using SweepM = std::tuple_element_t<SWEEP_KIND, std::tuple<matrix_a, matrix_b, accumulator>>;

    template <typename MatrixT, uint32_t BD, uint32_t BK, typename T, typename L>
    struct FragOf;
    template <uint32_t BD, uint32_t BK, typename T, typename L>
    struct FragOf<matrix_a, BD, BK, T, L>
    {
        static constexpr bool supported = detail::AtomK<sizeof(T), BK>::value != 0 && BD * BK * sizeof(T) <= 32768;
        template <typename = void>
        using type = fragment<matrix_a, BD, 16, BK, T, L>;
    };
    template <uint32_t BD, uint32_t BK, typename T, typename L>
    struct FragOf<matrix_b, BD, BK, T, L>
    {
        static constexpr bool supported = detail::AtomK<sizeof(T), BK>::value != 0 && BD * BK * sizeof(T) <= 32768;
        template <typename = void>
        using type = fragment<matrix_b, 16, BD, BK, T, L>;
    };
    template <uint32_t BD, uint32_t BK, typename T, typename L>
    struct FragOf<accumulator, BD, BK, T, L>
    {
        static constexpr bool supported = BK % 16 == 0 && BD * BK * sizeof(T) <= 32768;
        template <typename = void>
        using type = fragment<accumulator, BD, BK, 16, T, L>;
    };

    // every wave copies block (wave row, wave col) of a matrix of blocks
    template <typename Frag>
    __global__ void roundtrip_kernel(const typename Frag::element_type* src, typename Frag::element_type* dst, uint32_t rows,
                                     uint32_t cols, uint32_t ld_src, uint32_t ld_dst)
    {
        using Map     = GetMappingUtil_t<Frag>;
        const auto mc = Map::matrixCoord();
        if(get<0>(mc) >= rows || get<1>(mc) >= cols)
            return;
        Frag f;
        load_matrix_sync(f, Map::dataCoord(src, mc, ld_src), ld_src);
        store_matrix_sync(Map::dataCoord(dst, mc, ld_dst), f, ld_dst);
    }

    // all waves of a thread block copy ONE block together; blockIdx.x selects the block column
    template <typename Frag>
    __global__ void coop_kernel(const typename Frag::element_type* src, typename Frag::element_type* dst, uint32_t ld_src,
                                uint32_t ld_dst)
    {
        using Shape            = GetIOShape_t<Frag>;
        using DS               = GetDataLayout_t<Frag>;
        const uint32_t off_src = DS::fromMatrixCoord(make_coord2d(0u, blockIdx.x * Shape::BlockWidth), ld_src);
        const uint32_t off_dst = DS::fromMatrixCoord(make_coord2d(0u, blockIdx.x * Shape::BlockWidth), ld_dst);
        Frag           f;
        load_matrix_coop_sync(f, src + off_src, ld_src);
        store_matrix_coop_sync(dst + off_dst, f, ld_dst);
    }

    template <typename MatrixT, uint32_t BD, uint32_t BK, typename T, typename L>
    int run_case(int mode, Args const& a)
    {
        using Of = FragOf<MatrixT, BD, BK, T, L>;
        if constexpr(!Of::supported)
            return -3;
        else
        {
            using Frag  = typename Of::template type<>;
            using Shape = GetIOShape_t<Frag>;
            if(mode == 0)
            {
                a.shape[0] = Shape::BlockHeight;
                a.shape[1] = Shape::BlockWidth;
                a.shape[2] = sizeof(T);
                a.shape[3] = Frag::num_elements;
                return 0;
            }
            if(mode == 1)
            {
                dim3 block(a.waves_x * 32, a.waves_y);
                dim3 grid((a.rows / Shape::BlockHeight + a.waves_x - 1) / a.waves_x,
                          (a.cols / Shape::BlockWidth + a.waves_y - 1) / a.waves_y);
                roundtrip_kernel<Frag><<<grid, block>>>(static_cast<const T*>(a.src), static_cast<T*>(a.dst), a.rows, a.cols,
                                                        a.ld_src, a.ld_dst);
                return static_cast<int>(cudaDeviceSynchronize());
            }
            if(mode == 2)
            {
                coop_kernel<Frag><<<a.blocks, dim3(a.waves_x * 32, a.waves_y)>>>(static_cast<const T*>(a.src),
                                                                                static_cast<T*>(a.dst), a.ld_src, a.ld_dst);
                return static_cast<int>(cudaDeviceSynchronize());
            }
            return -1;
        }
    }

    template <typename MatrixT, uint32_t BD, uint32_t BK, typename T>
    int by_layout(int col, int mode, Args const& a)
    {
        return col ? run_case<MatrixT, BD, BK, T, col_major>(mode, a) : run_case<MatrixT, BD, BK, T, row_major>(mode, a);
    }
    template <typename MatrixT, uint32_t BD>
    int by_k(uint32_t bk, int col, int mode, Args const& a)
    {
        switch(bk)
        {
        case 8:
            return by_layout<MatrixT, BD, 8, SweepT>(col, mode, a);
        case 16:
            return by_layout<MatrixT, BD, 16, SweepT>(col, mode, a);
        case 32:
            return by_layout<MatrixT, BD, 32, SweepT>(col, mode, a);
        case 64:
            return by_layout<MatrixT, BD, 64, SweepT>(col, mode, a);
        case 128:
            return by_layout<MatrixT, BD, 128, SweepT>(col, mode, a);
        case 256:
            return by_layout<MatrixT, BD, 256, SweepT>(col, mode, a);
        default:
            return -1;
        }
    }
    template <typename MatrixT>
    int by_dim(uint32_t bd, uint32_t bk, int col, int mode, Args const& a)
    {
        switch(bd)
        {
        case 16:
            return by_k<MatrixT, 16>(bk, col, mode, a);
        case 32:
            return by_k<MatrixT, 32>(bk, col, mode, a);
        case 64:
            return by_k<MatrixT, 64>(bk, col, mode, a);
        case 128:
            return by_k<MatrixT, 128>(bk, col, mode, a);
        case 256:
            return by_k<MatrixT, 256>(bk, col, mode, a);
        default:
            return -1;
        }
    }
} // namespace

extern "C" int SWEEP_PIECE_NAME(SWEEP_KIND, SWEEP_TYPE)(uint32_t block_dim, uint32_t block_k, int col, int mode, Args const* a)
{
    return by_dim<SweepM>(block_dim, block_k, col, mode, *a);
}

#else // the dispatcher

#define DECLARE_PIECE(K, T) extern "C" int SWEEP_PIECE_NAME(K, T)(uint32_t, uint32_t, int, int, Args const*);
#define FOR_EACH_PIECE(X) X(0, 0) X(0, 1) X(0, 2) X(0, 3) X(1, 0) X(1, 1) X(1, 2) X(1, 3) X(2, 0) X(2, 1) X(2, 2) X(2, 3)
FOR_EACH_PIECE(DECLARE_PIECE)

// kind: 0 matrix_a, 1 matrix_b, 2 accumulator;  type: 0 i8, 1 f16, 2 f32, 3 f64;  col: data layout col_major
// mode: 0 write {block height, block width, element bytes, num_elements} to shape
//       1 load -> store round trip of a rows x cols matrix of blocks, one block per wave
//       2 cooperative load -> store of `blocks` blocks side by side, all waves of a thread block on one block
// Returns 0, a CUDA error code, -3 for a point this implementation does not offer, -1 for a bad selector.
extern "C" int frag_sweep(int kind, uint32_t block_dim, uint32_t block_k, int type, int col, int mode, const void* src,
                          void* dst, uint32_t rows, uint32_t cols, uint32_t ld_src, uint32_t ld_dst, uint32_t waves_x,
                          uint32_t waves_y, uint32_t blocks, uint32_t* shape)
{
    const Args a{src, dst, rows, cols, ld_src, ld_dst, waves_x, waves_y, blocks, shape};
#define CALL_PIECE(K, T)        \
    if(kind == K && type == T) \
        return SWEEP_PIECE_NAME(K, T)(block_dim, block_k, col, mode, &a);
    FOR_EACH_PIECE(CALL_PIECE)
    return -1;
}
#endif
