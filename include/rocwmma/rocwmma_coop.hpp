// Cooperative (multi-warp) fragment loads and stores.
//
// Same overload set as rocWMMA's rocwmma_coop.hpp:78-412.  `waveCount` warps share the movement
// of ONE block: warp `waveIndex` moves slice `waveIndex` of it and leaves the rest of its fragment
// untouched, so a load / store pair issued with the same (waveIndex, waveCount) on every
// participating warp moves the whole block collectively (global -> registers -> shared memory in
// perf_hgemm, samples/perf_hgemm.cpp:329-362).
//
// The unit of splitting here is one 32-bit register per lane (4 / 2 / 1 elements of 8- / 16- / 32-and-64-bit
// types): the fragment's elements are dealt out in contiguous, equally sized ranges of such units, identically for
// a fragment and for any re-interpretation of its registers (applyTranspose, applyDataLayout, the register-file
// view), so a cooperative load of one view followed by a cooperative store of another moves exactly the
// registers each warp holds.  When there are more warps than units the surplus warps do nothing, like the
// reference's waves beyond `maxWaves`
// (internal/coop_load.hpp:101-135).  The deprecated splitCount forms are accepted and ignore the
// split count, as the reference does (rocwmma_coop_impl.hpp:51-53).
#ifndef ROCWMMA_B200_COOP_API_HPP
#define ROCWMMA_B200_COOP_API_HPP

#include "rocwmma.hpp"

namespace rocwmma
{
    namespace detail
    {
        // Element range [begin, end) of the fragment that warp `waveIndex` of `waveCount` moves.
        template <typename Geometry, typename DataT>
        ROCWMMA_DEVICE inline void coop_range(uint32_t waveIndex, uint32_t waveCount, uint32_t& begin,
                                              uint32_t& end)
        {
            constexpr uint32_t U     = CoopUnit<DataT>::value;
            constexpr uint32_t units = Geometry::Size / U;
            static_assert(Geometry::Size % U == 0, "fragments hold whole 32-bit registers");
            const uint32_t per = (units + waveCount - 1u) / waveCount;
            const uint32_t b   = min(waveIndex * per, units);
            begin              = b * U;
            end                = min(b + per, units) * U;
        }
        // Default wave index / count: all warps of the thread block, row-major warp order
        // (reference: rocwmma_coop_impl.hpp:101-107).
        ROCWMMA_DEVICE inline void coop_defaults(uint32_t& waveIndex, uint32_t& waveCount)
        {
            const uint32_t wavesY = blockDim.y;
            waveIndex             = (threadIdx.x / Constants::AMDGCN_WAVE_SIZE) * wavesY + threadIdx.y;
            waveCount             = (blockDim.x / Constants::AMDGCN_WAVE_SIZE) * wavesY;
        }
    }

    // ---- loads ------------------------------------------------------------------------------
    template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void
        load_matrix_coop_sync(fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>& frag,
                              const DataT* data, uint32_t ldm, uint32_t waveIndex, uint32_t waveCount)
    {
        static_assert(!std::is_same<DataLayoutT, void>::value, "Cooperative loads need a static data layout");
        using G = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>::Geometry;
        uint32_t begin, end;
        detail::coop_range<G, DataT>(waveIndex, waveCount, begin, end);
        detail::move_atoms<true, std::is_same<DataLayoutT, col_major>::value, G, DataT>(
            frag.x, const_cast<DataT*>(data), ldm, begin, end);
    }

    template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT,
              typename DataLayoutT>
    [[deprecated("splitCount argument is deprecated and will be removed in a future release")]] ROCWMMA_DEVICE inline void
        load_matrix_coop_sync(fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>& frag,
                              const DataT* data, uint32_t ldm, uint32_t waveIndex, uint32_t waveCount,
                              uint32_t /*splitCount*/)
    {
        load_matrix_coop_sync(frag, data, ldm, waveIndex, waveCount);
    }

    template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void
        load_matrix_coop_sync(fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>& frag,
                              const DataT* data, uint32_t ldm)
    {
        uint32_t waveIndex, waveCount;
        detail::coop_defaults(waveIndex, waveCount);
        load_matrix_coop_sync(frag, data, ldm, waveIndex, waveCount);
    }

    template <uint32_t WaveCount, typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK,
              typename DataT, typename DataLayoutT>
    ROCWMMA_DEVICE inline void
        load_matrix_coop_sync(fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>& frag,
                              const DataT* data, uint32_t ldm, uint32_t waveIndex)
    {
        load_matrix_coop_sync(frag, data, ldm, waveIndex, WaveCount);
    }

    template <uint32_t WaveCount, uint32_t SplitCount, typename MatrixT, uint32_t BlockM, uint32_t BlockN,
              uint32_t BlockK, typename DataT, typename DataLayoutT>
    [[deprecated("SplitCount argument is deprecated and will be removed in a future release")]] ROCWMMA_DEVICE inline void
        load_matrix_coop_sync(fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>& frag,
                              const DataT* data, uint32_t ldm, uint32_t waveIndex)
    {
        load_matrix_coop_sync(frag, data, ldm, waveIndex, WaveCount);
    }

    // ---- stores -----------------------------------------------------------------------------
    template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void
        store_matrix_coop_sync(DataT* data, fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT> const& frag,
                               uint32_t ldm, uint32_t waveIndex, uint32_t waveCount)
    {
        static_assert(!std::is_same<DataLayoutT, void>::value, "Cooperative stores need a static data layout");
        using G = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>::Geometry;
        uint32_t begin, end;
        detail::coop_range<G, DataT>(waveIndex, waveCount, begin, end);
        detail::move_atoms<false, std::is_same<DataLayoutT, col_major>::value, G, DataT>(
            const_cast<DataT*>(frag.x), data, ldm, begin, end);
    }

    template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT,
              typename DataLayoutT>
    [[deprecated("splitCount argument is deprecated and will be removed in a future release")]] ROCWMMA_DEVICE inline void
        store_matrix_coop_sync(DataT* data, fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT> const& frag,
                               uint32_t ldm, uint32_t waveIndex, uint32_t waveCount, uint32_t /*splitCount*/)
    {
        store_matrix_coop_sync(data, frag, ldm, waveIndex, waveCount);
    }

    template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void
        store_matrix_coop_sync(DataT* data, fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT> const& frag,
                               uint32_t ldm)
    {
        uint32_t waveIndex, waveCount;
        detail::coop_defaults(waveIndex, waveCount);
        store_matrix_coop_sync(data, frag, ldm, waveIndex, waveCount);
    }

    template <uint32_t WaveCount, typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK,
              typename DataT, typename DataLayoutT>
    ROCWMMA_DEVICE inline void
        store_matrix_coop_sync(DataT* data, fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT> const& frag,
                               uint32_t ldm, uint32_t waveIndex)
    {
        store_matrix_coop_sync(data, frag, ldm, waveIndex, WaveCount);
    }

    template <uint32_t WaveCount, uint32_t SplitCount, typename MatrixT, uint32_t BlockM, uint32_t BlockN,
              uint32_t BlockK, typename DataT, typename DataLayoutT>
    [[deprecated("SplitCount argument is deprecated and will be removed in a future release")]] ROCWMMA_DEVICE inline void
        store_matrix_coop_sync(DataT* data, fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT> const& frag,
                               uint32_t ldm, uint32_t waveIndex)
    {
        store_matrix_coop_sync(data, frag, ldm, waveIndex, WaveCount);
    }
} // namespace rocwmma

#endif
