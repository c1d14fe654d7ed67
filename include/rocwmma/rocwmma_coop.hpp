// Cooperative (multi-warp) fragment loads and stores.
//
// Same overload set as rocWMMA's rocwmma_coop.hpp:78-412.  `waveCount` warps share the movement
// of ONE block: warp `waveIndex` moves slice `waveIndex` of it and leaves the rest of its fragment
// untouched, so a load / store pair issued with the same (waveIndex, waveCount) on every
// participating warp moves the whole block collectively (global -> registers -> shared memory in
// perf_hgemm, samples/perf_hgemm.cpp:329-362).
//
// A warp's slice always occupies the FIRST registers of its fragment (registers 0 .. slice size - 1 hold the slice's
// elements in order), whatever the wave index: only addresses depend on the wave index, so the compiler keeps a
// cooperative fragment in as many registers as one slice needs.  (The reference leaves the placement unspecified: a
// cooperatively loaded fragment is only good for a cooperative store with the same wave index and count.)
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
        // The same split with the wave count known at compile time: the slice LENGTH is then a constant (all waves
        // but possibly the last move `per` units), so the compiler sees that only the fragment's first registers are
        // ever touched.  f(begin, count) performs the move.
        template <typename Geometry, typename DataT, uint32_t WaveCount, typename F>
        ROCWMMA_DEVICE inline void coop_static(uint32_t waveIndex, F const& f)
        {
            constexpr uint32_t U     = CoopUnit<DataT>::value;
            constexpr uint32_t units = Geometry::Size / U;
            constexpr uint32_t per   = (units + WaveCount - 1u) / WaveCount;
            constexpr uint32_t full  = units / per; // waves with a whole slice
            constexpr uint32_t tail  = units - full * per; // units of the one wave after them (0: none)
            if(waveIndex < full)
                f(waveIndex * per * U, per * U);
            else if(tail != 0u && waveIndex == full)
                f(full * per * U, tail * U);
        }

        // Whether every slice of that split begins and ends on a run boundary of the fragment's layout.
        template <typename Geometry, typename DataT, uint32_t WaveCount>
        struct CoopStaticRunAligned
        {
            static constexpr uint32_t U     = CoopUnit<DataT>::value;
            static constexpr uint32_t units = Geometry::Size / U;
            static constexpr uint32_t per   = (units + WaveCount - 1u) / WaveCount;
            static constexpr bool     value = (per * U) % Geometry::Run == 0u;
        };

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
        detail::move_atoms<true, std::is_same<DataLayoutT, col_major>::value, G, DataT, detail::CoopUnit<DataT>::value % G::Run == 0>(
            frag.x, const_cast<DataT*>(data), ldm, begin, end - begin);
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
        static_assert(!std::is_same<DataLayoutT, void>::value, "Cooperative loads need a static data layout");
        using G = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>::Geometry;
        detail::coop_static<G, DataT, WaveCount>(waveIndex, [&](uint32_t begin, uint32_t count) {
            detail::move_atoms<true, std::is_same<DataLayoutT, col_major>::value, G, DataT,
                               detail::CoopStaticRunAligned<G, DataT, WaveCount>::value>(frag.x, const_cast<DataT*>(data), ldm, begin,
                                                                                       count);
        });
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
        detail::move_atoms<false, std::is_same<DataLayoutT, col_major>::value, G, DataT, detail::CoopUnit<DataT>::value % G::Run == 0>(
            const_cast<DataT*>(frag.x), data, ldm, begin, end - begin);
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
        static_assert(!std::is_same<DataLayoutT, void>::value, "Cooperative stores need a static data layout");
        using G = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>::Geometry;
        detail::coop_static<G, DataT, WaveCount>(waveIndex, [&](uint32_t begin, uint32_t count) {
            detail::move_atoms<false, std::is_same<DataLayoutT, col_major>::value, G, DataT,
                               detail::CoopStaticRunAligned<G, DataT, WaveCount>::value>(const_cast<DataT*>(frag.x), data, ldm, begin,
                                                                                       count);
        });
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
