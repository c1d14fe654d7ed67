// MappingUtil: maps the thread-block configuration onto warp / block / matrix / data coordinates.
// Same interface and conventions as rocWMMA's internal/mapping_util.hpp:144-206
// ((x, y) = (row, col); warp x = threadIdx.x / warp size, warp y = threadIdx.y), with the warp size 32.
// Data offsets are returned as uint32_t like the reference; kernels addressing more than 2^32
// elements must do their own 64-bit arithmetic.
#ifndef ROCWMMA_B200_MAPPING_UTIL_HPP
#define ROCWMMA_B200_MAPPING_UTIL_HPP

#include "layout.hpp"

namespace rocwmma
{
    namespace detail
    {
        // Warp ("wave") coordinates of the thread block.  TBlockX / TBlockY are the thread-block dimensions when
        // they are known at compile time (workgroupDim() is then a constant expression), else 0 for a run-time
        // query of blockDim (reference: internal/mapping_util.hpp:42-68, mapping_util_impl.hpp:70-121).
        // The functions are callable in host code too, where the thread coordinates read as zero: user code
        // declares `constexpr` helpers on top of them without a device qualifier.
        template <uint32_t TBlockX = 0u, uint32_t TBlockY = 0u>
        struct WaveSpace
        {
            using WaveCoordT      = Coord2d;
            using WorkgroupCoordT = Coord2d;
            using WorkgroupDimT   = Coord2d;

            ROCWMMA_HOST_DEVICE static inline uint32_t localLaneId()
            {
#if defined(__CUDA_ARCH__)
                return threadIdx.x & (Constants::AMDGCN_WAVE_SIZE - 1u);
#else
                return 0u;
#endif
            }
            ROCWMMA_HOST_DEVICE static inline WaveCoordT localWaveCoord()
            {
#if defined(__CUDA_ARCH__)
                return make_coord2d(threadIdx.x / Constants::AMDGCN_WAVE_SIZE, threadIdx.y);
#else
                return make_coord2d(0u, 0u);
#endif
            }
            ROCWMMA_HOST_DEVICE static inline WaveCoordT globalWaveCoord()
            {
#if defined(__CUDA_ARCH__)
                const uint32_t bx = TBlockX > 0u && TBlockY > 0u ? TBlockX : blockDim.x;
                const uint32_t by = TBlockX > 0u && TBlockY > 0u ? TBlockY : blockDim.y;
                return make_coord2d((blockIdx.x * bx + threadIdx.x) / Constants::AMDGCN_WAVE_SIZE,
                                    blockIdx.y * by + threadIdx.y);
#else
                return make_coord2d(0u, 0u);
#endif
            }
            ROCWMMA_HOST_DEVICE static inline WorkgroupCoordT workgroupCoord()
            {
#if defined(__CUDA_ARCH__)
                return make_coord2d(blockIdx.x, blockIdx.y);
#else
                return make_coord2d(0u, 0u);
#endif
            }
            template <bool IsConst = (TBlockX > 0u && TBlockY > 0u), std::enable_if_t<IsConst>* = nullptr>
            ROCWMMA_HOST_DEVICE constexpr static inline WorkgroupDimT workgroupDim()
            {
                return make_coord2d(TBlockX / Constants::AMDGCN_WAVE_SIZE, TBlockY);
            }
            template <bool IsConst = (TBlockX > 0u && TBlockY > 0u), std::enable_if_t<!IsConst>* = nullptr>
            ROCWMMA_HOST_DEVICE static inline WorkgroupDimT workgroupDim()
            {
#if defined(__CUDA_ARCH__)
                return make_coord2d(blockDim.x / Constants::AMDGCN_WAVE_SIZE, blockDim.y);
#else
                return make_coord2d(0u, 0u);
#endif
            }
        };
    } // namespace detail

    template <uint32_t BlockHeight, uint32_t BlockWidth, typename DataT, typename DataLayout>
    struct MappingUtil
    {
        using DataSpace     = detail::DataSpace<DataLayout>;
        using WaveCoordT    = Coord2d;
        using BlockCoordT   = Coord2d;
        using MatrixCoordT  = Coord2d;
        using WorkgroupDimT = Coord2d;

        ROCWMMA_DEVICE static inline uint32_t laneId()
        {
            return threadIdx.x & (Constants::AMDGCN_WAVE_SIZE - 1u);
        }
        // warp position inside the thread block
        ROCWMMA_DEVICE static inline WaveCoordT waveCoord()
        {
            return make_coord2d(threadIdx.x / Constants::AMDGCN_WAVE_SIZE, threadIdx.y);
        }
        // warp position in the grid = coordinate of the block this warp owns
        ROCWMMA_DEVICE static inline BlockCoordT blockCoord()
        {
            return make_coord2d((blockIdx.x * blockDim.x + threadIdx.x) / Constants::AMDGCN_WAVE_SIZE,
                                blockIdx.y * blockDim.y + threadIdx.y);
        }
        ROCWMMA_DEVICE static inline MatrixCoordT matrixCoord(BlockCoordT const& blockCoord)
        {
            return make_coord2d(get<0>(blockCoord) * BlockHeight, get<1>(blockCoord) * BlockWidth);
        }
        ROCWMMA_DEVICE static inline MatrixCoordT matrixCoord()
        {
            return matrixCoord(blockCoord());
        }
        ROCWMMA_DEVICE static inline WorkgroupDimT workgroupDim()
        {
            return make_coord2d(blockDim.x / Constants::AMDGCN_WAVE_SIZE, blockDim.y);
        }
        ROCWMMA_DEVICE static inline BlockCoordT blockCoordM(uint32_t m)
        {
            auto c    = blockCoord();
            get<0>(c) = m;
            return c;
        }
        ROCWMMA_DEVICE static inline BlockCoordT blockCoordN(uint32_t n)
        {
            auto c    = blockCoord();
            get<1>(c) = n;
            return c;
        }
        ROCWMMA_DEVICE static inline MatrixCoordT matrixCoordM(uint32_t m)
        {
            auto c    = matrixCoord();
            get<0>(c) = m;
            return c;
        }
        ROCWMMA_DEVICE static inline MatrixCoordT matrixCoordN(uint32_t n)
        {
            auto c    = matrixCoord();
            get<1>(c) = n;
            return c;
        }
        ROCWMMA_DEVICE static inline uint32_t dataOffset(MatrixCoordT const& matrixCoord, uint32_t ldm)
        {
            return DataSpace::fromMatrixCoord(matrixCoord, ldm);
        }
        ROCWMMA_DEVICE static inline DataT const* dataCoord(DataT const* baseAddr, MatrixCoordT const& c,
                                                            uint32_t ldm)
        {
            return baseAddr + dataOffset(c, ldm);
        }
        ROCWMMA_DEVICE static inline DataT* dataCoord(DataT* baseAddr, MatrixCoordT const& c, uint32_t ldm)
        {
            return baseAddr + dataOffset(c, ldm);
        }
        ROCWMMA_DEVICE static inline DataT const* dataCoord(DataT const* baseAddr, uint32_t ldm)
        {
            return dataCoord(baseAddr, matrixCoord(), ldm);
        }
        ROCWMMA_DEVICE static inline DataT* dataCoord(DataT* baseAddr, uint32_t ldm)
        {
            return dataCoord(baseAddr, matrixCoord(), ldm);
        }
    };
} // namespace rocwmma

#endif
