// Small utilities user kernels call directly (rocWMMA internal/utils.hpp:140-149,
// internal/constants.hpp:88-102): Coord2d with get<>/make_coord2d and element-wise arithmetic,
// ceilDiv, Log2, Constants.
#ifndef ROCWMMA_B200_UTILS_HPP
#define ROCWMMA_B200_UTILS_HPP

#include "config.hpp"
#include <type_traits>

namespace rocwmma
{
    struct Constants
    {
        // The "wave" of this implementation is the 32-thread CUDA warp.
        static constexpr uint32_t AMDGCN_WAVE_SIZE    = 32u;
        static constexpr uint32_t AMDGCN_WAVE_SIZE_32 = 32u;
        static constexpr uint32_t AMDGCN_WAVE_SIZE_64 = 64u;
        static constexpr uint32_t AMDGCN_DWORD_SIZE_BYTES = 4u;
        static constexpr uint32_t AMDGCN_LDS_MAX_SIZE_BYTES = 232448u; // 227 KiB opt-in per CTA
    };

    struct Coord2d
    {
        uint32_t v[2];
    };

    ROCWMMA_HOST_DEVICE constexpr inline Coord2d make_coord2d(uint32_t x, uint32_t y)
    {
        return Coord2d{{x, y}};
    }
    template <uint32_t I>
    ROCWMMA_HOST_DEVICE constexpr inline uint32_t& get(Coord2d& c)
    {
        static_assert(I < 2, "Coord2d has two components");
        return c.v[I];
    }
    template <uint32_t I>
    ROCWMMA_HOST_DEVICE constexpr inline uint32_t get(Coord2d const& c)
    {
        static_assert(I < 2, "Coord2d has two components");
        return c.v[I];
    }

#define ROCWMMA_B200_COORD_OP(OP)                                                              \
    ROCWMMA_HOST_DEVICE constexpr inline Coord2d operator OP(Coord2d const& a, Coord2d const& b) \
    {                                                                                          \
        return Coord2d{{a.v[0] OP b.v[0], a.v[1] OP b.v[1]}};                                  \
    }                                                                                          \
    ROCWMMA_HOST_DEVICE constexpr inline Coord2d operator OP(Coord2d const& a, uint32_t s)     \
    {                                                                                          \
        return Coord2d{{a.v[0] OP s, a.v[1] OP s}};                                            \
    }                                                                                          \
    ROCWMMA_HOST_DEVICE constexpr inline Coord2d operator OP(uint32_t s, Coord2d const& a)     \
    {                                                                                          \
        return Coord2d{{s OP a.v[0], s OP a.v[1]}};                                            \
    }
    ROCWMMA_B200_COORD_OP(+)
    ROCWMMA_B200_COORD_OP(-)
    ROCWMMA_B200_COORD_OP(*)
    ROCWMMA_B200_COORD_OP(/)
    ROCWMMA_B200_COORD_OP(%)
#undef ROCWMMA_B200_COORD_OP
    // compound forms (the reference's vector type has them: matrixCoord *= make_coord2d(BlocksX, BlocksY),
    // test/gemm/gemm_PGR0_LB0_MP0_MB_NC/device/kernel_device_func.hpp:110)
#define ROCWMMA_B200_COORD_ASSIGN_OP(OP)                                                        \
    ROCWMMA_HOST_DEVICE constexpr inline Coord2d& operator OP##=(Coord2d& a, Coord2d const& b) \
    {                                                                                          \
        a.v[0] OP## = b.v[0];                                                                  \
        a.v[1] OP## = b.v[1];                                                                  \
        return a;                                                                              \
    }                                                                                          \
    ROCWMMA_HOST_DEVICE constexpr inline Coord2d& operator OP##=(Coord2d& a, uint32_t s)       \
    {                                                                                          \
        a.v[0] OP## = s;                                                                       \
        a.v[1] OP## = s;                                                                       \
        return a;                                                                              \
    }
    ROCWMMA_B200_COORD_ASSIGN_OP(+)
    ROCWMMA_B200_COORD_ASSIGN_OP(-)
    ROCWMMA_B200_COORD_ASSIGN_OP(*)
    ROCWMMA_B200_COORD_ASSIGN_OP(/)
    ROCWMMA_B200_COORD_ASSIGN_OP(%)
#undef ROCWMMA_B200_COORD_ASSIGN_OP
    ROCWMMA_HOST_DEVICE constexpr inline bool operator==(Coord2d const& a, Coord2d const& b)
    {
        return a.v[0] == b.v[0] && a.v[1] == b.v[1];
    }
    ROCWMMA_HOST_DEVICE constexpr inline Coord2d swap(Coord2d const& a)
    {
        return Coord2d{{a.v[1], a.v[0]}};
    }

    template <typename IntT1, typename IntT2>
    ROCWMMA_HOST_DEVICE constexpr inline auto ceilDiv(IntT1 numerator, IntT2 divisor)
    {
        return (numerator + divisor - 1) / divisor;
    }

    template <uint32_t x>
    struct Log2
    {
        static constexpr uint32_t value = 1u + Log2<(x >> 1)>::value;
        static_assert((x & (x - 1u)) == 0u, "Log2 argument must be a power of two");
    };
    template <>
    struct Log2<1u>
    {
        static constexpr uint32_t value = 0u;
    };
} // namespace rocwmma

#endif
