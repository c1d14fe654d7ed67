// Data types of the device API (rocWMMA internal/types.hpp:48-62, :102-114).
//
// float16_t in the reference is the compiler's _Float16, which mixes freely with float in
// expressions such as `alpha * acc.x[i] + beta * c.x[i]` (samples/simple_hgemm.cpp:131-134).
// CUDA's __half makes `float * __half` ambiguous, so float16_t here is a 2-byte wrapper around
// the same bits with implicit conversions to and from float and no arithmetic of its own:
// mixed expressions are evaluated in fp32 and rounded once on assignment.
#ifndef ROCWMMA_B200_TYPES_HPP
#define ROCWMMA_B200_TYPES_HPP

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_fp16.h>
#include <cstdint>

#include "config.hpp"

namespace rocwmma
{
    struct __align__(2) float16_t
    {
        unsigned short bits;

        float16_t() = default;
        ROCWMMA_HOST_DEVICE float16_t(float f)
        {
            bits = __half_as_ushort(__float2half_rn(f));
        }
        ROCWMMA_HOST_DEVICE float16_t(double f)
            : float16_t(static_cast<float>(f))
        {
        }
        ROCWMMA_HOST_DEVICE float16_t(int v)
            : float16_t(static_cast<float>(v))
        {
        }
        ROCWMMA_HOST_DEVICE float16_t(unsigned v)
            : float16_t(static_cast<float>(v))
        {
        }
        ROCWMMA_HOST_DEVICE float16_t(__half h)
        {
            bits = __half_as_ushort(h);
        }
        ROCWMMA_HOST_DEVICE operator float() const
        {
            return __half2float(__ushort_as_half(bits));
        }
        ROCWMMA_HOST_DEVICE __half as_half() const
        {
            return __ushort_as_half(bits);
        }
    };
    static_assert(sizeof(float16_t) == 2, "float16_t must be two bytes");

    // bfloat16_t: the same kind of wrapper around the bf16 bits (the reference's is hip_bfloat16, a class with
    // float conversions, internal/types.hpp:52)
    struct __align__(2) bfloat16_t
    {
        unsigned short bits;

        bfloat16_t() = default;
        ROCWMMA_HOST_DEVICE bfloat16_t(float f)
        {
            bits = __bfloat16_as_ushort(__float2bfloat16_rn(f));
        }
        ROCWMMA_HOST_DEVICE bfloat16_t(double f)
            : bfloat16_t(static_cast<float>(f))
        {
        }
        ROCWMMA_HOST_DEVICE bfloat16_t(int v)
            : bfloat16_t(static_cast<float>(v))
        {
        }
        ROCWMMA_HOST_DEVICE bfloat16_t(unsigned v)
            : bfloat16_t(static_cast<float>(v))
        {
        }
        ROCWMMA_HOST_DEVICE operator float() const
        {
            return __bfloat162float(__ushort_as_bfloat16(bits));
        }
    };
    static_assert(sizeof(bfloat16_t) == 2, "bfloat16_t must be two bytes");

    // 8-bit floats in the OCP formats the tensor cores take: float8_t = e4m3, bfloat8_t = e5m2 (the reference's
    // float8_t / bfloat8_t on its OCP targets, internal/types.hpp:48-50).  Conversions saturate to the largest
    // finite value, like the hardware's.
    template <__nv_fp8_interpretation_t Format>
    struct __align__(1) fp8_base
    {
        unsigned char bits;

        fp8_base() = default;
        ROCWMMA_HOST_DEVICE fp8_base(float f)
        {
            bits = static_cast<unsigned char>(__nv_cvt_float_to_fp8(f, __NV_SATFINITE, Format));
        }
        ROCWMMA_HOST_DEVICE fp8_base(double f)
            : fp8_base(static_cast<float>(f))
        {
        }
        ROCWMMA_HOST_DEVICE fp8_base(int v)
            : fp8_base(static_cast<float>(v))
        {
        }
        ROCWMMA_HOST_DEVICE operator float() const
        {
            return __half2float(__half(__nv_cvt_fp8_to_halfraw(bits, Format)));
        }
    };
    using float8_t  = fp8_base<__NV_E4M3>;
    using bfloat8_t = fp8_base<__NV_E5M2>;
    static_assert(sizeof(float8_t) == 1 && sizeof(bfloat8_t) == 1, "8-bit floats must be one byte");

    // xfloat32_t: fp32 storage multiplied at TF32 precision (one tensor-core product instead of the three that
    // float32_t inputs take); the reference's xfloat32_t (internal/types.hpp:62).
    struct xfloat32_t
    {
        float value;

        xfloat32_t() = default;
        ROCWMMA_HOST_DEVICE xfloat32_t(float f)
            : value(f)
        {
        }
        ROCWMMA_HOST_DEVICE operator float() const
        {
            return value;
        }
    };
    static_assert(sizeof(xfloat32_t) == 4, "xfloat32_t must be four bytes");

    using hfloat16_t = __half;
    using float32_t  = float;
    using float64_t  = double;
    using int8_t     = ::int8_t;
    using uint8_t    = ::uint8_t;
    using int16_t    = ::int16_t;
    using int32_t    = ::int32_t;
    using uint32_t   = ::uint32_t;
    using int64_t    = ::int64_t;
    using uint64_t   = ::uint64_t;
    using index_t    = ::int32_t;

    // Printable names of the data types (reference: internal/utils.hpp:202-330); user code adds specialisations
    // for its own tag types (test/gemm/gemm_config.hpp:435-475).
    template <typename DataT>
    constexpr const char* dataTypeToString();
#define ROCWMMA_B200_TYPE_NAME(TYPE, NAME)                 \
    template <>                                            \
    constexpr const char* dataTypeToString<TYPE>()         \
    {                                                      \
        return NAME;                                       \
    }
    ROCWMMA_B200_TYPE_NAME(float16_t, "f16")
    ROCWMMA_B200_TYPE_NAME(hfloat16_t, "h16")
    ROCWMMA_B200_TYPE_NAME(bfloat16_t, "bf16")
    ROCWMMA_B200_TYPE_NAME(float8_t, "f8")
    ROCWMMA_B200_TYPE_NAME(bfloat8_t, "bf8")
    ROCWMMA_B200_TYPE_NAME(xfloat32_t, "xf32")
    ROCWMMA_B200_TYPE_NAME(float32_t, "f32")
    ROCWMMA_B200_TYPE_NAME(float64_t, "f64")
    ROCWMMA_B200_TYPE_NAME(int8_t, "i8")
    ROCWMMA_B200_TYPE_NAME(uint8_t, "u8")
    ROCWMMA_B200_TYPE_NAME(int16_t, "i16")
    ROCWMMA_B200_TYPE_NAME(int32_t, "i32")
    ROCWMMA_B200_TYPE_NAME(uint32_t, "u32")
    ROCWMMA_B200_TYPE_NAME(int64_t, "i64")
    ROCWMMA_B200_TYPE_NAME(uint64_t, "u64")
#undef ROCWMMA_B200_TYPE_NAME

    // Minimal fixed-size vector used as fragment storage (`*frag`, `frag.x`).
    template <typename T, uint32_t N>
    struct VecT
    {
        T data[N];
        ROCWMMA_HOST_DEVICE T& operator[](uint32_t i)
        {
            return data[i];
        }
        ROCWMMA_HOST_DEVICE T const& operator[](uint32_t i) const
        {
            return data[i];
        }
        ROCWMMA_HOST_DEVICE constexpr static uint32_t size()
        {
            return N;
        }
    };
} // namespace rocwmma

#endif
