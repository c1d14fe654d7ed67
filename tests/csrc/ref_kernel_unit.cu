// Compiles rocWMMA's OWN test GEMM kernels - gemm_PGR0_LB0_MP0_SB_NC and gemm_PGR0_LB0_MP0_MB_NC
// (test/gemm/gemm_PGR0_LB0_MP0_{SB,MB}_NC/device/kernel_device_func.hpp), unmodified - against this
// repository's <rocwmma/rocwmma.hpp>: the header drop-in claim, checked on the reference's source.
// The reference tree is only named on the include path at build time (-I <reference>/test/gemm); nothing of it
// lives in this repository, and the library is built only where that tree exists.
//
// The kernels include two harness headers written in terms of AMD architecture traits (build predicates, the
// LDS / cooperative configuration catalogue).  Their include guards are pre-defined here and the two guard
// templates the kernels consult are given as always-true stand-ins; everything else is the reference's code.
#include <rocwmma/rocwmma.hpp>
#include <rocwmma/rocwmma_coop.hpp>
#include <rocwmma/rocwmma_transforms.hpp>

#include <cstdint>

#define ROCWMMA_GEMM_TEST_DEVICE_PREDICATES
#define GEMM_CONFIG_HPP
namespace rocwmma
{
    template <uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename InputT, typename OutputT, typename ComputeT,
              uint32_t TBlockX, uint32_t TBlockY, uint32_t WaveSize, uint32_t ArchId>
    struct gemm_PGR0_LB0_MP0_SB_NC_guard
    {
        ROCWMMA_HOST_DEVICE static constexpr bool enableBuild()
        {
            return true;
        }
    };
    template <uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename InputT, typename OutputT, typename ComputeT,
              uint32_t BlocksX, uint32_t BlocksY, uint32_t TBlockX, uint32_t TBlockY, uint32_t WaveSize, uint32_t ArchId>
    struct gemm_PGR0_LB0_MP0_MB_NC_guard
    {
        ROCWMMA_HOST_DEVICE static constexpr bool enableBuild()
        {
            return true;
        }
    };
} // namespace rocwmma

#include "gemm_PGR0_LB0_MP0_SB_NC/device/kernel_device_func.hpp"
#undef ROCWMMA_GEMM_TEST_DEVICE_FUNC
#include "gemm_PGR0_LB0_MP0_MB_NC/device/kernel_device_func.hpp"

using namespace rocwmma;

namespace
{
    constexpr uint32_t TX = 128, TY = 2, WS = Constants::AMDGCN_WAVE_SIZE;

    // one wave per BlockM x BlockN block (SB) or per BlocksX x BlocksY blocks (MB): the reference's grid rule,
    // test/gemm/gemm_kernel_base_impl.hpp gridDim()
    template <uint32_t BM, uint32_t BN, uint32_t BK, uint32_t BX, uint32_t BY, typename InT, typename OutT, typename CmpT,
              typename LA, typename LB, typename LC>
    int run(int multi, uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b, const void* c, void* d,
            uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, double alpha, double beta)
    {
        const dim3 block(TX, TY);
        const uint32_t wx = TX / WS;
        if(multi)
        {
            const dim3 grid((m + BM * BX * wx - 1) / (BM * BX * wx), (n + BN * BY * TY - 1) / (BN * BY * TY));
            gemm_PGR0_LB0_MP0_MB_NC<BM, BN, BK, InT, OutT, CmpT, LA, LB, LC, LC, BX, BY, TX, TY, WS, 0>
                <<<grid, block>>>(m, n, k, static_cast<const InT*>(a), static_cast<const InT*>(b), static_cast<const OutT*>(c),
                                  static_cast<OutT*>(d), lda, ldb, ldc, ldd, static_cast<CmpT>(alpha), static_cast<CmpT>(beta));
        }
        else
        {
            const dim3 grid((m + BM * wx - 1) / (BM * wx), (n + BN * TY - 1) / (BN * TY));
            gemm_PGR0_LB0_MP0_SB_NC<BM, BN, BK, InT, OutT, CmpT, LA, LB, LC, LC, TX, TY, WS, 0>
                <<<grid, block>>>(m, n, k, static_cast<const InT*>(a), static_cast<const InT*>(b), static_cast<const OutT*>(c),
                                  static_cast<OutT*>(d), lda, ldb, ldc, ldd, static_cast<CmpT>(alpha), static_cast<CmpT>(beta));
        }
        return static_cast<int>(cudaGetLastError());
    }
} // namespace

// variant: 0 f16->f32 (A row, B col, C/D row)   1 f16->f16 compute f32 (A col, B row, C/D row)
//          2 f32 (A row, B col)                  3 f64 (A row, B col)        4 i8 -> i32 (A row, B col)
//          5 f16->f32, 32x32x16 blocks (A row, B col)
extern "C" int ref_test_gemm(int variant, int multi, uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b,
                             const void* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, double alpha,
                             double beta)
{
    switch(variant)
    {
    case 0:
        return run<16, 16, 16, 2, 2, float16_t, float32_t, float32_t, row_major, col_major, row_major>(
            multi, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta);
    case 1:
        return run<16, 16, 16, 2, 2, float16_t, float16_t, float32_t, col_major, row_major, row_major>(
            multi, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta);
    case 2:
        return run<16, 16, 16, 2, 2, float32_t, float32_t, float32_t, row_major, col_major, row_major>(
            multi, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta);
    case 3:
        return run<16, 16, 16, 2, 2, float64_t, float64_t, float64_t, row_major, col_major, row_major>(
            multi, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta);
    case 4:
        return run<16, 16, 16, 2, 2, int8_t, int32_t, int32_t, row_major, col_major, row_major>(
            multi, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta);
    case 5:
        return run<32, 32, 16, 1, 2, float16_t, float32_t, float32_t, row_major, col_major, row_major>(
            multi, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta);
    default:
        return -1;
    }
}
