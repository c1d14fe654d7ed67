// Compiles rocWMMA's OWN test GEMM kernels - gemm_PGR0_LB0_MP0_SB_NC, gemm_PGR0_LB0_MP0_MB_NC and the
// cooperative, double-buffered gemm_PGR1_LB2_MP0_MB_CP (test/gemm/gemm_PGR*/device/kernel_device_func.hpp),
// unmodified - against this repository's <rocwmma/rocwmma.hpp>: the header drop-in claim, checked on the
// reference's source.  The cooperative kernel is assembled, as in the reference's tests, from the harness
// templates of test/gemm (gemm_config.hpp, gemm_driver*.hpp, gemm_global_mapping*.hpp, gemm_local_mapping*.hpp,
// gemm_coop_schedule.hpp), which are compiled unmodified as well.
// The reference tree is only named on the include path at build time (-I <reference>/test/gemm); nothing of it
// lives in this repository, and the library is built only where that tree exists.
//
// The kernels also include a header of build predicates written in terms of AMD architecture traits.  Its
// include guard is pre-defined here and the three guard templates the kernels consult are given as always-true
// stand-ins; everything else is the reference's code.
#include <rocwmma/rocwmma.hpp>
#include <rocwmma/rocwmma_coop.hpp>
#include <rocwmma/rocwmma_transforms.hpp>

#include <cstdint>

#define ROCWMMA_GEMM_TEST_DEVICE_PREDICATES
#include "gemm_config.hpp"
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
    template <uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename InputT, typename OutputT, typename ComputeT,
              typename LayoutA, typename LayoutB, typename LayoutC, typename LayoutD, typename LayoutLds, typename GemmConfig,
              uint32_t BlocksX, uint32_t BlocksY, uint32_t TBlockX, uint32_t TBlockY, uint32_t WaveSize, uint32_t ArchId>
    struct gemm_PGR1_LB2_MP0_MB_CP_guard
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
#undef ROCWMMA_GEMM_TEST_DEVICE_FUNC
#include "gemm_PGR1_LB2_MP0_MB_CP/device/kernel_device_func.hpp"

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

namespace
{
    // The reference's launch rule for the cooperative kernel (test/gemm/gemm_PGR1_LB2_MP0_MB_CP/detail/kernel_impl.hpp
    // gridDim(), ldsUsage()): one macro tile of (TX / wave size * BX * BM) x (TY * BY * BN) per thread block, two
    // shared-memory buffers of (macro tile rows + macro tile columns) x BK inputs.
    template <typename Config, typename LLds, uint32_t BM, uint32_t BN, uint32_t BK, uint32_t BX, uint32_t BY, uint32_t TBX,
              uint32_t TBY, typename InT, typename OutT, typename CmpT, typename LA, typename LB>
    int run_coop(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b, const void* c, void* d, uint32_t lda,
                 uint32_t ldb, uint32_t ldc, uint32_t ldd, double alpha, double beta)
    {
        constexpr uint32_t macro_m = TBX / WS * BX * BM, macro_n = TBY * BY * BN;
        if(m % macro_m != 0 || n % macro_n != 0 || k % BK != 0 || k < BK)
            return -2; // the kernel has no tail handling: the reference's checkSizes() skips such runs
        const dim3     grid(m / macro_m, n / macro_n), block(TBX, TBY);
        const uint32_t lds = 2u * sizeof(InT) * (macro_m + macro_n) * BK;
        auto           kern
            = gemm_PGR1_LB2_MP0_MB_CP<BM, BN, BK, InT, OutT, CmpT, LA, LB, row_major, row_major, LLds, Config, BX, BY, TBX, TBY, WS, 0>;
        if(lds > 48u * 1024u)
            if(cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(lds)))
                return static_cast<int>(e);
        kern<<<grid, block, lds>>>(m, n, k, static_cast<const InT*>(a), static_cast<const InT*>(b), static_cast<const OutT*>(c),
                                   static_cast<OutT*>(d), lda, ldb, ldc, ldd, static_cast<CmpT>(alpha), static_cast<CmpT>(beta));
        return static_cast<int>(cudaGetLastError());
    }

    template <typename Config, typename LLds>
    int run_coop_variant(int variant, uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b, const void* c, void* d,
                         uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, double alpha, double beta)
    {
        switch(variant)
        {
        case 0: // 2 x 2 waves of 2 x 2 blocks
            return run_coop<Config, LLds, 16, 16, 16, 2, 2, 64, 2, float16_t, float32_t, float32_t, row_major, col_major>(
                m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta);
        case 1: // 4 x 2 waves of 2 x 2 blocks
            return run_coop<Config, LLds, 16, 16, 16, 2, 2, 128, 2, float16_t, float16_t, float32_t, col_major, row_major>(
                m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta);
        case 2: // 2 x 2 waves of 2 x 1 blocks
            return run_coop<Config, LLds, 16, 16, 16, 2, 1, 64, 2, float32_t, float32_t, float32_t, row_major, col_major>(
                m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta);
        case 3: // 2 x 4 waves of 1 x 2 blocks
            return run_coop<Config, LLds, 16, 16, 16, 1, 2, 64, 4, float64_t, float64_t, float64_t, row_major, col_major>(
                m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta);
        case 4: // 2 x 2 waves of 2 x 2 blocks, K = 32 per step
            return run_coop<Config, LLds, 16, 16, 32, 2, 2, 64, 2, int8_t, int32_t, int32_t, row_major, col_major>(
                m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta);
        case 5: // 2 x 4 waves of 1 x 2 blocks of 32 x 32 x 16, both inputs column-major
            return run_coop<Config, LLds, 32, 32, 16, 1, 2, 64, 4, float16_t, float32_t, float32_t, col_major, col_major>(
                m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta);
        default:
            return -1;
        }
    }
} // namespace

// config : 0 block-level / 1 wave-level / 2 workgroup-level cooperation (test/gemm/gemm_config.hpp), each with the
//          inputs kept as A | B^T (+0, "LdsNT") or A^T | B (+3, "LdsTN") in shared memory; 6 block-level with the
//          fragments' raw register files in shared memory ("LdsRF")
// lds_col: shared-memory data layout row_major (0) or col_major (1)
// variant: 0 f16->f32 (A row, B col)  1 f16->f16 compute f32 (A col, B row)  2 f32 (A row, B col)  3 f64 (A row, B col)
//          4 i8->i32, BlockK 32 (A row, B col)  5 f16->f32, 32x32x16 blocks (A col, B col);  C / D row-major
extern "C" int ref_test_gemm_coop(int config, int lds_col, int variant, uint32_t m, uint32_t n, uint32_t k, const void* a,
                                  const void* b, const void* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                                  double alpha, double beta)
{
    namespace CG = rocwmma::CooperativeGemm;
#define COOP_CASE(ID, CONFIG)                                                                                          \
    case ID:                                                                                                           \
        return lds_col ? run_coop_variant<CONFIG, col_major>(variant, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta) \
                       : run_coop_variant<CONFIG, row_major>(variant, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta);
    switch(config)
    {
        COOP_CASE(0, CG::BlockLevel::LdsNT)
        COOP_CASE(1, CG::WaveLevel::LdsNT)
        COOP_CASE(2, CG::WorkgroupLevel::LdsNT)
        COOP_CASE(3, CG::BlockLevel::LdsTN)
        COOP_CASE(4, CG::WaveLevel::LdsTN)
        COOP_CASE(5, CG::WorkgroupLevel::LdsTN)
        COOP_CASE(6, CG::BlockLevel::LdsRF)
    default:
        return -1;
    }
#undef COOP_CASE
}
