// Compiles the UNMODIFIED rocWMMA CPU reference (test/reference_impl.hpp: gemm_CPU,
// dlrm_fwd_CPU, dlrm_bwd_CPU) into oracle/_ref/libref.so behind C entry points that have
// the same signatures as oracle/ref_port.c.  Nothing from the reference is copied: its
// header is included from where it lies at build time (REF_ROOT/test on the include path).
//
// TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline); never linked by the product.
//
// The reference header expects HIP-side declarations.  The minimum it needs is declared
// here first; the HIP-only headers it includes are shadowed by empty files in this folder.
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <type_traits>

typedef unsigned int uint;

namespace rocwmma
{
    struct row_major {};
    struct col_major {};
    using float16_t = _Float16;
    using float32_t = float;
    using float64_t = double;

    struct HipDevice
    {
        static HipDevice* instance() { static HipDevice d; return &d; }
        uint32_t          warpSize() const { return 64u; }
    };

    template <typename T>
    struct PackTraits
    {
        using PackedT = uint32_t;
        enum : uint32_t { PackRatio = 1 };
    };

    namespace CrossLaneOps
    {
        struct Properties
        {
            enum : uint32_t
            {
                OP_GROUP_SIZE_WARP = 0xFFFFu,
                OP_DIR_L = 0, OP_DIR_R = 1,
                OP_ID_BCAST = 100, OP_ID_BLOCK_BCAST, OP_ID_REVERSE, OP_ID_SWAP,
                OP_ID_WFALL_BCAST, OP_ID_ROTATE, OP_ID_SHIFT, OP_ID_SHUFFLE, OP_ID_PERM_BYTE,
                OP_ID_MOVE, OP_ID_BLEND,
            };
        };
    }
}

#define ROCWMMA_TEST_HIP_DEVICE_HPP  // include guard of the reference's test/hip_device.hpp
#include "reference.hpp"             // resolved in REF_ROOT/test; pulls in reference_impl.hpp

using namespace rocwmma;

namespace
{
    // Dispatch the four runtime layout flags (0 = row_major, 1 = col_major) onto the
    // reference's compile-time layout parameters.
    template <typename In, typename Out, typename Cmp, typename LA, typename LB, typename LC>
    void gemm_ld(int ld, uint32_t m, uint32_t n, uint32_t k, const In* a, const In* b,
                 const Out* c, Out* d, Cmp alpha, Cmp beta)
    {
        if(ld) gemm_CPU<In, Out, Cmp, LA, LB, LC, col_major>(m, n, k, a, b, c, d, alpha, beta);
        else   gemm_CPU<In, Out, Cmp, LA, LB, LC, row_major>(m, n, k, a, b, c, d, alpha, beta);
    }
    template <typename In, typename Out, typename Cmp, typename LA, typename LB>
    void gemm_lc(int lc, int ld, uint32_t m, uint32_t n, uint32_t k, const In* a, const In* b,
                 const Out* c, Out* d, Cmp alpha, Cmp beta)
    {
        if(lc) gemm_ld<In, Out, Cmp, LA, LB, col_major>(ld, m, n, k, a, b, c, d, alpha, beta);
        else   gemm_ld<In, Out, Cmp, LA, LB, row_major>(ld, m, n, k, a, b, c, d, alpha, beta);
    }
    template <typename In, typename Out, typename Cmp, typename LA>
    void gemm_lb(int lb, int lc, int ld, uint32_t m, uint32_t n, uint32_t k, const In* a,
                 const In* b, const Out* c, Out* d, Cmp alpha, Cmp beta)
    {
        if(lb) gemm_lc<In, Out, Cmp, LA, col_major>(lc, ld, m, n, k, a, b, c, d, alpha, beta);
        else   gemm_lc<In, Out, Cmp, LA, row_major>(lc, ld, m, n, k, a, b, c, d, alpha, beta);
    }
    template <typename In, typename Out, typename Cmp>
    void gemm_any(uint32_t m, uint32_t n, uint32_t k, const In* a, const In* b, const Out* c,
                  Out* d, Cmp alpha, Cmp beta, int la, int lb, int lc, int ld, uint32_t m_rows)
    {
        // The reference always evaluates all m rows with natural leading dimensions.  A row
        // sub-block (timed CPU baseline on large problems) is only expressible for row-major
        // A/C/D, where the first m_rows rows are a smaller problem with the same strides.
        if(m_rows != 0 && m_rows < m && la == 0 && lc == 0 && ld == 0)
            m = m_rows;
        if(la) gemm_lb<In, Out, Cmp, col_major>(lb, lc, ld, m, n, k, a, b, c, d, alpha, beta);
        else   gemm_lb<In, Out, Cmp, row_major>(lb, lc, ld, m, n, k, a, b, c, d, alpha, beta);
    }
}

#define GEMM_ENTRY(NAME, IN_T, OUT_T, CMP_T)                                                   \
    extern "C" void NAME(uint32_t m, uint32_t n, uint32_t k, const IN_T* a, const IN_T* b,     \
                         const OUT_T* c, OUT_T* d, CMP_T alpha, CMP_T beta, int la, int lb,    \
                         int lc, int ld, uint32_t m_rows)                                      \
    {                                                                                          \
        gemm_any<IN_T, OUT_T, CMP_T>(m, n, k, a, b, c, d, alpha, beta, la, lb, lc, ld, m_rows);\
    }

GEMM_ENTRY(oracle_gemm_f16_f32, _Float16, float, float)
GEMM_ENTRY(oracle_gemm_f16_f16, _Float16, _Float16, float)
GEMM_ENTRY(oracle_gemm_i8_i32, int8_t, int32_t, int32_t)
GEMM_ENTRY(oracle_gemm_i8_i8, int8_t, int8_t, int32_t)
GEMM_ENTRY(oracle_gemm_f32, float, float, float)
GEMM_ENTRY(oracle_gemm_f64, double, double, double)

extern "C" void oracle_dlrm_fwd_f16(const _Float16* in, _Float16* out, uint32_t m, uint32_t k, uint32_t b)
{ dlrm_fwd_CPU<_Float16>(in, out, m, k, b); }
extern "C" void oracle_dlrm_fwd_f32(const float* in, float* out, uint32_t m, uint32_t k, uint32_t b)
{ dlrm_fwd_CPU<float>(in, out, m, k, b); }
extern "C" void oracle_dlrm_bwd_f16(const _Float16* in, const _Float16* up, _Float16* mlp, _Float16* grad,
                                    uint32_t m, uint32_t k, uint32_t b)
{ dlrm_bwd_CPU<_Float16>(in, up, mlp, grad, m, k, b); }
extern "C" void oracle_dlrm_bwd_f32(const float* in, const float* up, float* mlp, float* grad,
                                    uint32_t m, uint32_t k, uint32_t b)
{ dlrm_bwd_CPU<float>(in, up, mlp, grad, m, k, b); }

// The reference has no CPU gemv in test/reference_impl.hpp; the equivalent call is gemm_CPU
// with n = 1: A (m x k) in its layout, x as a k x 1 column, y as an m x 1 column.
extern "C" void oracle_gemv_f32(uint32_t m, uint32_t n, const float* a, uint32_t lda, int a_col_major,
                                const float* x, float* y, float alpha, float beta)
{
    (void)lda;
    if(a_col_major) gemm_CPU<float, float, float, col_major, col_major, col_major, col_major>(m, 1, n, a, x, y, y, alpha, beta);
    else            gemm_CPU<float, float, float, row_major, col_major, col_major, col_major>(m, 1, n, a, x, y, y, alpha, beta);
}
extern "C" void oracle_gemv_f64(uint32_t m, uint32_t n, const double* a, uint32_t lda, int a_col_major,
                                const double* x, double* y, double alpha, double beta)
{
    (void)lda;
    if(a_col_major) gemm_CPU<double, double, double, col_major, col_major, col_major, col_major>(m, 1, n, a, x, y, y, alpha, beta);
    else            gemm_CPU<double, double, double, row_major, col_major, col_major, col_major>(m, 1, n, a, x, y, y, alpha, beta);
}

#ifdef _OPENMP
#include <omp.h>
extern "C" int oracle_num_threads(void) { return omp_get_max_threads(); }
// launchers such as torchrun export OMP_NUM_THREADS=1; the timed baseline asks for all host threads
extern "C" void oracle_set_num_threads(int n) { if(n > 0) omp_set_num_threads(n); }
#else
extern "C" int oracle_num_threads(void) { return 1; }
extern "C" void oracle_set_num_threads(int) {}
#endif
