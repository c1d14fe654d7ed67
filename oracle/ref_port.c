/*
 * CPU restatement of the rocWMMA reference algorithms for the GEMM / DLRM / GEMV hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the parity checker: only tests/, the smoke
 * check and the cpu_baseline / reference arm of bench.py may build, load or call it.
 * The product library never links or falls back to anything in this directory.
 *
 * Parity status: PINNED.  Every function below is checked (tests/test_oracle.py)
 *   - bit-for-bit against the reference's own CPU code (test/reference_impl.hpp compiled
 *     into oracle/_ref/libref.so by oracle/Makefile) through fixtures generated here and
 *     committed under tests/golden/ (gen_golden.py), and
 *   - against the reference's shipped DLRM known-answer arrays (test/dlrm/data/, B=64,
 *     m=27, k=128) within the f16-output tolerance (they were produced on a GPU).
 *
 * Build: gcc -std=c11 -O3 -fopenmp -march=x86-64-v3 -ffp-contract=off -shared -fPIC
 * (-ffp-contract=off keeps "acc += a*b" as a separate multiply and add, the same
 *  arithmetic as the reference compiled with the same flag.)
 *
 * Each function cites the reference file:line it follows (paths relative to the
 * rocWMMA project root).
 */
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 f16;

/* layout flags: 0 = row_major, 1 = col_major (matches rocwmma::layout_t order,
 * library/include/rocwmma/rocwmma.hpp:104-108) */
static inline size_t idx2(uint32_t row, uint32_t col, uint32_t ld, int col_major)
{
    /* test/reference_impl.hpp:58-59 (rowMjr / colMjr lambdas) */
    return col_major ? (size_t)col * ld + row : (size_t)row * ld + col;
}

/*
 * gemm_CPU, test/reference_impl.hpp:36-81.
 *   lda..ldd are the natural leading dimensions (:53-56); OpenMP over rows (:66);
 *   acc = 0; for h ascending: acc += ComputeT(a[i,h]) * ComputeT(b[h,j]) (:72-76);
 *   d[i,j] = OutputT(alpha*acc + beta*ComputeT(c[i,j])) (:77-78).
 * m_rows lets a caller evaluate only the first m_rows rows of an m-row problem (rows are
 * independent in the reference loop); the leading dimensions still use the full m.
 */
#define DEFINE_GEMM(NAME, IN_T, OUT_T, CMP_T)                                                  \
    void NAME(uint32_t m, uint32_t n, uint32_t k, const IN_T* a, const IN_T* b,                \
              const OUT_T* c, OUT_T* d, CMP_T alpha, CMP_T beta, int la, int lb, int lc,       \
              int ld_, uint32_t m_rows)                                                        \
    {                                                                                          \
        uint32_t lda = la ? m : k, ldb = lb ? k : n, ldc = lc ? m : n, ldd = ld_ ? m : n;      \
        if(m_rows == 0 || m_rows > m)                                                          \
            m_rows = m;                                                                        \
        _Pragma("omp parallel for schedule(static)") for(int64_t i = 0; i < (int64_t)m_rows;   \
                                                         ++i)                                  \
        {                                                                                      \
            for(uint32_t j = 0; j < n; ++j)                                                    \
            {                                                                                  \
                CMP_T acc = (CMP_T)0;                                                          \
                for(uint32_t h = 0; h < k; ++h)                                                \
                    acc += (CMP_T)a[idx2((uint32_t)i, h, lda, la)]                             \
                           * (CMP_T)b[idx2(h, j, ldb, lb)];                                    \
                d[idx2((uint32_t)i, j, ldd, ld_)]                                              \
                    = (OUT_T)(alpha * acc + beta * (CMP_T)c[idx2((uint32_t)i, j, ldc, lc)]);   \
            }                                                                                  \
        }                                                                                      \
    }

DEFINE_GEMM(oracle_gemm_f16_f32, f16, float, float)
DEFINE_GEMM(oracle_gemm_f16_f16, f16, f16, float)
DEFINE_GEMM(oracle_gemm_i8_i32, int8_t, int32_t, int32_t)
DEFINE_GEMM(oracle_gemm_i8_i8, int8_t, int8_t, int32_t) /* the reference's <int8_t, int8_t, int32_t> set (test/gemm/gemm_common_test_params.hpp:53) */
DEFINE_GEMM(oracle_gemm_f32, float, float, float)
DEFINE_GEMM(oracle_gemm_f64, double, double, double)

/*
 * dlrm_fwd_CPU, test/reference_impl.hpp:83-119.
 *   output row = [input[b,0,0:k]] ++ [Z[i,j] for i in 0..m-1 for j < i], Z = X X^T with a
 *   float accumulator over h ascending (:104-109), cast to DataT when stored (:113).
 *   Output stride per sample = m(m-1)/2 + k (:87).
 */
#define DEFINE_DLRM_FWD(NAME, T)                                                               \
    void NAME(const T* input, T* output, uint32_t m, uint32_t k, uint32_t batch)               \
    {                                                                                          \
        size_t in_stride = (size_t)m * k, out_stride = (size_t)m * (m - 1) / 2 + k;            \
        _Pragma("omp parallel for schedule(static)") for(int64_t b = 0; b < (int64_t)batch;    \
                                                         ++b)                                  \
        {                                                                                      \
            const T* x = input + b * in_stride;                                                \
            T*       o = output + b * out_stride;                                              \
            for(uint32_t i = 0; i < k; ++i)                                                    \
                *o++ = x[i];                                                                   \
            for(uint32_t i = 0; i < m; ++i)                                                    \
                for(uint32_t j = 0; j < i; ++j)                                                \
                {                                                                              \
                    float acc = 0.0f;                                                          \
                    for(uint32_t h = 0; h < k; ++h)                                            \
                        acc += (float)x[(size_t)i * k + h] * (float)x[(size_t)j * k + h];      \
                    *o++ = (T)acc;                                                             \
                }                                                                              \
        }                                                                                      \
    }

DEFINE_DLRM_FWD(oracle_dlrm_fwd_f16, f16)
DEFINE_DLRM_FWD(oracle_dlrm_fwd_f32, float)

/*
 * dlrm_bwd_CPU, test/reference_impl.hpp:121-179.
 *   bottomMlpGrad[b,:] = upstream[b,0:k] (:139-142);
 *   T = symmetric m x m matrix rebuilt from the packed strict lower triangle, zero diagonal,
 *       stored in DataT (:145-161);
 *   grad[b,i,j] = DataT( sum_h float(T[i,h]) * float(X[b,h,j]) ), h ascending (:164-176).
 */
#define DEFINE_DLRM_BWD(NAME, T)                                                               \
    void NAME(const T* input, const T* upstream, T* bottom_mlp_grad, T* grad, uint32_t m,      \
              uint32_t k, uint32_t batch)                                                      \
    {                                                                                          \
        size_t in_stride = (size_t)m * k, up_stride = (size_t)m * (m - 1) / 2 + k;             \
        _Pragma("omp parallel") {                                                              \
            T* tri = (T*)malloc(sizeof(T) * (size_t)m * m);                                    \
            _Pragma("omp for schedule(static)") for(int64_t b = 0; b < (int64_t)batch; ++b)    \
            {                                                                                  \
                const T* x = input + b * in_stride;                                            \
                const T* u = upstream + b * up_stride;                                         \
                for(uint32_t j = 0; j < k; ++j)                                                \
                    bottom_mlp_grad[(size_t)b * k + j] = u[j];                                 \
                const T* up = u + k;                                                           \
                for(uint32_t i = 0; i < m; ++i)                                                \
                    for(uint32_t j = 0; j <= i; ++j)                                           \
                    {                                                                          \
                        if(i == j)                                                             \
                            tri[(size_t)i * m + j] = (T)0;                                     \
                        else                                                                   \
                        {                                                                      \
                            tri[(size_t)i * m + j] = *up;                                      \
                            tri[(size_t)j * m + i] = *up;                                      \
                            ++up;                                                              \
                        }                                                                      \
                    }                                                                          \
                for(uint32_t i = 0; i < m; ++i)                                                \
                    for(uint32_t j = 0; j < k; ++j)                                            \
                    {                                                                          \
                        float acc = 0.0f;                                                      \
                        for(uint32_t h = 0; h < m; ++h)                                        \
                            acc += (float)tri[(size_t)i * m + h] * (float)x[(size_t)h * k + j];\
                        grad[b * in_stride + (size_t)i * k + j] = (T)acc;                      \
                    }                                                                          \
            }                                                                                  \
            free(tri);                                                                         \
        }                                                                                      \
    }

DEFINE_DLRM_BWD(oracle_dlrm_bwd_f16, f16)
DEFINE_DLRM_BWD(oracle_dlrm_bwd_f32, float)

/*
 * sgemv_cpu_h / dgemv_cpu_h, samples/simple_sgemv.cpp:46-66 and samples/simple_dgemv.cpp:46-66:
 *   serial over rows, acc += a[i,h]*x[h] for h ascending, y[i] = alpha*acc + beta*y[i] in
 *   place.  The sample stores A column-major (lda = m, :55,:62); `a_col_major` selects that
 *   or the row-major storage the benchmark configuration uses (the arithmetic per row is
 *   the same).  OpenMP over rows only changes which thread computes a row, not the order of
 *   operations inside it.
 */
#define DEFINE_GEMV(NAME, T)                                                                   \
    void NAME(uint32_t m, uint32_t n, const T* a, uint32_t lda, int a_col_major, const T* x,   \
              T* y, T alpha, T beta)                                                           \
    {                                                                                          \
        _Pragma("omp parallel for schedule(static)") for(int64_t i = 0; i < (int64_t)m; ++i)   \
        {                                                                                      \
            T acc = (T)0;                                                                      \
            for(uint32_t h = 0; h < n; ++h)                                                    \
                acc += a[a_col_major ? (size_t)h * lda + i : (size_t)i * lda + h] * x[h];      \
            y[i] = alpha * acc + beta * y[i];                                                  \
        }                                                                                      \
    }

DEFINE_GEMV(oracle_gemv_f32, float)
DEFINE_GEMV(oracle_gemv_f64, double)

/*
 * Denominator of the acceptance metric for floating-point GEMM results:
 *   bound[i,j] = |alpha| * sum_h |a[i,h]| |b[h,j]| + |beta| |c[i,j]|   (accumulated in double)
 * so a test can check |d - ref| / bound <= tol.  Inputs are given as double arrays in
 * row-major logical order to keep this independent of storage type and layout.
 */
void oracle_gemm_abs_bound(uint32_t m, uint32_t n, uint32_t k, const double* a_rm,
                           const double* b_rm, const double* c_rm, double alpha, double beta,
                           double* bound_rm)
{
#pragma omp parallel for schedule(static)
    for(int64_t i = 0; i < (int64_t)m; ++i)
        for(uint32_t j = 0; j < n; ++j)
        {
            double acc = 0.0;
            for(uint32_t h = 0; h < k; ++h)
            {
                double av = a_rm[(size_t)i * k + h], bv = b_rm[(size_t)h * n + j];
                acc += (av < 0 ? -av : av) * (bv < 0 ? -bv : bv);
            }
            double cv = c_rm ? c_rm[(size_t)i * n + j] : 0.0;
            bound_rm[(size_t)i * n + j]
                = (alpha < 0 ? -alpha : alpha) * acc + (beta < 0 ? -beta : beta) * (cv < 0 ? -cv : cv);
        }
}

/* Thread count for the OpenMP loops above (launchers such as torchrun export OMP_NUM_THREADS=1). */
void oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if(n > 0)
        omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int oracle_num_threads(void)
{
    int n = 1;
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    n = omp_get_max_threads();
#endif
    return n;
}
