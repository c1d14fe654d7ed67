// Host driver of the tensor-core GEMM, mirroring gemm_test() of rocWMMA's samples/perf_hgemm.cpp:713-941:
// fill, copy to the device, 2 warm-up + 5 timed launches, TFlops/s, spot validation.
// Usage: perf_hgemm [m n k alpha beta [nt]]   (default 8192 8192 8192 1 1: A row-major, B col-major, C/D fp16;
//        "nt" selects the layouts the reference sample ships with: A col-major, B row-major, samples/perf_hgemm.cpp:264-271)
#include "common.hpp"

#include <string>

int main(int argc, char** argv)
{
    const uint32_t m = argc > 3 ? std::atoi(argv[1]) : 8192, n = argc > 3 ? std::atoi(argv[2]) : 8192,
                   k = argc > 3 ? std::atoi(argv[3]) : 8192;
    const float alpha = argc > 5 ? std::atof(argv[4]) : 1.0f, beta = argc > 5 ? std::atof(argv[5]) : 1.0f;
    const bool  nt    = argc > 6 && std::string(argv[6]) == "nt"; // A column-major (lda = m), B row-major (ldb = n)
    std::printf("Initializing host data...\n");
    std::vector<__half> a(size_t(m) * k), b(size_t(n) * k), c(size_t(m) * n), d(size_t(m) * n);
    // logical A[i][h], B[h][j]; storage index depends on the layout
    auto ai = [&](size_t i, size_t h) { return nt ? h * m + i : i * k + h; };
    auto bi = [&](size_t h, size_t j) { return nt ? h * n + j : j * k + h; };
    for(size_t i = 0; i < m; ++i)
        for(size_t h = 0; h < k; ++h) a[ai(i, h)] = __float2half(float(sample::uniform(1, i * k + h)));
    for(size_t h = 0; h < k; ++h)
        for(size_t j = 0; j < n; ++j) b[bi(h, j)] = __float2half(float(sample::uniform(2, h * n + j)));
    for(size_t i = 0; i < c.size(); ++i) c[i] = __float2half(float(sample::uniform(3, i)));
    std::printf("Initializing device data...\n");
    __half *da = sample::to_device(a), *db = sample::to_device(b), *dc = sample::to_device(c), *dd = nullptr;
    CHECK_CUDA(cudaMalloc(&dd, d.size() * sizeof(__half)));
    CHECK_CUDA(cudaMemset(dd, 0xFF, d.size() * sizeof(__half))); // NaN pattern: unwritten elements show up
    std::printf("Launching GEMM kernel...\n");
    const float ms = sample::time_launches(
        [&] {
            CHECK_B200(b200wmma_gemm_f16(m, n, k, da, db, dc, dd, nt ? m : k, nt ? n : k, n, n, alpha, beta,
                                         nt ? B200WMMA_COL_MAJOR : B200WMMA_ROW_MAJOR,
                                         nt ? B200WMMA_ROW_MAJOR : B200WMMA_COL_MAJOR, B200WMMA_ROW_MAJOR,
                                         B200WMMA_OUT_F16, nullptr));
        },
        2, 5);
    std::printf("MatM, MatN, MatK, alpha, beta, elapsedMs, TFlops/s\n%u, %u, %u, %g, %g, %.4f, %.1f\n", m, n, k, alpha,
                beta, ms, sample::tflops(m, n, k, ms));
    CHECK_CUDA(cudaMemcpy(d.data(), dd, d.size() * sizeof(__half), cudaMemcpyDeviceToHost));
    // spot validation: 8 rows, all columns, fp64 host recomputation
    double max_err = 0.0;
    for(uint32_t s = 0; s < 8; ++s)
    {
        const uint32_t i = (s == 7) ? m - 1 : uint32_t(sample::mix(42, s) % m);
        for(uint32_t j = 0; j < n; ++j)
        {
            double acc = 0.0, mag = 0.0;
            for(uint32_t h = 0; h < k; ++h)
            {
                const double av = __half2float(a[ai(i, h)]), bv = __half2float(b[bi(h, j)]);
                acc += av * bv;
                mag += std::fabs(av * bv);
            }
            const double cv = __half2float(c[size_t(i) * n + j]);
            const double ref = alpha * acc + beta * cv, bound = std::fabs(alpha) * mag + std::fabs(beta * cv);
            max_err = std::fmax(max_err, std::fabs(__half2float(d[size_t(i) * n + j]) - ref) / std::fmax(bound, 1e-30));
        }
    }
    CHECK_CUDA(cudaFree(da)); CHECK_CUDA(cudaFree(db)); CHECK_CUDA(cudaFree(dc)); CHECK_CUDA(cudaFree(dd));
    const int rc = sample::report("perf_hgemm", max_err, 2e-3);
    std::printf("Finished!\n");
    return rc;
}
