// Host driver of the fp64 GEMM (DMMA), mirroring gemm_test() of rocWMMA's samples/perf_dgemm.cpp (the perf_hgemm
// flow, samples/perf_hgemm.cpp:713-941, with fp64 types): fill, copy to the device, 2 warm-up + 5 timed launches,
// TFlops/s, spot validation.
// Usage: perf_dgemm [m n k alpha beta]   (default 4096 4096 4096 1 1: A row-major, B col-major, C/D row-major)
#include "common.hpp"

int main(int argc, char** argv)
{
    const uint32_t m = argc > 3 ? std::atoi(argv[1]) : 4096, n = argc > 3 ? std::atoi(argv[2]) : 4096,
                   k = argc > 3 ? std::atoi(argv[3]) : 4096;
    const double alpha = argc > 5 ? std::atof(argv[4]) : 1.0, beta = argc > 5 ? std::atof(argv[5]) : 1.0;
    std::printf("Initializing host data...\n");
    std::vector<double> a(size_t(m) * k), b(size_t(n) * k), c(size_t(m) * n), d(size_t(m) * n);
    for(size_t i = 0; i < a.size(); ++i) a[i] = sample::uniform(1, i);
    for(size_t h = 0; h < k; ++h)
        for(size_t j = 0; j < n; ++j) b[j * k + h] = sample::uniform(2, h * n + j); // B column-major
    for(size_t i = 0; i < c.size(); ++i) c[i] = sample::uniform(3, i);
    std::printf("Initializing device data...\n");
    double *da = sample::to_device(a), *db = sample::to_device(b), *dc = sample::to_device(c), *dd = nullptr;
    CHECK_CUDA(cudaMalloc(&dd, d.size() * sizeof(double)));
    CHECK_CUDA(cudaMemset(dd, 0xFF, d.size() * sizeof(double)));
    std::printf("Launching GEMM kernel...\n");
    const float ms = sample::time_launches(
        [&] {
            CHECK_B200(b200wmma_gemm_f64(m, n, k, da, db, dc, dd, k, k, n, n, alpha, beta, B200WMMA_ROW_MAJOR, B200WMMA_COL_MAJOR,
                                         B200WMMA_ROW_MAJOR, nullptr));
        },
        2, 5);
    std::printf("MatM, MatN, MatK, alpha, beta, elapsedMs, TFlops/s\n%u, %u, %u, %g, %g, %.4f, %.1f\n", m, n, k, alpha, beta, ms,
                sample::tflops(m, n, k, ms));
    CHECK_CUDA(cudaMemcpy(d.data(), dd, d.size() * sizeof(double), cudaMemcpyDeviceToHost));
    double max_err = 0.0;
    for(uint32_t s = 0; s < 8; ++s)
    {
        const uint32_t i = (s == 7) ? m - 1 : uint32_t(sample::mix(42, s) % m);
        for(uint32_t j = 0; j < n; ++j)
        {
            long double acc = 0.0L;
            double      mag = 0.0;
            for(uint32_t h = 0; h < k; ++h)
            {
                const double av = a[size_t(i) * k + h], bv = b[size_t(j) * k + h];
                acc += static_cast<long double>(av) * bv;
                mag += std::fabs(av * bv);
            }
            const double cv  = c[size_t(i) * n + j];
            const double ref = double(alpha * acc + beta * cv), bound = std::fabs(alpha) * mag + std::fabs(beta * cv);
            max_err = std::fmax(max_err, std::fabs(d[size_t(i) * n + j] - ref) / std::fmax(bound, 1e-30));
        }
    }
    CHECK_CUDA(cudaFree(da)); CHECK_CUDA(cudaFree(db)); CHECK_CUDA(cudaFree(dc)); CHECK_CUDA(cudaFree(dd));
    const int rc = sample::report("perf_dgemm", max_err, 1e-12);
    std::printf("Finished!\n");
    return rc;
}
