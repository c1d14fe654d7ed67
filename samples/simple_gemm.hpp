// Shared body of the fp32 / fp64 forms of the naive fragment-API GEMM hosts, mirroring gemm_test() of rocWMMA's
// samples/simple_sgemm.cpp:141-291 and samples/simple_dgemm.cpp:141-291 (the two differ in their element type only).
#pragma once
#include "common.hpp"

namespace sample
{
    // Launch = the C entry point of the element type; tol = acceptance bound relative to alpha * sum|a||b| + |beta c|
    template <typename T, typename Launch>
    int simple_gemm_main(const char* name, int argc, char** argv, Launch launch, double tol)
    {
        const uint32_t m = argc > 3 ? std::atoi(argv[1]) : 1024, n = argc > 3 ? std::atoi(argv[2]) : 1024,
                       k = argc > 3 ? std::atoi(argv[3]) : 1024;
        const T alpha = T(2), beta = T(2);
        if(m % 16 || n % 16 || k % 16)
        {
            std::printf("Unsupported size!\n");
            return 0;
        }
        std::vector<T> a(size_t(m) * k), b(size_t(n) * k), c(size_t(m) * n), d(size_t(m) * n);
        for(size_t i = 0; i < a.size(); ++i) a[i] = T(uniform(1, i));
        for(size_t i = 0; i < b.size(); ++i) b[i] = T(uniform(2, i)); // B column-major: element (h, j) at j * k + h
        for(size_t i = 0; i < c.size(); ++i) c[i] = T(uniform(3, i));
        T *da = to_device(a), *db = to_device(b), *dc = to_device(c), *dd = nullptr;
        CHECK_CUDA(cudaMalloc(&dd, d.size() * sizeof(T)));
        CHECK_CUDA(cudaMemset(dd, 0xFF, d.size() * sizeof(T)));
        const float ms = time_launches([&] { CHECK_B200(launch(m, n, k, da, db, dc, dd, k, k, n, n, alpha, beta, nullptr)); }, 1, 3);
        std::printf("BlkM, BlkN, BlkK, MatM, MatN, MatK, alpha, beta, elapsedMs, TFlops/s\n16, 16, 16, %u, %u, %u, %g, %g, %.4f, %.2f\n",
                    m, n, k, double(alpha), double(beta), ms, tflops(m, n, k, ms));
        CHECK_CUDA(cudaMemcpy(d.data(), dd, d.size() * sizeof(T), cudaMemcpyDeviceToHost));
        double max_err = 0.0;
        for(uint32_t s = 0; s < 16; ++s)
        {
            const uint32_t i = (s == 15) ? m - 1 : uint32_t(mix(43, s) % m);
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
                const double cv = c[size_t(i) * n + j], ref = double(alpha * acc + beta * cv);
                max_err = std::fmax(max_err, std::fabs(d[size_t(i) * n + j] - ref) / std::fmax(alpha * mag + std::fabs(beta * cv), 1e-30));
            }
        }
        CHECK_CUDA(cudaFree(da)); CHECK_CUDA(cudaFree(db)); CHECK_CUDA(cudaFree(dc)); CHECK_CUDA(cudaFree(dd));
        const int rc = report(name, max_err, tol);
        std::printf("Finished!\n");
        return rc;
    }
} // namespace sample
