// Shared body of simple_sgemv / simple_dgemv, mirroring sgemv_test() of rocWMMA's samples/simple_sgemv.cpp:157-273
// (y = alpha * A x + beta * y in place, then host validation as in sgemv_cpu_h, :46-66).
#pragma once
#include "common.hpp"

template <typename T, typename Launch>
int gemv_sample(const char* name, int argc, char** argv, double tol, Launch launch)
{
    const uint32_t m = argc > 2 ? std::atoi(argv[1]) : 32768, n = argc > 2 ? std::atoi(argv[2]) : 32768;
    const T        alpha = T(1.5), beta = T(0.5);
    std::printf("Initializing host data...\n");
    std::vector<T> a(size_t(m) * n), x(n), y(m), y0;
    for(size_t i = 0; i < a.size(); ++i) a[i] = T(sample::uniform(6, i));
    for(size_t i = 0; i < n; ++i) x[i] = T(sample::uniform(7, i));
    for(size_t i = 0; i < m; ++i) y[i] = T(sample::uniform(8, i));
    y0 = y;
    T *da = sample::to_device(a), *dx = sample::to_device(x), *dy = sample::to_device(y);
    std::printf("Launching %s kernel...\n", name);
    // validation run (in place on y), then timing runs on a scratch copy of y
    CHECK_B200(launch(m, n, da, n, B200WMMA_ROW_MAJOR, dx, dy, alpha, beta, nullptr));
    CHECK_CUDA(cudaMemcpy(y.data(), dy, m * sizeof(T), cudaMemcpyDeviceToHost));
    const float ms = sample::time_launches([&] { CHECK_B200(launch(m, n, da, n, B200WMMA_ROW_MAJOR, dx, dy, alpha, T(0), nullptr)); }, 2, 10);
    std::printf("MatM, MatN, elapsedMs, GB/s\n%u, %u, %.4f, %.0f\n", m, n, ms,
                double(sizeof(T)) * (double(m) * n + n + 2.0 * m) / (ms * 1e-3) / 1e9);
    double max_err = 0.0;
    for(uint32_t s = 0; s < 64; ++s)
    {
        const uint32_t i = (s == 63) ? m - 1 : uint32_t(sample::mix(45, s) % m);
        long double    acc = 0, mag = 0;
        for(uint32_t h = 0; h < n; ++h)
        {
            acc += (long double)a[size_t(i) * n + h] * x[h];
            mag += fabsl((long double)a[size_t(i) * n + h] * x[h]);
        }
        const long double ref = alpha * acc + beta * y0[i], bound = std::fabs(alpha) * mag + fabsl(beta * y0[i]);
        max_err = std::fmax(max_err, double(fabsl(y[i] - ref) / bound));
    }
    CHECK_CUDA(cudaFree(da)); CHECK_CUDA(cudaFree(dx)); CHECK_CUDA(cudaFree(dy));
    const int rc = sample::report(name, max_err, tol);
    std::printf("Finished!\n");
    return rc;
}
