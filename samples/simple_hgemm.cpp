// Host driver of the fragment-API GEMM, mirroring gemm_test() of rocWMMA's samples/simple_hgemm.cpp:141-291.
// Usage: simple_hgemm [m n k]   (default 1024^3, alpha = beta = 2, A row-major, B col-major, C/D fp32)
#include "common.hpp"

int main(int argc, char** argv)
{
    const uint32_t m = argc > 3 ? std::atoi(argv[1]) : 1024, n = argc > 3 ? std::atoi(argv[2]) : 1024,
                   k = argc > 3 ? std::atoi(argv[3]) : 1024;
    const float alpha = 2.0f, beta = 2.0f;
    if(m % 16 || n % 16 || k % 16)
    {
        std::printf("Unsupported size!\n");
        return 0;
    }
    std::vector<__half> a(size_t(m) * k), b(size_t(n) * k);
    std::vector<float>  c(size_t(m) * n), d(size_t(m) * n);
    for(size_t i = 0; i < a.size(); ++i) a[i] = __float2half(float(sample::uniform(1, i)));
    for(size_t i = 0; i < b.size(); ++i) b[i] = __float2half(float(sample::uniform(2, i)));
    for(size_t i = 0; i < c.size(); ++i) c[i] = float(sample::uniform(3, i));
    __half *da = sample::to_device(a), *db = sample::to_device(b);
    float * dc = sample::to_device(c), *dd = nullptr;
    CHECK_CUDA(cudaMalloc(&dd, d.size() * sizeof(float)));
    CHECK_CUDA(cudaMemset(dd, 0xFF, d.size() * sizeof(float)));
    const float ms = sample::time_launches(
        [&] { CHECK_B200(b200wmma_simple_hgemm(m, n, k, da, db, dc, dd, k, k, n, n, alpha, beta, B200WMMA_OUT_F32, nullptr)); },
        1, 3);
    std::printf("BlkM, BlkN, BlkK, MatM, MatN, MatK, alpha, beta, elapsedMs, TFlops/s\n16, 16, 16, %u, %u, %u, %g, %g, %.4f, %.2f\n",
                m, n, k, alpha, beta, ms, sample::tflops(m, n, k, ms));
    CHECK_CUDA(cudaMemcpy(d.data(), dd, d.size() * sizeof(float), cudaMemcpyDeviceToHost));
    double max_err = 0.0;
    for(uint32_t s = 0; s < 16; ++s)
    {
        const uint32_t i = (s == 15) ? m - 1 : uint32_t(sample::mix(43, s) % m);
        for(uint32_t j = 0; j < n; ++j)
        {
            double acc = 0.0, mag = 0.0;
            for(uint32_t h = 0; h < k; ++h)
            {
                const double av = __half2float(a[size_t(i) * k + h]), bv = __half2float(b[size_t(j) * k + h]);
                acc += av * bv;
                mag += std::fabs(av * bv);
            }
            const double cv = c[size_t(i) * n + j], ref = alpha * acc + beta * cv;
            max_err = std::fmax(max_err, std::fabs(d[size_t(i) * n + j] - ref) / std::fmax(alpha * mag + std::fabs(beta * cv), 1e-30));
        }
    }
    CHECK_CUDA(cudaFree(da)); CHECK_CUDA(cudaFree(db)); CHECK_CUDA(cudaFree(dc)); CHECK_CUDA(cudaFree(dd));
    const int rc = sample::report("simple_hgemm", max_err, 1e-3);
    std::printf("Finished!\n");
    return rc;
}
