// Host driver of the DLRM dot interaction, mirroring dlrm_test() of rocWMMA's samples/simple_dlrm.cpp:443-710:
// forward pass then backward pass, each timed and validated on the host.
// Usage: simple_dlrm [m k batch]   (default 27 128 16384; rows padded to 32, output width padded to a multiple of 8)
#include "common.hpp"

int main(int argc, char** argv)
{
    const uint32_t m = argc > 3 ? std::atoi(argv[1]) : 27, k = argc > 3 ? std::atoi(argv[2]) : 128,
                   B = argc > 3 ? std::atoi(argv[3]) : 16384;
    const uint32_t ms = 32, tri = m * (m - 1) / 2, w = (k + tri + 7) / 8 * 8;
    std::vector<__half> x(size_t(B) * ms * k, __float2half(0.f)), up(size_t(B) * w, __float2half(0.f));
    for(size_t b = 0; b < B; ++b)
    {
        for(uint32_t i = 0; i < m; ++i)
            for(uint32_t j = 0; j < k; ++j)
                x[(b * ms + i) * k + j] = __float2half(float(sample::normal(4, (b * ms + i) * k + j, 0.25)));
        for(uint32_t j = 0; j < k + tri; ++j)
            up[b * w + j] = __float2half(float(sample::normal(5, b * w + j, 0.1)));
    }
    std::vector<__half> out(size_t(B) * w), grad(size_t(B) * ms * k), mlp(size_t(B) * k);
    __half *dx = sample::to_device(x), *dup = sample::to_device(up), *dout, *dgrad, *dmlp;
    CHECK_CUDA(cudaMalloc(&dout, out.size() * 2)); CHECK_CUDA(cudaMalloc(&dgrad, grad.size() * 2)); CHECK_CUDA(cudaMalloc(&dmlp, mlp.size() * 2));
    CHECK_CUDA(cudaMemset(dgrad, 0, grad.size() * 2));

    const float fms = sample::time_launches([&] { CHECK_B200(b200wmma_dlrm_fwd(dx, dout, m, ms, k, B, w, nullptr)); }, 2, 10);
    const float bms = sample::time_launches(
        [&] { CHECK_B200(b200wmma_dlrm_bwd(dx, dup, dgrad, dmlp, m, ms, k, B, w, 0, nullptr)); }, 2, 10);
    std::printf("pass, m, k, batch, elapsedMs, samples/s, GB/s\n");
    std::printf("fwd, %u, %u, %u, %.4f, %.3e, %.0f\n", m, k, B, fms, B / (fms * 1e-3), B * double(m * k * 2 + w * 2) / (fms * 1e-3) / 1e9);
    std::printf("bwd, %u, %u, %u, %.4f, %.3e, %.0f\n", m, k, B, bms, B / (bms * 1e-3), B * double(2 * m * k * 2 + w * 2 + k * 2) / (bms * 1e-3) / 1e9);
    CHECK_CUDA(cudaMemcpy(out.data(), dout, out.size() * 2, cudaMemcpyDeviceToHost));
    CHECK_CUDA(cudaMemcpy(grad.data(), dgrad, grad.size() * 2, cudaMemcpyDeviceToHost));
    CHECK_CUDA(cudaMemcpy(mlp.data(), dmlp, mlp.size() * 2, cudaMemcpyDeviceToHost));

    double ferr = 0.0, berr = 0.0;
    auto   X    = [&](size_t b, uint32_t i, uint32_t j) { return double(__half2float(x[(b * ms + i) * k + j])); };
    for(uint32_t s = 0; s < 32; ++s)
    {
        const size_t b = (s == 31) ? B - 1 : size_t(sample::mix(44, s) % B);
        for(uint32_t j = 0; j < k; ++j)
        {
            if(__half2float(out[b * w + j]) != float(X(b, 0, j))) ferr = 1.0;         // pass-through is a copy
            if(__half2float(mlp[b * k + j]) != __half2float(up[b * w + j])) berr = 1.0;
        }
        std::vector<double> T(size_t(m) * m, 0.0);
        uint32_t            p = k;
        for(uint32_t i = 0; i < m; ++i)
            for(uint32_t j = 0; j < i; ++j, ++p)
            {
                double acc = 0.0, mag = 0.0;
                for(uint32_t h = 0; h < k; ++h) { acc += X(b, i, h) * X(b, j, h); mag += std::fabs(X(b, i, h) * X(b, j, h)); }
                ferr = std::fmax(ferr, std::fabs(__half2float(out[b * w + p]) - acc) / std::fmax(mag, 1e-30));
                T[i * m + j] = T[j * m + i] = __half2float(up[b * w + p]);
            }
        for(uint32_t i = 0; i < m; ++i)
            for(uint32_t j = 0; j < k; ++j)
            {
                double acc = 0.0, mag = 0.0;
                for(uint32_t h = 0; h < m; ++h) { acc += T[i * m + h] * X(b, h, j); mag += std::fabs(T[i * m + h] * X(b, h, j)); }
                berr = std::fmax(berr, std::fabs(__half2float(grad[(b * ms + i) * k + j]) - acc) / std::fmax(mag, 1e-30));
            }
    }
    CHECK_CUDA(cudaFree(dx)); CHECK_CUDA(cudaFree(dup)); CHECK_CUDA(cudaFree(dout)); CHECK_CUDA(cudaFree(dgrad)); CHECK_CUDA(cudaFree(dmlp));
    int rc = sample::report("simple_dlrm forward", ferr, 2e-3);
    rc |= sample::report("simple_dlrm backward", berr, 2e-3);
    std::printf("Finished!\n");
    return rc;
}
