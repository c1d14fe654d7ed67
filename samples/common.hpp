// Shared helpers of the sample hosts: CUDA / library error checks, seeded fills, event timing and a
// small host-side spot check.  The samples mirror the host drivers of rocWMMA's samples
// (samples/common.hpp:34-46 error macro, :133-143 TFlops helper, :180-224 fills, :227-272 host check)
// on top of this library's C ABI.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../include/rocwmma_b200.h"

#define CHECK_CUDA(expr)                                                                              \
    do                                                                                                \
    {                                                                                                 \
        cudaError_t e_ = (expr);                                                                      \
        if(e_ != cudaSuccess)                                                                         \
        {                                                                                             \
            std::fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
            std::exit(EXIT_FAILURE);                                                                  \
        }                                                                                             \
    } while(0)

#define CHECK_B200(expr)                                                                              \
    do                                                                                                \
    {                                                                                                 \
        int s_ = (expr);                                                                              \
        if(s_ != B200WMMA_OK)                                                                         \
        {                                                                                             \
            std::fprintf(stderr, "rocwmma_b200 error %d (%s) at %s:%d\n", s_, b200wmma_last_error_string(), \
                         __FILE__, __LINE__);                                                         \
            std::exit(EXIT_FAILURE);                                                                  \
        }                                                                                             \
    } while(0)

namespace sample
{
    // Counter-based generator shared with the Python side (rocwmma_b200/datagen.py).
    inline uint64_t mix(uint64_t seed, uint64_t idx)
    {
        uint64_t z = seed * 0x9E3779B97F4A7C15ull + idx;
        z          = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z          = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    inline double uniform(uint64_t seed, uint64_t idx) // [-1, 1)
    {
        return 2.0 * (static_cast<double>(mix(seed, idx) >> 40) * 0x1.0p-24) - 1.0;
    }
    inline double normal(uint64_t seed, uint64_t idx, double sigma)
    {
        const double u1 = (static_cast<double>(mix(seed, 2 * idx) >> 40) + 0.5) * 0x1.0p-24;
        const double u2 = static_cast<double>(mix(seed, 2 * idx + 1) >> 40) * 0x1.0p-24;
        return sigma * std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2);
    }

    template <typename T>
    T* to_device(const std::vector<T>& h)
    {
        T* d = nullptr;
        CHECK_CUDA(cudaMalloc(&d, h.size() * sizeof(T)));
        CHECK_CUDA(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
        return d;
    }

    // Runs `launch` warm + timed times on the default stream; returns the mean time per launch in ms.
    template <typename F>
    float time_launches(F&& launch, int warm, int timed)
    {
        cudaEvent_t e0, e1;
        CHECK_CUDA(cudaEventCreate(&e0));
        CHECK_CUDA(cudaEventCreate(&e1));
        for(int i = 0; i < warm; ++i)
            launch();
        CHECK_CUDA(cudaEventRecord(e0));
        for(int i = 0; i < timed; ++i)
            launch();
        CHECK_CUDA(cudaEventRecord(e1));
        CHECK_CUDA(cudaEventSynchronize(e1));
        float ms = 0.f;
        CHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        CHECK_CUDA(cudaEventDestroy(e0));
        CHECK_CUDA(cudaEventDestroy(e1));
        int      st = 0;
        unsigned detail = 0;
        CHECK_B200(b200wmma_device_status(nullptr, &st, &detail));
        if(st != 0)
        {
            std::fprintf(stderr, "device status %d (detail 0x%08x)\n", st, detail);
            std::exit(EXIT_FAILURE);
        }
        return ms / timed;
    }

    inline double tflops(double m, double n, double k, double ms)
    {
        return 2.0 * m * n * k / (ms * 1e-3) / 1e12;
    }

    inline int report(const char* what, double max_err, double tol)
    {
        const bool ok = max_err <= tol && std::isfinite(max_err);
        std::printf("%s: max relative error %.3e (tolerance %.1e) -> %s\n", what, max_err, tol, ok ? "PASSED" : "FAILED");
        return ok ? 0 : 1;
    }
}
