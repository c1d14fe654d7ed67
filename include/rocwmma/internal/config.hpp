// Compile-time configuration of the warp-32 rocWMMA-compatible device API.
// Mirrors the macro surface of rocWMMA's internal/config.hpp (:48-219) that user kernels touch.
#ifndef ROCWMMA_B200_CONFIG_HPP
#define ROCWMMA_B200_CONFIG_HPP

#include <cuda_runtime.h>
#include <cstdint>

#if defined(__CUDA_ARCH__)
#define ROCWMMA_ARCH_HOST 0
#else
#define ROCWMMA_ARCH_HOST 1
#endif

// No AMD target is ever active here; user code that branches on these takes its generic path.
#define ROCWMMA_ARCH_GFX9 0
#define ROCWMMA_ARCH_GFX11 0
#define ROCWMMA_ARCH_GFX12 0
#define ROCWMMA_ARCH_SM100 1
#define ROCWMMA_WAVE64_MODE 0
#define ROCWMMA_WAVE32_MODE 1

#define ROCWMMA_DEVICE __device__
#define ROCWMMA_HOST __host__
#define ROCWMMA_HOST_DEVICE __host__ __device__
#define ROCWMMA_KERNEL __global__

// HIP's spelling of the dynamic shared-memory array, used by kernels written for the reference
// (samples/perf_hgemm.cpp:345, test/gemm/gemm_PGR1_LB2_MP0_MB_CP/device/kernel_device_func.hpp:191)
#ifndef HIP_DYNAMIC_SHARED
#define HIP_DYNAMIC_SHARED(type, var) extern __shared__ type var[];
#endif

#endif
