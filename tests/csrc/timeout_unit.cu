// Exercises the bounded-wait machinery of the kernels (rocwmma_b200/csrc/ptx_sm100.cuh) without
// faulting or hanging anything: one CTA waits on an mbarrier that nothing ever arrives on, with a
// 1 ms limit instead of the kernels' 2 s.  The wait must give up, set the CTA abort flag, record
// {5 = DEVICE_TIMEOUT, detail} in the status word it was given and let the kernel return normally,
// leaving the context usable.  A second kernel shows the other outcome: the barrier is satisfied
// (one thread arrives) and the wait returns true with the status word untouched.
#include <cuda_runtime.h>
#include <cstdint>

#include "../../rocwmma_b200/csrc/ptx_sm100.cuh"

using namespace b200wmma;

__global__ void wait_kernel(unsigned* status, unsigned* result, int arrive, unsigned long long timeout_ns)
{
    __shared__ __align__(8) unsigned long long bar;
    __shared__ unsigned                       abort_flag;
    const uint32_t bar_addr = ptx::smem_u32(&bar);
    if(threadIdx.x == 0)
    {
        abort_flag = 0;
        ptx::mbar_init(bar_addr, 1);
        ptx::fence_barrier_init();
    }
    __syncthreads();
    if(threadIdx.x == 1 && arrive)
        ptx::mbar_arrive(bar_addr);
    bool ok = true;
    if(threadIdx.x == 0)
        ok = ptx::mbar_wait_bounded(bar_addr, 0, &abort_flag, status, 0xABC00000u | blockIdx.x, timeout_ns);
    // a second waiter must leave through the CTA-wide abort flag once the first one gave up
    if(threadIdx.x == 32)
        ok = ptx::mbar_wait_bounded(bar_addr, 0, &abort_flag, status, 0xDEF00000u | blockIdx.x, 4ull * timeout_ns);
    __syncthreads();
    if(threadIdx.x == 0)
    {
        result[0] = ok ? 1u : 0u;
        result[1] = abort_flag;
    }
}

// status, result: device pointers to 4 and 2 unsigned words.
extern "C" int timeout_unit_run(unsigned* status, unsigned* result, int arrive, unsigned long long timeout_ns)
{
    wait_kernel<<<1, 64>>>(status, result, arrive, timeout_ns);
    return static_cast<int>(cudaDeviceSynchronize());
}
