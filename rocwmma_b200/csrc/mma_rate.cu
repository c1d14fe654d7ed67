// Issue rate of the warp-level tensor-core instructions the fragment API and the fp64 GEMM are built on, measured on
// the device the caller is on: every SM runs warps that issue the instruction back to back from registers (no memory
// traffic), so the result is the rate the instruction's pipe sustains at the clock the GPU runs at under that load.
// It is the denominator for the throughput of the fragment-API kernels and of the fp64 GEMM.  No reference counterpart.
#include "common.cuh"

namespace b200wmma
{
    namespace rate
    {
        constexpr int WARPS = 16, MI = 2, NJ = 4; // the register tile of the fp64 GEMM's warps: 2 x 4 accumulators

        // kind 0: m16n8k16 f16 x f16 -> f32;  kind 1: m16n8k8 f64
        template <int KIND>
        __global__ void __launch_bounds__(WARPS * 32) issue_loop(double* sink, int iters, double seed)
        {
            if constexpr(KIND == 0)
            {
                float    acc[MI][NJ][4];
                uint32_t a[MI][4], b[NJ][2];
                for(int i = 0; i < MI; ++i)
                    for(int q = 0; q < 4; ++q)
                        a[i][q] = 0x3C003C00u + threadIdx.x + i + q; // two fp16 values near 1
                for(int j = 0; j < NJ; ++j)
                    for(int q = 0; q < 2; ++q)
                        b[j][q] = 0x3C003C00u + 3u * threadIdx.x + j + q;
                for(int i = 0; i < MI; ++i)
                    for(int j = 0; j < NJ; ++j)
                        for(int e = 0; e < 4; ++e)
                            acc[i][j][e] = 0.f;
                for(int it = 0; it < iters; ++it)
                {
#pragma unroll
                    for(int i = 0; i < MI; ++i)
#pragma unroll
                        for(int j = 0; j < NJ; ++j)
                            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
                                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                         : "+f"(acc[i][j][0]), "+f"(acc[i][j][1]), "+f"(acc[i][j][2]), "+f"(acc[i][j][3])
                                         : "r"(a[i][0]), "r"(a[i][1]), "r"(a[i][2]), "r"(a[i][3]), "r"(b[j][0]), "r"(b[j][1]));
                }
                float s = 0.f;
                for(int i = 0; i < MI; ++i)
                    for(int j = 0; j < NJ; ++j)
                        for(int e = 0; e < 4; ++e)
                            s += acc[i][j][e];
                if(s == 12345.678f) // never true: keeps the loop alive without a store on the measured path
                    sink[threadIdx.x] = s;
            }
            else
            {
                double acc[MI][NJ][4], a[MI][4], b[NJ][2];
                for(int i = 0; i < MI; ++i)
                    for(int q = 0; q < 4; ++q)
                        a[i][q] = seed * (threadIdx.x + i + q);
                for(int j = 0; j < NJ; ++j)
                    for(int q = 0; q < 2; ++q)
                        b[j][q] = seed * (3 * threadIdx.x + j + q);
                for(int i = 0; i < MI; ++i)
                    for(int j = 0; j < NJ; ++j)
                        for(int e = 0; e < 4; ++e)
                            acc[i][j][e] = 0.0;
                for(int it = 0; it < iters; ++it)
                {
#pragma unroll
                    for(int i = 0; i < MI; ++i)
#pragma unroll
                        for(int j = 0; j < NJ; ++j)
                            asm volatile("mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 "
                                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                         : "+d"(acc[i][j][0]), "+d"(acc[i][j][1]), "+d"(acc[i][j][2]), "+d"(acc[i][j][3])
                                         : "d"(a[i][0]), "d"(a[i][1]), "d"(a[i][2]), "d"(a[i][3]), "d"(b[j][0]), "d"(b[j][1]));
                }
                double s = 0.0;
                for(int i = 0; i < MI; ++i)
                    for(int j = 0; j < NJ; ++j)
                        for(int e = 0; e < 4; ++e)
                            s += acc[i][j][e];
                if(s == 12345.678)
                    sink[threadIdx.x] = s;
            }
        }
    } // namespace rate
} // namespace b200wmma

extern "C" int b200wmma_measure_mma_sync_rate(int kind, double* tflops, void* stream)
{
    using namespace b200wmma;
    using namespace b200wmma::rate;
    clear_error();
    B200_REQUIRE(kind == 0 || kind == 1, B200WMMA_ERR_INVALID_ARG, "measure_mma_sync_rate: kind must be 0 (f16 m16n8k16) or 1 (f64 m16n8k8)");
    B200_REQUIRE(tflops, B200WMMA_ERR_INVALID_ARG, "measure_mma_sync_rate: tflops must be non-null");
    if(int e = require_sm100())
        return e;
    int dev = 0, sms = 0;
    B200_CHECK_CUDA(cudaGetDevice(&dev));
    B200_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    cudaStream_t st = as_stream(stream);
    double*      sink = nullptr;
    B200_CHECK_CUDA(cudaMalloc(&sink, WARPS * 32 * sizeof(double)));
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaError_t err = cudaEventCreate(&e0);
    if(err == cudaSuccess)
        err = cudaEventCreate(&e1);
    // a few milliseconds per launch: kind 0 issues 4096 flop per instruction, kind 1 2048
    const int    iters         = kind == 0 ? 60000 : 6000;
    const double flop_per_inst = kind == 0 ? 2.0 * 16 * 8 * 16 : 2.0 * 16 * 8 * 8;
    float        best_ms       = 0.f;
    for(int rep = 0; rep < 3 && err == cudaSuccess; ++rep) // the first launch warms up; the faster of the next two counts
    {
        cudaEventRecord(e0, st);
        if(kind == 0)
            issue_loop<0><<<sms, WARPS * 32, 0, st>>>(sink, iters, 1e-9);
        else
            issue_loop<1><<<sms, WARPS * 32, 0, st>>>(sink, iters, 1e-9);
        cudaEventRecord(e1, st);
        err = cudaEventSynchronize(e1);
        float ms = 0.f;
        if(err == cudaSuccess)
            err = cudaEventElapsedTime(&ms, e0, e1);
        if(rep > 0 && (best_ms == 0.f || ms < best_ms))
            best_ms = ms;
    }
    if(e0)
        cudaEventDestroy(e0);
    if(e1)
        cudaEventDestroy(e1);
    cudaFree(sink);
    B200_CHECK_CUDA(err);
    *tflops = flop_per_inst * MI * NJ * iters * WARPS * sms / (best_ms * 1e-3) / 1e12;
    return B200WMMA_OK;
}
