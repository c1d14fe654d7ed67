// Host driver of the fp32 fragment-API GEMM (sgemm_rocwmma_d, samples/simple_sgemm.cpp:81-139).
// Usage: simple_sgemm [m n k]   (default 1024^3, alpha = beta = 2, A row-major, B col-major, C/D row-major)
#include "simple_gemm.hpp"

int main(int argc, char** argv)
{
    return sample::simple_gemm_main<float>("simple_sgemm", argc, argv, b200wmma_simple_sgemm, 5e-6);
}
