// Host driver of the fp64 fragment-API GEMM (dgemm_rocwmma_d, samples/simple_dgemm.cpp:81-139).
// Usage: simple_dgemm [m n k]   (default 1024^3, alpha = beta = 2, A row-major, B col-major, C/D row-major)
#include "simple_gemm.hpp"

int main(int argc, char** argv)
{
    return sample::simple_gemm_main<double>("simple_dgemm", argc, argv, b200wmma_simple_dgemm, 1e-12);
}
