// Usage: simple_sgemv [m n]   (default 32768 x 32768, row-major A, alpha = 1.5, beta = 0.5)
#include "simple_gemv.hpp"
int main(int argc, char** argv)
{
    return gemv_sample<float>("simple_sgemv", argc, argv, 1e-3, b200wmma_gemv_f32);
}
