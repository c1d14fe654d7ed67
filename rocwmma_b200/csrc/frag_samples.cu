// Placeholder until the fragment-API sample kernels are added.
#include "common.cuh"
extern "C" int b200wmma_simple_hgemm(uint32_t, uint32_t, uint32_t, const void*, const void*, const void*, void*,
                                     uint32_t, uint32_t, uint32_t, uint32_t, float, float, int, void*)
{
    return b200wmma::set_error(B200WMMA_ERR_UNSUPPORTED, "simple_hgemm: not built yet");
}
extern "C" int b200wmma_perf_hgemm_fragment(uint32_t, uint32_t, uint32_t, const void*, const void*, const void*,
                                            void*, uint32_t, uint32_t, uint32_t, uint32_t, float, float, void*)
{
    return b200wmma::set_error(B200WMMA_ERR_UNSUPPORTED, "perf_hgemm_fragment: not built yet");
}
