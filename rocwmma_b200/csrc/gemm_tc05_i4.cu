// Host side of the packed-int4 GEMM that unpacks in the load path (gemm_tc05_i4.cuh).
//
// rocWMMA v1.6.0 has no int4 path; the semantics are those of its int8 GEMM (gemm_rocwmma_d pattern,
// samples/perf_hgemm.cpp:515-711 with int8 inputs / int32 compute as in
// test/gemm/gemm_common_test_params.hpp:51-147) applied to the sign-extended operands, bit-exact in int32.
#include "gemm_tc05_i4.cuh"
#include "tuning.cuh"

namespace b200wmma
{
    int launch_gemm_tc05_i4(uint32_t m, uint32_t n, uint32_t k, const uint8_t* a_packed, const uint8_t* b_packed,
                            const int32_t* c, int32_t* d, uint32_t lda_bytes, uint32_t ldb_bytes, uint32_t ldc, uint32_t ldd,
                            int32_t alpha, int32_t beta, cudaStream_t stream)
    {
        using namespace tc05;
        B200_REQUIRE(m && n && k, B200WMMA_ERR_INVALID_ARG, "gemm_i4: m, n, k must be non-zero");
        B200_REQUIRE(a_packed && b_packed && d, B200WMMA_ERR_INVALID_ARG, "gemm_i4: a_packed, b_packed, d must be non-null");
        B200_REQUIRE(c || beta == 0, B200WMMA_ERR_INVALID_ARG, "gemm_i4: c may be null only when beta == 0");
        B200_REQUIRE(k % 32 == 0, B200WMMA_ERR_UNSUPPORTED, "gemm_i4: k must be a multiple of 32 (16 packed bytes)");
        B200_REQUIRE(lda_bytes >= k / 2 && ldb_bytes >= k / 2 && ldd >= n && (!c || ldc >= n), B200WMMA_ERR_INVALID_ARG,
                     "gemm_i4: leading dimension smaller than the row it strides");
        B200_REQUIRE(aligned16(a_packed) && aligned16(b_packed) && lda_bytes % 16 == 0 && ldb_bytes % 16 == 0,
                     B200WMMA_ERR_ALIGNMENT, "gemm_i4: packed rows must be 16-byte aligned (TMA requirement)");
        if(int e = require_sm100())
            return e;
        unsigned* status = nullptr;
        if(int e = status_word_ptr(&status))
            return e;
        int dev = 0, sms = 0;
        B200_CHECK_CUDA(cudaGetDevice(&dev));
        B200_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));

        CUtensorMap tm_a, tm_b;
        if(int e = make_bytes_tmap(&tm_a, a_packed, m, k / 2, lda_bytes, tc05i4::RAW_ROW_BYTES, tc05i4::CTA_M,
                                   CU_TENSOR_MAP_SWIZZLE_NONE))
            return e;
        if(int e = make_bytes_tmap(&tm_b, b_packed, n, k / 2, ldb_bytes, tc05i4::RAW_ROW_BYTES, tc05i4::HALF_N,
                                   CU_TENSOR_MAP_SWIZZLE_NONE))
            return e;
        auto row_align = [](const void* p, uint32_t ld) {
            return (reinterpret_cast<uintptr_t>(p) % 16) == 0 && (static_cast<uint64_t>(ld) * 4) % 16 == 0;
        };
        const int   vec_ok = (row_align(d, ldd) && (!c || row_align(c, ldc))) ? 1 : 0;
        CUtensorMap tm_c = tm_a, tm_d = tm_a; // placeholders, never dereferenced when vec_ok == 0
        if(vec_ok)
        {
            if(int e = make_rowbox_tmap(&tm_d, 4, d, m, n, ldd))
                return e;
            tm_c = tm_d;
            if(c)
                if(int e = make_rowbox_tmap(&tm_c, 4, c, m, n, ldc))
                    return e;
        }

        // nibbles as 16 * v (cheaper to unpack, exact while 256 * |sum| fits int32) or sign-extended
        const bool          scaled = k < 131072u;
        auto                kern   = scaled ? tc05i4::gemm_tc05_i4_kernel<true> : tc05i4::gemm_tc05_i4_kernel<false>;
        static int          max_clusters_dev[2][MAX_DEVICES];
        int&                max_clusters = max_clusters_dev[scaled ? 1 : 0][current_device_slot()];
        cudaLaunchConfig_t  cfg          = {};
        cudaLaunchAttribute attr[1];
        attr[0].id               = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.blockDim             = dim3(tc05i4::NUM_THREADS);
        cfg.dynamicSmemBytes     = tc05i4::SMEM_BYTES;
        cfg.stream               = stream;
        cfg.attrs                = attr;
        cfg.numAttrs             = 1;
        if(max_clusters == 0)
        {
            B200_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tc05i4::SMEM_BYTES));
            cfg.gridDim = dim3(static_cast<unsigned>(sms) & ~1u);
            int nc      = 0;
            B200_CHECK_CUDA(cudaOccupancyMaxActiveClusters(&nc, kern, &cfg));
            B200_REQUIRE(nc > 0, B200WMMA_ERR_CUDA, "no two-CTA cluster of the int4 GEMM kernel fits on this device");
            max_clusters = nc;
        }
        const uint32_t tiles_m = ceil_div(m, tc05i4::PAIR_M), tiles_n = ceil_div(n, tc05i4::TILE_N);
        const uint32_t pairs   = min(tiles_m * tiles_n, static_cast<uint32_t>(max_clusters));
        cfg.gridDim            = dim3(2 * pairs);
        const int      gm      = tuning::get(tuning::GEMM_GROUP_M);
        B200_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, tm_a, tm_b, tm_c, tm_d, c, d, m, n, k / 2, ldc, ldd, alpha, beta, tiles_m,
                                           tiles_n, vec_ok, gm > 0 ? static_cast<uint32_t>(gm) : tc05i4::GROUP_M, status));
        return B200WMMA_OK;
    }
} // namespace b200wmma
