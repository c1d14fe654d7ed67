// Host side of the sparse tensor-core GEMM (kernel in gemm_tc05_sp.cuh): operand checks, the five
// TMA tensor maps and the cluster launch.
#include "gemm_tc05_sp.cuh"

namespace b200wmma
{
    // The kernel moves K in whole 128-wide boxes with TMA: every row start and pitch a multiple of 16
    // bytes, k a multiple of 128 (metadata rows are k/8 bytes: 16 bytes per slab).
    bool sp24_direct_ok(uint32_t k, const void* a_vals, const void* a_meta, const void* b, uint32_t lda_vals,
                        uint32_t ld_meta, uint32_t ldb)
    {
        return k % tc05s::HALF_K == 0 && aligned16(a_vals) && aligned16(a_meta) && aligned16(b) && lda_vals % 16 == 0
               && ld_meta % 16 == 0 && ldb % 16 == 0;
    }

    size_t sp24_packed_meta_bytes(uint32_t m, uint32_t k)
    {
        return static_cast<size_t>(ceil_div(m, tc05s::CTA_M)) * ceil_div(k, tc05s::SLAB_K) * tc05s::E_STAGE_BYTES;
    }

    int launch_sp24_repack_meta(uint32_t m, uint32_t k, const uint8_t* a_meta, uint32_t ld_meta, void* packed,
                                size_t packed_bytes, cudaStream_t stream)
    {
        using namespace tc05s;
        B200_REQUIRE(m && k, B200WMMA_ERR_INVALID_ARG, "sp24_repack_meta: m, k must be non-zero");
        B200_REQUIRE(a_meta && packed, B200WMMA_ERR_INVALID_ARG, "sp24_repack_meta: a_meta, packed must be non-null");
        B200_REQUIRE(k % HALF_K == 0, B200WMMA_ERR_UNSUPPORTED, "sp24_repack_meta: k must be a multiple of 128");
        B200_REQUIRE(ld_meta >= k / 8, B200WMMA_ERR_INVALID_ARG, "sp24_repack_meta: ld_meta smaller than k/8");
        B200_REQUIRE(aligned16(a_meta) && ld_meta % 16 == 0 && aligned16(packed), B200WMMA_ERR_ALIGNMENT,
                     "sp24_repack_meta: metadata rows and the destination must be 16-byte aligned");
        B200_REQUIRE(packed_bytes >= sp24_packed_meta_bytes(m, k), B200WMMA_ERR_INVALID_ARG,
                     "sp24_repack_meta: destination too small (%zu < %zu bytes)", packed_bytes, sp24_packed_meta_bytes(m, k));
        if(int e = require_sm100())
            return e;
        const uint32_t num_kb = ceil_div(k, SLAB_K);
        repack_meta_kernel<<<dim3(num_kb, ceil_div(m, CTA_M)), 256, 0, stream>>>(a_meta, static_cast<uint8_t*>(packed), m, k,
                                                                                 ld_meta, num_kb);
        B200_CHECK_CUDA(cudaGetLastError());
        return B200WMMA_OK;
    }

    // meta_is_packed: `a_meta` is the re-tiled copy made by launch_sp24_repack_meta (ld_meta unused).  Otherwise
    // it is the caller's row-major array; if `scratch` can hold the re-tiled copy it is made first.
    int launch_gemm_tc05_i8_sp24(uint32_t m, uint32_t n, uint32_t k, const int8_t* a_vals, const uint8_t* a_meta,
                                 bool meta_is_packed, const int8_t* b, const int32_t* c, int32_t* d, uint32_t lda_vals,
                                 uint32_t ld_meta, uint32_t ldb, uint32_t ldc, uint32_t ldd, int32_t alpha, int32_t beta,
                                 void* scratch, size_t scratch_bytes, cudaStream_t stream)
    {
        using namespace tc05s;
        B200_REQUIRE(m && n && k, B200WMMA_ERR_INVALID_ARG, "gemm_i8_sp24: m, n, k must be non-zero");
        B200_REQUIRE(a_vals && a_meta && b && d, B200WMMA_ERR_INVALID_ARG,
                     "gemm_i8_sp24: a_vals, a_meta, b, d must be non-null");
        B200_REQUIRE(c || beta == 0, B200WMMA_ERR_INVALID_ARG, "gemm_i8_sp24: c may be null only when beta == 0");
        if(meta_is_packed)
            ld_meta = (k / 8 + 15u) & ~15u; // not used for addressing; keeps the shared checks below meaningful
        B200_REQUIRE(lda_vals >= k / 2 && ld_meta >= k / 8 && ldb >= k && ldd >= n && (!c || ldc >= n),
                     B200WMMA_ERR_INVALID_ARG, "gemm_i8_sp24: leading dimension smaller than the row it strides");
        B200_REQUIRE(sp24_direct_ok(k, a_vals, a_meta, b, lda_vals, ld_meta, ldb), B200WMMA_ERR_ALIGNMENT,
                     "gemm_i8_sp24: the sparse tensor-core path needs k %% 128 == 0 and 16-byte aligned rows");
        if(int e = require_sm100())
            return e;
        unsigned* status = nullptr;
        if(int e = status_word_ptr(&status))
            return e;

        auto row_align = [](const void* p, uint32_t ld) {
            return (reinterpret_cast<uintptr_t>(p) % 16) == 0 && (static_cast<uint64_t>(ld) * 4) % 16 == 0;
        };
        const int vec_ok = (row_align(d, ldd) && (!c || row_align(c, ldc))) ? 1 : 0;

        // With scratch for a re-tiled copy of the metadata (1/8 byte per element of A) the kernel fetches it in
        // 128-byte rows; without, in the 16-byte rows of the caller's array (8 x the requests).
        const uint32_t num_kb   = ceil_div(k, SLAB_K);
        const bool     retile   = !meta_is_packed && scratch != nullptr && aligned16(scratch)
                            && scratch_bytes >= sp24_packed_meta_bytes(m, k);
        const bool  e_packed = meta_is_packed || retile;
        const void* e_src    = meta_is_packed ? static_cast<const void*>(a_meta) : scratch;
        if(retile)
            if(int e = launch_sp24_repack_meta(m, k, a_meta, ld_meta, scratch, scratch_bytes, stream))
                return e;
        CUtensorMap tm_a, tm_e, tm_b;
        if(int e = make_bytes_tmap(&tm_a, a_vals, m, k / 2, lda_vals, A_ROW_BYTES, CTA_M, CU_TENSOR_MAP_SWIZZLE_128B))
            return e;
        if(e_packed)
        {
            if(int e = make_bytes_tmap(&tm_e, e_src, ceil_div(m, CTA_M) * num_kb * E_PACKED_ROWS, 128, 128, 128, E_PACKED_ROWS,
                                       CU_TENSOR_MAP_SWIZZLE_NONE))
                return e;
        }
        else if(int e = make_bytes_tmap(&tm_e, a_meta, m, k / 8, ld_meta, E_ROW_BYTES, CTA_M, CU_TENSOR_MAP_SWIZZLE_NONE))
            return e;
        if(int e = make_bytes_tmap(&tm_b, b, n, k, ldb, HALF_K, HALF_N, CU_TENSOR_MAP_SWIZZLE_128B))
            return e;
        CUtensorMap tm_c = tm_a, tm_d = tm_a; // placeholders, never dereferenced when vec_ok == 0
        if(vec_ok != 0)
        {
            if(int e = make_rowbox_tmap(&tm_d, 4, d, m, n, ldd, EPI_ROW_BYTES))
                return e;
            tm_c = tm_d;
            if(c)
                if(int e = make_rowbox_tmap(&tm_c, 4, c, m, n, ldc, EPI_ROW_BYTES))
                    return e;
        }

        int dev = 0, sms = 0;
        B200_CHECK_CUDA(cudaGetDevice(&dev));
        B200_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        auto kern = e_packed ? gemm_tc05_sp_kernel<true> : gemm_tc05_sp_kernel<false>;
        static int max_clusters_dev[2][MAX_DEVICES];
        int&       max_clusters = max_clusters_dev[e_packed ? 1 : 0][current_device_slot()];
        const uint32_t tiles_m = ceil_div(m, PAIR_M), tiles_n = ceil_div(n, TILE_N);
        cudaLaunchConfig_t  cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id               = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.blockDim         = dim3(NUM_THREADS);
        cfg.dynamicSmemBytes = SMEM_BYTES;
        cfg.stream           = stream;
        cfg.attrs            = attr;
        cfg.numAttrs         = 1;
        if(max_clusters == 0)
        {
            B200_CHECK_CUDA(
                cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
            cfg.gridDim = dim3(static_cast<unsigned>(sms) & ~1u);
            int nc      = 0;
            B200_CHECK_CUDA(cudaOccupancyMaxActiveClusters(&nc, kern, &cfg));
            B200_REQUIRE(nc > 0, B200WMMA_ERR_CUDA, "no two-CTA cluster of the sparse GEMM kernel fits on this device");
            max_clusters = nc;
        }
        const uint32_t pairs = min(tiles_m * tiles_n, static_cast<uint32_t>(max_clusters));
        cfg.gridDim          = dim3(2 * pairs);
        B200_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, tm_a, tm_e, tm_b, tm_c, tm_d, c, d, m, n, k, ldc, ldd,
                                           alpha, beta, tiles_m, tiles_n, vec_ok, static_cast<uint32_t>(GROUP_M), status));
        return B200WMMA_OK;
    }
} // namespace b200wmma
