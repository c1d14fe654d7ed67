// GEMM kernels written against this repository's rocWMMA-compatible fragment API
// (<rocwmma/rocwmma.hpp>, <rocwmma/rocwmma_coop.hpp>, <rocwmma/rocwmma_transforms.hpp>), i.e. the
// way a rocWMMA user writes kernels.  They exist to prove the device API end to end:
//
//   simple_hgemm         the naive "one 16x16 output block per wave" GEMM of
//                        samples/simple_hgemm.cpp:81-139 (A row major, B column major, C/D row major,
//                        fp32 accumulation, D = alpha*A*B + beta*C computed element-wise on fragments).
//   perf_hgemm_fragment  the cooperative / shared-memory double-buffered pipeline of
//                        samples/perf_hgemm.cpp:515-711 with the layouts that sample ships with
//                        (A column major, B row major, C/D row major, LDS column major).
//
// The fast GEMM of this library is the tcgen05 kernel (gemm_tc05.cu); these two go through
// warp-level mma.sync fragments like any user kernel would.
#include "common.cuh"
#include "tuning.cuh"

#include <rocwmma/rocwmma.hpp>
#include <rocwmma/rocwmma_coop.hpp>
#include <rocwmma/rocwmma_transforms.hpp>

namespace b200wmma
{
    namespace fragk
    {
        using namespace rocwmma;

        // --------------------------------- simple_hgemm ---------------------------------------
        constexpr uint32_t SB_M = 16, SB_N = 16, SB_K = 16;
        constexpr uint32_t S_TBLOCK_X = 4 * Constants::AMDGCN_WAVE_SIZE, S_TBLOCK_Y = 4;

        // The same kernel body serves hgemm_rocwmma_d (InT = float16_t, CmpT = float32_t), sgemm_rocwmma_d
        // (samples/simple_sgemm.cpp:81-139, all float32_t) and dgemm_rocwmma_d (samples/simple_dgemm.cpp:81-139,
        // all float64_t): the three samples differ in their types only.
        template <typename InT, typename OutT, typename CmpT>
        ROCWMMA_KERNEL void simple_gemm_kernel(uint32_t m, uint32_t n, uint32_t k, InT const* a, InT const* b,
                                               OutT const* c, OutT* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                                               uint32_t ldd, CmpT alpha, CmpT beta)
        {
            fragment<matrix_a, SB_M, SB_N, SB_K, InT, row_major> fragA;
            fragment<matrix_b, SB_M, SB_N, SB_K, InT, col_major> fragB;
            fragment<accumulator, SB_M, SB_N, SB_K, OutT>        fragC; // layout given at run time
            fragment<accumulator, SB_M, SB_N, SB_K, CmpT>        fragAcc;
            fill_fragment(fragAcc, CmpT(0));

            // one output block per wave: wave grid position -> block position
            const uint32_t waveRow = (blockIdx.x * blockDim.x + threadIdx.x) / Constants::AMDGCN_WAVE_SIZE;
            const uint32_t waveCol = blockIdx.y * blockDim.y + threadIdx.y;
            const uint32_t row0 = waveRow * SB_M, col0 = waveCol * SB_N;
            if(row0 >= m || col0 >= n)
                return;

            for(uint32_t kk = 0; kk < k; kk += SB_K)
            {
                load_matrix_sync(fragA, a + (static_cast<size_t>(row0) * lda + kk), lda);
                load_matrix_sync(fragB, b + (static_cast<size_t>(col0) * ldb + kk), ldb);
                mma_sync(fragAcc, fragA, fragB, fragAcc);
            }
            load_matrix_sync(fragC, c + (static_cast<size_t>(row0) * ldc + col0), ldc, mem_row_major);
            for(uint32_t i = 0; i < fragC.num_elements; ++i)
                fragC.x[i] = alpha * fragAcc.x[i] + beta * fragC.x[i];
            store_matrix_sync(d + (static_cast<size_t>(row0) * ldd + col0), fragC, ldd, mem_row_major);
        }

        // ------------------------------ perf_hgemm on fragments --------------------------------
        // 8 warps as 4 (x) by 2 (y); each warp owns a 32 x 64 tile = 2 x 4 blocks of 16 x 16;
        // the thread block owns a 128 x 128 macro tile and walks K in slabs of SLAB_K (a multiple of the blocks' K = 16):
        // one cooperative global read, one shared-memory write and one barrier per slab, SLAB_K / 16 rounds of block
        // multiplies on it.  The sample's own slab is one block deep (samples/perf_hgemm.cpp:264-271), and so is the
        // default here; deeper slabs are selectable for measurement (see the launch code for what they cost).
        constexpr uint32_t P_M = 16, P_N = 16, P_K = 16;
        constexpr uint32_t P_BLOCKS_X = 2, P_BLOCKS_Y = 4;
        constexpr uint32_t P_TBLOCK_X = 128, P_TBLOCK_Y = 2;
        constexpr uint32_t P_WARPS_X = P_TBLOCK_X / Constants::AMDGCN_WAVE_SIZE, P_WARPS_Y = P_TBLOCK_Y;
        constexpr uint32_t P_WARP_TILE_X = P_BLOCKS_X * P_M, P_WARP_TILE_Y = P_BLOCKS_Y * P_N;
        constexpr uint32_t P_MACRO_X = P_WARPS_X * P_WARP_TILE_X, P_MACRO_Y = P_WARPS_Y * P_WARP_TILE_Y;
        constexpr uint32_t P_WARPS = P_WARPS_X * P_WARPS_Y;

        using PIn = float16_t;
        using POut = float16_t;
        using PCmp = float32_t;
        using PLayoutA = col_major;
        using PLayoutB = row_major;
        using PLayoutC = row_major;
        using PLayoutLds = col_major;

        using MmaA   = fragment<matrix_a, P_M, P_N, P_K, PIn, PLayoutA>;
        using MmaB   = fragment<matrix_b, P_M, P_N, P_K, PIn, PLayoutB>;
        using MmaC   = fragment<accumulator, P_M, P_N, P_K, POut, PLayoutC>;
        using MmaAcc = fragment<accumulator, P_M, P_N, P_K, PCmp>;
        using LdsReadA = ApplyDataLayout_t<MmaA, PLayoutLds>;
        using LdsReadB = ApplyDataLayout_t<ApplyTranspose_t<MmaB>, PLayoutLds>;
        template <uint32_t SLAB_K>
        struct PSlab
        {
            // whole-macro-tile K slabs read cooperatively from global memory
            using GlobalA = fragment<matrix_a, P_MACRO_X, P_N, SLAB_K, PIn, PLayoutA>;
            using GlobalB = fragment<matrix_b, P_M, P_MACRO_Y, SLAB_K, PIn, PLayoutB>;
            // shared memory holds A and B^T stacked, both as "matrix_a"-shaped column-major blocks
            using LdsWriteA = ApplyDataLayout_t<GlobalA, PLayoutLds>;
            using LdsWriteB = ApplyDataLayout_t<ApplyTranspose_t<GlobalB>, PLayoutLds>;
            static constexpr uint32_t LDS_HEIGHT = GetIOShape_t<LdsWriteA>::BlockHeight + GetIOShape_t<LdsWriteB>::BlockHeight;
            static constexpr uint32_t LDS_WIDTH  = SLAB_K;
            // leading dimension of the shared-memory block, padded by 16 bytes: consecutive K rows then start in
            // different banks, which the 8 x 8 matrix loads and stores (eight 16-byte rows per instruction phase) need
            // to be conflict-free
            static constexpr uint32_t LDS_PAD   = 16 / sizeof(PIn);
            static constexpr uint32_t LDS_LD    = (std::is_same<PLayoutLds, row_major>::value ? LDS_WIDTH : LDS_HEIGHT) + LDS_PAD;
            static constexpr uint32_t LDS_ALLOC = LDS_LD * (std::is_same<PLayoutLds, row_major>::value ? LDS_HEIGHT : LDS_WIDTH);
        };

        template <uint32_t SLAB_K>
        ROCWMMA_KERNEL void __launch_bounds__(P_TBLOCK_X* P_TBLOCK_Y)
            perf_hgemm_fragment_kernel(uint32_t m, uint32_t n, uint32_t k, PIn const* a, PIn const* b,
                                       POut const* c, POut* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                                       uint32_t ldd, PCmp alpha, PCmp beta)
        {
            using S         = PSlab<SLAB_K>;
            using GlobalA   = typename S::GlobalA;
            using GlobalB   = typename S::GlobalB;
            using LdsWriteA = typename S::LdsWriteA;
            using LdsWriteB = typename S::LdsWriteB;
            constexpr uint32_t P_LDS_LD = S::LDS_LD;
            extern __shared__ __align__(16) unsigned char lds_raw[];
            PIn* ldsLo = reinterpret_cast<PIn*>(lds_raw);
            PIn* ldsHi = ldsLo + S::LDS_ALLOC;

            const auto warpCoord  = make_coord2d(threadIdx.x / Constants::AMDGCN_WAVE_SIZE, threadIdx.y);
            const auto warpOffset = warpCoord * make_coord2d(P_WARP_TILE_X, P_WARP_TILE_Y);
            const auto macroCoord = make_coord2d(blockIdx.x, blockIdx.y) * make_coord2d(P_MACRO_X, P_MACRO_Y);
            const auto tileCoord  = macroCoord + warpOffset;
            if(get<0>(tileCoord) + P_WARP_TILE_X > m || get<1>(tileCoord) + P_WARP_TILE_Y > n)
                return; // host guarantees whole macro tiles; nothing to synchronise with in that case
            const uint32_t warpIndex = get<0>(warpCoord) * P_WARPS_Y + get<1>(warpCoord);

            using MapGA = GetDataLayout_t<GlobalA>;
            using MapGB = GetDataLayout_t<GlobalB>;
            using MapLA = GetDataLayout_t<LdsWriteA>;
            using MapLB = GetDataLayout_t<LdsWriteB>;
            size_t       offA  = MapGA::fromMatrixCoord(make_coord2d(get<0>(macroCoord), 0u), lda);
            size_t       offB  = MapGB::fromMatrixCoord(make_coord2d(0u, get<1>(macroCoord)), ldb);
            const size_t stepA = MapGA::fromMatrixCoord(make_coord2d(0u, SLAB_K), lda);
            const size_t stepB = MapGB::fromMatrixCoord(make_coord2d(SLAB_K, 0u), ldb);

            const uint32_t ldsWriteA = 0u;
            const uint32_t ldsWriteB = MapLA::fromMatrixCoord(make_coord2d(GetIOShape_t<LdsWriteA>::BlockHeight, 0u), P_LDS_LD);
            const uint32_t ldsReadA  = ldsWriteA + MapLA::fromMatrixCoord(make_coord2d(get<0>(warpOffset), 0u), P_LDS_LD);
            const uint32_t ldsReadB  = ldsWriteB + MapLB::fromMatrixCoord(make_coord2d(get<1>(warpOffset), 0u), P_LDS_LD);
            const uint32_t blockStepA = GetDataLayout_t<LdsReadA>::fromMatrixCoord(make_coord2d(GetIOShape_t<LdsReadA>::BlockHeight, 0u), P_LDS_LD);
            const uint32_t blockStepB = GetDataLayout_t<LdsReadB>::fromMatrixCoord(make_coord2d(GetIOShape_t<LdsReadB>::BlockHeight, 0u), P_LDS_LD);
            const uint32_t kStep      = GetDataLayout_t<LdsReadA>::fromMatrixCoord(make_coord2d(0u, P_K), P_LDS_LD); // one block deeper into the slab

            GlobalA grA;
            GlobalB grB;
            auto globalRead = [&]() {
                load_matrix_coop_sync<P_WARPS>(grA, a + offA, lda, warpIndex);
                load_matrix_coop_sync<P_WARPS>(grB, b + offB, ldb, warpIndex);
                offA += stepA;
                offB += stepB;
            };
            auto ldsWrite = [&](PIn* lds) {
                store_matrix_coop_sync<P_WARPS>(lds + ldsWriteA, applyDataLayout<PLayoutLds, P_WARPS>(grA), P_LDS_LD, warpIndex);
                store_matrix_coop_sync<P_WARPS>(lds + ldsWriteB, applyDataLayout<PLayoutLds, P_WARPS>(applyTranspose(grB)),
                                                P_LDS_LD, warpIndex);
            };

            MmaAcc acc[P_BLOCKS_X][P_BLOCKS_Y];
#pragma unroll
            for(uint32_t i = 0; i < P_BLOCKS_X; ++i)
#pragma unroll
                for(uint32_t j = 0; j < P_BLOCKS_Y; ++j)
                    fill_fragment(acc[i][j], 0.0f);

            auto ldsStep = [&](PIn const* lds) {
#pragma unroll
                for(uint32_t ks = 0; ks < SLAB_K / P_K; ++ks)
                {
                    MmaA fa[P_BLOCKS_X];
                    MmaB fb[P_BLOCKS_Y];
#pragma unroll
                    for(uint32_t i = 0; i < P_BLOCKS_X; ++i)
                    {
                        LdsReadA tmp;
                        load_matrix_sync(tmp, lds + ldsReadA + i * blockStepA + ks * kStep, P_LDS_LD);
                        fa[i] = applyDataLayout<PLayoutA>(tmp);
                    }
#pragma unroll
                    for(uint32_t j = 0; j < P_BLOCKS_Y; ++j)
                    {
                        LdsReadB tmp;
                        load_matrix_sync(tmp, lds + ldsReadB + j * blockStepB + ks * kStep, P_LDS_LD);
                        fb[j] = applyDataLayout<PLayoutB>(applyTranspose(tmp));
                    }
#pragma unroll
                    for(uint32_t i = 0; i < P_BLOCKS_X; ++i)
#pragma unroll
                        for(uint32_t j = 0; j < P_BLOCKS_Y; ++j)
                            mma_sync(acc[i][j], fa[i], fb[j], acc[i][j]);
                }
            };

            // prologue: first K slab through registers into the low buffer
            globalRead();
            ldsWrite(ldsLo);
            synchronize_workgroup();

            for(uint32_t kk = SLAB_K; kk < k; kk += SLAB_K)
            {
                globalRead(); // prefetch slab kk while slab kk - SLAB_K is multiplied
                ldsStep(ldsLo);
                ldsWrite(ldsHi);
                synchronize_workgroup();
                PIn* t = ldsLo;
                ldsLo  = ldsHi;
                ldsHi  = t;
            }
            ldsStep(ldsLo);

            using MapC = GetDataLayout_t<MmaC>;
            const size_t   cBase = MapC::fromMatrixCoord(tileCoord, ldc), dBase = MapC::fromMatrixCoord(tileCoord, ldd);
#pragma unroll
            for(uint32_t i = 0; i < P_BLOCKS_X; ++i)
#pragma unroll
                for(uint32_t j = 0; j < P_BLOCKS_Y; ++j)
                {
                    MmaC fc;
                    load_matrix_sync(fc, c + cBase + MapC::fromMatrixCoord(make_coord2d(i * P_M, j * P_N), ldc), ldc);
                    for(uint32_t e = 0; e < fc.num_elements; ++e)
                        fc.x[e] = static_cast<POut>(alpha * acc[i][j].x[e] + beta * static_cast<PCmp>(fc.x[e]));
                    store_matrix_sync(d + dBase + MapC::fromMatrixCoord(make_coord2d(i * P_M, j * P_N), ldd), fc, ldd);
                }
        }
    } // namespace fragk
} // namespace b200wmma

using namespace b200wmma;

extern "C" int b200wmma_simple_hgemm(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b,
                                     const void* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                                     uint32_t ldd, float alpha, float beta, int out_type, void* stream)
{
    clear_error();
    B200_REQUIRE(a && b && c && d, B200WMMA_ERR_INVALID_ARG, "simple_hgemm: a, b, c, d must be non-null");
    B200_REQUIRE(m && n && k, B200WMMA_ERR_INVALID_ARG, "simple_hgemm: m, n, k must be non-zero");
    // same size rule as the sample's host check (samples/simple_hgemm.cpp:144-149)
    B200_REQUIRE(m % fragk::SB_M == 0 && n % fragk::SB_N == 0 && k % fragk::SB_K == 0, B200WMMA_ERR_UNSUPPORTED,
                 "simple_hgemm: m, n, k must be multiples of 16");
    B200_REQUIRE(out_type == B200WMMA_OUT_F16 || out_type == B200WMMA_OUT_F32, B200WMMA_ERR_INVALID_ARG,
                 "simple_hgemm: out_type must be 0 (f16) or 1 (f32)");
    B200_REQUIRE(lda >= k && ldb >= k && ldc >= n && ldd >= n, B200WMMA_ERR_INVALID_ARG,
                 "simple_hgemm: leading dimension too small");
    if(int e = require_sm100())
        return e;
    const dim3 block(fragk::S_TBLOCK_X, fragk::S_TBLOCK_Y);
    const dim3 grid(ceil_div(m, fragk::SB_M * fragk::S_TBLOCK_X / rocwmma::Constants::AMDGCN_WAVE_SIZE),
                    ceil_div(n, fragk::SB_N * fragk::S_TBLOCK_Y));
    auto       A = static_cast<const rocwmma::float16_t*>(a);
    auto       B = static_cast<const rocwmma::float16_t*>(b);
    if(out_type == B200WMMA_OUT_F16)
        fragk::simple_gemm_kernel<rocwmma::float16_t, rocwmma::float16_t, float><<<grid, block, 0, as_stream(stream)>>>(
            m, n, k, A, B, static_cast<const rocwmma::float16_t*>(c), static_cast<rocwmma::float16_t*>(d), lda, ldb,
            ldc, ldd, alpha, beta);
    else
        fragk::simple_gemm_kernel<rocwmma::float16_t, float, float><<<grid, block, 0, as_stream(stream)>>>(
            m, n, k, A, B, static_cast<const float*>(c), static_cast<float*>(d), lda, ldb, ldc, ldd, alpha, beta);
    B200_CHECK_CUDA(cudaGetLastError());
    return B200WMMA_OK;
}

namespace
{
    // shared by the fp32 / fp64 forms of the naive sample
    template <typename T>
    int simple_gemm_same_type(const char* who, uint32_t m, uint32_t n, uint32_t k, const T* a, const T* b, const T* c, T* d,
                              uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, T alpha, T beta, void* stream)
    {
        clear_error();
        B200_REQUIRE(a && b && c && d, B200WMMA_ERR_INVALID_ARG, "%s: a, b, c, d must be non-null", who);
        B200_REQUIRE(m && n && k, B200WMMA_ERR_INVALID_ARG, "%s: m, n, k must be non-zero", who);
        // same size rule as the samples' host check (samples/simple_sgemm.cpp:144-149)
        B200_REQUIRE(m % fragk::SB_M == 0 && n % fragk::SB_N == 0 && k % fragk::SB_K == 0, B200WMMA_ERR_UNSUPPORTED,
                     "%s: m, n, k must be multiples of 16", who);
        B200_REQUIRE(lda >= k && ldb >= k && ldc >= n && ldd >= n, B200WMMA_ERR_INVALID_ARG,
                     "%s: leading dimension too small", who);
        if(int e = require_sm100())
            return e;
        const dim3 block(fragk::S_TBLOCK_X, fragk::S_TBLOCK_Y);
        const dim3 grid(ceil_div(m, fragk::SB_M * fragk::S_TBLOCK_X / rocwmma::Constants::AMDGCN_WAVE_SIZE),
                        ceil_div(n, fragk::SB_N * fragk::S_TBLOCK_Y));
        fragk::simple_gemm_kernel<T, T, T><<<grid, block, 0, as_stream(stream)>>>(m, n, k, a, b, c, d, lda, ldb, ldc, ldd,
                                                                                 alpha, beta);
        B200_CHECK_CUDA(cudaGetLastError());
        return B200WMMA_OK;
    }
} // namespace

extern "C" int b200wmma_simple_sgemm(uint32_t m, uint32_t n, uint32_t k, const float* a, const float* b, const float* c,
                                     float* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, float alpha,
                                     float beta, void* stream)
{
    return simple_gemm_same_type<float>("simple_sgemm", m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, stream);
}

extern "C" int b200wmma_simple_dgemm(uint32_t m, uint32_t n, uint32_t k, const double* a, const double* b, const double* c,
                                     double* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, double alpha,
                                     double beta, void* stream)
{
    return simple_gemm_same_type<double>("simple_dgemm", m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, stream);
}

extern "C" int b200wmma_perf_hgemm_fragment(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b,
                                            const void* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                                            uint32_t ldd, float alpha, float beta, void* stream)
{
    clear_error();
    B200_REQUIRE(a && b && c && d, B200WMMA_ERR_INVALID_ARG, "perf_hgemm_fragment: a, b, c, d must be non-null");
    B200_REQUIRE(m && n && k, B200WMMA_ERR_INVALID_ARG, "perf_hgemm_fragment: m, n, k must be non-zero");
    // the sample's own size rule (samples/perf_hgemm.cpp:757-762): whole macro tiles, whole K steps
    B200_REQUIRE(m % fragk::P_MACRO_X == 0 && n % fragk::P_MACRO_Y == 0 && k % fragk::P_K == 0,
                 B200WMMA_ERR_UNSUPPORTED, "perf_hgemm_fragment: m, n must be multiples of 128 and k of 16");
    B200_REQUIRE(lda >= m && ldb >= n && ldc >= n && ldd >= n, B200WMMA_ERR_INVALID_ARG,
                 "perf_hgemm_fragment: leading dimension too small (A is column major, B row major)");
    if(int e = require_sm100())
        return e;
    const dim3   block(fragk::P_TBLOCK_X, fragk::P_TBLOCK_Y);
    const dim3   grid(m / fragk::P_MACRO_X, n / fragk::P_MACRO_Y);
    const int  forced = tuning::get(tuning::FRAG_PERF_SLAB_K);
    const auto launch = [&](auto slab) {
        constexpr uint32_t SLAB_K = decltype(slab)::value;
        const size_t       lds    = 2 * fragk::PSlab<SLAB_K>::LDS_ALLOC * sizeof(fragk::PIn);
        static bool        attr_ok_dev[MAX_DEVICES];
        bool&              attr_ok = attr_ok_dev[current_device_slot()];
        if(lds > 48 * 1024 && !attr_ok)
        {
            if(cudaFuncSetAttribute(fragk::perf_hgemm_fragment_kernel<SLAB_K>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(lds))
               != cudaSuccess)
                return;
            attr_ok = true;
        }
        fragk::perf_hgemm_fragment_kernel<SLAB_K><<<grid, block, lds, as_stream(stream)>>>(
            m, n, k, static_cast<const fragk::PIn*>(a), static_cast<const fragk::PIn*>(b),
            static_cast<const fragk::POut*>(c), static_cast<fragk::POut*>(d), lda, ldb, ldc, ldd, alpha, beta);
    };
    // One block deep, as in the sample, unless b200wmma_set_tuning asks for a deeper slab that divides k.  Measured at
    // 8192^3 on one B200: slabs of 16 / 32 / 64 give 81 / 49 / 48 TFLOP/s - the deeper slabs need 206 / 240 registers
    // per thread, one thread block per SM instead of two, and lose more to occupancy than they gain per barrier.
    uint32_t slab = 16u;
    if((forced == 16 || forced == 32 || forced == 64) && k % static_cast<uint32_t>(forced) == 0)
        slab = static_cast<uint32_t>(forced);
    if(slab == 64)
        launch(std::integral_constant<uint32_t, 64>{});
    else if(slab == 32)
        launch(std::integral_constant<uint32_t, 32>{});
    else
        launch(std::integral_constant<uint32_t, 16>{});
    B200_CHECK_CUDA(cudaGetLastError());
    return B200WMMA_OK;
}
