// Pieces shared by the one-CTA and the two-CTA tcgen05 GEMM kernels: operand kinds, the
// instruction descriptor, tile rasterisation, the alpha/beta epilogue on one row chunk, and the
// host-side TMA tensor-map construction.
#pragma once
#include "common.cuh"
#include "ptx_sm100.cuh"

#include <cuda_bf16.h>
#include <type_traits>

namespace b200wmma
{
    namespace tc05
    {
        constexpr uint32_t BLOCK_K_BYTES   = 128; // one 128-byte swizzle row: 64 fp16 / 128 int8
        constexpr uint64_t WAIT_TIMEOUT_NS = 2000000000ull; // 2 s: far beyond any healthy wait

        enum Kind : int
        {
            KIND_F16  = 0, // fp16 x fp16 -> fp32
            KIND_I8   = 1, // int8 x int8 -> int32
            KIND_BF16 = 2, // bf16 x bf16 -> fp32
            KIND_E4M3 = 3, // OCP fp8 e4m3 x e4m3 -> fp32
            KIND_E5M2 = 4 // OCP fp8 e5m2 x e5m2 -> fp32
        };
        // bytes per input element
        template <int KIND>
        __host__ __device__ constexpr uint32_t elem_bytes()
        {
            return (KIND == KIND_F16 || KIND == KIND_BF16) ? 2u : 1u;
        }
        enum Role : uint32_t
        {
            ROLE_PRODUCER = 1,
            ROLE_MMA      = 2,
            ROLE_EPILOGUE = 3
        };

        // tcgen05 instruction descriptor (32-bit): D format bits [4,6), A format [7,10),
        // B format [10,13), A/B major bits 15/16 (0 = K-major), N>>3 at [17,23), M>>4 at [24,29).
        template <int KIND, uint32_t MMA_M, uint32_t MMA_N, bool A_MN = false, bool B_MN = false>
        __host__ __device__ constexpr uint32_t make_idesc()
        {
            uint32_t d = 0;
            if(KIND == KIND_F16)
            {
                d |= 1u << 4; // D = F32;  A = B = F16 (format 0)
            }
            else if(KIND == KIND_BF16)
            {
                d |= 1u << 4; // D = F32
                d |= 1u << 7; // A = BF16 (format 1 of kind::f16)
                d |= 1u << 10; // B = BF16
            }
            else if(KIND == KIND_E4M3)
            {
                d |= 1u << 4; // D = F32;  A = B = E4M3 (format 0 of kind::f8f6f4)
            }
            else if(KIND == KIND_E5M2)
            {
                d |= 1u << 4; // D = F32
                d |= 1u << 7; // A = E5M2 (format 1 of kind::f8f6f4)
                d |= 1u << 10; // B = E5M2
            }
            else
            {
                d |= 2u << 4; // D = S32
                d |= 1u << 7; // A = signed 8-bit
                d |= 1u << 10; // B = signed 8-bit
            }
            d |= (A_MN ? 1u : 0u) << 15; // A major: 0 = K-major, 1 = MN-major
            d |= (B_MN ? 1u : 0u) << 16; // B major
            d |= (MMA_N >> 3) << 17;
            d |= (MMA_M >> 4) << 24;
            return d;
        }

        // Rasterisation: tiles are walked in bands of `GROUP_M` row tiles; inside a band the row index
        // varies fastest, so CTAs running at the same time share a few B column slabs and the
        // band's A rows stay hot in L2 while the band sweeps across N.
        __device__ __forceinline__ void tile_coords(uint32_t  tile,
                                                    uint32_t  tiles_m,
                                                    uint32_t  tiles_n,
                                                    uint32_t  GROUP_M,
                                                    uint32_t& m_idx,
                                                    uint32_t& n_idx)
        {
            const uint32_t group_size = GROUP_M * tiles_n;
            const uint32_t group      = tile / group_size;
            const uint32_t first_m    = group * GROUP_M;
            const uint32_t gm         = min(tiles_m - first_m, GROUP_M);
            const uint32_t within     = tile - group * group_size;
            m_idx                     = first_m + within % gm;
            n_idx                     = within / gm;
        }

        // ---- epilogue element helpers -----------------------------------------------------
        __device__ __forceinline__ float epi(float acc, float c, float alpha, float beta)
        {
            return alpha * acc + beta * c;
        }
        __device__ __forceinline__ int32_t epi(int32_t acc, int32_t c, int32_t alpha, int32_t beta)
        {
            // wrap-around int32 arithmetic, as the reference's int32 ComputeT does
            return static_cast<int32_t>(static_cast<uint32_t>(alpha) * static_cast<uint32_t>(acc)
                                        + static_cast<uint32_t>(beta) * static_cast<uint32_t>(c));
        }

        // Two 16-bit outputs in one 32-bit word: widening of a C word and rounding of a D pair, for fp16 and bf16.
        template <typename T>
        struct Pack16;
        template <>
        struct Pack16<__half>
        {
            __device__ static __forceinline__ float2 widen(uint32_t w)
            {
                return __half22float2(*reinterpret_cast<const __half2*>(&w));
            }
            __device__ static __forceinline__ uint32_t narrow(float x, float y)
            {
                const __half2 h = __floats2half2_rn(x, y);
                return *reinterpret_cast<const uint32_t*>(&h);
            }
        };
        template <>
        struct Pack16<__nv_bfloat16>
        {
            __device__ static __forceinline__ float2 widen(uint32_t w)
            {
                return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
            }
            __device__ static __forceinline__ uint32_t narrow(float x, float y)
            {
                const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
                return *reinterpret_cast<const uint32_t*>(&h);
            }
        };

        // 16- or 32-byte global accesses of VW 32-bit words.  C is read once and D written once,
        // so both use the streaming (evict-first) policy and leave L2 to the A / B slabs.
        template <int VW>
        __device__ __forceinline__ void ldg_words(const void* p, uint32_t (&w)[VW])
        {
            if constexpr(VW == 8)
                asm volatile("ld.global.cs.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                             : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]),
                               "=r"(w[7])
                             : "l"(p));
            else
                asm volatile("ld.global.cs.v4.b32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                             : "l"(p));
        }
        template <int VW>
        __device__ __forceinline__ void stg_words(void* p, const uint32_t (&w)[VW])
        {
            if constexpr(VW == 8)
                asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(w[0]), "r"(w[1]),
                             "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                             : "memory");
            else
                asm volatile("st.global.cs.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                             "r"(w[3])
                             : "memory");
        }

        // Vector path of one thread's 32 consecutive output columns: VW words per access.
        template <typename OutT, typename ScalarT, int VW>
        __device__ __forceinline__ void epilogue_row_chunk_vec(const uint32_t (&v)[32],
                                                               const OutT* __restrict__ c_row,
                                                               OutT* __restrict__ d_row, ScalarT alpha,
                                                               ScalarT beta, bool read_c)
        {
            constexpr int EPW   = 4 / sizeof(OutT); // output elements per 32-bit word
            constexpr int WORDS = 32 / EPW; // words covering 32 columns
            const uint32_t* cw_ptr = reinterpret_cast<const uint32_t*>(c_row);
            uint32_t*       dw_ptr = reinterpret_cast<uint32_t*>(d_row);
#pragma unroll
            for(int g = 0; g < WORDS / VW; ++g)
            {
                uint32_t cw[VW], ow[VW];
#pragma unroll
                for(int j = 0; j < VW; ++j)
                    cw[j] = 0u;
                if(read_c)
                    ldg_words<VW>(cw_ptr + g * VW, cw);
#pragma unroll
                for(int j = 0; j < VW; ++j)
                {
                    const int w = g * VW + j;
                    if constexpr(EPW == 2)
                    {
                        const float2 cf = Pack16<OutT>::widen(cw[j]);
                        const float  x0 = epi(__uint_as_float(v[2 * w]), cf.x, alpha, beta);
                        const float  x1 = epi(__uint_as_float(v[2 * w + 1]), cf.y, alpha, beta);
                        ow[j]           = Pack16<OutT>::narrow(x0, x1);
                    }
                    else if constexpr(std::is_same<OutT, float>::value)
                        ow[j] = __float_as_uint(epi(__uint_as_float(v[w]), __uint_as_float(cw[j]), alpha, beta));
                    else
                        ow[j] = static_cast<uint32_t>(
                            epi(static_cast<int32_t>(v[w]), static_cast<int32_t>(cw[j]), alpha, beta));
                }
                stg_words<VW>(dw_ptr + g * VW, ow);
            }
        }

        // One-byte integer outputs: the thread's 32 columns are 32 contiguous bytes of its row; with 16-byte aligned rows
        // they are read and written as two 16-byte accesses (one 32-byte access when vec == 2) instead of 32 single
        // bytes.  Each byte is the low byte of alpha * acc + beta * int32(c), as the element-wise path computes it.
        template <typename ScalarT, int VW>
        __device__ __forceinline__ void epilogue_row_chunk_bytes(const uint32_t (&v)[32], const int8_t* __restrict__ c_row,
                                                                 int8_t* __restrict__ d_row, ScalarT alpha, ScalarT beta,
                                                                 bool read_c)
        {
#pragma unroll
            for(int g = 0; g < 8 / VW; ++g)
            {
                uint32_t cw[VW], ow[VW];
#pragma unroll
                for(int j = 0; j < VW; ++j)
                    cw[j] = 0u;
                if(read_c)
                    ldg_words<VW>(reinterpret_cast<const uint32_t*>(c_row) + g * VW, cw);
#pragma unroll
                for(int j = 0; j < VW; ++j)
                {
                    uint32_t o = 0u;
#pragma unroll
                    for(int b = 0; b < 4; ++b)
                    {
                        const int32_t cv = static_cast<int8_t>((cw[j] >> (8 * b)) & 0xFFu);
                        const int32_t r  = epi(static_cast<int32_t>(v[4 * (g * VW + j) + b]), cv, alpha, beta);
                        o |= (static_cast<uint32_t>(r) & 0xFFu) << (8 * b);
                    }
                    ow[j] = o;
                }
                stg_words<VW>(reinterpret_cast<uint32_t*>(d_row) + g * VW, ow);
            }
        }

        // One thread's 32 consecutive output columns of one row.
        // OutT = __half: acc is fp32 bits.  OutT = float: fp32.  OutT = int32_t: int32.
        // vec: 0 = element-wise, 1 = 16-byte accesses, 2 = 32-byte accesses (rows aligned accordingly).
        template <typename OutT, typename ScalarT>
        __device__ __forceinline__ void epilogue_row_chunk(const uint32_t (&v)[32],
                                                           const OutT* __restrict__ c_row,
                                                           OutT* __restrict__ d_row,
                                                           uint32_t ncols, // valid columns (<= 32)
                                                           ScalarT  alpha,
                                                           ScalarT  beta,
                                                           bool     read_c,
                                                           int      vec)
        {
            if constexpr(std::is_same<OutT, int8_t>::value)
            {
                if(ncols == 32 && vec == 2)
                    return epilogue_row_chunk_bytes<ScalarT, 8>(v, c_row, d_row, alpha, beta, read_c);
                if(ncols == 32 && vec == 1)
                    return epilogue_row_chunk_bytes<ScalarT, 4>(v, c_row, d_row, alpha, beta, read_c);
            }
            if(sizeof(OutT) >= 2 && ncols == 32 && vec == 2)
                epilogue_row_chunk_vec<OutT, ScalarT, 8>(v, c_row, d_row, alpha, beta, read_c);
            else if(sizeof(OutT) >= 2 && ncols == 32 && vec == 1)
                epilogue_row_chunk_vec<OutT, ScalarT, 4>(v, c_row, d_row, alpha, beta, read_c);
            else
            {
#pragma unroll
                for(int j = 0; j < 32; ++j)
                {
                    if(static_cast<uint32_t>(j) < ncols)
                    {
                        if constexpr(std::is_integral<OutT>::value)
                        {
                            // int32 compute; a narrower output type keeps the low bits, as the reference's
                            // static_cast<OutputT> does (test/reference_impl.hpp:77-78)
                            const int32_t cvv = read_c ? static_cast<int32_t>(c_row[j]) : 0;
                            d_row[j] = static_cast<OutT>(epi(static_cast<int32_t>(v[j]), cvv, alpha, beta));
                        }
                        else
                        {
                            const float cvv = read_c ? static_cast<float>(c_row[j]) : 0.0f;
                            d_row[j]
                                = static_cast<OutT>(epi(__uint_as_float(v[j]), cvv, alpha, beta));
                        }
                    }
                }
            }
        }

        // Epilogue of one accumulator: the calling warp drains its 32-lane quadrant of a
        // 128-lane x TILE_N-column accumulator (one output row per thread, 32 columns per step),
        // applies alpha / beta and stores D.  `tmem_acc` is the accumulator's tensor-memory address
        // (lane 0, first column); row_base / col_base locate the CTA's 128 x TILE_N block in D.
        // All 32 lanes must call it together (tcgen05.ld is warp-collective).
        template <typename OutT, typename ScalarT, uint32_t TILE_N, int ACC_SHIFT = 0>
        __device__ __forceinline__ void drain_accumulator(uint32_t tmem_acc, uint32_t quad, uint32_t lane,
                                                          uint32_t row_base, uint32_t col_base, uint32_t m,
                                                          uint32_t n, const OutT* __restrict__ c,
                                                          OutT* __restrict__ d, uint32_t ldc, uint32_t ldd,
                                                          ScalarT alpha, ScalarT beta, bool read_c, int vec_ok)
        {
            const uint32_t row    = row_base + quad * 32u + lane;
            const bool     row_ok = row < m;
            const OutT*    c_row  = c + static_cast<size_t>(row) * ldc + col_base;
            OutT*          d_row  = d + static_cast<size_t>(row) * ldd + col_base;
#pragma unroll 1
            for(uint32_t ch = 0; ch < TILE_N / 32; ++ch)
            {
                uint32_t v[32];
                ptx::tmem_ld_32x32b_x32(tmem_acc + ((quad * 32u) << 16) + ch * 32u, v);
                ptx::tmem_ld_wait();
                if constexpr(ACC_SHIFT != 0) // integer accumulators of operands that carry a power-of-two scale
                {
#pragma unroll
                    for(int i = 0; i < 32; ++i)
                        v[i] = static_cast<uint32_t>(static_cast<int32_t>(v[i]) >> ACC_SHIFT);
                }
                const uint32_t col0 = col_base + ch * 32u;
                if(row_ok && col0 < n)
                {
                    const uint32_t ncols = min(32u, n - col0);
                    epilogue_row_chunk<OutT, ScalarT>(v, c_row + ch * 32u, d_row + ch * 32u, ncols, alpha, beta,
                                                      read_c, vec_ok);
                }
            }
        }

        // ---- host side ------------------------------------------------------------------
        typedef CUresult (*EncodeTiledFn)(CUtensorMap*,
                                          CUtensorMapDataType,
                                          cuuint32_t,
                                          void*,
                                          const cuuint64_t*,
                                          const cuuint64_t*,
                                          const cuuint32_t*,
                                          const cuuint32_t*,
                                          CUtensorMapInterleave,
                                          CUtensorMapSwizzle,
                                          CUtensorMapL2promotion,
                                          CUtensorMapFloatOOBfill);

        static EncodeTiledFn get_encode_fn()
        {
            static EncodeTiledFn fn = []() -> EncodeTiledFn {
                void*                           p = nullptr;
                cudaDriverEntryPointQueryResult q;
                if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q)
                       != cudaSuccess
                   || q != cudaDriverEntryPointSuccess)
                    return nullptr;
                return reinterpret_cast<EncodeTiledFn>(p);
            }();
            return fn;
        }

        // K-major operand: `rows` rows of `k_elems` contiguous elements, row pitch ld elements.
        // Box = one 128-byte K slab x box_rows rows, 128-byte swizzle, zero fill out of bounds.
        static int make_kmajor_tmap(CUtensorMap*        out,
                                    CUtensorMapDataType dtype,
                                    uint32_t            elem_bytes,
                                    const void*         ptr,
                                    uint32_t            rows,
                                    uint32_t            k_elems,
                                    uint32_t            ld,
                                    uint32_t            box_rows)
        {
            EncodeTiledFn fn = get_encode_fn();
            B200_REQUIRE(fn != nullptr, B200WMMA_ERR_CUDA, "cuTensorMapEncodeTiled not available");
            cuuint64_t gdim[2]    = {k_elems, rows};
            cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
            cuuint32_t box[2]     = {BLOCK_K_BYTES / elem_bytes, box_rows};
            cuuint32_t estr[2]    = {1, 1};
            CUresult   r          = fn(out,
                            dtype,
                            2,
                            const_cast<void*>(ptr),
                            gdim,
                            gstride,
                            box,
                            estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            B200_REQUIRE(r == CUDA_SUCCESS,
                         B200WMMA_ERR_CUDA,
                         "cuTensorMapEncodeTiled failed with CUresult %d",
                         static_cast<int>(r));
            return B200WMMA_OK;
        }

        // Byte matrix (`rows` rows of `row_bytes` bytes, pitch `pitch_bytes`) tiled in boxes of
        // box_bytes x box_rows with the given swizzle; zero fill out of bounds.
        static int make_bytes_tmap(CUtensorMap* out, const void* ptr, uint32_t rows, uint32_t row_bytes,
                                   uint64_t pitch_bytes, uint32_t box_bytes, uint32_t box_rows, CUtensorMapSwizzle swizzle)
        {
            EncodeTiledFn fn = get_encode_fn();
            B200_REQUIRE(fn != nullptr, B200WMMA_ERR_CUDA, "cuTensorMapEncodeTiled not available");
            cuuint64_t gdim[2]    = {row_bytes, rows};
            cuuint64_t gstride[1] = {pitch_bytes};
            cuuint32_t box[2]     = {box_bytes, box_rows};
            cuuint32_t estr[2]    = {1, 1};
            CUresult   r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            B200_REQUIRE(r == CUDA_SUCCESS, B200WMMA_ERR_CUDA,
                         "cuTensorMapEncodeTiled (byte matrix) failed with CUresult %d", static_cast<int>(r));
            return B200WMMA_OK;
        }

        // MN-major operand: `k_extent` rows of `mn_extent` contiguous elements, row pitch ld elements
        // (a column-major A or a row-major B).  Box = 128 bytes of MN x one K slab of rows.
        static int make_mnmajor_tmap(CUtensorMap* out, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* ptr,
                                     uint32_t mn_extent, uint32_t k_extent, uint32_t ld)
        {
            EncodeTiledFn fn = get_encode_fn();
            B200_REQUIRE(fn != nullptr, B200WMMA_ERR_CUDA, "cuTensorMapEncodeTiled not available");
            cuuint64_t gdim[2]    = {mn_extent, k_extent};
            cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
            cuuint32_t box[2]     = {128u / elem_bytes, BLOCK_K_BYTES / elem_bytes};
            cuuint32_t estr[2]    = {1, 1};
            CUresult   r          = fn(out, dtype, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            B200_REQUIRE(r == CUDA_SUCCESS, B200WMMA_ERR_CUDA,
                         "cuTensorMapEncodeTiled (MN-major operand) failed with CUresult %d", static_cast<int>(r));
            return B200WMMA_OK;
        }

        // Row-major output matrix (rows x cols, pitch ld elements) tiled in boxes of 64 bytes x 32 rows
        // with the 64-byte swizzle: the staging tiles of the TMA epilogue.
        // row_bytes: 64 (default), or 128 with the 128-byte swizzle.
        static int make_rowbox_tmap(CUtensorMap* out, uint32_t elem_bytes, const void* ptr, uint32_t rows,
                                    uint32_t cols, uint32_t ld, uint32_t row_bytes = 64)
        {
            EncodeTiledFn fn = get_encode_fn();
            B200_REQUIRE(fn != nullptr, B200WMMA_ERR_CUDA, "cuTensorMapEncodeTiled not available");
            const CUtensorMapDataType dt
                = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
            cuuint64_t gdim[2]    = {cols, rows};
            cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
            cuuint32_t box[2]     = {row_bytes / elem_bytes, 32u};
            cuuint32_t estr[2]    = {1, 1};
            CUresult   r          = fn(out, dt, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE,
                            row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            B200_REQUIRE(r == CUDA_SUCCESS, B200WMMA_ERR_CUDA,
                         "cuTensorMapEncodeTiled (output boxes) failed with CUresult %d", static_cast<int>(r));
            return B200WMMA_OK;
        }
    } // namespace tc05
} // namespace b200wmma
