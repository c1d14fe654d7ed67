// Integer GEMM on compressed operands: 2:4 structured-sparse int8 A, and packed int4 A / B.
//
// rocWMMA v1.6.0 has no sparse or int4 path; the semantics are those of the dense int8 GEMM
// (gemm_rocwmma_d pattern, samples/perf_hgemm.cpp:515-711 with int8 inputs / int32 compute as
// in test/gemm/gemm_common_test_params.hpp:51-147) applied to the densified / sign-extended
// operands, bit-exact in int32.
//
// The sparse GEMM runs on the sparse tensor-core path (gemm_tc05_sp.cuh: compressed values and
// metadata straight into tcgen05.mma.sp) whenever k is a multiple of 128 and the rows are 16-byte
// aligned.  Otherwise the compressed operand is expanded to K-major int8 in a caller-provided device
// workspace with one streaming pass (16-byte loads and stores) and the dense tcgen05 int8 GEMM runs on
// the expanded operand.  The int4 GEMM (the sm_100 tensor cores have no 4-bit integer kind) unpacks to
// int8 inside its own kernel, between the TMA load and the MMA (gemm_tc05_i4.cuh).
#include "common.cuh"
#include "tuning.cuh"

#include <mutex>

namespace b200wmma
{
    namespace i8var
    {
        constexpr int THREADS = 256;

        // One thread expands 8 groups of a row: 16 value bytes + 4 metadata bytes -> 32 dense bytes.
        // vals row pitch ldv (bytes), meta row pitch ldm (bytes), dense row pitch k (bytes).
        __global__ void __launch_bounds__(THREADS)
            expand_sp24_kernel(const int8_t* __restrict__ vals, const uint8_t* __restrict__ meta,
                               int8_t* __restrict__ dense, uint32_t m, uint32_t k, size_t ldv,
                               size_t ldm)
        {
            const uint32_t units_per_row = k >> 5; // 32 dense elements per unit
            const size_t   total         = static_cast<size_t>(m) * units_per_row;
            for(size_t u = static_cast<size_t>(blockIdx.x) * THREADS + threadIdx.x; u < total;
                u += static_cast<size_t>(gridDim.x) * THREADS)
            {
                const uint32_t row  = static_cast<uint32_t>(u / units_per_row);
                const uint32_t unit = static_cast<uint32_t>(u - static_cast<size_t>(row) * units_per_row);
                const uint4    v = __ldcs(reinterpret_cast<const uint4*>(vals + row * ldv + unit * 16));
                const uint32_t md = __ldcs(reinterpret_cast<const uint32_t*>(meta + row * ldm + unit * 4));
                const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
                uint32_t       out[8];
#pragma unroll
                for(int gi = 0; gi < 8; ++gi)
                {
                    // group gi: values at bytes 2*gi, 2*gi+1; nibble gi of the metadata word
                    const uint32_t pair = (vw[gi >> 1] >> ((gi & 1) * 16)) & 0xFFFFu;
                    const uint32_t nib  = (md >> (4 * gi)) & 0xFu;
                    const uint32_t i0 = nib & 3u, i1 = nib >> 2;
                    out[gi] = ((pair & 0xFFu) << (8 * i0)) | ((pair >> 8) << (8 * i1));
                }
                uint4* dst = reinterpret_cast<uint4*>(dense + static_cast<size_t>(row) * k + unit * 32);
                dst[0]     = make_uint4(out[0], out[1], out[2], out[3]);
                dst[1]     = make_uint4(out[4], out[5], out[6], out[7]);
            }
        }

        static uint32_t grid_for(size_t units)
        {
            const size_t want = (units + THREADS - 1) / THREADS;
            return static_cast<uint32_t>(want < 148u * 16u ? (want ? want : 1) : 148u * 16u);
        }
        static size_t round256(size_t x)
        {
            return (x + 255) & ~static_cast<size_t>(255);
        }
        // b200wmma_set_tuning("sp24_force_expand", 1) sends every sparse GEMM through the densifying pass (comparison aid).
        static bool force_expansion()
        {
            return tuning::get(tuning::SP24_FORCE_EXPAND) != 0;
        }
    } // namespace i8var
} // namespace b200wmma

using namespace b200wmma;

extern "C" size_t b200wmma_gemm_i8_sp24_workspace_bytes(uint32_t m, uint32_t n, uint32_t k)
{
    (void)n;
    // enough for either use: the densified A (m x k) or the re-tiled metadata of the sparse tensor-core path
    const size_t dense = i8var::round256(static_cast<size_t>(m) * k), meta = i8var::round256(sp24_packed_meta_bytes(m, k));
    return dense > meta ? dense : meta;
}

extern "C" size_t b200wmma_sp24_packed_meta_bytes(uint32_t m, uint32_t k)
{
    return sp24_packed_meta_bytes(m, k);
}

extern "C" int b200wmma_sp24_repack_meta(uint32_t m, uint32_t k, const uint8_t* a_meta, uint32_t ld_meta, void* packed,
                                         size_t packed_bytes, void* stream)
{
    clear_error();
    return launch_sp24_repack_meta(m, k, a_meta, ld_meta, packed, packed_bytes, as_stream(stream));
}

extern "C" int b200wmma_gemm_i8_sp24_packed(uint32_t m, uint32_t n, uint32_t k, const int8_t* a_vals,
                                            const void* a_meta_packed, const int8_t* b, const int32_t* c, int32_t* d,
                                            uint32_t lda_vals, uint32_t ldb, uint32_t ldc, uint32_t ldd, int32_t alpha,
                                            int32_t beta, void* stream)
{
    clear_error();
    B200_REQUIRE(k % 128 == 0, B200WMMA_ERR_UNSUPPORTED, "gemm_i8_sp24_packed: k must be a multiple of 128");
    return launch_gemm_tc05_i8_sp24(m, n, k, a_vals, static_cast<const uint8_t*>(a_meta_packed), true, b, c, d, lda_vals, 0, ldb,
                                    ldc, ldd, alpha, beta, nullptr, 0, as_stream(stream));
}

extern "C" size_t b200wmma_gemm_i4_workspace_bytes(uint32_t m, uint32_t n, uint32_t k)
{
    (void)m, (void)n, (void)k;
    return 0; // the int4 GEMM unpacks inside the kernel: no scratch
}

extern "C" int b200wmma_gemm_i8_sp24(uint32_t m, uint32_t n, uint32_t k, const int8_t* a_vals,
                                     const uint8_t* a_meta, const int8_t* b, const int32_t* c,
                                     int32_t* d, uint32_t lda_vals, uint32_t ld_meta, uint32_t ldb,
                                     uint32_t ldc, uint32_t ldd, int32_t alpha, int32_t beta,
                                     void* workspace, size_t workspace_bytes, void* stream)
{
    clear_error();
    B200_REQUIRE(m && n && k, B200WMMA_ERR_INVALID_ARG, "gemm_i8_sp24: m, n, k must be non-zero");
    B200_REQUIRE(a_vals && a_meta && b && d, B200WMMA_ERR_INVALID_ARG,
                 "gemm_i8_sp24: a_vals, a_meta, b, d must be non-null");
    B200_REQUIRE(k % 32 == 0, B200WMMA_ERR_UNSUPPORTED, "gemm_i8_sp24: k must be a multiple of 32");
    B200_REQUIRE(lda_vals >= k / 2 && ld_meta >= k / 8, B200WMMA_ERR_INVALID_ARG,
                 "gemm_i8_sp24: lda_vals / ld_meta smaller than k/2 / k/8");
    // Sparse tensor-core path: compressed A goes to the tensor cores as it is, no scratch involved.
    if(!i8var::force_expansion() && sp24_direct_ok(k, a_vals, a_meta, b, lda_vals, ld_meta, ldb))
        return launch_gemm_tc05_i8_sp24(m, n, k, a_vals, a_meta, false, b, c, d, lda_vals, ld_meta, ldb, ldc, ldd, alpha, beta,
                                        workspace, workspace_bytes, as_stream(stream));
    // Otherwise (k not a multiple of 128, or rows that TMA cannot address): densify A into the
    // workspace and run the dense int8 kernel.
    B200_REQUIRE(workspace, B200WMMA_ERR_INVALID_ARG,
                 "gemm_i8_sp24: this shape / alignment needs the workspace (k %% 128 != 0 or rows not 16-byte aligned)");
    B200_REQUIRE(aligned16(a_vals) && lda_vals % 16 == 0 && (reinterpret_cast<uintptr_t>(a_meta) & 3) == 0
                     && ld_meta % 4 == 0 && aligned16(workspace),
                 B200WMMA_ERR_ALIGNMENT,
                 "gemm_i8_sp24: value rows must be 16-byte aligned, metadata rows 4-byte aligned");
    B200_REQUIRE(workspace_bytes >= b200wmma_gemm_i8_sp24_workspace_bytes(m, n, k), B200WMMA_ERR_INVALID_ARG,
                 "gemm_i8_sp24: workspace too small (%zu < %zu bytes)", workspace_bytes,
                 b200wmma_gemm_i8_sp24_workspace_bytes(m, n, k));
    if(int e = require_sm100())
        return e;
    int8_t*      dense = static_cast<int8_t*>(workspace);
    const size_t units = static_cast<size_t>(m) * (k / 32);
    i8var::expand_sp24_kernel<<<i8var::grid_for(units), i8var::THREADS, 0, as_stream(stream)>>>(
        a_vals, a_meta, dense, m, k, lda_vals, ld_meta);
    B200_CHECK_CUDA(cudaGetLastError());
    return launch_gemm_tc05_i8(m, n, k, dense, b, c, d, k, ldb, ldc, ldd, alpha, beta, B200WMMA_ROW_MAJOR,
                               B200WMMA_COL_MAJOR, B200WMMA_ROW_MAJOR, as_stream(stream));
}

extern "C" int b200wmma_gemm_i4(uint32_t m, uint32_t n, uint32_t k, const uint8_t* a_packed,
                                const uint8_t* b_packed, const int32_t* c, int32_t* d,
                                uint32_t lda_bytes, uint32_t ldb_bytes, uint32_t ldc, uint32_t ldd,
                                int32_t alpha, int32_t beta, void* workspace, size_t workspace_bytes,
                                void* stream)
{
    clear_error();
    (void)workspace, (void)workspace_bytes; // kept in the signature; the kernel unpacks in its load path and needs none
    return launch_gemm_tc05_i4(m, n, k, a_packed, b_packed, c, d, lda_bytes, ldb_bytes, ldc, ldd, alpha, beta,
                               as_stream(stream));
}

// ---------------------------------------------------------------------------------------------
// 2:4-sparse int8 GEMM for callers that have no way to hand over scratch memory.
//
// The kernel signature rocWMMA-style harnesses launch is (m, n, k, a, b, c, d, lda, ldb, ldc, ldd,
// alpha, beta): inputs, outputs and nothing else.  A harness built around that signature, or an
// application that gave all device memory to its own arena at start-up, can neither pass a
// workspace pointer nor call cudaMalloc on the library's behalf.  For those callers the expanded
// copy of A lives in a fixed array inside this library instead of in caller memory.
// ---------------------------------------------------------------------------------------------
namespace b200wmma
{
    namespace i8var
    {
        // Resident in every GPU that loads the library, from load until the process exits.
        static __device__ __align__(256) unsigned char g_sp24_static_scratch[B200WMMA_SP24_STATIC_SCRATCH_BYTES];

        // Device address of the array for the current device.  In host code the array's name is only a
        // handle for the runtime, never an address a kernel may use: it is resolved once per device,
        // with that device current, and cached.
        static int static_scratch_address(int8_t** out, cudaStream_t stream)
        {
            static int8_t*    cache[64];
            static std::mutex mu;
            int               dev = 0;
            B200_CHECK_CUDA(cudaGetDevice(&dev));
            B200_REQUIRE(dev >= 0 && dev < 64, B200WMMA_ERR_UNSUPPORTED, "device index %d out of range", dev);
            // The array of the CURRENT device is used: a stream of another device would run the kernels there with
            // this device's address.
            if(stream != nullptr)
            {
                int sdev = dev;
                if(cudaStreamGetDevice(stream, &sdev) == cudaSuccess)
                    B200_REQUIRE(sdev == dev, B200WMMA_ERR_INVALID_ARG,
                                 "gemm_i8_sp24_static: the stream belongs to device %d but device %d is current", sdev, dev);
                else
                    (void)cudaGetLastError();
            }
            std::lock_guard<std::mutex> lock(mu);
            if(!cache[dev] || !status_word_ready())
            {
                // first call on this device: the look-ups below (and the status word's, inside the GEMM launch) are
                // not stream operations and must not happen while the stream is being captured
                cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
                if(cudaStreamIsCapturing(stream, &cap) == cudaSuccess)
                    B200_REQUIRE(cap == cudaStreamCaptureStatusNone, B200WMMA_ERR_INVALID_ARG,
                                 "gemm_i8_sp24_static: the first call on a device sets the library up and cannot be part of a "
                                 "stream capture; call it once before capturing");
                else
                    (void)cudaGetLastError();
            }
            if(!cache[dev])
            {
                void* p = nullptr;
                B200_CHECK_CUDA(cudaGetSymbolAddress(&p, g_sp24_static_scratch));
                B200_REQUIRE(p != nullptr && aligned16(p), B200WMMA_ERR_CUDA,
                             "static scratch array resolved to an unusable address");
                cache[dev] = static_cast<int8_t*>(p);
            }
            *out = cache[dev];
            return B200WMMA_OK;
        }
    } // namespace i8var
} // namespace b200wmma

extern "C" int b200wmma_gemm_i8_sp24_static(uint32_t m, uint32_t n, uint32_t k, const int8_t* a_vals,
                                            const uint8_t* a_meta, const int8_t* b, const int32_t* c,
                                            int32_t* d, uint32_t lda_vals, uint32_t ld_meta, uint32_t ldb,
                                            uint32_t ldc, uint32_t ldd, int32_t alpha, int32_t beta,
                                            void* stream)
{
    clear_error();
    B200_REQUIRE(m && n && k, B200WMMA_ERR_INVALID_ARG, "gemm_i8_sp24_static: m, n, k must be non-zero");
    B200_REQUIRE(a_vals && a_meta && b && d, B200WMMA_ERR_INVALID_ARG,
                 "gemm_i8_sp24_static: a_vals, a_meta, b, d must be non-null");
    B200_REQUIRE(k % 32 == 0, B200WMMA_ERR_UNSUPPORTED, "gemm_i8_sp24_static: k must be a multiple of 32");
    B200_REQUIRE(static_cast<uint64_t>(m) * k <= B200WMMA_SP24_STATIC_SCRATCH_BYTES, B200WMMA_ERR_UNSUPPORTED,
                 "gemm_i8_sp24_static: m * k = %llu exceeds the built-in scratch of %llu bytes; "
                 "use b200wmma_gemm_i8_sp24 with a caller-provided workspace",
                 static_cast<unsigned long long>(static_cast<uint64_t>(m) * k),
                 static_cast<unsigned long long>(B200WMMA_SP24_STATIC_SCRATCH_BYTES));
    B200_REQUIRE(lda_vals >= k / 2 && ld_meta >= k / 8, B200WMMA_ERR_INVALID_ARG,
                 "gemm_i8_sp24_static: lda_vals / ld_meta smaller than k/2 / k/8");
    B200_REQUIRE(aligned16(a_vals) && lda_vals % 16 == 0 && (reinterpret_cast<uintptr_t>(a_meta) & 3) == 0
                     && ld_meta % 4 == 0,
                 B200WMMA_ERR_ALIGNMENT,
                 "gemm_i8_sp24_static: value rows must be 16-byte aligned, metadata rows 4-byte aligned");
    if(int e = require_sm100())
        return e;
    int8_t* dense = nullptr;
    if(int e = i8var::static_scratch_address(&dense, as_stream(stream)))
        return e;
    // The expansion writes all m * k bytes it later reads (zeros included), so nothing left in the array
    // by an earlier call can leak into this one and nothing needs clearing first.
    const size_t units = static_cast<size_t>(m) * (k / 32);
    i8var::expand_sp24_kernel<<<i8var::grid_for(units), i8var::THREADS, 0, as_stream(stream)>>>(
        a_vals, a_meta, dense, m, k, lda_vals, ld_meta);
    B200_CHECK_CUDA(cudaGetLastError());
    return launch_gemm_tc05_i8(m, n, k, dense, b, c, d, k, ldb, ldc, ldd, alpha, beta, B200WMMA_ROW_MAJOR,
                               B200WMMA_COL_MAJOR, B200WMMA_ROW_MAJOR, as_stream(stream));
}
