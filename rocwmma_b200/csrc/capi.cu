// C ABI of rocwmma_b200: argument validation, error strings, the per-device status word,
// the dense GEMM entry points, and the host-buffer drivers that mirror the reference samples'
// host functions (allocate / copy in / launch / copy out).
#include "common.cuh"

#include <cstring>
#include <mutex>
#include <new>
#include <vector>

namespace b200wmma
{
    // {code, detail, reserved, reserved}: written by kernels whose bounded waits give up.
    __device__ unsigned g_status_word[4];

    static thread_local char tl_error[512] = "";

    int set_error(int code, const char* fmt, ...)
    {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
        va_end(ap);
        return code;
    }
    void clear_error()
    {
        tl_error[0] = '\0';
    }

    int require_sm100()
    {
        int         dev = -1;
        cudaError_t e   = cudaGetDevice(&dev);
        if(e != cudaSuccess)
            return set_error(B200WMMA_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
        static int cached_major[64];
        if(dev >= 0 && dev < 64 && cached_major[dev] == 0)
        {
            int major = 0;
            e         = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
            if(e != cudaSuccess)
                return set_error(B200WMMA_ERR_CUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
            cached_major[dev] = major;
        }
        const int major = (dev >= 0 && dev < 64) ? cached_major[dev] : 0;
        if(major != 10)
            return set_error(B200WMMA_ERR_NO_DEVICE,
                             "device %d has compute capability major %d; this library contains "
                             "sm_100a code only and has no fallback path",
                             dev, major);
        return B200WMMA_OK;
    }

    int status_word_ptr(unsigned** out)
    {
        static unsigned*  cache[64];
        static std::mutex mu;
        int               dev = 0;
        B200_CHECK_CUDA(cudaGetDevice(&dev));
        B200_REQUIRE(dev >= 0 && dev < 64, B200WMMA_ERR_UNSUPPORTED, "device index %d out of range", dev);
        std::lock_guard<std::mutex> lock(mu);
        if(!cache[dev])
        {
            void* p = nullptr;
            B200_CHECK_CUDA(cudaGetSymbolAddress(&p, g_status_word));
            B200_CHECK_CUDA(cudaMemset(p, 0, sizeof(unsigned) * 4));
            cache[dev] = static_cast<unsigned*>(p);
        }
        *out = cache[dev];
        return B200WMMA_OK;
    }

    static int check_layouts(const char* who, int la, int lb, int lcd)
    {
        B200_REQUIRE((la == 0 || la == 1) && (lb == 0 || lb == 1) && (lcd == 0 || lcd == 1),
                     B200WMMA_ERR_INVALID_ARG, "%s: layout flags must be 0 (row) or 1 (col)", who);
        return B200WMMA_OK;
    }
} // namespace b200wmma

using namespace b200wmma;

extern "C" const char* b200wmma_last_error_string(void)
{
    return tl_error;
}

extern "C" int b200wmma_version(void)
{
    return 100; // 0.1.0
}

extern "C" int b200wmma_device_status(void* stream, int* out_status, unsigned* out_detail)
{
    clear_error();
    B200_REQUIRE(out_status, B200WMMA_ERR_INVALID_ARG, "device_status: out_status must be non-null");
    unsigned* dev_ptr = nullptr;
    if(int e = status_word_ptr(&dev_ptr))
        return e;
    B200_CHECK_CUDA(cudaStreamSynchronize(as_stream(stream)));
    unsigned host[4] = {0, 0, 0, 0};
    B200_CHECK_CUDA(cudaMemcpy(host, dev_ptr, sizeof(host), cudaMemcpyDeviceToHost));
    if(host[0] != 0)
        B200_CHECK_CUDA(cudaMemset(dev_ptr, 0, sizeof(host)));
    *out_status = static_cast<int>(host[0]);
    if(out_detail)
        *out_detail = host[1];
    return B200WMMA_OK;
}

extern "C" int b200wmma_gemm_f16(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b,
                                 const void* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                                 uint32_t ldd, float alpha, float beta, int layout_a, int layout_b,
                                 int layout_cd, int out_type, void* stream)
{
    clear_error();
    if(int e = check_layouts("gemm_f16", layout_a, layout_b, layout_cd))
        return e;
    return launch_gemm_tc05_f16(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, layout_a, layout_b,
                                layout_cd, out_type, as_stream(stream));
}

extern "C" int b200wmma_gemm_bf16(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b, const float* c,
                                  float* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, float alpha,
                                  float beta, int layout_a, int layout_b, int layout_cd, void* stream)
{
    clear_error();
    if(int e = check_layouts("gemm_bf16", layout_a, layout_b, layout_cd))
        return e;
    return launch_gemm_tc05_bf16(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, layout_a, layout_b, layout_cd,
                                 as_stream(stream));
}

extern "C" int b200wmma_gemm_fp8(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b, const float* c,
                                 float* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, float alpha,
                                 float beta, int layout_a, int layout_b, int layout_cd, int fp8_format, void* stream)
{
    clear_error();
    if(int e = check_layouts("gemm_fp8", layout_a, layout_b, layout_cd))
        return e;
    return launch_gemm_tc05_fp8(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, layout_a, layout_b, layout_cd,
                                fp8_format, as_stream(stream));
}

extern "C" size_t b200wmma_gemm_f32_workspace_bytes(uint32_t m, uint32_t n, uint32_t k)
{
    return gemm_f32_workspace_bytes(m, n, k);
}

extern "C" int b200wmma_gemm_f32(uint32_t m, uint32_t n, uint32_t k, const float* a, const float* b, const float* c,
                                 float* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, float alpha, float beta,
                                 int layout_a, int layout_b, int layout_cd, void* workspace, size_t workspace_bytes,
                                 void* stream)
{
    clear_error();
    if(int e = check_layouts("gemm_f32", layout_a, layout_b, layout_cd))
        return e;
    B200_REQUIRE(layout_a == B200WMMA_ROW_MAJOR && layout_b == B200WMMA_COL_MAJOR && layout_cd == B200WMMA_ROW_MAJOR,
                 B200WMMA_ERR_UNSUPPORTED, "gemm_f32: A row-major, B column-major, C/D row-major only");
    return launch_gemm_tc05_f32(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, workspace, workspace_bytes,
                                as_stream(stream));
}

extern "C" int b200wmma_gemm_i8(uint32_t m, uint32_t n, uint32_t k, const int8_t* a, const int8_t* b,
                                const int32_t* c, int32_t* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                                uint32_t ldd, int32_t alpha, int32_t beta, int layout_a, int layout_b,
                                int layout_cd, void* stream)
{
    clear_error();
    if(int e = check_layouts("gemm_i8", layout_a, layout_b, layout_cd))
        return e;
    return launch_gemm_tc05_i8(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, layout_a, layout_b, layout_cd,
                               as_stream(stream));
}

// ---------------------------------------------------------------------------------------------
// Host-buffer drivers
// ---------------------------------------------------------------------------------------------
struct b200wmma_ctx
{
    static constexpr int NBUF = 4;
    cudaStream_t         stream    = nullptr; // compute stream (and the only one for the small drivers)
    cudaStream_t         s_in = nullptr, s_out = nullptr; // copy-in / copy-out streams of the pipelined GEMM driver
    cudaStream_t         s_bc = nullptr; // broadcasts of the multi-GPU GEMM driver (created on first use)
    std::vector<cudaEvent_t> events;      // reusable, timing disabled
    void*                buf[NBUF] = {nullptr, nullptr, nullptr, nullptr};
    size_t               cap[NBUF] = {0, 0, 0, 0};
    int                  device    = 0;
};

namespace
{
    int ctx_reserve(b200wmma_ctx* ctx, int i, size_t bytes)
    {
        if(bytes <= ctx->cap[i])
            return B200WMMA_OK;
        if(ctx->buf[i])
        {
            B200_CHECK_CUDA(cudaFree(ctx->buf[i]));
            ctx->buf[i] = nullptr;
            ctx->cap[i] = 0;
        }
        B200_CHECK_CUDA(cudaMalloc(&ctx->buf[i], bytes));
        ctx->cap[i] = bytes;
        return B200WMMA_OK;
    }
    int ctx_check(b200wmma_ctx* ctx)
    {
        B200_REQUIRE(ctx, B200WMMA_ERR_INVALID_ARG, "ctx must be non-null");
        B200_CHECK_CUDA(cudaSetDevice(ctx->device));
        return B200WMMA_OK;
    }
    // Extent in elements of a strided 2-D region: (outer - 1) * ld + inner.
    size_t extent(uint32_t outer, uint32_t inner, uint32_t ld)
    {
        return outer ? static_cast<size_t>(outer - 1) * ld + inner : 0;
    }
    int finish(b200wmma_ctx* ctx)
    {
        int      st     = 0;
        unsigned detail = 0;
        if(int e = b200wmma_device_status(ctx->stream, &st, &detail))
            return e;
        if(st != 0)
            return set_error(st, "device-side bounded wait gave up (detail 0x%08x)", detail);
        return B200WMMA_OK;
    }
}


namespace
{
    int ctx_events(b200wmma_ctx* ctx, size_t count)
    {
        while(ctx->events.size() < count)
        {
            cudaEvent_t ev = nullptr;
            B200_CHECK_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
            ctx->events.push_back(ev);
        }
        return B200WMMA_OK;
    }

    // Host-buffer GEMM as a three-stream pipeline over blocks of rows.  B is copied once; then for each
    // block of rows: copy A / C rows in (copy-in stream), multiply (compute stream), copy the D rows out
    // (copy-out stream).  Row blocks of a row-major A / C / D are contiguous, and rows of a GEMM are
    // independent, so the copies of block i+1 and of block i-1 overlap the kernel of block i and the two
    // copy directions overlap each other.  `launch(rows, a_dev, c_dev, d_dev)` enqueues one block.
    // With a multi-GPU handle (`mg`), A is the operand every rank needs whole: only rank `root` uploads it from its
    // host copy, block by block, and each block is broadcast to the other ranks over NCCL on the copy-in stream
    // (NVLink instead of one PCIe upload per rank); `a` is ignored on the other ranks.  root = -1: every rank holds A
    // on the host, and row block i is uploaded and broadcast by rank i mod nranks, so the upload is shared out as well.
    // Every rank must make the call.
    template <typename Launch>
    int gemm_host_pipeline(b200wmma_ctx* ctx, uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b,
                           const void* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                           size_t in_es, size_t out_es, bool use_c, Launch launch, b200wmma_mg* mg = nullptr, int root = 0)
    {
        const int my_rank = mg ? b200wmma_mg_rank(mg) : 0, nranks = mg ? b200wmma_mg_size(mg) : 1;
        const size_t ba = extent(m, k, lda) * in_es, bb = extent(n, k, ldb) * in_es;
        const size_t bc = extent(m, n, ldc) * out_es, bd = extent(m, n, ldd) * out_es;
        if(int e = ctx_reserve(ctx, 0, ba)) return e;
        if(int e = ctx_reserve(ctx, 1, bb)) return e;
        if(int e = ctx_reserve(ctx, 2, use_c ? bc : 16)) return e;
        if(int e = ctx_reserve(ctx, 3, bd)) return e;
        const uint32_t block_rows = 1024; // 64 pair tiles of 512 x 256 at n = 8192: one round of the GEMM kernel
        const uint32_t blocks     = (m + block_rows - 1) / block_rows;
        if(int e = ctx_events(ctx, 3 * static_cast<size_t>(blocks) + 1)) return e;
        if(mg && !ctx->s_bc)
            B200_CHECK_CUDA(cudaStreamCreateWithFlags(&ctx->s_bc, cudaStreamNonBlocking));
        char*       da = static_cast<char*>(ctx->buf[0]);
        char*       dc = static_cast<char*>(ctx->buf[2]);
        char*       dd = static_cast<char*>(ctx->buf[3]);
        const char* ha = static_cast<const char*>(a);
        const char* hc = static_cast<const char*>(c);
        char*       hd = static_cast<char*>(d);

        B200_CHECK_CUDA(cudaMemcpyAsync(ctx->buf[1], b, bb, cudaMemcpyHostToDevice, ctx->s_in));
        for(uint32_t i = 0; i < blocks; ++i)
        {
            const uint32_t r0 = i * block_rows, rows = (m - r0 < block_rows) ? m - r0 : block_rows;
            const size_t   oa = static_cast<size_t>(r0) * lda * in_es, oc = static_cast<size_t>(r0) * ldc * out_es,
                         od = static_cast<size_t>(r0) * ldd * out_es;
            const int blk_root = root >= 0 ? root : static_cast<int>(i % static_cast<uint32_t>(nranks));
            if(mg == nullptr || my_rank == blk_root)
                B200_CHECK_CUDA(cudaMemcpyAsync(da + oa, ha + oa, extent(rows, k, lda) * in_es, cudaMemcpyHostToDevice, ctx->s_in));
            if(mg)
            {
                // the broadcasts run on a stream of their own, so that this rank's later uploads do not queue behind
                // a broadcast that waits for another rank's upload
                cudaEvent_t ev_up = ctx->events[2 * static_cast<size_t>(blocks) + 1 + i];
                if(my_rank == blk_root)
                {
                    B200_CHECK_CUDA(cudaEventRecord(ev_up, ctx->s_in));
                    B200_CHECK_CUDA(cudaStreamWaitEvent(ctx->s_bc, ev_up, 0));
                }
                if(int e = b200wmma_mg_broadcast(mg, da + oa, extent(rows, k, lda) * in_es, blk_root, ctx->s_bc))
                    return e;
                B200_CHECK_CUDA(cudaEventRecord(ev_up, ctx->s_bc)); // reused: now "block i of A is on this device"
                B200_CHECK_CUDA(cudaStreamWaitEvent(ctx->stream, ev_up, 0));
            }
            if(use_c)
                B200_CHECK_CUDA(cudaMemcpyAsync(dc + oc, hc + oc, extent(rows, n, ldc) * out_es, cudaMemcpyHostToDevice, ctx->s_in));
            cudaEvent_t ev_in = ctx->events[2 * i], ev_done = ctx->events[2 * i + 1];
            B200_CHECK_CUDA(cudaEventRecord(ev_in, ctx->s_in)); // B (first block) and this block's rows are on the device
            B200_CHECK_CUDA(cudaStreamWaitEvent(ctx->stream, ev_in, 0));
            if(int e = launch(rows, da + oa, use_c ? dc + oc : nullptr, dd + od))
                return e;
            B200_CHECK_CUDA(cudaEventRecord(ev_done, ctx->stream));
            B200_CHECK_CUDA(cudaStreamWaitEvent(ctx->s_out, ev_done, 0));
            B200_CHECK_CUDA(cudaMemcpyAsync(hd + od, dd + od, extent(rows, n, ldd) * out_es, cudaMemcpyDeviceToHost, ctx->s_out));
        }
        B200_CHECK_CUDA(cudaStreamSynchronize(ctx->s_out));
        B200_CHECK_CUDA(cudaStreamSynchronize(ctx->s_in));
        if(mg)
            B200_CHECK_CUDA(cudaStreamSynchronize(ctx->s_bc));
        return finish(ctx);
    }
}

extern "C" int b200wmma_ctx_create(b200wmma_ctx** out_ctx)
{
    clear_error();
    B200_REQUIRE(out_ctx, B200WMMA_ERR_INVALID_ARG, "ctx_create: out_ctx must be non-null");
    if(int e = require_sm100())
        return e;
    b200wmma_ctx* ctx = new(std::nothrow) b200wmma_ctx();
    B200_REQUIRE(ctx, B200WMMA_ERR_CUDA, "ctx_create: out of host memory");
    cudaError_t e = cudaGetDevice(&ctx->device);
    if(e == cudaSuccess)
        e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if(e == cudaSuccess)
        e = cudaStreamCreateWithFlags(&ctx->s_in, cudaStreamNonBlocking);
    if(e == cudaSuccess)
        e = cudaStreamCreateWithFlags(&ctx->s_out, cudaStreamNonBlocking);
    if(e != cudaSuccess)
    {
        if(ctx->stream) cudaStreamDestroy(ctx->stream);
        if(ctx->s_in) cudaStreamDestroy(ctx->s_in);
        delete ctx;
        return set_error(B200WMMA_ERR_CUDA, "ctx_create: %s", cudaGetErrorString(e));
    }
    *out_ctx = ctx;
    return B200WMMA_OK;
}

extern "C" int b200wmma_ctx_destroy(b200wmma_ctx* ctx)
{
    clear_error();
    if(!ctx)
        return B200WMMA_OK;
    cudaSetDevice(ctx->device);
    for(int i = 0; i < b200wmma_ctx::NBUF; ++i)
        if(ctx->buf[i])
            cudaFree(ctx->buf[i]);
    for(cudaEvent_t ev : ctx->events)
        cudaEventDestroy(ev);
    if(ctx->stream)
        cudaStreamDestroy(ctx->stream);
    if(ctx->s_in)
        cudaStreamDestroy(ctx->s_in);
    if(ctx->s_bc)
        cudaStreamDestroy(ctx->s_bc);
    if(ctx->s_out)
        cudaStreamDestroy(ctx->s_out);
    delete ctx;
    return B200WMMA_OK;
}

extern "C" int b200wmma_gemm_f16_host(b200wmma_ctx* ctx, uint32_t m, uint32_t n, uint32_t k,
                                      const void* a, const void* b, const void* c, void* d,
                                      uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                                      float alpha, float beta, int layout_a, int layout_b,
                                      int layout_cd, int out_type)
{
    clear_error();
    if(int e = ctx_check(ctx))
        return e;
    if(int e = check_layouts("gemm_f16_host", layout_a, layout_b, layout_cd))
        return e;
    B200_REQUIRE(layout_a == B200WMMA_ROW_MAJOR && layout_b == B200WMMA_COL_MAJOR && layout_cd == B200WMMA_ROW_MAJOR,
                 B200WMMA_ERR_UNSUPPORTED,
                 "gemm_f16_host: the row-block pipeline needs A row-major, B column-major, C/D row-major");
    B200_REQUIRE(a && b && d && m && n && k, B200WMMA_ERR_INVALID_ARG, "gemm_f16_host: null pointer or zero size");
    B200_REQUIRE(out_type == 0 || out_type == 1, B200WMMA_ERR_INVALID_ARG, "gemm_f16_host: bad out_type");
    B200_REQUIRE(lda >= k && ldb >= k && ldd >= n && ldc >= n, B200WMMA_ERR_INVALID_ARG,
                 "gemm_f16_host: leading dimension too small");
    const size_t osz   = out_type == B200WMMA_OUT_F16 ? 2 : 4;
    const bool   use_c = c != nullptr && beta != 0.0f;
    B200_REQUIRE(c || beta == 0.0f, B200WMMA_ERR_INVALID_ARG, "gemm_f16_host: c may be null only when beta == 0");
    return gemm_host_pipeline(ctx, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, 2, osz, use_c,
                              [&](uint32_t rows, const void* da, const void* dc, void* dd) {
                                  return launch_gemm_tc05_f16(rows, n, k, da, ctx->buf[1], dc, dd, lda, ldb, ldc, ldd, alpha,
                                                              use_c ? beta : 0.0f, B200WMMA_ROW_MAJOR, B200WMMA_COL_MAJOR,
                                                              B200WMMA_ROW_MAJOR, out_type, ctx->stream);
                              });
}

extern "C" int b200wmma_gemm_f16_host_mg(b200wmma_ctx* ctx, b200wmma_mg* mg, int root, uint32_t m, uint32_t n, uint32_t k,
                                         const void* a, const void* b, const void* c, void* d, uint32_t lda, uint32_t ldb,
                                         uint32_t ldc, uint32_t ldd, float alpha, float beta, int out_type)
{
    clear_error();
    if(int e = ctx_check(ctx))
        return e;
    B200_REQUIRE(mg, B200WMMA_ERR_INVALID_ARG, "gemm_f16_host_mg: mg must be a live handle");
    B200_REQUIRE(root >= -1 && root < b200wmma_mg_size(mg), B200WMMA_ERR_INVALID_ARG, "gemm_f16_host_mg: bad root %d", root);
    const bool needs_a = root < 0 || b200wmma_mg_rank(mg) == root;
    B200_REQUIRE((a || !needs_a) && b && d && m && n && k, B200WMMA_ERR_INVALID_ARG,
                 "gemm_f16_host_mg: null pointer or zero size");
    B200_REQUIRE(out_type == 0 || out_type == 1, B200WMMA_ERR_INVALID_ARG, "gemm_f16_host_mg: bad out_type");
    B200_REQUIRE(lda >= k && ldb >= k && ldd >= n && ldc >= n, B200WMMA_ERR_INVALID_ARG,
                 "gemm_f16_host_mg: leading dimension too small");
    const size_t osz   = out_type == B200WMMA_OUT_F16 ? 2 : 4;
    const bool   use_c = c != nullptr && beta != 0.0f;
    B200_REQUIRE(c || beta == 0.0f, B200WMMA_ERR_INVALID_ARG, "gemm_f16_host_mg: c may be null only when beta == 0");
    return gemm_host_pipeline(
        ctx, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, 2, osz, use_c,
        [&](uint32_t rows, const void* da, const void* dc, void* dd) {
            return launch_gemm_tc05_f16(rows, n, k, da, ctx->buf[1], dc, dd, lda, ldb, ldc, ldd, alpha, use_c ? beta : 0.0f,
                                        B200WMMA_ROW_MAJOR, B200WMMA_COL_MAJOR, B200WMMA_ROW_MAJOR, out_type, ctx->stream);
        },
        mg, root);
}

extern "C" int b200wmma_gemm_i8_host(b200wmma_ctx* ctx, uint32_t m, uint32_t n, uint32_t k,
                                     const int8_t* a, const int8_t* b, const int32_t* c, int32_t* d,
                                     uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                                     int32_t alpha, int32_t beta, int layout_a, int layout_b,
                                     int layout_cd)
{
    clear_error();
    if(int e = ctx_check(ctx))
        return e;
    if(int e = check_layouts("gemm_i8_host", layout_a, layout_b, layout_cd))
        return e;
    B200_REQUIRE(layout_a == B200WMMA_ROW_MAJOR && layout_b == B200WMMA_COL_MAJOR && layout_cd == B200WMMA_ROW_MAJOR,
                 B200WMMA_ERR_UNSUPPORTED,
                 "gemm_i8_host: the row-block pipeline needs A row-major, B column-major, C/D row-major");
    B200_REQUIRE(a && b && d && m && n && k, B200WMMA_ERR_INVALID_ARG, "gemm_i8_host: null pointer or zero size");
    B200_REQUIRE(lda >= k && ldb >= k && ldd >= n && ldc >= n, B200WMMA_ERR_INVALID_ARG,
                 "gemm_i8_host: leading dimension too small");
    const bool use_c = c != nullptr && beta != 0;
    B200_REQUIRE(c || beta == 0, B200WMMA_ERR_INVALID_ARG, "gemm_i8_host: c may be null only when beta == 0");
    return gemm_host_pipeline(ctx, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, 1, 4, use_c,
                              [&](uint32_t rows, const void* da, const void* dc, void* dd) {
                                  return launch_gemm_tc05_i8(rows, n, k, static_cast<const int8_t*>(da),
                                                             static_cast<const int8_t*>(ctx->buf[1]),
                                                             static_cast<const int32_t*>(dc), static_cast<int32_t*>(dd), lda,
                                                             ldb, ldc, ldd, alpha, use_c ? beta : 0, B200WMMA_ROW_MAJOR,
                                                             B200WMMA_COL_MAJOR, B200WMMA_ROW_MAJOR, ctx->stream);
                              });
}

extern "C" int b200wmma_gemm_i8_host_mg(b200wmma_ctx* ctx, b200wmma_mg* mg, int root, uint32_t m, uint32_t n, uint32_t k,
                                        const int8_t* a, const int8_t* b, const int32_t* c, int32_t* d, uint32_t lda,
                                        uint32_t ldb, uint32_t ldc, uint32_t ldd, int32_t alpha, int32_t beta)
{
    clear_error();
    if(int e = ctx_check(ctx))
        return e;
    B200_REQUIRE(mg, B200WMMA_ERR_INVALID_ARG, "gemm_i8_host_mg: mg must be a live handle");
    B200_REQUIRE(root >= -1 && root < b200wmma_mg_size(mg), B200WMMA_ERR_INVALID_ARG, "gemm_i8_host_mg: bad root %d", root);
    const bool needs_a = root < 0 || b200wmma_mg_rank(mg) == root;
    B200_REQUIRE((a || !needs_a) && b && d && m && n && k, B200WMMA_ERR_INVALID_ARG,
                 "gemm_i8_host_mg: null pointer or zero size");
    B200_REQUIRE(lda >= k && ldb >= k && ldd >= n && ldc >= n, B200WMMA_ERR_INVALID_ARG,
                 "gemm_i8_host_mg: leading dimension too small");
    const bool use_c = c != nullptr && beta != 0;
    B200_REQUIRE(c || beta == 0, B200WMMA_ERR_INVALID_ARG, "gemm_i8_host_mg: c may be null only when beta == 0");
    return gemm_host_pipeline(
        ctx, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, 1, 4, use_c,
        [&](uint32_t rows, const void* da, const void* dc, void* dd) {
            return launch_gemm_tc05_i8(rows, n, k, static_cast<const int8_t*>(da), static_cast<const int8_t*>(ctx->buf[1]),
                                       static_cast<const int32_t*>(dc), static_cast<int32_t*>(dd), lda, ldb, ldc, ldd, alpha,
                                       use_c ? beta : 0, B200WMMA_ROW_MAJOR, B200WMMA_COL_MAJOR, B200WMMA_ROW_MAJOR,
                                       ctx->stream);
        },
        mg, root);
}

extern "C" int b200wmma_dlrm_fwd_host(b200wmma_ctx* ctx, const void* input, void* output, uint32_t m,
                                      uint32_t m_stride, uint32_t k, uint32_t batch, uint32_t out_stride)
{
    clear_error();
    if(int e = ctx_check(ctx))
        return e;
    B200_REQUIRE(input && output && m && k && batch && m_stride >= m, B200WMMA_ERR_INVALID_ARG,
                 "dlrm_fwd_host: null pointer or bad size");
    const size_t bi = static_cast<size_t>(batch) * m_stride * k * 2;
    const size_t bo = static_cast<size_t>(batch) * out_stride * 2;
    if(int e = ctx_reserve(ctx, 0, bi)) return e;
    if(int e = ctx_reserve(ctx, 3, bo)) return e;
    B200_CHECK_CUDA(cudaMemcpyAsync(ctx->buf[0], input, bi, cudaMemcpyHostToDevice, ctx->stream));
    if(int e = b200wmma_dlrm_fwd(ctx->buf[0], ctx->buf[3], m, m_stride, k, batch, out_stride, ctx->stream))
        return e;
    B200_CHECK_CUDA(cudaMemcpyAsync(output, ctx->buf[3], bo, cudaMemcpyDeviceToHost, ctx->stream));
    return finish(ctx);
}

extern "C" int b200wmma_dlrm_bwd_host(b200wmma_ctx* ctx, const void* input, const void* upstream,
                                      void* grad, void* bottom_mlp_grad, uint32_t m, uint32_t m_stride,
                                      uint32_t k, uint32_t batch, uint32_t upstream_stride,
                                      int fuse_mlp_into_row0)
{
    clear_error();
    if(int e = ctx_check(ctx))
        return e;
    B200_REQUIRE(input && upstream && grad && m && k && batch && m_stride >= m, B200WMMA_ERR_INVALID_ARG,
                 "dlrm_bwd_host: null pointer or bad size");
    const size_t bi = static_cast<size_t>(batch) * m_stride * k * 2;
    const size_t bu = static_cast<size_t>(batch) * upstream_stride * 2;
    const size_t bm = static_cast<size_t>(batch) * k * 2;
    if(int e = ctx_reserve(ctx, 0, bi)) return e;
    if(int e = ctx_reserve(ctx, 1, bu)) return e;
    if(int e = ctx_reserve(ctx, 2, bm)) return e;
    if(int e = ctx_reserve(ctx, 3, bi)) return e;
    B200_CHECK_CUDA(cudaMemcpyAsync(ctx->buf[0], input, bi, cudaMemcpyHostToDevice, ctx->stream));
    B200_CHECK_CUDA(cudaMemcpyAsync(ctx->buf[1], upstream, bu, cudaMemcpyHostToDevice, ctx->stream));
    // rows m..m_stride-1 of grad are not written by the kernel: keep what the host passed in
    if(m_stride != m)
        B200_CHECK_CUDA(cudaMemcpyAsync(ctx->buf[3], grad, bi, cudaMemcpyHostToDevice, ctx->stream));
    if(int e = b200wmma_dlrm_bwd(ctx->buf[0], ctx->buf[1], ctx->buf[3], bottom_mlp_grad ? ctx->buf[2] : nullptr,
                                 m, m_stride, k, batch, upstream_stride, fuse_mlp_into_row0, ctx->stream))
        return e;
    B200_CHECK_CUDA(cudaMemcpyAsync(grad, ctx->buf[3], bi, cudaMemcpyDeviceToHost, ctx->stream));
    if(bottom_mlp_grad)
        B200_CHECK_CUDA(cudaMemcpyAsync(bottom_mlp_grad, ctx->buf[2], bm, cudaMemcpyDeviceToHost, ctx->stream));
    return finish(ctx);
}

template <typename T, typename Fn>
static int gemv_host(b200wmma_ctx* ctx, uint32_t m, uint32_t n, const T* a, uint32_t lda, int layout_a,
                     const T* x, T* y, T alpha, T beta, Fn launch)
{
    if(int e = ctx_check(ctx))
        return e;
    B200_REQUIRE(a && x && y && m && n, B200WMMA_ERR_INVALID_ARG, "gemv_host: null pointer or zero size");
    B200_REQUIRE(layout_a == 0 || layout_a == 1, B200WMMA_ERR_INVALID_ARG, "gemv_host: bad layout");
    B200_REQUIRE(lda >= (layout_a == 0 ? n : m), B200WMMA_ERR_INVALID_ARG, "gemv_host: lda too small");
    const size_t ba = (layout_a == 0 ? extent(m, n, lda) : extent(n, m, lda)) * sizeof(T);
    if(int e = ctx_reserve(ctx, 0, ba)) return e;
    if(int e = ctx_reserve(ctx, 1, n * sizeof(T))) return e;
    if(int e = ctx_reserve(ctx, 3, m * sizeof(T))) return e;
    B200_CHECK_CUDA(cudaMemcpyAsync(ctx->buf[0], a, ba, cudaMemcpyHostToDevice, ctx->stream));
    B200_CHECK_CUDA(cudaMemcpyAsync(ctx->buf[1], x, n * sizeof(T), cudaMemcpyHostToDevice, ctx->stream));
    B200_CHECK_CUDA(cudaMemcpyAsync(ctx->buf[3], y, m * sizeof(T), cudaMemcpyHostToDevice, ctx->stream));
    if(int e = launch(m, n, static_cast<const T*>(ctx->buf[0]), lda, layout_a,
                      static_cast<const T*>(ctx->buf[1]), static_cast<T*>(ctx->buf[3]), alpha, beta,
                      ctx->stream))
        return e;
    B200_CHECK_CUDA(cudaMemcpyAsync(y, ctx->buf[3], m * sizeof(T), cudaMemcpyDeviceToHost, ctx->stream));
    return finish(ctx);
}

extern "C" int b200wmma_gemv_f32_host(b200wmma_ctx* ctx, uint32_t m, uint32_t n, const float* a,
                                      uint32_t lda, int layout_a, const float* x, float* y, float alpha,
                                      float beta)
{
    clear_error();
    return gemv_host<float>(ctx, m, n, a, lda, layout_a, x, y, alpha, beta, b200wmma_gemv_f32);
}

extern "C" int b200wmma_gemv_f64_host(b200wmma_ctx* ctx, uint32_t m, uint32_t n, const double* a,
                                      uint32_t lda, int layout_a, const double* x, double* y,
                                      double alpha, double beta)
{
    clear_error();
    return gemv_host<double>(ctx, m, n, a, lda, layout_a, x, y, alpha, beta, b200wmma_gemv_f64);
}
