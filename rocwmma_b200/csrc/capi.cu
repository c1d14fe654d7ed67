// C ABI of rocwmma_b200: argument validation, error strings, the per-device status word,
// the dense GEMM entry points, and the host-buffer drivers that mirror the reference samples'
// host functions (allocate / copy in / launch / copy out).
#include "common.cuh"
#include "tuning.cuh"

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
        static int        cached_major[64];
        static std::mutex mu;
        int               major = 0;
        {
            std::lock_guard<std::mutex> lock(mu);
            if(dev >= 0 && dev < 64 && cached_major[dev] == 0)
            {
                int v = 0;
                e     = cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, dev);
                if(e != cudaSuccess)
                    return set_error(B200WMMA_ERR_CUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
                cached_major[dev] = v;
            }
            major = (dev >= 0 && dev < 64) ? cached_major[dev] : 0;
        }
        if(major != 10)
            return set_error(B200WMMA_ERR_NO_DEVICE,
                             "device %d has compute capability major %d; this library contains "
                             "sm_100a code only and has no fallback path",
                             dev, major);
        return B200WMMA_OK;
    }

    static unsigned*  g_status_cache[64];
    static std::mutex g_status_mu;

    bool status_word_ready()
    {
        int dev = 0;
        if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
            return false;
        std::lock_guard<std::mutex> lock(g_status_mu);
        return g_status_cache[dev] != nullptr;
    }

    int status_word_ptr(unsigned** out)
    {
        unsigned**  cache = g_status_cache;
        std::mutex& mu    = g_status_mu;
        int         dev   = 0;
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

    namespace tuning
    {
        static std::atomic<int> g_values[NUM_KEYS];
        int get(Key k)
        {
            return g_values[k].load(std::memory_order_relaxed);
        }
        void set(Key k, int value)
        {
            g_values[k].store(value, std::memory_order_relaxed);
        }
    } // namespace tuning

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

extern "C" int b200wmma_set_tuning(const char* key, int value)
{
    clear_error();
    B200_REQUIRE(key, B200WMMA_ERR_INVALID_ARG, "set_tuning: key must be non-null");
    static const struct
    {
        const char*  name;
        tuning::Key  key;
        int          lo, hi;
    } table[] = {{"gemm_tile_variant", tuning::GEMM_TILE_VARIANT, 0, 3},
                 {"gemm_group_m", tuning::GEMM_GROUP_M, 0, 1024},
                 {"sp24_force_expand", tuning::SP24_FORCE_EXPAND, 0, 1},
                 {"gemm_mma_order", tuning::GEMM_MMA_ORDER, 0, 2},
                 {"gemm_split_tail", tuning::GEMM_SPLIT_TAIL, 0, 2},
                 {"gemm_split_fixup", tuning::GEMM_SPLIT_FIXUP, 0, 4096},
                 {"dlrm_bwd_stages", tuning::DLRM_BWD_STAGES, 0, 3},
                 {"dlrm_bwd_warps", tuning::DLRM_BWD_WARPS, 0, 12},
                 {"dlrm_fwd_stages", tuning::DLRM_FWD_STAGES, 0, 3},
                 {"dlrm_fwd_warps", tuning::DLRM_FWD_WARPS, 0, 12},
                 {"gemm_f64_kernel", tuning::GEMM_F64_KERNEL, 0, 2},
                 {"frag_perf_slab_k", tuning::FRAG_PERF_SLAB_K, 0, 64},
                 {"gemv_rows", tuning::GEMV_ROWS, 0, 4},
                 {"gemv_col_vn", tuning::GEMV_COL_VN, 0, 4}};
    for(const auto& t : table)
        if(std::strcmp(key, t.name) == 0)
        {
            B200_REQUIRE(value >= t.lo && value <= t.hi, B200WMMA_ERR_INVALID_ARG, "set_tuning: %s takes %d..%d, got %d", key,
                         t.lo, t.hi, value);
            tuning::set(t.key, value);
            return B200WMMA_OK;
        }
    return set_error(B200WMMA_ERR_INVALID_ARG, "set_tuning: unknown key '%s'", key);
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

extern "C" size_t b200wmma_gemm_split_workspace_bytes(void)
{
    return gemm_split_workspace_bytes();
}

extern "C" int b200wmma_gemm_f16_ws(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b, const void* c, void* d,
                                    uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, float alpha, float beta,
                                    int layout_a, int layout_b, int layout_cd, int out_type, void* workspace,
                                    size_t workspace_bytes, void* stream)
{
    clear_error();
    if(int e = check_layouts("gemm_f16_ws", layout_a, layout_b, layout_cd))
        return e;
    return launch_gemm_tc05_f16(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, layout_a, layout_b, layout_cd, out_type,
                                as_stream(stream), workspace, workspace_bytes);
}

extern "C" int b200wmma_gemm_i8_ws(uint32_t m, uint32_t n, uint32_t k, const int8_t* a, const int8_t* b, const int32_t* c,
                                   int32_t* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, int32_t alpha,
                                   int32_t beta, int layout_a, int layout_b, int layout_cd, void* workspace,
                                   size_t workspace_bytes, void* stream)
{
    clear_error();
    if(int e = check_layouts("gemm_i8_ws", layout_a, layout_b, layout_cd))
        return e;
    return launch_gemm_tc05_i8(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, layout_a, layout_b, layout_cd,
                               as_stream(stream), workspace, workspace_bytes);
}

extern "C" int b200wmma_gemm_bf16(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b, const float* c,
                                  float* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, float alpha,
                                  float beta, int layout_a, int layout_b, int layout_cd, void* stream)
{
    clear_error();
    if(int e = check_layouts("gemm_bf16", layout_a, layout_b, layout_cd))
        return e;
    return launch_gemm_tc05_bf16(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, layout_a, layout_b, layout_cd,
                                 B200WMMA_OUT_F32, as_stream(stream));
}

extern "C" int b200wmma_gemm_bf16_out(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b, const void* c, void* d,
                                      uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, float alpha, float beta,
                                      int layout_a, int layout_b, int layout_cd, int out_type, void* stream)
{
    clear_error();
    if(int e = check_layouts("gemm_bf16_out", layout_a, layout_b, layout_cd))
        return e;
    return launch_gemm_tc05_bf16(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, layout_a, layout_b, layout_cd, out_type,
                                 as_stream(stream));
}

extern "C" int b200wmma_gemm_i8_i8(uint32_t m, uint32_t n, uint32_t k, const int8_t* a, const int8_t* b, const int8_t* c,
                                   int8_t* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, int32_t alpha,
                                   int32_t beta, int layout_a, int layout_b, int layout_cd, void* stream)
{
    clear_error();
    if(int e = check_layouts("gemm_i8_i8", layout_a, layout_b, layout_cd))
        return e;
    return launch_gemm_tc05_i8_i8(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, layout_a, layout_b, layout_cd,
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
    const bool a_mn = layout_a == B200WMMA_COL_MAJOR, b_mn = layout_b == B200WMMA_ROW_MAJOR;
    if(layout_cd == B200WMMA_ROW_MAJOR)
        return launch_gemm_tc05_f32(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, workspace, workspace_bytes,
                                    as_stream(stream), a_mn, b_mn);
    // column-major C / D: the transposed problem D^T = alpha * B^T A^T + beta * C^T (B^T is K-contiguous exactly when B was)
    return launch_gemm_tc05_f32(n, m, k, b, a, c, d, ldb, lda, ldc, ldd, alpha, beta, workspace, workspace_bytes,
                                as_stream(stream), b_mn, a_mn);
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
// A failed call inside a host driver, after copies from / to the caller's buffers may already be queued: drain the
// stream first, so that nothing of the call is still in flight when the error is returned.
#define HOST_CHECK_CUDA(ctx, expr)                                                                          \
    do                                                                                                      \
    {                                                                                                       \
        cudaError_t _e = (expr);                                                                            \
        if(_e != cudaSuccess)                                                                               \
        {                                                                                                   \
            cudaStreamSynchronize((ctx)->stream);                                                           \
            return ::b200wmma::set_error(B200WMMA_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                 \
                                         cudaGetErrorString(_e), __FILE__, __LINE__);                       \
        }                                                                                                   \
    } while(0)

struct b200wmma_ctx
{
    static constexpr int NBUF = 5; // A, B, C, D, split-K scratch of the GEMM kernel
    cudaStream_t         stream    = nullptr; // compute stream (and the only one for the small drivers)
    cudaStream_t         s_in = nullptr, s_out = nullptr; // copy-in / copy-out streams of the pipelined GEMM driver
    cudaStream_t         s_bc = nullptr; // broadcasts of the multi-GPU GEMM driver (created on first use)
    std::vector<cudaEvent_t> events;      // reusable
    void*                buf[NBUF] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    size_t               cap[NBUF] = {0, 0, 0, 0, 0};
    int                  device    = 0;
    float                stage_ms[5] = {0, 0, 0, 0, 0}; // upload span, exchange, compute, copy-out, total of the last GEMM host call
    bool                 stage_valid = false;
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
            B200_CHECK_CUDA(cudaEventCreate(&ev)); // timing enabled: the drivers report per-stage times from them
            ctx->events.push_back(ev);
        }
        return B200WMMA_OK;
    }

    // Host-buffer GEMM as a pipeline over chunks of rows on three (multi-GPU: four) streams.  B is copied once; then
    // for each chunk of rows: copy A / C rows in (copy-in stream), multiply (compute stream), copy the D rows out
    // (copy-out stream).  Row chunks of a row-major A / C / D are contiguous, and rows of a GEMM are independent, so the
    // copies of chunk i+1 and of chunk i-1 overlap the kernel of chunk i and the two copy directions overlap each other.
    // `launch(rows, a_dev, c_dev, d_dev)` enqueues one chunk.
    //
    // With a multi-GPU handle (`mg`), A is the operand every rank needs whole.
    //   root = -1: every rank holds A on the host.  The rows are cut into a few chunks; of each chunk every rank uploads
    //     one equal slice (1 / nranks of the rows) and one all-gather per chunk, on a stream of its own, assembles the
    //     chunk on every GPU over NVLink: a rank moves A / nranks over PCIe, and the first multiply starts after the
    //     first chunk instead of after all of A.
    //   root >= 0: only rank `root` reads its host copy, chunk by chunk, and broadcasts each chunk; `a` is ignored on
    //     the other ranks.
    // Every rank must make the call with the same m, k, lda and root.
    //
    // Everything that can be rejected is checked before the first copy is queued.  If a CUDA or NCCL call fails after
    // that, the streams are drained before the error is returned, so no copy is still reading or writing the caller's
    // host buffers when the call returns; in the multi-GPU form the other ranks may then be left waiting inside a
    // collective, and every rank has to destroy the handle (b200wmma_mg_destroy) to recover.
    template <typename Launch>
    int gemm_host_pipeline(b200wmma_ctx* ctx, uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b,
                           const void* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                           size_t in_es, size_t out_es, bool use_c, Launch launch, b200wmma_mg* mg = nullptr, int root = 0,
                           uint32_t b_outer = 0, uint32_t b_inner = 0)
    {
        // b_outer x b_inner: the stored shape of B when it is not the column-major n x k (a row-major B is k x n)
        if(b_outer == 0)
            b_outer = n, b_inner = k;
        const int my_rank = mg ? b200wmma_mg_rank(mg) : 0, nranks = mg ? b200wmma_mg_size(mg) : 1;
        // ---- checks that precede any queued work (the kernels' own launch checks repeat some of these) ----
        B200_REQUIRE((static_cast<uint64_t>(lda) * in_es) % 16 == 0 && (static_cast<uint64_t>(ldb) * in_es) % 16 == 0,
                     B200WMMA_ERR_ALIGNMENT,
                     "gemm host driver: the row pitches of A and B must be multiples of 16 bytes (TMA requirement)");
        if(mg)
            B200_REQUIRE(mg_device(mg) == ctx->device, B200WMMA_ERR_INVALID_ARG,
                         "gemm host driver: the context was created on device %d, the multi-GPU handle on device %d",
                         ctx->device, mg_device(mg));
        if(int e = require_sm100())
            return e;

        // ---- row chunks ----
        // single GPU: 1024 rows (64 pair tiles of 512 x 256 at n = 8192: one round of the GEMM kernel).
        // multi GPU : up to 4 chunks, each nranks equal slices of whole rows (a multiple of 128 rows per slice).
        uint32_t chunk_rows = 1024, slice_rows = 0;
        if(mg && nranks > 1)
        {
            uint32_t nchunk = m / (static_cast<uint32_t>(nranks) * 256u);
            nchunk          = nchunk < 1 ? 1 : (nchunk > 4 ? 4 : nchunk);
            slice_rows      = (m + nchunk * nranks - 1) / (nchunk * nranks);
            slice_rows      = (slice_rows + 127u) & ~127u;
            chunk_rows      = slice_rows * static_cast<uint32_t>(nranks);
        }
        // chunk i covers rows [bounds[i], bounds[i + 1]).  Single GPU: the call ends with the multiply and the copy-out of
        // the LAST chunk, which nothing overlaps (the uploads are over by then), so the last 1024 rows go as 512 + 256 +
        // 256: the tail after the last upload shrinks from a 16 MiB copy-out to a 4 MiB one.
        std::vector<uint32_t> bounds;
        for(uint32_t r = 0; r < m; r += chunk_rows)
            bounds.push_back(r);
        if(!(mg && nranks > 1) && bounds.size() >= 2 && m - bounds.back() >= 512)
        {
            const uint32_t last = bounds.back(), span = m - last;
            const uint32_t half = (span / 2 + 127u) & ~127u, quarter = ((span - half) / 2 + 127u) & ~127u;
            bounds.push_back(last + half);
            if(quarter != 0 && last + half + quarter < m)
                bounds.push_back(last + half + quarter);
        }
        bounds.push_back(m);
        const uint32_t chunks = static_cast<uint32_t>(bounds.size()) - 1u;
        const uint32_t padded_rows = ((m + chunk_rows - 1) / chunk_rows) * chunk_rows; // multi GPU: whole chunks
        // A on the device is sized in whole chunks: the last all-gather may move (never-read) rows past m
        const size_t ba = mg && nranks > 1 ? static_cast<size_t>(padded_rows) * lda * in_es : extent(m, k, lda) * in_es;
        const size_t bb = extent(b_outer, b_inner, ldb) * in_es;
        const size_t bc = extent(m, n, ldc) * out_es, bd = extent(m, n, ldd) * out_es;
        if(int e = ctx_reserve(ctx, 0, ba)) return e;
        if(int e = ctx_reserve(ctx, 1, bb)) return e;
        if(int e = ctx_reserve(ctx, 2, use_c ? bc : 16)) return e;
        if(int e = ctx_reserve(ctx, 3, bd)) return e;
        if(int e = ctx_reserve(ctx, 4, gemm_split_workspace_bytes())) return e;
        // events per chunk: A in, exchange begin, exchange end, C in, compute begin, compute end, copy-out end; +3 overall
        constexpr size_t PER = 7;
        if(int e = ctx_events(ctx, PER * static_cast<size_t>(chunks) + 3)) return e;
        if(mg && !ctx->s_bc)
            B200_CHECK_CUDA(cudaStreamCreateWithFlags(&ctx->s_bc, cudaStreamNonBlocking));
        char*       da = static_cast<char*>(ctx->buf[0]);
        char*       dc = static_cast<char*>(ctx->buf[2]);
        char*       dd = static_cast<char*>(ctx->buf[3]);
        const char* ha = static_cast<const char*>(a);
        const char* hc = static_cast<const char*>(c);
        char*       hd = static_cast<char*>(d);
        cudaEvent_t ev_start = ctx->events[PER * chunks], ev_b = ctx->events[PER * chunks + 1],
                    ev_in_end = ctx->events[PER * chunks + 2];
        ctx->stage_valid = false;

        int         rc   = B200WMMA_OK;
        cudaError_t cerr = cudaSuccess;
#define PIPE_CUDA(expr)                                                                                     \
    do                                                                                                      \
    {                                                                                                       \
        cerr = (expr);                                                                                      \
        if(cerr != cudaSuccess)                                                                             \
        {                                                                                                   \
            rc = set_error(B200WMMA_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(cerr),     \
                           __FILE__, __LINE__);                                                             \
            goto drain;                                                                                     \
        }                                                                                                   \
    } while(0)

        PIPE_CUDA(cudaEventRecord(ev_start, ctx->s_in));
        for(uint32_t i = 0; i < chunks; ++i)
        {
            const uint32_t r0 = bounds[i], rows = bounds[i + 1] - bounds[i];
            const size_t   oa = static_cast<size_t>(r0) * lda * in_es, oc = static_cast<size_t>(r0) * ldc * out_es,
                         od = static_cast<size_t>(r0) * ldd * out_es;
            cudaEvent_t* ev = &ctx->events[PER * i]; // [0] A in, [1] exch begin, [2] exch end, [3] C in, [4] / [5] compute, [6] out
            // ---- A rows of the chunk: the whole chunk (single GPU / the root), or this rank's slice of it ----
            if(!mg || nranks == 1)
                PIPE_CUDA(cudaMemcpyAsync(da + oa, ha + oa, extent(rows, k, lda) * in_es, cudaMemcpyHostToDevice, ctx->s_in));
            else if(root >= 0)
            {
                if(my_rank == root)
                    PIPE_CUDA(cudaMemcpyAsync(da + oa, ha + oa, extent(rows, k, lda) * in_es, cudaMemcpyHostToDevice, ctx->s_in));
            }
            else
            {
                const uint32_t s0 = r0 + static_cast<uint32_t>(my_rank) * slice_rows; // first row of this rank's slice
                if(s0 < m)
                {
                    const uint32_t srows = (m - s0 < slice_rows) ? m - s0 : slice_rows;
                    const size_t   os    = static_cast<size_t>(s0) * lda * in_es;
                    PIPE_CUDA(cudaMemcpyAsync(da + os, ha + os, extent(srows, k, lda) * in_es, cudaMemcpyHostToDevice, ctx->s_in));
                }
            }
            PIPE_CUDA(cudaEventRecord(ev[0], ctx->s_in));
            if(i == 0)
            {
                PIPE_CUDA(cudaMemcpyAsync(ctx->buf[1], b, bb, cudaMemcpyHostToDevice, ctx->s_in));
                PIPE_CUDA(cudaEventRecord(ev_b, ctx->s_in));
                PIPE_CUDA(cudaStreamWaitEvent(ctx->stream, ev_b, 0));
            }
            // ---- exchange: the chunk reaches every rank over NVLink, on a stream of its own so that this rank's later
            //      uploads do not queue behind a collective that waits for another rank ----
            if(mg && nranks > 1)
            {
                PIPE_CUDA(cudaStreamWaitEvent(ctx->s_bc, ev[0], 0));
                PIPE_CUDA(cudaEventRecord(ev[1], ctx->s_bc));
                if(root >= 0)
                    rc = mg_broadcast_here(mg, da + oa, extent(rows, k, lda) * in_es, root, ctx->s_bc);
                else
                    rc = mg_allgather_here(mg, da + oa, static_cast<size_t>(slice_rows) * lda * in_es, ctx->s_bc);
                if(rc != B200WMMA_OK)
                    goto drain;
                PIPE_CUDA(cudaEventRecord(ev[2], ctx->s_bc)); // "chunk i of A is on this device"
                PIPE_CUDA(cudaStreamWaitEvent(ctx->stream, ev[2], 0));
            }
            else
                PIPE_CUDA(cudaStreamWaitEvent(ctx->stream, ev[0], 0));
            if(use_c)
                PIPE_CUDA(cudaMemcpyAsync(dc + oc, hc + oc, extent(rows, n, ldc) * out_es, cudaMemcpyHostToDevice, ctx->s_in));
            PIPE_CUDA(cudaEventRecord(ev[3], ctx->s_in));
            PIPE_CUDA(cudaStreamWaitEvent(ctx->stream, ev[3], 0));
            PIPE_CUDA(cudaEventRecord(ev[4], ctx->stream));
            rc = launch(rows, da + oa, use_c ? dc + oc : nullptr, dd + od);
            if(rc != B200WMMA_OK)
                goto drain;
            PIPE_CUDA(cudaEventRecord(ev[5], ctx->stream));
            PIPE_CUDA(cudaStreamWaitEvent(ctx->s_out, ev[5], 0));
            PIPE_CUDA(cudaMemcpyAsync(hd + od, dd + od, extent(rows, n, ldd) * out_es, cudaMemcpyDeviceToHost, ctx->s_out));
            PIPE_CUDA(cudaEventRecord(ev[6], ctx->s_out));
        }
        PIPE_CUDA(cudaEventRecord(ev_in_end, ctx->s_in));
#undef PIPE_CUDA
    drain:
        // both exits: nothing of this call may still be in flight when it returns
        {
            cudaError_t e1 = cudaStreamSynchronize(ctx->s_out), e2 = cudaStreamSynchronize(ctx->s_in),
                        e3 = mg && ctx->s_bc ? cudaStreamSynchronize(ctx->s_bc) : cudaSuccess,
                        e4 = cudaStreamSynchronize(ctx->stream);
            if(rc == B200WMMA_OK)
                for(cudaError_t e : {e1, e2, e3, e4})
                    if(e != cudaSuccess)
                    {
                        rc = set_error(B200WMMA_ERR_CUDA, "gemm host driver: %s", cudaGetErrorString(e));
                        break;
                    }
        }
        if(rc != B200WMMA_OK)
            return rc;
        // ---- per-stage device times of this call (ms): upload span, exchange, compute, copy-out (sums), total span ----
        {
            float up = 0, ex = 0, cp = 0, out = 0, total = 0, t = 0;
            bool  ok = cudaEventElapsedTime(&up, ev_start, ev_in_end) == cudaSuccess;
            for(uint32_t i = 0; ok && i < chunks; ++i)
            {
                cudaEvent_t* ev = &ctx->events[PER * i];
                if(mg && nranks > 1)
                {
                    ok = cudaEventElapsedTime(&t, ev[1], ev[2]) == cudaSuccess;
                    ex += t;
                }
                ok = ok && cudaEventElapsedTime(&t, ev[4], ev[5]) == cudaSuccess;
                cp += t;
                ok = ok && cudaEventElapsedTime(&t, ev[5], ev[6]) == cudaSuccess;
                out += t;
            }
            ok = ok && cudaEventElapsedTime(&total, ev_start, ctx->events[PER * (chunks - 1) + 6]) == cudaSuccess;
            ctx->stage_ms[0] = up, ctx->stage_ms[1] = ex, ctx->stage_ms[2] = cp, ctx->stage_ms[3] = out, ctx->stage_ms[4] = total;
            ctx->stage_valid = ok;
        }
        return finish(ctx);
    }
}

namespace
{
    // Host-buffer GEMM for the layouts in which a chunk of rows is not contiguous in every matrix (column-major A, C or D):
    // all of A, B and C go up, one GEMM runs, D comes back.  `launch(a_dev, b_dev, c_dev, d_dev)` enqueues the GEMM.
    // ea, eb, ec, ed: element counts of the stored matrices.
    template <typename Launch>
    int gemm_host_whole(b200wmma_ctx* ctx, const void* a, const void* b, const void* c, void* d, size_t ba, size_t bb, size_t bc,
                        size_t bd, bool use_c, Launch launch)
    {
        if(int e = require_sm100())
            return e;
        if(int e = ctx_reserve(ctx, 0, ba)) return e;
        if(int e = ctx_reserve(ctx, 1, bb)) return e;
        if(int e = ctx_reserve(ctx, 2, use_c ? bc : 16)) return e;
        if(int e = ctx_reserve(ctx, 3, bd)) return e;
        if(int e = ctx_reserve(ctx, 4, gemm_split_workspace_bytes())) return e;
        ctx->stage_valid = false;
        HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(ctx->buf[0], a, ba, cudaMemcpyHostToDevice, ctx->stream));
        HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(ctx->buf[1], b, bb, cudaMemcpyHostToDevice, ctx->stream));
        if(use_c)
            HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(ctx->buf[2], c, bc, cudaMemcpyHostToDevice, ctx->stream));
        if(int e = launch(ctx->buf[0], ctx->buf[1], use_c ? ctx->buf[2] : nullptr, ctx->buf[3]))
        {
            cudaStreamSynchronize(ctx->stream);
            return e;
        }
        HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(d, ctx->buf[3], bd, cudaMemcpyDeviceToHost, ctx->stream));
        return finish(ctx);
    }
}

extern "C" int b200wmma_ctx_last_stage_ms(b200wmma_ctx* ctx, float* out_ms5)
{
    clear_error();
    B200_REQUIRE(ctx && out_ms5, B200WMMA_ERR_INVALID_ARG, "ctx_last_stage_ms: ctx and out_ms5 must be non-null");
    B200_REQUIRE(ctx->stage_valid, B200WMMA_ERR_UNSUPPORTED,
                 "ctx_last_stage_ms: no stage times (the last call on this context was not a GEMM host driver, or it failed)");
    for(int i = 0; i < 5; ++i)
        out_ms5[i] = ctx->stage_ms[i];
    return B200WMMA_OK;
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
    B200_REQUIRE(a && b && d && m && n && k, B200WMMA_ERR_INVALID_ARG, "gemm_f16_host: null pointer or zero size");
    B200_REQUIRE(out_type == 0 || out_type == 1, B200WMMA_ERR_INVALID_ARG, "gemm_f16_host: bad out_type");
    const size_t osz   = out_type == B200WMMA_OUT_F16 ? 2 : 4;
    const bool   use_c = c != nullptr && beta != 0.0f;
    B200_REQUIRE(c || beta == 0.0f, B200WMMA_ERR_INVALID_ARG, "gemm_f16_host: c may be null only when beta == 0");
    const bool a_col = layout_a == B200WMMA_COL_MAJOR, b_col = layout_b == B200WMMA_COL_MAJOR, cd_col = layout_cd == B200WMMA_COL_MAJOR;
    B200_REQUIRE(lda >= (a_col ? m : k) && ldb >= (b_col ? k : n) && ldd >= (cd_col ? m : n) && (!c || ldc >= (cd_col ? m : n)),
                 B200WMMA_ERR_INVALID_ARG, "gemm_f16_host: leading dimension too small");
    if(a_col || cd_col)
        // a chunk of rows is not contiguous in these layouts: whole matrices up, one GEMM, D back
        return gemm_host_whole(ctx, a, b, c, d, extent(a_col ? k : m, a_col ? m : k, lda) * 2, extent(b_col ? n : k, b_col ? k : n, ldb) * 2,
                               extent(cd_col ? n : m, cd_col ? m : n, ldc) * osz, extent(cd_col ? n : m, cd_col ? m : n, ldd) * osz, use_c,
                               [&](const void* da, const void* db, const void* dc, void* dd) {
                                   return launch_gemm_tc05_f16(m, n, k, da, db, dc, dd, lda, ldb, ldc, ldd, alpha, use_c ? beta : 0.0f,
                                                               layout_a, layout_b, layout_cd, out_type, ctx->stream, ctx->buf[4],
                                                               ctx->cap[4]);
                               });
    return gemm_host_pipeline(ctx, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, 2, osz, use_c,
                              [&](uint32_t rows, const void* da, const void* dc, void* dd) {
                                  return launch_gemm_tc05_f16(rows, n, k, da, ctx->buf[1], dc, dd, lda, ldb, ldc, ldd, alpha,
                                                              use_c ? beta : 0.0f, B200WMMA_ROW_MAJOR, layout_b,
                                                              B200WMMA_ROW_MAJOR, out_type, ctx->stream, ctx->buf[4], ctx->cap[4]);
                              },
                              nullptr, 0, b_col ? n : k, b_col ? k : n);
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
                                        B200WMMA_ROW_MAJOR, B200WMMA_COL_MAJOR, B200WMMA_ROW_MAJOR, out_type, ctx->stream, ctx->buf[4], ctx->cap[4]);
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
    B200_REQUIRE(a && b && d && m && n && k, B200WMMA_ERR_INVALID_ARG, "gemm_i8_host: null pointer or zero size");
    const bool use_c = c != nullptr && beta != 0;
    B200_REQUIRE(c || beta == 0, B200WMMA_ERR_INVALID_ARG, "gemm_i8_host: c may be null only when beta == 0");
    const bool a_col = layout_a == B200WMMA_COL_MAJOR, b_col = layout_b == B200WMMA_COL_MAJOR, cd_col = layout_cd == B200WMMA_COL_MAJOR;
    B200_REQUIRE(lda >= (a_col ? m : k) && ldb >= (b_col ? k : n) && ldd >= (cd_col ? m : n) && (!c || ldc >= (cd_col ? m : n)),
                 B200WMMA_ERR_INVALID_ARG, "gemm_i8_host: leading dimension too small");
    if(a_col || cd_col)
        return gemm_host_whole(ctx, a, b, c, d, extent(a_col ? k : m, a_col ? m : k, lda), extent(b_col ? n : k, b_col ? k : n, ldb),
                               extent(cd_col ? n : m, cd_col ? m : n, ldc) * 4, extent(cd_col ? n : m, cd_col ? m : n, ldd) * 4, use_c,
                               [&](const void* da, const void* db, const void* dc, void* dd) {
                                   return launch_gemm_tc05_i8(m, n, k, static_cast<const int8_t*>(da), static_cast<const int8_t*>(db),
                                                              static_cast<const int32_t*>(dc), static_cast<int32_t*>(dd), lda, ldb, ldc,
                                                              ldd, alpha, use_c ? beta : 0, layout_a, layout_b, layout_cd, ctx->stream,
                                                              ctx->buf[4], ctx->cap[4]);
                               });
    return gemm_host_pipeline(ctx, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, 1, 4, use_c,
                              [&](uint32_t rows, const void* da, const void* dc, void* dd) {
                                  return launch_gemm_tc05_i8(rows, n, k, static_cast<const int8_t*>(da),
                                                             static_cast<const int8_t*>(ctx->buf[1]),
                                                             static_cast<const int32_t*>(dc), static_cast<int32_t*>(dd), lda,
                                                             ldb, ldc, ldd, alpha, use_c ? beta : 0, B200WMMA_ROW_MAJOR,
                                                             layout_b, B200WMMA_ROW_MAJOR, ctx->stream, ctx->buf[4],
                                                             ctx->cap[4]);
                              },
                              nullptr, 0, b_col ? n : k, b_col ? k : n);
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
                                       ctx->stream, ctx->buf[4], ctx->cap[4]);
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
    HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(ctx->buf[0], input, bi, cudaMemcpyHostToDevice, ctx->stream));
    if(int e = b200wmma_dlrm_fwd(ctx->buf[0], ctx->buf[3], m, m_stride, k, batch, out_stride, ctx->stream))
    {
        cudaStreamSynchronize(ctx->stream); // the input copy must not outlive the call
        return e;
    }
    HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(output, ctx->buf[3], bo, cudaMemcpyDeviceToHost, ctx->stream));
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
    HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(ctx->buf[0], input, bi, cudaMemcpyHostToDevice, ctx->stream));
    HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(ctx->buf[1], upstream, bu, cudaMemcpyHostToDevice, ctx->stream));
    // rows m..m_stride-1 of grad are not written by the kernel: keep what the host passed in
    if(m_stride != m)
        HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(ctx->buf[3], grad, bi, cudaMemcpyHostToDevice, ctx->stream));
    if(int e = b200wmma_dlrm_bwd(ctx->buf[0], ctx->buf[1], ctx->buf[3], bottom_mlp_grad ? ctx->buf[2] : nullptr,
                                 m, m_stride, k, batch, upstream_stride, fuse_mlp_into_row0, ctx->stream))
    {
        cudaStreamSynchronize(ctx->stream);
        return e;
    }
    HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(grad, ctx->buf[3], bi, cudaMemcpyDeviceToHost, ctx->stream));
    if(bottom_mlp_grad)
        HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(bottom_mlp_grad, ctx->buf[2], bm, cudaMemcpyDeviceToHost, ctx->stream));
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
    HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(ctx->buf[0], a, ba, cudaMemcpyHostToDevice, ctx->stream));
    HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(ctx->buf[1], x, n * sizeof(T), cudaMemcpyHostToDevice, ctx->stream));
    HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(ctx->buf[3], y, m * sizeof(T), cudaMemcpyHostToDevice, ctx->stream));
    if(int e = launch(m, n, static_cast<const T*>(ctx->buf[0]), lda, layout_a,
                      static_cast<const T*>(ctx->buf[1]), static_cast<T*>(ctx->buf[3]), alpha, beta,
                      ctx->stream))
    {
        cudaStreamSynchronize(ctx->stream);
        return e;
    }
    HOST_CHECK_CUDA(ctx, cudaMemcpyAsync(y, ctx->buf[3], m * sizeof(T), cudaMemcpyDeviceToHost, ctx->stream));
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
