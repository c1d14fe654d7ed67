// Shared host/device plumbing for the rocwmma_b200 kernels: status codes, the thread-local
// error string, argument checks, the per-device status word that bounded device-side waits
// report into, and small PTX wrappers (mbarrier, TMA, tcgen05) used by the tensor-core GEMM.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/rocwmma_b200.h"

namespace b200wmma
{
    // ---- host-side error reporting -------------------------------------------------------
    int  set_error(int code, const char* fmt, ...);
    void clear_error();

#define B200_CHECK_CUDA(expr)                                                                 \
    do                                                                                        \
    {                                                                                         \
        cudaError_t _e = (expr);                                                              \
        if(_e != cudaSuccess)                                                                 \
            return ::b200wmma::set_error(B200WMMA_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,   \
                                         cudaGetErrorString(_e), __FILE__, __LINE__);         \
    } while(0)

#define B200_REQUIRE(cond, code, ...)                                                         \
    do                                                                                        \
    {                                                                                         \
        if(!(cond))                                                                           \
            return ::b200wmma::set_error(code, __VA_ARGS__);                                  \
    } while(0)

    // The current device must be a Blackwell sm_100 part: the kernels are built for sm_100a
    // only and there is no fallback path.
    int require_sm100();

    // Device-resident status word {code, detail}; one copy per device (module global).
    // Kernels with bounded waits get its device address from here.
    int status_word_ptr(unsigned** out_dev_ptr);
    // true once status_word_ptr has resolved (and cleared) the word of the current device
    bool status_word_ready();

    static inline bool aligned16(const void* p)
    {
        return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
    }
    static inline cudaStream_t as_stream(void* s)
    {
        return reinterpret_cast<cudaStream_t>(s);
    }
    // Kernel attributes and occupancy results are per device: caches of them are arrays indexed by
    // the current device (a process may drive several GPUs).
    constexpr int MAX_DEVICES = 64;
    static inline int current_device_slot()
    {
        int dev = 0;
        cudaGetDevice(&dev);
        return (dev >= 0 && dev < MAX_DEVICES) ? dev : 0;
    }
    static inline uint32_t ceil_div(uint32_t a, uint32_t b)
    {
        return (a + b - 1) / b;
    }

    // ---- kernel launchers implemented in the .cu files --------------------------------
    int launch_gemm_tc05_f16(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b,
                             const void* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                             uint32_t ldd, float alpha, float beta, int layout_a, int layout_b,
                             int layout_cd, int out_type, cudaStream_t stream, void* split_ws = nullptr,
                             size_t split_ws_bytes = 0);
    // bytes of scratch with which the 512 x 256 GEMM kernel may split the tiles of its last, partial round along K
    size_t gemm_split_workspace_bytes();
    int launch_gemm_tc05_bf16(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b, const void* c, void* d,
                              uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, float alpha, float beta, int layout_a,
                              int layout_b, int layout_cd, int out_type, cudaStream_t stream);
    // int8 inputs, int32 compute, int8 C / D (the int32 result cast to int8)
    int launch_gemm_tc05_i8_i8(uint32_t m, uint32_t n, uint32_t k, const int8_t* a, const int8_t* b, const int8_t* c, int8_t* d,
                               uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, int32_t alpha, int32_t beta, int layout_a,
                               int layout_b, int layout_cd, cudaStream_t stream);
    int launch_gemm_tc05_fp8(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b, const float* c, float* d,
                             uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, float alpha, float beta, int layout_a,
                             int layout_b, int layout_cd, int fp8_format, cudaStream_t stream);
    // fp32 inputs, 3 x TF32 on the tensor cores; C / D row major, a_mn / b_mn: operand stored with M / N contiguous
    size_t gemm_f32_workspace_bytes(uint32_t m, uint32_t n, uint32_t k);
    int    launch_gemm_tc05_f32(uint32_t m, uint32_t n, uint32_t k, const float* a, const float* b, const float* c, float* d,
                                uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, float alpha, float beta,
                                void* workspace, size_t workspace_bytes, cudaStream_t stream, bool a_mn = false,
                                bool b_mn = false);
    int launch_gemm_tc05_i8(uint32_t m, uint32_t n, uint32_t k, const int8_t* a,
                            const int8_t* b, const int32_t* c, int32_t* d, uint32_t lda,
                            uint32_t ldb, uint32_t ldc, uint32_t ldd, int32_t alpha,
                            int32_t beta, int layout_a, int layout_b, int layout_cd,
                            cudaStream_t stream, void* split_ws = nullptr, size_t split_ws_bytes = 0);
    // packed int4 operands (two per byte along K), unpacked to int8 in the kernel's load path
    int launch_gemm_tc05_i4(uint32_t m, uint32_t n, uint32_t k, const uint8_t* a_packed, const uint8_t* b_packed,
                            const int32_t* c, int32_t* d, uint32_t lda_bytes, uint32_t ldb_bytes, uint32_t ldc, uint32_t ldd,
                            int32_t alpha, int32_t beta, cudaStream_t stream);
    // DLRM dot interaction for shapes beyond the one-warp-per-sample kernels (dlrm_general.cu)
    int launch_dlrm_fwd_general(const void* input, void* output, uint32_t m, uint32_t m_stride, uint32_t k, uint32_t batch,
                                uint32_t out_stride, bool f32, cudaStream_t stream);
    int launch_dlrm_bwd_general(const void* input, const void* upstream, void* grad, void* bottom_mlp_grad, uint32_t m,
                                uint32_t m_stride, uint32_t k, uint32_t batch, uint32_t upstream_stride, int fuse, bool f32,
                                cudaStream_t stream);
    // 2:4-sparse int8 GEMM on compressed A (values + metadata) without a densified copy.
    // sp24_direct_ok() tells whether the operands meet its shape / alignment rules.
    bool sp24_direct_ok(uint32_t k, const void* a_vals, const void* a_meta, const void* b, uint32_t lda_vals,
                        uint32_t ld_meta, uint32_t ldb);
    int  launch_gemm_tc05_i8_sp24(uint32_t m, uint32_t n, uint32_t k, const int8_t* a_vals, const uint8_t* a_meta,
                                  bool meta_is_packed, const int8_t* b, const int32_t* c, int32_t* d, uint32_t lda_vals,
                                  uint32_t ld_meta, uint32_t ldb, uint32_t ldc, uint32_t ldd, int32_t alpha, int32_t beta,
                                  void* scratch, size_t scratch_bytes, cudaStream_t stream);
    int  launch_sp24_repack_meta(uint32_t m, uint32_t k, const uint8_t* a_meta, uint32_t ld_meta, void* packed,
                                 size_t packed_bytes, cudaStream_t stream);
    // bytes of scratch with which the kernel fetches the metadata in wide rows (a re-tiled copy)
    size_t sp24_packed_meta_bytes(uint32_t m, uint32_t k);
    // multi-GPU handle internals for the host-buffer drivers (multi_gpu.cu); the *_here forms assume that the handle's
    // device is already current.  mg_allgather_here: rank r's bytes_per_rank bytes lie at buf + r * bytes_per_rank.
    int mg_device(const b200wmma_mg* mg);
    int mg_broadcast_here(b200wmma_mg* mg, void* buf, size_t bytes, int root, cudaStream_t stream);
    int mg_allgather_here(b200wmma_mg* mg, void* buf, size_t bytes_per_rank, cudaStream_t stream);
} // namespace b200wmma
