"""Python host mirror of the rocWMMA sample / test-harness entry points for the hot path.

Every function here forwards to the C ABI (include/rocwmma_b200.h) with device pointers taken
from torch CUDA tensors and the current torch stream.  torch is plumbing only (memory, streams);
all arithmetic happens in the hand-written kernels.  Argument names and meaning follow the
reference kernels: gemm_rocwmma_d (samples/perf_hgemm.cpp:515-528), dlrmDotFwd / dlrmDotBwd
(samples/simple_dlrm.cpp:184-192, :349-360), sgemv_rocwmma_d (samples/simple_sgemv.cpp:103-116).
"""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import B200WmmaError, check, lib

ROW_MAJOR, COL_MAJOR = 0, 1
OUT_F16, OUT_F32 = 0, 1


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t, dtype, name):
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == dtype):
        raise TypeError(f"{name} must be a CUDA tensor of dtype {dtype}")


def set_tuning(key: str, value: int):
    """b200wmma_set_tuning: override the library's kernel selection (0 = built-in choice)."""
    check(lib().b200wmma_set_tuning(key.encode(), int(value)))


def device_status():
    """Synchronise the current stream and return (status, detail) of the device status word."""
    st, detail = C.c_int(0), C.c_uint(0)
    check(lib().b200wmma_device_status(_stream(), C.byref(st), C.byref(detail)))
    return st.value, detail.value


def gemm_split_workspace_bytes():
    """Bytes of scratch with which gemm_f16 / gemm_i8 may split the tiles of a partial last round along K."""
    return lib().b200wmma_gemm_split_workspace_bytes()


def gemm_f16(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta,
             layout_a=ROW_MAJOR, layout_b=COL_MAJOR, layout_cd=ROW_MAJOR, workspace=None):
    """D = alpha * A x B + beta * C; fp16 inputs, fp32 accumulate, D/C fp16 or fp32 (by d.dtype).
    workspace: optional uint8 CUDA tensor of gemm_split_workspace_bytes() bytes (b200wmma_gemm_f16_ws)."""
    _need(a, torch.float16, "a"); _need(b, torch.float16, "b")
    out_type = OUT_F16 if d.dtype == torch.float16 else OUT_F32
    _need(d, torch.float16 if out_type == OUT_F16 else torch.float32, "d")
    if c is not None:
        _need(c, d.dtype, "c")
    if workspace is not None:
        _need(workspace, torch.uint8, "workspace")
        check(lib().b200wmma_gemm_f16_ws(m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc, ldd, alpha, beta,
                                         layout_a, layout_b, layout_cd, out_type, _ptr(workspace), workspace.numel(), _stream()))
        return
    check(lib().b200wmma_gemm_f16(m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc, ldd,
                                  alpha, beta, layout_a, layout_b, layout_cd, out_type, _stream()))


def gemm_f32_workspace_bytes(m, n, k):
    return lib().b200wmma_gemm_f32_workspace_bytes(m, n, k)


def gemm_f32(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, workspace,
             layout_a=ROW_MAJOR, layout_b=COL_MAJOR, layout_cd=ROW_MAJOR):
    """fp32 GEMM (3 x TF32 on the tensor cores), every layout combination."""
    _need(a, torch.float32, "a"); _need(b, torch.float32, "b"); _need(d, torch.float32, "d")
    _need(workspace, torch.uint8, "workspace")
    if c is not None:
        _need(c, torch.float32, "c")
    check(lib().b200wmma_gemm_f32(m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc, ldd, alpha, beta,
                                  layout_a, layout_b, layout_cd, _ptr(workspace), workspace.numel(), _stream()))


FP8_E4M3, FP8_E5M2 = 0, 1


OUT_BF16 = 2


def gemm_bf16(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta,
              layout_a=ROW_MAJOR, layout_b=COL_MAJOR, layout_cd=ROW_MAJOR):
    """bfloat16 inputs, fp32 accumulate, C / D fp32 or bfloat16 (by d.dtype)."""
    _need(a, torch.bfloat16, "a"); _need(b, torch.bfloat16, "b")
    if d.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("d must be float32 or bfloat16")
    _need(d, d.dtype, "d")
    if c is not None:
        _need(c, d.dtype, "c")
    if d.dtype == torch.float32:
        check(lib().b200wmma_gemm_bf16(m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc, ldd,
                                       alpha, beta, layout_a, layout_b, layout_cd, _stream()))
    else:
        check(lib().b200wmma_gemm_bf16_out(m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc, ldd,
                                           alpha, beta, layout_a, layout_b, layout_cd, OUT_BF16, _stream()))


def gemm_i8_i8(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta,
               layout_a=ROW_MAJOR, layout_b=COL_MAJOR, layout_cd=ROW_MAJOR):
    """int8 inputs, int32 compute, int8 C / D (the int32 result cast to int8)."""
    _need(a, torch.int8, "a"); _need(b, torch.int8, "b"); _need(d, torch.int8, "d")
    if c is not None:
        _need(c, torch.int8, "c")
    check(lib().b200wmma_gemm_i8_i8(m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc, ldd,
                                    alpha, beta, layout_a, layout_b, layout_cd, _stream()))


def gemm_fp8(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta,
             layout_a=ROW_MAJOR, layout_b=COL_MAJOR, layout_cd=ROW_MAJOR):
    """OCP fp8 inputs (both torch.float8_e4m3fn or both torch.float8_e5m2), fp32 accumulate, fp32 C / D."""
    if a.dtype not in (torch.float8_e4m3fn, torch.float8_e5m2):
        raise TypeError("a must be float8_e4m3fn or float8_e5m2")
    _need(a, a.dtype, "a"); _need(b, a.dtype, "b"); _need(d, torch.float32, "d")
    if c is not None:
        _need(c, torch.float32, "c")
    fmt = FP8_E4M3 if a.dtype == torch.float8_e4m3fn else FP8_E5M2
    check(lib().b200wmma_gemm_fp8(m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc, ldd,
                                  alpha, beta, layout_a, layout_b, layout_cd, fmt, _stream()))


def gemm_i8(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta,
            layout_a=ROW_MAJOR, layout_b=COL_MAJOR, layout_cd=ROW_MAJOR, workspace=None):
    _need(a, torch.int8, "a"); _need(b, torch.int8, "b"); _need(d, torch.int32, "d")
    if c is not None:
        _need(c, torch.int32, "c")
    if workspace is not None:
        _need(workspace, torch.uint8, "workspace")
        check(lib().b200wmma_gemm_i8_ws(m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc, ldd, alpha, beta,
                                        layout_a, layout_b, layout_cd, _ptr(workspace), workspace.numel(), _stream()))
        return
    check(lib().b200wmma_gemm_i8(m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc, ldd,
                                 alpha, beta, layout_a, layout_b, layout_cd, _stream()))


def gemm_f64(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta,
             layout_a=ROW_MAJOR, layout_b=COL_MAJOR, layout_cd=ROW_MAJOR):
    for t, nm in ((a, "a"), (b, "b"), (d, "d")):
        _need(t, torch.float64, nm)
    if c is not None:
        _need(c, torch.float64, "c")
    check(lib().b200wmma_gemm_f64(m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc, ldd,
                                  alpha, beta, layout_a, layout_b, layout_cd, _stream()))


def gemm_i8_sp24_workspace_bytes(m, n, k):
    return lib().b200wmma_gemm_i8_sp24_workspace_bytes(m, n, k)


def gemm_i8_sp24(m, n, k, a_vals, a_meta, b, c, d, lda_vals, ld_meta, ldb, ldc, ldd, alpha, beta, workspace):
    _need(a_vals, torch.int8, "a_vals"); _need(a_meta, torch.uint8, "a_meta")
    _need(b, torch.int8, "b"); _need(d, torch.int32, "d")
    if workspace is not None:          # needed only off the sparse tensor-core path (k % 128 != 0, unaligned rows)
        _need(workspace, torch.uint8, "workspace")
    check(lib().b200wmma_gemm_i8_sp24(m, n, k, _ptr(a_vals), _ptr(a_meta), _ptr(b), _ptr(c), _ptr(d),
                                      lda_vals, ld_meta, ldb, ldc, ldd, alpha, beta,
                                      _ptr(workspace), 0 if workspace is None else workspace.numel(), _stream()))


def sp24_packed_meta_bytes(m, k):
    return lib().b200wmma_sp24_packed_meta_bytes(m, k)


def sp24_repack_meta(m, k, a_meta, ld_meta, packed):
    """Re-tile the 2:4 metadata of A once (A reused across calls); feed `packed` to gemm_i8_sp24_packed."""
    _need(a_meta, torch.uint8, "a_meta"); _need(packed, torch.uint8, "packed")
    check(lib().b200wmma_sp24_repack_meta(m, k, _ptr(a_meta), ld_meta, _ptr(packed), packed.numel(), _stream()))


def gemm_i8_sp24_packed(m, n, k, a_vals, a_meta_packed, b, c, d, lda_vals, ldb, ldc, ldd, alpha, beta):
    _need(a_vals, torch.int8, "a_vals"); _need(a_meta_packed, torch.uint8, "a_meta_packed")
    _need(b, torch.int8, "b"); _need(d, torch.int32, "d")
    check(lib().b200wmma_gemm_i8_sp24_packed(m, n, k, _ptr(a_vals), _ptr(a_meta_packed), _ptr(b), _ptr(c), _ptr(d),
                                             lda_vals, ldb, ldc, ldd, alpha, beta, _stream()))


def gemm_i4_workspace_bytes(m, n, k):
    return lib().b200wmma_gemm_i4_workspace_bytes(m, n, k)


def gemm_i4(m, n, k, a_packed, b_packed, c, d, lda_bytes, ldb_bytes, ldc, ldd, alpha, beta, workspace=None):
    _need(a_packed, torch.uint8, "a_packed"); _need(b_packed, torch.uint8, "b_packed")
    _need(d, torch.int32, "d")
    if workspace is not None:
        _need(workspace, torch.uint8, "workspace")
    check(lib().b200wmma_gemm_i4(m, n, k, _ptr(a_packed), _ptr(b_packed), _ptr(c), _ptr(d),
                                 lda_bytes, ldb_bytes, ldc, ldd, alpha, beta,
                                 _ptr(workspace), 0 if workspace is None else workspace.numel(), _stream()))


def simple_sgemm(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta):
    """sgemm_rocwmma_d (samples/simple_sgemm.cpp:81-139) on this repo's fragment headers."""
    for t, nm in ((a, "a"), (b, "b"), (c, "c"), (d, "d")):
        _need(t, torch.float32, nm)
    check(lib().b200wmma_simple_sgemm(m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc, ldd, alpha, beta,
                                      _stream()))


def simple_dgemm(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta):
    """dgemm_rocwmma_d (samples/simple_dgemm.cpp:81-139) on this repo's fragment headers."""
    for t, nm in ((a, "a"), (b, "b"), (c, "c"), (d, "d")):
        _need(t, torch.float64, nm)
    check(lib().b200wmma_simple_dgemm(m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc, ldd, alpha, beta,
                                      _stream()))


def simple_hgemm(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta):
    """hgemm_rocwmma_d (samples/simple_hgemm.cpp:81-139) on this repo's fragment headers."""
    _need(a, torch.float16, "a"); _need(b, torch.float16, "b")
    out_type = OUT_F16 if d.dtype == torch.float16 else OUT_F32
    _need(c, d.dtype, "c")
    check(lib().b200wmma_simple_hgemm(m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc, ldd,
                                      alpha, beta, out_type, _stream()))


def measure_mma_sync_rate(kind):
    """TFLOP/s at which the device issues mma.sync from registers: kind 0 = m16n8k16 fp16 -> fp32, 1 = m16n8k8 fp64."""
    out = C.c_double(0.0)
    check(lib().b200wmma_measure_mma_sync_rate(int(kind), C.byref(out), _stream()))
    return out.value


def perf_hgemm_fragment(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta):
    for t, nm in ((a, "a"), (b, "b"), (c, "c"), (d, "d")):
        _need(t, torch.float16, nm)
    check(lib().b200wmma_perf_hgemm_fragment(m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d),
                                             lda, ldb, ldc, ldd, alpha, beta, _stream()))


def dlrm_dot_fwd(input, output, m, m_stride, k, batch, out_stride):
    """fp16 or fp32 data (by input.dtype)."""
    dt = input.dtype
    if dt not in (torch.float16, torch.float32):
        raise TypeError("input must be float16 or float32")
    _need(input, dt, "input"); _need(output, dt, "output")
    fn = lib().b200wmma_dlrm_fwd if dt == torch.float16 else lib().b200wmma_dlrm_fwd_f32
    check(fn(_ptr(input), _ptr(output), m, m_stride, k, batch, out_stride, _stream()))


def dlrm_dot_bwd(input, upstream, grad, bottom_mlp_grad, m, m_stride, k, batch, upstream_stride,
                 fuse_mlp_into_row0=False):
    dt = input.dtype
    if dt not in (torch.float16, torch.float32):
        raise TypeError("input must be float16 or float32")
    _need(input, dt, "input"); _need(upstream, dt, "upstream")
    _need(grad, dt, "grad")
    if bottom_mlp_grad is not None:
        _need(bottom_mlp_grad, dt, "bottom_mlp_grad")
    fn = lib().b200wmma_dlrm_bwd if dt == torch.float16 else lib().b200wmma_dlrm_bwd_f32
    check(fn(_ptr(input), _ptr(upstream), _ptr(grad), _ptr(bottom_mlp_grad),
             m, m_stride, k, batch, upstream_stride, int(fuse_mlp_into_row0), _stream()))


def gemv(m, n, a, lda, x, y, alpha, beta, layout_a=ROW_MAJOR):
    """y = alpha * A x + beta * y in place; fp32 or fp64 by a.dtype."""
    if a.dtype == torch.float32:
        fn = lib().b200wmma_gemv_f32
    elif a.dtype == torch.float64:
        fn = lib().b200wmma_gemv_f64
    else:
        raise TypeError("gemv: a must be float32 or float64")
    _need(a, a.dtype, "a"); _need(x, a.dtype, "x"); _need(y, a.dtype, "y")
    check(fn(m, n, _ptr(a), lda, layout_a, _ptr(x), _ptr(y), alpha, beta, _stream()))


class HostContext:
    """b200wmma_ctx: cached device buffers + stream for the host-buffer drivers (`*_host`)."""

    def __init__(self):
        self._h = C.c_void_p()
        check(lib().b200wmma_ctx_create(C.byref(self._h)))

    def close(self):
        if self._h:
            lib().b200wmma_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _hp(t):
        """Host pointer of a CPU torch tensor or numpy array (None passes through)."""
        if t is None:
            return None
        if isinstance(t, torch.Tensor):
            assert not t.is_cuda
            return C.c_void_p(t.data_ptr())
        return C.c_void_p(t.ctypes.data)

    def last_stage_ms(self):
        """Device times of the last GEMM host call: dict of upload / exchange / compute / download / total ms."""
        out = (C.c_float * 5)()
        check(lib().b200wmma_ctx_last_stage_ms(self._h, out))
        return dict(zip(("upload", "exchange", "compute", "download", "total"), (float(x) for x in out)))

    def gemm_f16(self, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, out_type,
                 layout_a=ROW_MAJOR, layout_b=COL_MAJOR, layout_cd=ROW_MAJOR):
        check(lib().b200wmma_gemm_f16_host(self._h, m, n, k, self._hp(a), self._hp(b), self._hp(c), self._hp(d),
                                           lda, ldb, ldc, ldd, alpha, beta, layout_a, layout_b, layout_cd, out_type))

    def gemm_f16_mg(self, mg, root, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, out_type):
        """Column-sharded form: n, b, c, d are this rank's block; only rank `root` reads `a` (may be None elsewhere);
        A travels to the other ranks over NCCL inside the pipeline.  Collective over `mg` (a MultiGpu)."""
        check(lib().b200wmma_gemm_f16_host_mg(self._h, mg._h, root, m, n, k, self._hp(a), self._hp(b), self._hp(c),
                                              self._hp(d), lda, ldb, ldc, ldd, alpha, beta, out_type))

    def gemm_i8_mg(self, mg, root, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta):
        """Column-sharded int8 form of gemm_f16_mg."""
        check(lib().b200wmma_gemm_i8_host_mg(self._h, mg._h, root, m, n, k, self._hp(a), self._hp(b), self._hp(c),
                                             self._hp(d), lda, ldb, ldc, ldd, alpha, beta))

    def gemm_i8(self, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta,
                layout_a=ROW_MAJOR, layout_b=COL_MAJOR, layout_cd=ROW_MAJOR):
        check(lib().b200wmma_gemm_i8_host(self._h, m, n, k, self._hp(a), self._hp(b), self._hp(c), self._hp(d),
                                          lda, ldb, ldc, ldd, alpha, beta, layout_a, layout_b, layout_cd))

    def dlrm_fwd(self, input, output, m, m_stride, k, batch, out_stride):
        check(lib().b200wmma_dlrm_fwd_host(self._h, self._hp(input), self._hp(output), m, m_stride, k, batch, out_stride))

    def dlrm_bwd(self, input, upstream, grad, bottom_mlp_grad, m, m_stride, k, batch, upstream_stride, fuse):
        check(lib().b200wmma_dlrm_bwd_host(self._h, self._hp(input), self._hp(upstream), self._hp(grad),
                                           self._hp(bottom_mlp_grad), m, m_stride, k, batch, upstream_stride, int(fuse)))

    def gemv(self, m, n, a, lda, x, y, alpha, beta, layout_a=ROW_MAJOR, double=False):
        fn = lib().b200wmma_gemv_f64_host if double else lib().b200wmma_gemv_f32_host
        check(fn(self._h, m, n, self._hp(a), lda, layout_a, self._hp(x), self._hp(y), alpha, beta))


def shard_range(total, parts, index, granule=1):
    """(begin, count) of part `index` of `parts` over `total` units (b200wmma_shard_range)."""
    begin, count = C.c_uint64(), C.c_uint64()
    check(lib().b200wmma_shard_range(total, parts, index, granule, C.byref(begin), C.byref(count)))
    return begin.value, count.value


class MultiGpu:
    """One rank of a one-process-per-GPU group on the library's own NCCL plumbing (b200wmma_mg_*).

    Rank 0 calls MultiGpu.unique_id() and ships the bytes to the other ranks by any means; every rank then
    constructs MultiGpu(id_bytes, rank, nranks) with its device current."""

    ID_BYTES = 128

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(MultiGpu.ID_BYTES)
        check(lib().b200wmma_mg_unique_id(buf))
        return buf.raw

    def __init__(self, id_bytes: bytes, rank: int, nranks: int):
        if len(id_bytes) != self.ID_BYTES:
            raise ValueError("id_bytes must be the 128 bytes of MultiGpu.unique_id()")
        self._h = C.c_void_p()
        check(lib().b200wmma_mg_create(C.byref(self._h), id_bytes, rank, nranks))
        self.rank, self.nranks = rank, nranks

    def broadcast(self, t, root=0):
        """In place, on the current torch stream."""
        if not t.is_cuda or not t.is_contiguous():
            raise ValueError("broadcast needs a contiguous CUDA tensor")
        check(lib().b200wmma_mg_broadcast(self._h, _ptr(t), t.numel() * t.element_size(), root, _stream()))

    def allgather(self, t):
        """In place, on the current torch stream: rank r contributes the r-th of nranks equal pieces of `t`."""
        if not t.is_cuda or not t.is_contiguous():
            raise ValueError("allgather needs a contiguous CUDA tensor")
        nbytes = t.numel() * t.element_size()
        if nbytes % self.nranks:
            raise ValueError("allgather: the buffer does not split into nranks equal pieces")
        check(lib().b200wmma_mg_allgather(self._h, _ptr(t), nbytes // self.nranks, _stream()))

    def close(self):
        if self._h:
            check(lib().b200wmma_mg_destroy(self._h))
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
