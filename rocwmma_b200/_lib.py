"""ctypes binding of librocwmma_b200.so (the C ABI declared in include/rocwmma_b200.h).

There is no CPU implementation behind this module: if the shared library has not been built
(`python -m rocwmma_b200.build`) importing `lib()` raises."""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "librocwmma_b200.so")

u32, i32, f32, f64, vp, sz = C.c_uint32, C.c_int32, C.c_float, C.c_double, C.c_void_p, C.c_size_t

# name -> (restype, argtypes); mirrors include/rocwmma_b200.h one to one
SIGNATURES = {
    "b200wmma_last_error_string": (C.c_char_p, []),
    "b200wmma_version": (C.c_int, []),
    "b200wmma_set_tuning": (C.c_int, [C.c_char_p, C.c_int]),
    "b200wmma_device_status": (C.c_int, [vp, C.POINTER(C.c_int), C.POINTER(C.c_uint)]),
    "b200wmma_gemm_f16": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, f32, f32,
                                    C.c_int, C.c_int, C.c_int, C.c_int, vp]),
    "b200wmma_gemm_i8": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, i32, i32,
                                   C.c_int, C.c_int, C.c_int, vp]),
    "b200wmma_gemm_split_workspace_bytes": (sz, []),
    "b200wmma_gemm_f16_ws": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, f32, f32,
                                       C.c_int, C.c_int, C.c_int, C.c_int, vp, sz, vp]),
    "b200wmma_gemm_i8_ws": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, i32, i32,
                                      C.c_int, C.c_int, C.c_int, vp, sz, vp]),
    "b200wmma_gemm_f32_workspace_bytes": (sz, [u32, u32, u32]),
    "b200wmma_gemm_f32": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, f32, f32,
                                    C.c_int, C.c_int, C.c_int, vp, sz, vp]),
    "b200wmma_gemm_bf16": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, f32, f32,
                                     C.c_int, C.c_int, C.c_int, vp]),
    "b200wmma_gemm_bf16_out": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, f32, f32,
                                         C.c_int, C.c_int, C.c_int, C.c_int, vp]),
    "b200wmma_gemm_i8_i8": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, i32, i32,
                                      C.c_int, C.c_int, C.c_int, vp]),
    "b200wmma_gemm_fp8": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, f32, f32,
                                    C.c_int, C.c_int, C.c_int, C.c_int, vp]),
    "b200wmma_gemm_f64": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, f64, f64,
                                    C.c_int, C.c_int, C.c_int, vp]),
    "b200wmma_gemm_i8_sp24_workspace_bytes": (sz, [u32, u32, u32]),
    "b200wmma_gemm_i8_sp24": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32,
                                        i32, i32, vp, sz, vp]),
    "b200wmma_gemm_i8_sp24_static": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32,
                                               i32, i32, vp]),
    "b200wmma_sp24_packed_meta_bytes": (sz, [u32, u32]),
    "b200wmma_sp24_repack_meta": (C.c_int, [u32, u32, vp, u32, vp, sz, vp]),
    "b200wmma_gemm_i8_sp24_packed": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, vp, u32, u32, u32, u32, i32, i32, vp]),
    "b200wmma_gemm_i4_workspace_bytes": (sz, [u32, u32, u32]),
    "b200wmma_gemm_i4": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, i32, i32,
                                   vp, sz, vp]),
    "b200wmma_simple_sgemm": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, f32, f32, vp]),
    "b200wmma_simple_dgemm": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, f64, f64, vp]),
    "b200wmma_simple_hgemm": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, f32, f32,
                                        C.c_int, vp]),
    "b200wmma_perf_hgemm_fragment": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32,
                                               f32, f32, vp]),
    "b200wmma_measure_mma_sync_rate": (C.c_int, [C.c_int, C.POINTER(C.c_double), vp]),
    "b200wmma_dlrm_fwd": (C.c_int, [vp, vp, u32, u32, u32, u32, u32, vp]),
    "b200wmma_dlrm_bwd": (C.c_int, [vp, vp, vp, vp, u32, u32, u32, u32, u32, C.c_int, vp]),
    "b200wmma_dlrm_fwd_f32": (C.c_int, [vp, vp, u32, u32, u32, u32, u32, vp]),
    "b200wmma_dlrm_bwd_f32": (C.c_int, [vp, vp, vp, vp, u32, u32, u32, u32, u32, C.c_int, vp]),
    "b200wmma_gemv_f32": (C.c_int, [u32, u32, vp, u32, C.c_int, vp, vp, f32, f32, vp]),
    "b200wmma_gemv_f64": (C.c_int, [u32, u32, vp, u32, C.c_int, vp, vp, f64, f64, vp]),
    "b200wmma_mg_unique_id": (C.c_int, [vp]),
    "b200wmma_mg_create": (C.c_int, [C.POINTER(vp), vp, C.c_int, C.c_int]),
    "b200wmma_mg_broadcast": (C.c_int, [vp, vp, C.c_size_t, C.c_int, vp]),
    "b200wmma_mg_allgather": (C.c_int, [vp, vp, C.c_size_t, vp]),
    "b200wmma_mg_destroy": (C.c_int, [vp]),
    "b200wmma_mg_rank": (C.c_int, [vp]),
    "b200wmma_mg_size": (C.c_int, [vp]),
    "b200wmma_gemm_f16_host_mg": (C.c_int, [vp, vp, C.c_int, u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, f32, f32,
                                            C.c_int]),
    "b200wmma_gemm_i8_host_mg": (C.c_int, [vp, vp, C.c_int, u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, i32, i32]),
    "b200wmma_shard_range": (C.c_int, [C.c_uint64, u32, u32, u32, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "b200wmma_ctx_create": (C.c_int, [C.POINTER(vp)]),
    "b200wmma_ctx_destroy": (C.c_int, [vp]),
    "b200wmma_ctx_last_stage_ms": (C.c_int, [vp, C.POINTER(C.c_float)]),
    "b200wmma_gemm_f16_host": (C.c_int, [vp, u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, f32, f32,
                                         C.c_int, C.c_int, C.c_int, C.c_int]),
    "b200wmma_gemm_i8_host": (C.c_int, [vp, u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, i32, i32,
                                        C.c_int, C.c_int, C.c_int]),
    "b200wmma_dlrm_fwd_host": (C.c_int, [vp, vp, vp, u32, u32, u32, u32, u32]),
    "b200wmma_dlrm_bwd_host": (C.c_int, [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, C.c_int]),
    "b200wmma_gemv_f32_host": (C.c_int, [vp, u32, u32, vp, u32, C.c_int, vp, vp, f32, f32]),
    "b200wmma_gemv_f64_host": (C.c_int, [vp, u32, u32, vp, u32, C.c_int, vp, vp, f64, f64]),
}

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m rocwmma_b200.build`. "
                "rocwmma_b200 has no CPU or PyTorch fallback.")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


class B200WmmaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"rocwmma_b200 error {code}: {message}")
        self.code = code


def check(code: int) -> None:
    if code != 0:
        raise B200WmmaError(code, lib().b200wmma_last_error_string().decode())
