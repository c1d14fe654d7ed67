"""numpy-facing loader for the two CPU checkers.  TEST INFRASTRUCTURE ONLY.

  port()      -> oracle/libref_port.so : this repo's C restatement (ref_port.c)
  reference() -> oracle/_ref/libref.so : the rocWMMA reference's own test/reference_impl.hpp,
                                         compiled by oracle/Makefile where the reference tree exists
Both export the same C entry points, so every helper below takes `impl` = port() or reference().
Array arguments are C-contiguous numpy arrays holding the matrices in their stated memory layout
with natural leading dimensions (as the reference's gemm_CPU assumes, test/reference_impl.hpp:53-56).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_PATH = os.path.join(_HERE, "libref_port.so")
REF_PATH = os.path.join(_HERE, "_ref", "libref.so")

_u32, _vp = C.c_uint32, C.c_void_p
_GEMM_SCALARS = {
    "oracle_gemm_f16_f32": C.c_float, "oracle_gemm_f16_f16": C.c_float, "oracle_gemm_i8_i32": C.c_int32, "oracle_gemm_i8_i8": C.c_int32,
    "oracle_gemm_f32": C.c_float, "oracle_gemm_f64": C.c_double,
}


def build() -> None:
    """(Re)build the checkers with oracle/Makefile (the reference part only where its tree exists)."""
    subprocess.run(["make", "-s", "-C", _HERE], check=True)


def _load(path):
    h = C.CDLL(path)
    for name, st in _GEMM_SCALARS.items():
        fn = getattr(h, name)
        fn.restype = None
        fn.argtypes = [_u32, _u32, _u32, _vp, _vp, _vp, _vp, st, st, C.c_int, C.c_int, C.c_int, C.c_int, _u32]
    for name in ("oracle_dlrm_fwd_f16", "oracle_dlrm_fwd_f32"):
        getattr(h, name).restype = None
        getattr(h, name).argtypes = [_vp, _vp, _u32, _u32, _u32]
    for name in ("oracle_dlrm_bwd_f16", "oracle_dlrm_bwd_f32"):
        getattr(h, name).restype = None
        getattr(h, name).argtypes = [_vp, _vp, _vp, _vp, _u32, _u32, _u32]
    h.oracle_gemv_f32.restype = None
    h.oracle_gemv_f32.argtypes = [_u32, _u32, _vp, _u32, C.c_int, _vp, _vp, C.c_float, C.c_float]
    h.oracle_gemv_f64.restype = None
    h.oracle_gemv_f64.argtypes = [_u32, _u32, _vp, _u32, C.c_int, _vp, _vp, C.c_double, C.c_double]
    h.oracle_num_threads.restype = C.c_int
    h.oracle_num_threads.argtypes = []
    h.oracle_set_num_threads.restype = None
    h.oracle_set_num_threads.argtypes = [C.c_int]
    if hasattr(h, "oracle_gemm_abs_bound"):
        h.oracle_gemm_abs_bound.restype = None
        h.oracle_gemm_abs_bound.argtypes = [_u32, _u32, _u32, _vp, _vp, _vp, C.c_double, C.c_double, _vp]
    return h


_cache = {}


def port():
    if "port" not in _cache:
        if not os.path.exists(PORT_PATH):
            build()
        _cache["port"] = _load(PORT_PATH)
    return _cache["port"]


def have_reference() -> bool:
    return os.path.exists(REF_PATH)


def reference():
    if "ref" not in _cache:
        if not have_reference():
            raise RuntimeError("oracle/_ref/libref.so not built (needs the reference tree; see oracle/Makefile)")
        _cache["ref"] = _load(REF_PATH)
    return _cache["ref"]


def _p(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


def _c(a):
    assert a is None or a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a


_GEMM_FN = {
    (np.float16, np.float32): "oracle_gemm_f16_f32", (np.float16, np.float16): "oracle_gemm_f16_f16",
    (np.int8, np.int32): "oracle_gemm_i8_i32", (np.int8, np.int8): "oracle_gemm_i8_i8", (np.float32, np.float32): "oracle_gemm_f32",
    (np.float64, np.float64): "oracle_gemm_f64",
}


def gemm(impl, m, n, k, a, b, c, alpha, beta, out_dtype, la=0, lb=1, lc=0, ld=0, m_rows=0):
    """D = alpha*A*B + beta*C with the reference's loop order.  a: m*k elements, b: k*n, c: m*n, each in
    its own layout (flags 0=row,1=col).  Returns d as a flat array of m*n (or m_rows*n when row-major D
    and m_rows given) elements in layout ld."""
    name = _GEMM_FN[(a.dtype.type, np.dtype(out_dtype).type)]
    rows = m if not m_rows else m_rows
    d = np.zeros(m * n if ld else rows * n, dtype=out_dtype)
    if c is None:
        c = np.zeros(m * n, dtype=out_dtype)
        beta = 0
    getattr(impl, name)(m, n, k, _p(_c(a)), _p(_c(b)), _p(_c(c)), _p(d), alpha, beta, la, lb, lc, ld, m_rows)
    return d


def dlrm_fwd(impl, x, m, k, batch):
    """x: [batch, m, k] fp16/fp32 -> [batch, k + m(m-1)/2]."""
    fn = impl.oracle_dlrm_fwd_f16 if x.dtype == np.float16 else impl.oracle_dlrm_fwd_f32
    out = np.zeros((batch, k + m * (m - 1) // 2), dtype=x.dtype)
    fn(_p(_c(x)), _p(out), m, k, batch)
    return out


def dlrm_bwd(impl, x, upstream, m, k, batch):
    """Returns (grad [batch, m, k], bottom_mlp_grad [batch, k])."""
    fn = impl.oracle_dlrm_bwd_f16 if x.dtype == np.float16 else impl.oracle_dlrm_bwd_f32
    grad = np.zeros((batch, m, k), dtype=x.dtype)
    mlp = np.zeros((batch, k), dtype=x.dtype)
    fn(_p(_c(x)), _p(_c(upstream)), _p(mlp), _p(grad), m, k, batch)
    return grad, mlp


def gemv(impl, m, n, a, x, y, alpha, beta, a_col_major=False):
    """Returns alpha*A*x + beta*y (y is not modified)."""
    out = np.array(y, copy=True)
    lda = m if a_col_major else n
    fn = impl.oracle_gemv_f32 if a.dtype == np.float32 else impl.oracle_gemv_f64
    fn(m, n, _p(_c(a)), lda, int(a_col_major), _p(_c(x)), _p(out), alpha, beta)
    return out


def gemm_abs_bound(m, n, k, a_rm, b_rm, c_rm, alpha, beta):
    """|alpha| * sum_h |a||b| + |beta||c| per output element, in float64, row-major logical inputs."""
    a64 = np.ascontiguousarray(a_rm, dtype=np.float64)
    b64 = np.ascontiguousarray(b_rm, dtype=np.float64)
    c64 = None if c_rm is None else np.ascontiguousarray(c_rm, dtype=np.float64)
    out = np.zeros((m, n), dtype=np.float64)
    port().oracle_gemm_abs_bound(m, n, k, _p(a64), _p(b64), _p(c64), float(alpha), float(beta), _p(out))
    return out


def num_threads(impl) -> int:
    return impl.oracle_num_threads()


def use_all_host_threads(impl) -> int:
    """Let the OpenMP loops use every hardware thread this process may run on; returns the count."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    impl.oracle_set_num_threads(n)
    return impl.oracle_num_threads()
