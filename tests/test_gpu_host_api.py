"""The host-buffer drivers (`b200wmma_*_host`, the mirrors of the reference samples' gemm_test / dlrm_test /
sgemv_test): host pointers in, host pointers out, copies and kernels pipelined inside the call."""
import numpy as np
import pytest
import torch

from conftest import TOL_F16_OUT, TOL_F32_OUT, TOL_F64_OUT, gemm_rel_err
from oracle import cpu_ref as R
from rocwmma_b200 import api
from rocwmma_b200 import datagen as G

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = api.HostContext()
    yield c
    c.close()


@pytest.mark.parametrize("m,n,k,out_np,beta", [(2500, 512, 256, np.float16, 1.0), (1024, 768, 128, np.float32, 2.0),
                                               (3000, 264, 72, np.float16, 0.0)])
def test_gemm_f16_host_row_block_pipeline(ctx, m, n, k, out_np, beta):
    """m spans several 1024-row blocks (ragged last block): every block goes through copy-in / multiply / copy-out."""
    a = G.uniform_np(1, (m, k), np.float16); b = G.uniform_np(2, (k, n), np.float16); c = G.uniform_np(3, (m, n), out_np)
    bs = np.ascontiguousarray(b.T)
    d = np.full((m, n), np.nan, dtype=out_np)
    for _ in range(2):  # second call reuses the cached device buffers, streams and events
        d[:] = np.nan
        ctx.gemm_f16(m, n, k, a, bs, c if beta else None, d, k, k, n, n, 1.5, beta, 0 if out_np == np.float16 else 1)
        ref = R.gemm(R.port(), m, n, k, a.ravel(), bs.ravel(), c.ravel() if beta else None, 1.5, beta, out_np).reshape(m, n)
        bound = R.gemm_abs_bound(m, n, k, a, b, c if beta else None, 1.5, beta)
        assert gemm_rel_err(d, ref, bound) <= (TOL_F16_OUT if out_np == np.float16 else TOL_F32_OUT)


_HOST_LAYOUTS = [(la, lb, lcd) for la in (0, 1) for lb in (0, 1) for lcd in (0, 1)]


@pytest.mark.parametrize("la,lb,lcd", _HOST_LAYOUTS, ids=["".join("RC"[x] for x in t) for t in _HOST_LAYOUTS])
def test_gemm_host_all_layouts(ctx, la, lb, lcd):
    """Every layout combination through the host-buffer drivers (the reference's NN / NT / TN / TT sweep): row-major
    A / C / D are pipelined over row chunks (m spans several), the other layouts go whole; fp16 and int8."""
    m, n, k = 2304, 320, 256
    store = lambda x, col: np.ascontiguousarray(x.T if col else x)
    lda, ldb, ldcd = (m if la else k), (k if lb else n), (m if lcd else n)
    a = G.uniform_np(1, (m, k), np.float16); b = G.uniform_np(2, (k, n), np.float16); c = G.uniform_np(3, (m, n), np.float16)
    sa, sb, sc = store(a, la), store(b, lb), store(c, lcd)
    d = np.full(sc.shape, np.nan, np.float16)
    ctx.gemm_f16(m, n, k, sa, sb, sc, d, lda, ldb, ldcd, ldcd, 1.5, 0.5, 0, la, lb, lcd)
    ref = R.gemm(R.port(), m, n, k, sa.ravel(), sb.ravel(), sc.ravel(), 1.5, 0.5, np.float16, la, lb, lcd, lcd)
    bound = store(R.gemm_abs_bound(m, n, k, a, b, c, 1.5, 0.5), lcd).ravel()
    assert gemm_rel_err(d.ravel(), ref, bound) <= TOL_F16_OUT
    ai = G.int8_np(1, (m, k)); bi = G.int8_np(2, (k, n)); ci = G.int8_np(3, (m, n)).astype(np.int32) * 77
    sa, sb, sc = store(ai, la), store(bi, lb), store(ci, lcd)
    di = np.zeros(sc.shape, np.int32)
    ctx.gemm_i8(m, n, k, sa, sb, sc, di, lda, ldb, ldcd, ldcd, 2, -1, la, lb, lcd)
    assert np.array_equal(di.ravel(), R.gemm(R.port(), m, n, k, sa.ravel(), sb.ravel(), sc.ravel(), 2, -1, np.int32, la, lb, lcd, lcd))


def test_gemm_f16_host_in_place(ctx):
    m, n, k = 2100, 256, 128
    a = G.uniform_np(1, (m, k), np.float16); b = G.uniform_np(2, (k, n), np.float16); c = G.uniform_np(3, (m, n), np.float16)
    bs = np.ascontiguousarray(b.T)
    cd = c.copy()
    ctx.gemm_f16(m, n, k, a, bs, cd, cd, k, k, n, n, 1.0, 1.0, 0)
    ref = R.gemm(R.port(), m, n, k, a.ravel(), bs.ravel(), c.ravel(), 1.0, 1.0, np.float16).reshape(m, n)
    assert gemm_rel_err(cd, ref, R.gemm_abs_bound(m, n, k, a, b, c, 1.0, 1.0)) <= TOL_F16_OUT


def test_gemm_i8_host_bit_exact(ctx):
    m, n, k = 2300, 320, 512
    a = G.int8_np(1, (m, k)); bs = np.ascontiguousarray(G.int8_np(2, (k, n)).T)
    c = G.int8_np(3, (m, n)).astype(np.int32) * 99
    d = np.zeros((m, n), np.int32)
    ctx.gemm_i8(m, n, k, a, bs, c, d, k, k, n, n, 2, -3)
    assert np.array_equal(d, R.gemm(R.port(), m, n, k, a.ravel(), bs.ravel(), c.ravel(), 2, -3, np.int32).reshape(m, n))


def test_dlrm_and_gemv_host(ctx):
    B, m, k, w = 300, 27, 128, 480
    x = np.zeros((B, 32, k), np.float16); x[:, :m] = G.normal_np(4, (B, m, k), 0.25, np.float16)
    up = np.zeros((B, w), np.float16); up[:, :479] = G.normal_np(5, (B, 479), 0.1, np.float16)
    out = np.zeros((B, w), np.float16); grad = np.zeros((B, 32, k), np.float16); mlp = np.zeros((B, k), np.float16)
    ctx.dlrm_fwd(x, out, m, 32, k, B, w)
    ctx.dlrm_bwd(x, up, grad, mlp, m, 32, k, B, w, False)
    xr = np.ascontiguousarray(x[:, :m])
    rf = R.dlrm_fwd(R.port(), xr, m, k, B)
    rg, rm = R.dlrm_bwd(R.port(), xr, np.ascontiguousarray(up[:, :479]), m, k, B)
    assert np.abs(out[:, :479].astype(np.float32) - rf.astype(np.float32)).max() <= 2e-2
    assert np.abs(grad[:, :m].astype(np.float32) - rg.astype(np.float32)).max() <= 2e-2
    assert np.array_equal(mlp, rm) and (grad[:, m:] == 0).all()
    for dt, tol, dbl in ((np.float32, TOL_F32_OUT, False), (np.float64, TOL_F64_OUT, True)):
        M, N = 700, 1536
        a = G.uniform_np(6, (M, N), dt); xv = G.uniform_np(7, (N,), dt); y0 = G.uniform_np(8, (M,), dt)
        y = y0.copy()
        ctx.gemv(M, N, a, N, xv, y, 1.5, 0.5, double=dbl)
        ref = R.gemv(R.port(), M, N, a.ravel(), xv, y0, dt(1.5), dt(0.5))
        bound = 1.5 * (np.abs(a.astype(np.float64)) @ np.abs(xv.astype(np.float64))) + 0.5 * np.abs(y0)
        assert np.max(np.abs(y.astype(np.float64) - ref) / bound) <= tol


def test_host_driver_rejects_bad_layout_flags_and_pitches(ctx):
    """Layout flags outside {0, 1} and a leading dimension smaller than the column it strides are argument errors."""
    from rocwmma_b200 import _lib
    import ctypes as C
    L = _lib.lib()
    a = np.zeros((128, 64), np.float16); d = np.zeros((128, 128), np.float16)
    p = lambda x: C.c_void_p(x.ctypes.data)
    assert L.b200wmma_gemm_f16_host(ctx._h, 128, 128, 64, p(a), p(a), None, p(d), 128, 64, 128, 128, 1.0, 0.0, 2, 1, 0, 0) == 1
    # column-major A needs lda >= m
    assert L.b200wmma_gemm_f16_host(ctx._h, 128, 128, 64, p(a), p(a), None, p(d), 64, 64, 128, 128, 1.0, 0.0, 1, 1, 0, 0) == 1
    assert b"leading dimension" in L.b200wmma_last_error_string()
