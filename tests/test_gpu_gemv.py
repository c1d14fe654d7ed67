"""GPU parity of the streaming GEMV kernels (through the C ABI) against the CPU oracle.
Metric: |y - ref| / (|alpha| sum|a||x| + |beta||y0|) <= 1e-3 (fp32) / 1e-12 (fp64)."""
import os

import numpy as np
import pytest
import torch

import gen_golden as GG
from conftest import TOL_F32_OUT, TOL_F64_OUT
from gpu_util import assert_status_ok, dev
from oracle import cpu_ref as R
from rocwmma_b200 import api
from rocwmma_b200 import datagen as G

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def rel_err(got, ref, a, x, y0, alpha, beta):
    bound = abs(alpha) * (np.abs(a.astype(np.float64)) @ np.abs(x.astype(np.float64))) + abs(beta) * np.abs(y0.astype(np.float64))
    assert np.isfinite(got).all()
    return float(np.max(np.abs(got.astype(np.float64) - ref.astype(np.float64)) / np.maximum(bound, 1e-300)))


def run(m, n, dt, col, lda_pad=0, alpha=1.5, beta=0.5):
    a = G.uniform_np(G.SEED_GEMV_A, (m, n), dt)
    x = G.uniform_np(G.SEED_GEMV_X, (n,), dt)
    y0 = G.uniform_np(G.SEED_GEMV_Y, (m,), dt)
    store = np.ascontiguousarray(a.T if col else a)
    lda = store.shape[1] + lda_pad
    padded = np.full((store.shape[0], lda), np.nan, dtype=dt)
    padded[:, :store.shape[1]] = store
    y = dev(np.concatenate([y0, np.full(8, 123.0, dtype=dt)]))  # guard elements after y
    api.gemv(m, n, dev(padded), lda, dev(x), y, alpha, beta, api.COL_MAJOR if col else api.ROW_MAJOR)
    assert_status_ok()
    yh = y.cpu().numpy()
    assert (yh[m:] == 123.0).all()
    ref = R.gemv(R.port(), m, n, store.ravel(), x, y0, dt(alpha), dt(beta), col)
    return rel_err(yh[:m], ref, a, x, y0, alpha, beta)


@pytest.mark.parametrize("dt,tol", [(np.float32, TOL_F32_OUT), (np.float64, TOL_F64_OUT)], ids=["f32", "f64"])
@pytest.mark.parametrize("m,n,lda_pad", [(1, 1, 0), (4, 1024, 0), (37, 200, 0), (1000, 4096, 0), (130, 515, 1),
                                         (64, 2048, 4), (4099, 1000, 0)])
@pytest.mark.parametrize("col", [False, True], ids=["row", "col"])
def test_gemv_vs_oracle(dt, tol, m, n, lda_pad, col):
    assert run(m, n, dt, col, lda_pad) <= tol


@pytest.mark.parametrize("dt,tol", [(np.float32, TOL_F32_OUT), (np.float64, TOL_F64_OUT)], ids=["f32", "f64"])
@pytest.mark.parametrize("m,n,lda_pad", [(5, 1024, 0), (130, 515, 1), (1001, 4096, 4)])
def test_gemv_four_rows_per_cta_kernel(dt, tol, m, n, lda_pad):
    """The row-major kernel's other shape (four rows of A per thread block, ragged last block), selected by tuning key."""
    api.set_tuning("gemv_rows", 4)
    try:
        assert run(m, n, dt, False, lda_pad) <= tol
    finally:
        api.set_tuning("gemv_rows", 0)


@pytest.mark.parametrize("dt,tol,vn", [(np.float32, TOL_F32_OUT, 2), (np.float32, TOL_F32_OUT, 4), (np.float64, TOL_F64_OUT, 2)],
                         ids=["f32x2", "f32x4", "f64x2"])
@pytest.mark.parametrize("m,n,lda_pad", [(130, 515, 2), (1000, 4096, 0), (4099, 1000, 1)])
def test_gemv_col_major_wider_lanes(dt, tol, vn, m, n, lda_pad):
    """The column-major kernel with 2 or 4 consecutive rows per lane (selected by tuning key; where the pitch does not
    allow the vector loads the library falls back to one row per lane), ragged last block included."""
    api.set_tuning("gemv_col_vn", vn)
    try:
        assert run(m, n, dt, True, lda_pad) <= tol
    finally:
        api.set_tuning("gemv_col_vn", 0)


def test_gemv_reference_fixtures():
    gold = np.load(os.path.join(GOLD, "gemv_ref.npz"))
    for case in GG.GEMV_CASES:
        name, m, n, dt, col = case
        a, x, y0, sa = GG.gemv_inputs(case)
        y = dev(y0)
        lda = m if col else n
        api.gemv(m, n, dev(sa), lda, dev(x), y, 1.5, 0.5, api.COL_MAJOR if col else api.ROW_MAJOR)
        tol = TOL_F32_OUT if dt == np.float32 else TOL_F64_OUT
        assert rel_err(y.cpu().numpy(), gold[name], a, x, y0, 1.5, 0.5) <= tol, name
    assert_status_ok()


@pytest.mark.parametrize("dt,tdt,tol", [(np.float32, torch.float32, TOL_F32_OUT), (np.float64, torch.float64, TOL_F64_OUT)],
                         ids=["f32", "f64"])
def test_gemv_full_size_32768(dt, tdt, tol):
    """M=N=32768 (4 GiB / 8 GiB matrix): 64 seeded-random rows against the oracle, plus linearity over
    the whole vector: gemv(A, x, y; alpha, beta) - beta*y == alpha * gemv(A, x, 0; 1, 0)."""
    m = n = 32768
    a = G.fill_torch(torch.empty((m, n), dtype=tdt, device="cuda"), G.SEED_GEMV_A, "uniform")
    x = G.fill_torch(torch.empty(n, dtype=tdt, device="cuda"), G.SEED_GEMV_X, "uniform")
    y0 = G.fill_torch(torch.empty(m, dtype=tdt, device="cuda"), G.SEED_GEMV_Y, "uniform")
    y = y0.clone()
    api.gemv(m, n, a, n, x, y, 1.5, 0.5)
    z = torch.zeros_like(y0)
    api.gemv(m, n, a, n, x, z, 1.0, 0.0)
    assert_status_ok()
    lin = (y - 0.5 * y0 - 1.5 * z).abs().max().item()
    assert lin <= (1e-3 if dt == np.float32 else 1e-11)
    rows = np.unique((G.raw_np(55, 64) % np.uint64(m)).astype(np.int64))
    idx = torch.from_numpy(rows).cuda()
    ah, xh, y0h = a[idx].cpu().numpy(), x.cpu().numpy(), y0[idx].cpu().numpy()
    ref = R.gemv(R.port(), len(rows), n, ah.ravel(), xh, y0h, dt(1.5), dt(0.5))
    assert rel_err(y[idx].cpu().numpy(), ref, ah, xh, y0h, 1.5, 0.5) <= tol
