"""rocWMMA's own test GEMM kernels (test/gemm/gemm_PGR0_LB0_MP0_{SB,MB}_NC and gemm_PGR1_LB2_MP0_MB_CP,
device/kernel_device_func.hpp), compiled unmodified against this repository's <rocwmma/rocwmma.hpp>
(tests/csrc/ref_kernel_unit.cu, built by __graft_entry__.build() where the reference tree exists), run on the GPU
and checked against the oracle.  This is the header drop-in claim exercised on the reference's own source:
fragment, fill_fragment, load / store_matrix_sync, mma_sync, synchronize_workgroup, MappingUtil and the Coord2d
arithmetic; for the cooperative kernel also load / store_matrix_coop_sync, applyTranspose / applyDataLayout,
WaveSpace, the fragment accessors and the reference's whole block- / wave- / workgroup-level configuration
catalogue (test/gemm/gemm_config.hpp) with its global and shared-memory mappings."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from conftest import TOL_F16_OUT, TOL_F32_OUT, TOL_F64_OUT, gemm_rel_err
from gpu_util import dev, nan_filled
from oracle import cpu_ref as R
from rocwmma_b200 import datagen as G

pytestmark = pytest.mark.gpu
LIB = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libref_kernel_unit.so")

# variant -> (input dtype, output dtype, layout A, layout B, tolerance or None for exact)
VARIANTS = {
    0: (np.float16, np.float32, 0, 1, TOL_F32_OUT),
    1: (np.float16, np.float16, 1, 0, TOL_F16_OUT),
    2: (np.float32, np.float32, 0, 1, 5e-6),
    3: (np.float64, np.float64, 0, 1, TOL_F64_OUT),
    4: (np.int8, np.int32, 0, 1, None),
    5: (np.float16, np.float32, 0, 1, TOL_F32_OUT),
}


def _lib():
    if not os.path.exists(LIB):
        pytest.skip("tests/libref_kernel_unit.so is built only where the reference tree is present")
    lib = C.CDLL(LIB)
    lib.ref_test_gemm.restype = C.c_int
    lib.ref_test_gemm.argtypes = [C.c_int, C.c_int, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p,
                                  C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_double, C.c_double]
    lib.ref_test_gemm_coop.restype = C.c_int
    lib.ref_test_gemm_coop.argtypes = [C.c_int, C.c_int, C.c_int, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p,
                                       C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_double,
                                       C.c_double]
    return lib


def _case(variant_table, variant, m, n, k):
    in_t, out_t, la, lb, tol = variant_table[variant]
    if in_t == np.int8:
        a, b = G.int8_np(1, (m, k)), G.int8_np(2, (k, n))
        c = G.int8_np(3, (m, n)).astype(np.int32) * 100
        alpha, beta = 2, -1
    else:
        a, b, c = G.uniform_np(1, (m, k), in_t), G.uniform_np(2, (k, n), in_t), G.uniform_np(3, (m, n), out_t)
        alpha, beta = 2.0, 0.5
    store = lambda x, col: np.ascontiguousarray(x.T if col else x)
    sa, sb = store(a, la), store(b, lb)
    lda, ldb = (m if la else k), (k if lb else n)
    d = nan_filled((m, n), {np.float32: torch.float32, np.float16: torch.float16, np.float64: torch.float64,
                            np.int32: torch.int32}[out_t])
    return in_t, out_t, la, lb, tol, a, b, c, sa, sb, lda, ldb, d, alpha, beta


def _check(got, case, m, n, k):
    in_t, out_t, la, lb, tol, a, b, c, sa, sb, lda, ldb, d, alpha, beta = case
    ref = R.gemm(R.port(), m, n, k, sa.ravel(), sb.ravel(), c.ravel(), alpha, beta, out_t, la, lb, 0, 0).reshape(m, n)
    if tol is None:
        assert np.array_equal(got, ref)
    else:
        assert gemm_rel_err(got, ref, R.gemm_abs_bound(m, n, k, a, b, c, alpha, beta)) <= tol


# the cooperative kernel's variants: as above except 4 (BlockK 32) and 5 (both inputs column-major)
COOP_VARIANTS = dict(VARIANTS)
COOP_VARIANTS[5] = (np.float16, np.float32, 1, 1, TOL_F32_OUT)
COOP_CONFIGS = ["block_LdsNT", "wave_LdsNT", "workgroup_LdsNT", "block_LdsTN", "wave_LdsTN", "workgroup_LdsTN", "block_LdsRF"]


@pytest.mark.parametrize("lds_col", [0, 1], ids=["lds_row_major", "lds_col_major"])
@pytest.mark.parametrize("config", range(7), ids=COOP_CONFIGS)
@pytest.mark.parametrize("variant", sorted(COOP_VARIANTS))
def test_reference_cooperative_kernel_on_these_headers(variant, config, lds_col):
    """gemm_PGR1_LB2_MP0_MB_CP: global prefetch, two shared-memory buffers, cooperative loads - in each of the
    reference's seven cooperation / shared-memory configurations and both shared-memory data layouts."""
    lib = _lib()
    m, n, k = 256, 512, 96  # multiples of every variant's macro tile (at most 128 x 256) and K step
    case = _case(COOP_VARIANTS, variant, m, n, k)
    in_t, out_t, la, lb, tol, a, b, c, sa, sb, lda, ldb, d, alpha, beta = case
    da, db, dc = dev(sa), dev(sb), dev(c)
    rc = lib.ref_test_gemm_coop(config, lds_col, variant, m, n, k, da.data_ptr(), db.data_ptr(), dc.data_ptr(), d.data_ptr(),
                                lda, ldb, n, n, float(alpha), float(beta))
    torch.cuda.synchronize()
    assert rc == 0
    _check(d.cpu().numpy(), case, m, n, k)


def test_reference_cooperative_kernel_rejects_ragged_sizes():
    """The kernel has no tail handling; like the reference's checkSizes() the wrapper refuses sizes that are not whole
    macro tiles instead of launching."""
    lib = _lib()
    assert lib.ref_test_gemm_coop(0, 0, 0, 100, 64, 64, None, None, None, None, 64, 64, 64, 64, 1.0, 0.0) == -2


@pytest.mark.parametrize("multi", [0, 1], ids=["single_block", "multi_block"])
@pytest.mark.parametrize("variant", sorted(VARIANTS))
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (512, 384, 208)])
def test_reference_test_kernels_on_these_headers(variant, multi, m, n, k):
    lib = _lib()
    in_t, out_t, la, lb, tol = VARIANTS[variant]
    if in_t == np.int8:
        a, b = G.int8_np(1, (m, k)), G.int8_np(2, (k, n))
        c = G.int8_np(3, (m, n)).astype(np.int32) * 100
        alpha, beta = 2, -1
    else:
        a, b, c = G.uniform_np(1, (m, k), in_t), G.uniform_np(2, (k, n), in_t), G.uniform_np(3, (m, n), out_t)
        alpha, beta = 2.0, 0.5
    store = lambda x, col: np.ascontiguousarray(x.T if col else x)
    sa, sb = store(a, la), store(b, lb)
    lda, ldb = (m if la else k), (k if lb else n)
    d = nan_filled((m, n), {np.float32: torch.float32, np.float16: torch.float16, np.float64: torch.float64,
                            np.int32: torch.int32}[out_t])
    da, db, dc = dev(sa), dev(sb), dev(c)
    rc = lib.ref_test_gemm(variant, multi, m, n, k, da.data_ptr(), db.data_ptr(), dc.data_ptr(), d.data_ptr(), lda, ldb, n, n,
                           float(alpha), float(beta))
    torch.cuda.synchronize()
    assert rc == 0
    ref = R.gemm(R.port(), m, n, k, sa.ravel(), sb.ravel(), c.ravel(), alpha, beta, out_t, la, lb, 0, 0).reshape(m, n)
    got = d.cpu().numpy()
    if tol is None:
        assert np.array_equal(got, ref)
    else:
        assert gemm_rel_err(got, ref, R.gemm_abs_bound(m, n, k, a, b, c, alpha, beta)) <= tol
