"""GPU tests of the rocWMMA-compatible fragment API (include/rocwmma/*.hpp) through the test kernels
in tests/csrc/frag_unit.cu, and of the two fragment-API GEMMs exported by the C ABI.

Shapes of the checks follow the reference's unit suites: load->store round trip reproduces the
input; cooperative round trip with 1..8 waves; fill; stores leave everything outside the block
untouched (marker check); naive one-block-per-wave GEMM against the CPU oracle for every
supported type pair (int8 bit-exact; floating point within the stated tolerances)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from conftest import TOL_F16_OUT, TOL_F32_OUT, TOL_F64_OUT, gemm_rel_err
from gpu_util import assert_status_ok, dev, nan_filled
from oracle import cpu_ref as R
from rocwmma_b200 import api
from rocwmma_b200 import datagen as G

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))

# id -> (numpy dtype, layout col_major?) ; must match ROUNDTRIP_CASES in tests/csrc/frag_unit.cu
RT_CASES = {
    0: (np.float16, 0), 1: (np.float16, 1), 2: (np.float16, 0), 3: (np.float16, 1), 4: (np.float32, 0),
    5: (np.float32, 1), 6: (np.int8, 0), 7: (np.int8, 1), 8: (np.int8, 1), 9: (np.int32, 0),
    10: (np.float64, 0), 11: (np.float64, 0), 12: (np.float64, 1), 13: (np.float32, 0), 14: (np.float32, 1),
    15: (np.float16, 1), 16: (np.float16, 0), 17: (np.float16, 0), 18: (np.float16, 1), 19: (np.float16, 0),
    20: (np.float16, 1), 21: (np.int8, 0), 22: (np.float16, 0),
}
# id -> (in dtype, out dtype, A col?, B col?, tol or None for exact)
GEMM_CASES = {
    0: (np.float16, np.float32, 0, 1, TOL_F32_OUT), 1: (np.float16, np.float16, 0, 1, TOL_F16_OUT),
    2: (np.float16, np.float32, 1, 0, TOL_F32_OUT), 3: (np.float16, np.float32, 0, 0, TOL_F32_OUT),
    4: (np.float16, np.float32, 1, 1, TOL_F32_OUT), 5: (np.float16, np.float16, 0, 1, 4 * TOL_F16_OUT),
    6: (np.int8, np.int32, 0, 1, None), 7: (np.int8, np.int32, 1, 0, None),
    8: (np.float64, np.float64, 0, 1, TOL_F64_OUT), 9: (np.float64, np.float64, 1, 0, TOL_F64_OUT),
    10: (np.float32, np.float32, 0, 1, 1e-5), 11: (np.float32, np.float32, 1, 0, 1e-5),
    12: (np.float16, np.float32, 0, 1, TOL_F32_OUT), 13: (np.float16, np.float32, 0, 1, TOL_F32_OUT),
    # the reference's minimum BlockK (8 for 16-bit inputs, 4 for fp32), bfloat16 inputs, a BlockK that is not a multiple of 16
    14: (np.float16, np.float32, 0, 1, TOL_F32_OUT), 15: (np.float16, np.float16, 1, 0, TOL_F16_OUT),
    16: (np.float32, np.float32, 0, 1, 1e-5), 17: (np.float32, np.float32, 1, 0, 1e-5),
    18: ("bf16", np.float32, 0, 1, TOL_F32_OUT), 19: ("bf16", np.float32, 1, 0, TOL_F32_OUT),
    20: ("bf16", np.float32, 0, 0, 2e-2),  # bf16 compute: the accumulator is rounded to bf16 after every K step
    21: (np.float16, np.float32, 0, 1, TOL_F32_OUT),
    # OCP fp8 inputs (exact products, fp32 accumulation) and xfloat32 (inputs rounded to TF32: 2^-11 relative each)
    22: ("e4m3", np.float32, 0, 1, TOL_F32_OUT), 23: ("e5m2", np.float32, 1, 0, TOL_F32_OUT),
    24: ("xf32", np.float32, 0, 1, 2e-3), 25: ("xf32", np.float32, 1, 0, 2e-3),
    # the reference's minimum K of 32 x 32 blocks for int8 (8) and fp32 (2): atoms without an mma.sync shape of their own
    26: (np.int8, np.int32, 0, 1, None), 27: (np.int8, np.int32, 1, 0, None),
    28: (np.float32, np.float32, 0, 1, 1e-5), 29: (np.float32, np.float32, 1, 0, 1e-5),
    30: ("xf32", np.float32, 0, 0, 2e-3), 31: (np.int8, np.int32, 0, 0, None),
}
_TORCH_LOWP = {"bf16": torch.bfloat16, "e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


@pytest.fixture(scope="module")
def unit():
    path = os.path.join(HERE, "libfrag_unit.so")
    assert os.path.exists(path), "tests/libfrag_unit.so missing: run __graft_entry__.build()"
    h = C.CDLL(path)
    u32, vp = C.c_uint32, C.c_void_p
    h.frag_unit_block_shape.argtypes = [C.c_int] + [C.POINTER(u32)] * 4
    h.frag_unit_roundtrip.argtypes = [C.c_int, vp, vp, u32, u32, u32, u32, u32, u32]
    h.frag_unit_coop_roundtrip.argtypes = [C.c_int, vp, vp, u32, u32, u32, u32, u32, C.c_int]
    h.frag_unit_fill.argtypes = [C.c_int, vp, u32, C.c_double]
    h.frag_unit_transpose.argtypes = [C.c_int, vp, vp, u32]
    h.frag_unit_gemm.argtypes = [C.c_int, u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, u32, C.c_double, C.c_double, u32, u32]
    h.frag_unit_gemm_block.argtypes = [C.c_int] + [C.POINTER(u32)] * 3
    return h


def shape_of(unit, cid):
    v = [C.c_uint32() for _ in range(4)]
    assert unit.frag_unit_block_shape(cid, *[C.byref(x) for x in v]) == 0
    return tuple(x.value for x in v)


def rand_matrix(rows, cols, dt, seed):
    if np.issubdtype(dt, np.integer):
        return (G.raw_np(seed, rows * cols) % np.uint64(251)).astype(np.int64).astype(dt).reshape(rows, cols)
    return G.uniform_np(seed, (rows, cols), dt)


MARK = {np.float16: 777.0, np.float32: 777.0, np.float64: 777.0, np.int8: 99, np.int32: 99999}


def stored(mat, col, ld, dt):
    """Place logical `mat` into a padded buffer with leading dimension ld in the given layout, marker elsewhere."""
    r, c = mat.shape
    outer, inner = (c, r) if col else (r, c)
    buf = np.full((outer + 3, ld), MARK[dt], dtype=dt)  # 3 guard lines after the matrix
    buf[:outer, :inner] = mat.T if col else mat
    return buf


@pytest.mark.parametrize("cid", sorted(RT_CASES))
@pytest.mark.parametrize("waves", [(1, 1), (2, 2), (4, 1)], ids=["1w", "2x2w", "4x1w"])
def test_load_store_roundtrip_and_contamination(unit, cid, waves):
    dt, col = RT_CASES[cid]
    bh, bw, eb, ne = shape_of(unit, cid)
    assert eb == np.dtype(dt).itemsize and ne == bh * bw // 32  # num_elements = BlockDim * BlockK / 32
    rows, cols = bh * 3, bw * 2
    mat = rand_matrix(rows, cols, dt, 100 + cid)
    inner = rows if col else cols
    ld_src, ld_dst = inner + 8, inner + 24
    src = stored(mat, col, ld_src, dt)
    dst = dev(np.full(((cols if col else rows) + 3, ld_dst), MARK[dt], dtype=dt))
    assert unit.frag_unit_roundtrip(cid, dev(src).data_ptr(), dst.data_ptr(), rows, cols, ld_src, ld_dst, *waves) == 0
    got = dst.cpu().numpy()
    expect = stored(mat, col, ld_dst, dt)
    assert np.array_equal(got, expect)  # block reproduced AND every padding / guard element untouched


def test_load_store_unaligned_base(unit):
    """Odd element offsets and leading dimensions force the scalar path of load/store."""
    for cid in (0, 3, 4, 6, 12):
        dt, col = RT_CASES[cid]
        bh, bw, _, _ = shape_of(unit, cid)
        mat = rand_matrix(bh, bw, dt, 300 + cid)
        inner = bh if col else bw
        ld = inner + 3
        src = np.full((max(bh, bw) + 4) * ld + 1, MARK[dt], dtype=dt)
        body = stored(mat, col, ld, dt)
        src[1:1 + body.size] = body.ravel()
        s = dev(src)
        d = dev(np.full(src.shape, MARK[dt], dtype=dt))
        es = np.dtype(dt).itemsize
        assert unit.frag_unit_roundtrip(cid, s.data_ptr() + es, d.data_ptr() + es, bh, bw, ld, ld, 1, 1) == 0
        assert np.array_equal(d.cpu().numpy(), src)


@pytest.mark.parametrize("cid", [0, 3, 6, 8, 15, 16, 17, 18, 19, 21])
@pytest.mark.parametrize("waves", [(1, 1), (2, 1), (2, 2), (4, 2), (3, 1)], ids=["1", "2", "4", "8", "3"])
@pytest.mark.parametrize("default_args", [0, 1])
def test_coop_roundtrip(unit, cid, waves, default_args):
    dt, col = RT_CASES[cid]
    bh, bw, _, _ = shape_of(unit, cid)
    blocks = 3
    rows, cols = bh, bw * blocks
    mat = rand_matrix(rows, cols, dt, 200 + cid)
    inner = rows if col else cols
    ld_src, ld_dst = inner + 8, inner + 16
    src = stored(mat, col, ld_src, dt)
    dst = dev(np.full(((cols if col else rows) + 3, ld_dst), MARK[dt], dtype=dt))
    assert unit.frag_unit_coop_roundtrip(cid, dev(src).data_ptr(), dst.data_ptr(), ld_src, ld_dst, blocks, *waves, default_args) == 0
    assert np.array_equal(dst.cpu().numpy(), stored(mat, col, ld_dst, dt))


@pytest.mark.parametrize("cid", [0, 5, 6, 9, 12, 13, 17, 20])
def test_fill_fragment(unit, cid):
    dt, col = RT_CASES[cid]
    bh, bw, _, _ = shape_of(unit, cid)
    inner = bh if col else bw
    ld = inner + 8
    dst = dev(np.full(((bw if col else bh) + 3, ld), MARK[dt], dtype=dt))
    assert unit.frag_unit_fill(cid, dst.data_ptr(), ld, -3.0) == 0
    assert np.array_equal(dst.cpu().numpy(), stored(np.full((bh, bw), -3, dtype=dt), col, ld, dt))


@pytest.mark.parametrize("cid,shape,dt", [(0, (16, 16), np.float16), (1, (32, 64), np.int8), (2, (16, 8), np.float64)])
def test_apply_transpose_is_a_reinterpretation(unit, cid, shape, dt):
    """A (row major, M x K) and its transpose as matrix_b (column major, K x M) are the same memory."""
    mat = rand_matrix(shape[0], shape[1], dt, 400 + cid)
    ld = shape[1]
    dst = dev(np.zeros_like(mat))
    assert unit.frag_unit_transpose(cid, dev(mat).data_ptr(), dst.data_ptr(), ld) == 0
    assert np.array_equal(dst.cpu().numpy(), mat)


@pytest.mark.parametrize("cid", sorted(GEMM_CASES))
def test_naive_fragment_gemm(unit, cid):
    it, ot, acol, bcol, tol = GEMM_CASES[cid]
    v = [C.c_uint32() for _ in range(3)]
    assert unit.frag_unit_gemm_block(cid, *[C.byref(x) for x in v]) == 0
    bm, bn, bk = (x.value for x in v)
    m, n, k = bm * 5, bn * 3, bk * 7
    if it == np.int8:
        a = G.int8_np(1, (m, k)); b = G.int8_np(2, (k, n)); c = G.int8_np(3, (m, n)).astype(np.int32) * 7
        alpha, beta = 2, 3
    elif it in _TORCH_LOWP:
        # rounded once to the narrow type: these ARE the inputs; the oracle gets them widened exactly to fp32
        a = torch.from_numpy(G.uniform_np(1, (m, k), np.float32)).to(_TORCH_LOWP[it]).to(torch.float32).numpy()
        b = torch.from_numpy(G.uniform_np(2, (k, n), np.float32)).to(_TORCH_LOWP[it]).to(torch.float32).numpy()
        c = G.uniform_np(3, (m, n), ot)
        alpha, beta = 2.0, 0.5
    elif it == "xf32":
        a = G.uniform_np(1, (m, k), np.float32); b = G.uniform_np(2, (k, n), np.float32); c = G.uniform_np(3, (m, n), ot)
        alpha, beta = 2.0, 0.5
    else:
        a = G.uniform_np(1, (m, k), it); b = G.uniform_np(2, (k, n), it); c = G.uniform_np(3, (m, n), ot)
        alpha, beta = 2.0, 0.5
    sa = np.ascontiguousarray(a.T if acol else a)
    sb = np.ascontiguousarray(b.T if bcol else b)
    d = dev(np.full((m, n), MARK[ot], dtype=ot))
    dev_in = (lambda x: dev(x).to(_TORCH_LOWP[it])) if it in _TORCH_LOWP else dev
    da, db = dev_in(sa), dev_in(sb)
    assert unit.frag_unit_gemm(cid, m, n, k, da.data_ptr(), db.data_ptr(), dev(c).data_ptr(), d.data_ptr(),
                               sa.shape[1], sb.shape[1], n, n, alpha, beta, 2, 2) == 0
    ref = R.gemm(R.port(), m, n, k, sa.ravel(), sb.ravel(), c.ravel(), alpha, beta, ot, acol, bcol).reshape(m, n)
    got = d.cpu().numpy()
    if tol is None:
        assert np.array_equal(got, ref)
    else:
        bound = R.gemm_abs_bound(m, n, k, a, b, c, alpha, beta)
        assert gemm_rel_err(got, ref, bound) <= tol


@pytest.mark.parametrize("out_np", [np.float32, np.float16], ids=["f32out", "f16out"])
def test_simple_hgemm_config1(out_np):
    """The fragment-API correctness gate: M=N=K=1024, A row / B col fp16, C/D fp32 (and the sample's own
    fp16), alpha=beta=2, 16x16x16 blocks, full-matrix check against the oracle."""
    m = n = k = 1024
    a = G.uniform_np(G.SEED_A, (m, k), np.float16); b = G.uniform_np(G.SEED_B, (k, n), np.float16)
    c = G.uniform_np(G.SEED_C, (m, n), out_np)
    bs = np.ascontiguousarray(b.T)
    d = nan_filled((m, n), torch.float32 if out_np == np.float32 else torch.float16)
    api.simple_hgemm(m, n, k, dev(a), dev(bs), dev(c), d, k, k, n, n, 2.0, 2.0)
    assert_status_ok()
    ref = R.gemm(R.port(), m, n, k, a.ravel(), bs.ravel(), c.ravel(), 2.0, 2.0, out_np).reshape(m, n)
    bound = R.gemm_abs_bound(m, n, k, a, b, c, 2.0, 2.0)
    assert gemm_rel_err(d.cpu().numpy(), ref, bound) <= (TOL_F32_OUT if out_np == np.float32 else TOL_F16_OUT)


@pytest.mark.parametrize("np_t", [np.float32, np.float64], ids=["sgemm", "dgemm"])
@pytest.mark.parametrize("m,n,k", [(64, 64, 16), (256, 384, 208), (1024, 512, 512)])
def test_simple_sgemm_dgemm(np_t, m, n, k):
    """The fp32 / fp64 forms of the naive fragment GEMM (samples/simple_sgemm.cpp, samples/simple_dgemm.cpp):
    fp32 fragments multiply through three TF32 products, so they are held to 5e-6, far inside the 1e-3 acceptance bound for fp32 outputs."""
    a = G.uniform_np(G.SEED_A, (m, k), np_t); b = G.uniform_np(G.SEED_B, (k, n), np_t); c = G.uniform_np(G.SEED_C, (m, n), np_t)
    bs = np.ascontiguousarray(b.T)
    d = nan_filled((m, n), torch.float32 if np_t == np.float32 else torch.float64)
    fn = api.simple_sgemm if np_t == np.float32 else api.simple_dgemm
    fn(m, n, k, dev(a), dev(bs), dev(c), d, k, k, n, n, 2.0, 2.0)
    assert_status_ok()
    ref = R.gemm(R.port(), m, n, k, a.ravel(), bs.ravel(), c.ravel(), 2.0, 2.0, np_t).reshape(m, n)
    bound = R.gemm_abs_bound(m, n, k, a, b, c, 2.0, 2.0)
    assert gemm_rel_err(d.cpu().numpy(), ref, bound) <= (5e-6 if np_t == np.float32 else TOL_F64_OUT)


@pytest.mark.parametrize("m,n,k", [(128, 128, 16), (256, 384, 512), (1024, 1024, 1024)])
def test_perf_hgemm_fragment_pipeline(m, n, k):
    """perf_hgemm's cooperative / double-buffered pipeline on the fragment API: A col-major, B row-major."""
    a = G.uniform_np(G.SEED_A, (m, k), np.float16); b = G.uniform_np(G.SEED_B, (k, n), np.float16)
    c = G.uniform_np(G.SEED_C, (m, n), np.float16)
    sa = np.ascontiguousarray(a.T)  # column major: k rows of m
    d = nan_filled((m, n), torch.float16)
    api.perf_hgemm_fragment(m, n, k, dev(sa), dev(b), dev(c), d, m, n, n, n, 2.0, 2.0)
    assert_status_ok()
    ref = R.gemm(R.port(), m, n, k, sa.ravel(), b.ravel(), c.ravel(), 2.0, 2.0, np.float16, 1, 0).reshape(m, n)
    bound = R.gemm_abs_bound(m, n, k, a, b, c, 2.0, 2.0)
    assert gemm_rel_err(d.cpu().numpy(), ref, bound) <= TOL_F16_OUT


def test_measured_mma_sync_rates_are_plausible():
    """b200wmma_measure_mma_sync_rate: the register-only issue loops of the two warp-level tensor-core instructions the
    fragment layer and the fp64 GEMM are built on.  On a B200 the fp16 instruction issues at several hundred TFLOP/s
    and the fp64 one at 30-40; both repeat to within a few per cent."""
    from rocwmma_b200 import api
    f16 = [api.measure_mma_sync_rate(0) for _ in range(2)]
    f64 = [api.measure_mma_sync_rate(1) for _ in range(2)]
    assert 200.0 < min(f16) and max(f16) < 1200.0, f16
    assert 20.0 < min(f64) and max(f64) < 45.0, f64
    assert abs(f16[0] - f16[1]) / f16[0] < 0.1 and abs(f64[0] - f64[1]) / f64[0] < 0.1
