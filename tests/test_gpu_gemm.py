"""GPU parity of the tcgen05 GEMM entry points (through the C ABI) against the CPU oracle.

fp16 results are judged with |d - ref| / (|alpha| sum|a||b| + |beta||c|) <= 1e-3 (fp32 out) / 2e-3 (fp16 out);
fp64 with 1e-12; int8 / int4 / 2:4-sparse must be bit-exact."""
import os

import numpy as np
import pytest
import torch

import gen_golden as GG
from conftest import TOL_F16_OUT, TOL_F32_OUT, TOL_F64_OUT, gemm_rel_err
from gpu_util import assert_status_ok, dev, nan_filled, oracle_gemm_rows
from oracle import cpu_ref as R
from rocwmma_b200 import api
from rocwmma_b200 import datagen as G

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def run_f16(m, n, k, alpha, beta, out_np, seed_shift=0, ldd_pad=0):
    a = G.uniform_np(G.SEED_A + seed_shift, (m, k), np.float16)
    b = G.uniform_np(G.SEED_B + seed_shift, (k, n), np.float16)
    c = G.uniform_np(G.SEED_C + seed_shift, (m, n), out_np)
    bs = np.ascontiguousarray(b.T)  # column-major storage: n rows of k
    tdt = torch.float16 if out_np == np.float16 else torch.float32
    ldd = n + ldd_pad
    d = nan_filled((m, ldd), tdt)
    api.gemm_f16(m, n, k, dev(a), dev(bs), dev(c), d, k, k, n, ldd, alpha, beta)
    assert_status_ok()
    dh = d.cpu().numpy()
    ref = oracle_gemm_rows(a, bs, c, alpha, beta, out_np, n, k)
    bound = R.gemm_abs_bound(m, n, k, a, b, c, alpha, beta)
    err = gemm_rel_err(dh[:, :n], ref, bound)
    tol = TOL_F16_OUT if out_np == np.float16 else TOL_F32_OUT
    assert err <= tol, f"rel err {err:.3e} > {tol}"
    if ldd_pad:  # contamination: the guard columns keep their marker
        assert np.isnan(dh[:, n:]).all()
    return err


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 256), (256, 512, 512), (384, 256, 1024),
                                   (128, 256, 8), (2048, 2048, 512)])
def test_gemm_f16_f16out(m, n, k):
    run_f16(m, n, k, 1.0, 1.0, np.float16)


@pytest.mark.parametrize("m,n,k", [(100, 200, 72), (1, 8, 8), (129, 257, 136), (300, 40, 200)])
def test_gemm_f16_ragged(m, n, k):
    run_f16(m, n, k, 2.0, 2.0, np.float32, seed_shift=10)
    run_f16(m, n, k, 1.0, 1.0, np.float16, seed_shift=20, ldd_pad=8)


def test_gemm_f16_config1_1024_f32out():
    """M=N=K=1024, A row / B col fp16, C/D fp32, alpha=beta=2: full-matrix check."""
    run_f16(1024, 1024, 1024, 2.0, 2.0, np.float32)


def test_gemm_f16_beta0_null_c_and_inplace():
    m, n, k = 256, 256, 128
    a = G.uniform_np(1, (m, k), np.float16); b = G.uniform_np(2, (k, n), np.float16)
    bs = np.ascontiguousarray(b.T)
    d = nan_filled((m, n), torch.float16)
    api.gemm_f16(m, n, k, dev(a), dev(bs), None, d, k, k, n, n, 1.5, 0.0)
    ref = oracle_gemm_rows(a, bs, None, 1.5, 0.0, np.float16, n, k)
    bound = R.gemm_abs_bound(m, n, k, a, b, None, 1.5, 0.0)
    assert gemm_rel_err(d.cpu().numpy(), ref, bound) <= TOL_F16_OUT
    # c == d (in place)
    c = G.uniform_np(3, (m, n), np.float16)
    cd = dev(c)
    api.gemm_f16(m, n, k, dev(a), dev(bs), cd, cd, k, k, n, n, 1.0, 1.0)
    ref = oracle_gemm_rows(a, bs, c, 1.0, 1.0, np.float16, n, k)
    bound = R.gemm_abs_bound(m, n, k, a, b, c, 1.0, 1.0)
    assert gemm_rel_err(cd.cpu().numpy(), ref, bound) <= TOL_F16_OUT
    assert_status_ok()


def test_gemm_f16_integer_inputs_exact():
    """Small signed integers as the reference's test fill uses (test/device/common.hpp:203-240): every
    product and partial sum is exactly representable, so the result must equal the oracle bit for bit."""
    m, n, k = 256, 512, 256
    i, j = np.meshgrid(np.arange(m), np.arange(k), indexing="ij")
    a = (((i * k + j) % 5) * np.where(((i * k + j) % 5) % 3 == 0, -1, 1)).astype(np.float16)
    i, j = np.meshgrid(np.arange(k), np.arange(n), indexing="ij")
    b = (((i * n + j) % 3) * np.where(((i * n + j) % 3) % 3 == 0, -1, 1)).astype(np.float16)
    c = np.ones((m, n), np.float32)
    bs = np.ascontiguousarray(b.T)
    d = nan_filled((m, n), torch.float32)
    api.gemm_f16(m, n, k, dev(a), dev(bs), dev(c), d, k, k, n, n, 2.0, 2.0)
    ref = oracle_gemm_rows(a, bs, c, 2.0, 2.0, np.float32, n, k)
    assert np.array_equal(d.cpu().numpy(), ref)
    assert_status_ok()


def _lds(m, n, k, la, lb, lcd):
    return (m if la else k), (n if not lb else k), (m if lcd else n)


def test_gemm_reference_fixtures():
    """The committed outputs of the reference's own gemm_CPU (tests/golden/gemm_ref.npz), every layout case."""
    gold = np.load(os.path.join(GOLD, "gemm_ref.npz"))
    for case in GG.GEMM_CASES:
        name, m, n, k, it, ot, alpha, beta, la, lb, lc, ld = case
        if it == np.float32 or lc != ld:
            continue
        a, b, c, sa, sb, sc = GG.gemm_inputs(case)
        lda, ldb, ldcd = _lds(m, n, k, la, lb, lc)
        ref = gold[name]
        shape = (n, m) if lc else (m, n)
        if it == np.float64 and (la, lb, lc) != (0, 1, 0):
            continue
        if it == np.float16:
            d = nan_filled(shape, torch.float16 if ot == np.float16 else torch.float32)
            api.gemm_f16(m, n, k, dev(sa), dev(sb), dev(sc), d, lda, ldb, ldcd, ldcd, alpha, beta, la, lb, lc)
            bound = R.gemm_abs_bound(m, n, k, a, b, c, alpha, beta)
            bound = np.ascontiguousarray(bound.T if lc else bound).ravel()
            assert gemm_rel_err(d.cpu().numpy().ravel(), ref, bound) <= (TOL_F16_OUT if ot == np.float16 else TOL_F32_OUT), name
        elif it == np.int8 and ot == np.int8:
            d = nan_filled(shape, torch.int8)
            api.gemm_i8_i8(m, n, k, dev(sa), dev(sb), dev(sc), d, lda, ldb, ldcd, ldcd, alpha, beta, la, lb, lc)
            assert np.array_equal(d.cpu().numpy().ravel(), ref), name
        elif it == np.int8:
            d = nan_filled(shape, torch.int32)
            api.gemm_i8(m, n, k, dev(sa), dev(sb), dev(sc), d, lda, ldb, ldcd, ldcd, alpha, beta, la, lb, lc)
            assert np.array_equal(d.cpu().numpy().ravel(), ref), name
        elif it == np.float64:
            d = nan_filled((m, n), torch.float64)
            api.gemm_f64(m, n, k, dev(sa), dev(sb), dev(sc), d, k, k, n, n, alpha, beta)
            bound = R.gemm_abs_bound(m, n, k, a, b, c, alpha, beta)
            assert gemm_rel_err(d.cpu().numpy(), ref.reshape(m, n), bound) <= TOL_F64_OUT, name
    assert_status_ok()


LAYOUTS = [(la, lb, lcd) for la in (0, 1) for lb in (0, 1) for lcd in (0, 1)]


@pytest.mark.parametrize("la,lb,lcd", LAYOUTS, ids=["".join("RC"[x] for x in t) for t in LAYOUTS])
@pytest.mark.parametrize("m,n,k", [(512, 256, 128), (608, 336, 208), (80, 1104, 272)])
def test_gemm_all_layouts(la, lb, lcd, m, n, k):
    """Every combination of row / column-major A, B and C/D (the reference sweeps NN/NT/TN/TT,
    docs/api-reference/api-reference-guide.rst:169-187): fp16 within tolerance, int8 bit-exact.
    Column-major A / row-major B go through MN-major tensor-core descriptors; column-major C/D through the
    transposed problem."""
    lda, ldb, ldcd = _lds(m, n, k, la, lb, lcd)
    store = lambda x, col: np.ascontiguousarray(x.T if col else x)
    # fp16
    a = G.uniform_np(1, (m, k), np.float16); b = G.uniform_np(2, (k, n), np.float16); c = G.uniform_np(3, (m, n), np.float16)
    sa, sb, sc = store(a, la), store(b, lb), store(c, lcd)
    d = nan_filled(sc.shape, torch.float16)
    api.gemm_f16(m, n, k, dev(sa), dev(sb), dev(sc), d, lda, ldb, ldcd, ldcd, 2.0, 0.5, la, lb, lcd)
    ref = R.gemm(R.port(), m, n, k, sa.ravel(), sb.ravel(), sc.ravel(), 2.0, 0.5, np.float16, la, lb, lcd, lcd)
    bound = store(R.gemm_abs_bound(m, n, k, a, b, c, 2.0, 0.5), lcd).ravel()
    assert gemm_rel_err(d.cpu().numpy().ravel(), ref, bound) <= TOL_F16_OUT
    # int8
    ai = G.int8_np(1, (m, k)); bi = G.int8_np(2, (k, n)); ci = G.int8_np(3, (m, n)).astype(np.int32) * 1000
    sa, sb, sc = store(ai, la), store(bi, lb), store(ci, lcd)
    di = nan_filled(sc.shape, torch.int32)
    api.gemm_i8(m, n, k, dev(sa), dev(sb), dev(sc), di, lda, ldb, ldcd, ldcd, 3, -1, la, lb, lcd)
    refi = R.gemm(R.port(), m, n, k, sa.ravel(), sb.ravel(), sc.ravel(), 3, -1, np.int32, la, lb, lcd, lcd)
    assert np.array_equal(di.cpu().numpy().ravel(), refi)
    assert_status_ok()


TOL_F32X3 = 5e-6   # three TF32 products: ~2^-21 per product; a single TF32 product (2^-11) would miss this by far


@pytest.mark.parametrize("m,n,k,alpha,beta", [(512, 256, 256, 1.0, 0.0), (640, 300, 100, 2.0, 0.5), (200, 1000, 512, -1.5, 1.0),
                                              (1024, 1024, 1024, 2.0, 2.0)])
def test_gemm_f32_three_tf32(m, n, k, alpha, beta):
    """fp32 GEMM of the sgemm samples (samples/simple_sgemm.cpp, samples/perf_sgemm.cpp) against the reference's
    fp32 gemm_CPU arithmetic.  The tolerance is far tighter than the 1e-3 acceptance bound for fp32 outputs so that a plain TF32 product,
    which keeps 10 mantissa bits, could not pass."""
    a = G.uniform_np(G.SEED_A, (m, k), np.float32); b = G.uniform_np(G.SEED_B, (k, n), np.float32)
    c = G.uniform_np(G.SEED_C, (m, n), np.float32)
    bs = np.ascontiguousarray(b.T)
    ws = torch.empty(api.gemm_f32_workspace_bytes(m, n, k), dtype=torch.uint8, device="cuda")
    d = nan_filled((m, n), torch.float32)
    api.gemm_f32(m, n, k, dev(a), dev(bs), dev(c) if beta else None, d, k, k, n, n, alpha, beta, ws)
    assert_status_ok()
    ref = oracle_gemm_rows(a, bs, c if beta else None, alpha, beta, np.float32, n, k)
    bound = R.gemm_abs_bound(m, n, k, a, b, c if beta else np.zeros_like(c), alpha, beta)
    assert gemm_rel_err(d.cpu().numpy(), ref, bound) <= TOL_F32X3


@pytest.mark.parametrize("la,lb,lcd", LAYOUTS, ids=["".join("RC"[x] for x in t) for t in LAYOUTS])
@pytest.mark.parametrize("m,n,k", [(512, 256, 128), (301, 203, 100)])
def test_gemm_f32_all_layouts(la, lb, lcd, m, n, k):
    """fp32 GEMM in every layout combination (the split pre-pass absorbs column-major A / row-major B; column-major
    C / D is the transposed problem), ragged extents included, at the fp32-class tolerance."""
    a = G.uniform_np(G.SEED_A, (m, k), np.float32); b = G.uniform_np(G.SEED_B, (k, n), np.float32)
    c = G.uniform_np(G.SEED_C, (m, n), np.float32)
    def store(x, col, mult):   # natural storage, pitch rounded up to `mult` elements
        t = np.ascontiguousarray(x.T if col else x)
        ld = (t.shape[1] + mult - 1) // mult * mult
        out = np.full((t.shape[0], ld), np.nan, np.float32)
        out[:, :t.shape[1]] = t
        return out, ld
    (sa, lda), (sb, ldb), (sc, ldc) = store(a, la, 4), store(b, lb, 4), store(c, lcd, 1)
    ws = torch.empty(api.gemm_f32_workspace_bytes(m, n, k), dtype=torch.uint8, device="cuda")
    d = nan_filled(sc.shape, torch.float32)
    api.gemm_f32(m, n, k, dev(sa), dev(sb), dev(sc), d, lda, ldb, ldc, ldc, 1.5, 0.5, ws, la, lb, lcd)
    assert_status_ok()
    nat = lambda x, col: np.ascontiguousarray(x.T if col else x)
    ref = R.gemm(R.port(), m, n, k, nat(a, la).ravel(), nat(b, lb).ravel(), nat(c, lcd).ravel(), 1.5, 0.5, np.float32,
                 la, lb, lcd, lcd).reshape(nat(c, lcd).shape)
    bound = nat(R.gemm_abs_bound(m, n, k, a, b, c, 1.5, 0.5), lcd)
    assert gemm_rel_err(d.cpu().numpy()[:, :ref.shape[1]], ref, bound) <= TOL_F32X3


@pytest.mark.parametrize("la,lb,lcd", [(0, 1, 0), (1, 0, 0), (0, 0, 1), (1, 1, 1)], ids=["RCR", "CRR", "RRC", "CCC"])
@pytest.mark.parametrize("m,n,k,alpha,beta", [(512, 256, 256, 1, 0), (608, 336, 208, 3, -2), (144, 80, 96, 1, 1)])
def test_gemm_i8_int8_outputs(la, lb, lcd, m, n, k, alpha, beta):
    """The reference's <int8_t, int8_t, int32_t> set (test/gemm/gemm_common_test_params.hpp:53): int32 compute, the
    result cast to int8 as gemm_CPU's static_cast does.  Bit-exact against the oracle in the same layouts.  The C / D
    pitches of these shapes are multiples of 32 and of 16 only: the drain's 32-byte and 16-byte forms."""
    lda, ldb, ldcd = _lds(m, n, k, la, lb, lcd)
    store = lambda x, col: np.ascontiguousarray(x.T if col else x)
    a = G.int8_np(G.SEED_A, (m, k)); b = G.int8_np(G.SEED_B, (k, n)); c = G.int8_np(G.SEED_C, (m, n))
    sa, sb, sc = store(a, la), store(b, lb), store(c, lcd)
    d = nan_filled(sc.shape, torch.int8)
    api.gemm_i8_i8(m, n, k, dev(sa), dev(sb), dev(sc) if beta else None, d, lda, ldb, ldcd, ldcd, alpha, beta, la, lb, lcd)
    assert_status_ok()
    ref = R.gemm(R.port(), m, n, k, sa.ravel(), sb.ravel(), sc.ravel() if beta else None, alpha, beta, np.int8, la, lb, lcd, lcd)
    assert np.array_equal(d.cpu().numpy().ravel(), ref)


@pytest.mark.parametrize("lcd", [0, 1], ids=["RCR", "RCC"])
def test_gemm_i8_int8_outputs_unaligned_rows(lcd):
    """int8 C / D whose rows are not 16-byte aligned (pitch 75 resp. 200): the drain goes byte by byte."""
    m, n, k, alpha, beta = 200, 75, 128, 2, 1
    store = lambda x, col: np.ascontiguousarray(x.T if col else x)
    a = G.int8_np(G.SEED_A, (m, k)); b = G.int8_np(G.SEED_B, (k, n)); c = G.int8_np(G.SEED_C, (m, n))
    sa, sb, sc = a, store(b, 1), store(c, lcd)
    ldcd = m if lcd else n
    d = nan_filled(sc.shape, torch.int8)
    api.gemm_i8_i8(m, n, k, dev(sa), dev(sb), dev(sc), d, k, k, ldcd, ldcd, alpha, beta, 0, 1, lcd)
    assert_status_ok()
    ref = R.gemm(R.port(), m, n, k, sa.ravel(), sb.ravel(), sc.ravel(), alpha, beta, np.int8, 0, 1, lcd, lcd)
    assert np.array_equal(d.cpu().numpy().ravel(), ref)


TOL_BF16_OUT = 4e-3   # bf16 keeps 8 significant bits: one rounding of the result is up to 2^-9 of its magnitude


@pytest.mark.parametrize("la,lb,lcd", [(0, 1, 0), (1, 0, 0), (0, 0, 1), (1, 1, 1)], ids=["RCR", "CRR", "RRC", "CCC"])
@pytest.mark.parametrize("m,n,k", [(512, 256, 256), (608, 336, 208), (80, 1104, 272)])
def test_gemm_bf16_bf16_outputs(la, lb, lcd, m, n, k):
    """The reference's <bfloat16_t, bfloat16_t, float32_t> set (test/gemm/gemm_common_test_params.hpp:89-94): bf16 C and
    D, fp32 compute.  The reference build here has no bfloat16 type, so the oracle is gemm_CPU's fp32 arithmetic on the
    exactly widened inputs, with its final cast to bf16 applied by torch (round to nearest even, like the type's own)."""
    lda, ldb, ldcd = _lds(m, n, k, la, lb, lcd)
    store = lambda x, col: np.ascontiguousarray(x.T if col else x)
    bf = torch.bfloat16
    ta = torch.from_numpy(G.uniform_np(1, (m, k), np.float32)).to(bf)
    tb = torch.from_numpy(G.uniform_np(2, (k, n), np.float32)).to(bf)
    tc = torch.from_numpy(G.uniform_np(3, (m, n), np.float32)).to(bf)
    a, b, c = (t.to(torch.float32).numpy() for t in (ta, tb, tc))
    lay = lambda tt, col: (tt.t().contiguous() if col else tt.contiguous()).cuda()
    dc = lay(tc, lcd)
    d = torch.full(dc.shape, float("nan"), dtype=bf, device="cuda")
    api.gemm_bf16(m, n, k, lay(ta, la), lay(tb, lb), dc, d, lda, ldb, ldcd, ldcd, 2.0, 0.5, la, lb, lcd)
    assert_status_ok()
    ref32 = R.gemm(R.port(), m, n, k, store(a, la).ravel(), store(b, lb).ravel(), store(c, lcd).ravel(), 2.0, 0.5, np.float32,
                   la, lb, lcd, lcd)
    ref = torch.from_numpy(ref32).to(bf).to(torch.float32).numpy()
    bound = store(R.gemm_abs_bound(m, n, k, a, b, c, 2.0, 0.5), lcd).ravel()
    assert gemm_rel_err(d.to(torch.float32).cpu().numpy().ravel(), ref, bound) <= TOL_BF16_OUT


_LOWP = {"bf16": torch.bfloat16, "e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


@pytest.mark.parametrize("kind", sorted(_LOWP))
@pytest.mark.parametrize("la,lb,lcd", [(0, 1, 0), (1, 0, 0), (0, 0, 1), (1, 1, 1)], ids=["RCR", "CRR", "RRC", "CCC"])
@pytest.mark.parametrize("m,n,k", [(512, 256, 256), (608, 336, 208), (80, 1104, 272)])
def test_gemm_bf16_fp8_inputs(kind, la, lb, lcd, m, n, k):
    """bfloat16 / OCP fp8 inputs with fp32 accumulation and fp32 C / D (the reference's bfloat16_t, float8 and
    bfloat8 input types, docs/api-reference/api-reference-guide.rst:84-143).  The oracle is the reference's
    gemm_CPU arithmetic on the inputs widened exactly to fp32: acc += float(a) * float(b) in ascending k."""
    tdt = _LOWP[kind]
    lda, ldb, ldcd = _lds(m, n, k, la, lb, lcd)
    store = lambda x, col: np.ascontiguousarray(x.T if col else x)
    ta = torch.from_numpy(G.uniform_np(1, (m, k), np.float32)).to(tdt)       # rounded once; these ARE the inputs
    tb = torch.from_numpy(G.uniform_np(2, (k, n), np.float32)).to(tdt)
    a, b = ta.to(torch.float32).numpy(), tb.to(torch.float32).numpy()         # exact widening
    c = G.uniform_np(3, (m, n), np.float32)
    dev_lowp = lambda tt, col: (tt.t().contiguous() if col else tt.contiguous()).cuda()
    sc = store(c, lcd)
    d = nan_filled(sc.shape, torch.float32)
    fn = api.gemm_bf16 if kind == "bf16" else api.gemm_fp8
    fn(m, n, k, dev_lowp(ta, la), dev_lowp(tb, lb), dev(sc), d, lda, ldb, ldcd, ldcd, 2.0, 0.5, la, lb, lcd)
    assert_status_ok()
    ref = R.gemm(R.port(), m, n, k, store(a, la).ravel(), store(b, lb).ravel(), sc.ravel(), 2.0, 0.5, np.float32,
                 la, lb, lcd, lcd)
    bound = store(R.gemm_abs_bound(m, n, k, a, b, c, 2.0, 0.5), lcd).ravel()
    assert gemm_rel_err(d.cpu().numpy().ravel(), ref, bound) <= TOL_F32_OUT


@pytest.mark.parametrize("m,n,k,alpha,beta", [(128, 256, 128, 1, 0), (256, 256, 1024, 1, 0), (128, 512, 16384, 1, 0),
                                              (100, 72, 144, 3, -2), (513, 300, 272, 1, 1)])
def test_gemm_i8_bit_exact(m, n, k, alpha, beta):
    a = G.int8_np(G.SEED_A, (m, k)); b = G.int8_np(G.SEED_B, (k, n))
    c = G.int8_np(G.SEED_C, (m, n)).astype(np.int32) * 12345
    bs = np.ascontiguousarray(b.T)
    d = nan_filled((m, n), torch.int32)
    api.gemm_i8(m, n, k, dev(a), dev(bs), dev(c) if beta else None, d, k, k, n, n, alpha, beta)
    assert_status_ok()
    ref = oracle_gemm_rows(a, bs, c if beta else None, alpha, beta, np.int32, n, k)
    assert np.array_equal(d.cpu().numpy(), ref)


# k % 128 == 0 with 16-byte aligned rows runs on the sparse tensor cores (512 x 224 pair tiles, 256 K per slab:
# the shapes cross tile edges in M and N, include ragged ones and K tails of half a slab); with a workspace
# the metadata is re-tiled first, without (next test) it is read as it is.  The other shapes take the
# densify-then-dense path.
@pytest.mark.parametrize("m,n,k,alpha,beta", [(128, 256, 128, 1, 0), (200, 136, 512, 1, 0), (256, 256, 4096, 1, 0),
                                              (1100, 500, 384, 3, -2), (513, 225, 256, 1, 1), (64, 1000, 128, -1, 1),
                                              (300, 200, 96, 1, 0), (130, 72, 160, 2, 1)])
def test_gemm_i8_sparse24_bit_exact(m, n, k, alpha, beta):
    dense = G.int8_np(G.SEED_A, (m, k)); b = G.int8_np(G.SEED_B, (k, n))
    c = G.int8_np(G.SEED_C, (m, n)).astype(np.int32) * 54321
    vals, meta, densified = G.sparsify_24_np(dense)
    bs = np.ascontiguousarray(b.T)
    ws = torch.empty(api.gemm_i8_sp24_workspace_bytes(m, n, k), dtype=torch.uint8, device="cuda")
    d = nan_filled((m, n), torch.int32)
    api.gemm_i8_sp24(m, n, k, dev(vals), dev(meta), dev(bs), dev(c) if beta else None, d, k // 2, k // 8, k, n, n,
                     alpha, beta, ws)
    assert_status_ok()
    ref = oracle_gemm_rows(densified, bs, c if beta else None, alpha, beta, np.int32, n, k)
    assert np.array_equal(d.cpu().numpy(), ref)


@pytest.mark.parametrize("m,n,k", [(300, 260, 384), (1024, 448, 1024)])
def test_gemm_i8_sparse24_metadata_retiled_once(m, n, k):
    """Metadata re-tiled once (b200wmma_sp24_repack_meta), then two GEMMs with different B on the packed copy."""
    dense = G.int8_np(G.SEED_A, (m, k))
    vals, meta, densified = G.sparsify_24_np(dense)
    packed = torch.empty(api.sp24_packed_meta_bytes(m, k), dtype=torch.uint8, device="cuda")
    api.sp24_repack_meta(m, k, dev(meta), k // 8, packed)
    for seed in (G.SEED_B, G.SEED_C):
        bs = np.ascontiguousarray(G.int8_np(seed, (k, n)).T)
        d = nan_filled((m, n), torch.int32)
        api.gemm_i8_sp24_packed(m, n, k, dev(vals), packed, dev(bs), None, d, k // 2, k, n, n, 1, 0)
        assert_status_ok()
        assert np.array_equal(d.cpu().numpy(), oracle_gemm_rows(densified, bs, None, 1, 0, np.int32, n, k))


def test_gemm_i8_sparse24_padded_pitches_no_workspace():
    """Row pitches larger than the rows (values, metadata, B, C, D), D rows not 16-byte aligned (element-wise
    epilogue), and no workspace: the sparse tensor-core path needs none."""
    m, n, k = 700, 451, 640
    lda, ldm, ldb, ldc, ldd = k // 2 + 64, k // 8 + 16, k + 128, n + 5, n + 3
    dense = G.int8_np(G.SEED_A, (m, k)); b = G.int8_np(G.SEED_B, (k, n))
    c = G.int8_np(G.SEED_C, (m, n)).astype(np.int32) * 777
    vals, meta, densified = G.sparsify_24_np(dense)
    bs = np.ascontiguousarray(b.T)
    pad = lambda x, ld, fill: np.concatenate([x, np.full((x.shape[0], ld - x.shape[1]), fill, x.dtype)], axis=1)
    d = torch.full((m, ldd), -7, dtype=torch.int32, device="cuda")
    api.gemm_i8_sp24(m, n, k, dev(pad(vals, lda, 99)), dev(pad(meta, ldm, 0xEE)), dev(pad(bs, ldb, 55)),
                     dev(pad(c, ldc, 1 << 30)), d, lda, ldm, ldb, ldc, ldd, 2, 3, None)
    assert_status_ok()
    ref = oracle_gemm_rows(densified, bs, c, 2, 3, np.int32, n, k)
    out = d.cpu().numpy()
    assert np.array_equal(out[:, :n], ref)
    assert np.all(out[:, n:] == -7)          # nothing written past the row ends


def test_gemm_i8_sparse24_full_size_row_sample():
    """M=N=8192, K=16384, 2:4-sparse A: 32 seeded-random rows bit-exact against the oracle on the densified
    rows, and the exact column-sum checksum over the whole output."""
    m, n, k = 8192, 8192, 16384
    dense = G.fill_torch(torch.empty((m, k), dtype=torch.int8, device="cuda"), G.SEED_A, "int8")
    vals = torch.empty((m, k // 2), dtype=torch.int8, device="cuda")
    meta = torch.empty((m, k // 8), dtype=torch.uint8, device="cuda")
    densified = torch.empty((m, k), dtype=torch.int8, device="cuda")
    for r0 in range(0, m, 1024):                      # compress on the host in row chunks
        v, md, dn = G.sparsify_24_np(dense[r0:r0 + 1024].cpu().numpy(), row_start=r0)
        vals[r0:r0 + 1024] = torch.from_numpy(v).cuda()
        meta[r0:r0 + 1024] = torch.from_numpy(md).cuda()
        densified[r0:r0 + 1024] = torch.from_numpy(dn).cuda()
    del dense
    bs = G.fill_torch(torch.empty((n, k), dtype=torch.int8, device="cuda"), G.SEED_B, "int8")
    d = nan_filled((m, n), torch.int32)
    ws = torch.empty(api.gemm_i8_sp24_workspace_bytes(m, n, k), dtype=torch.uint8, device="cuda")
    api.gemm_i8_sp24(m, n, k, vals, meta, bs, None, d, k // 2, k // 8, k, n, n, 1, 0, ws)
    assert_status_ok()
    rows = _rows_sample(m, 32, 97)
    idx = torch.from_numpy(rows).cuda()
    ref = oracle_gemm_rows(densified[idx].cpu().numpy(), bs.cpu().numpy(), None, 1, 0, np.int32, n, k)
    assert np.array_equal(d[idx].cpu().numpy(), ref)
    col = d.to(torch.int64).sum(dim=0)
    a_sum = densified.to(torch.float64).sum(dim=0)
    expect = bs.to(torch.float64) @ a_sum
    assert torch.equal(col.to(torch.float64), expect)


@pytest.mark.parametrize("m,n,k,alpha,beta", [(128, 256, 128, 1, 0), (200, 136, 512, 1, 0), (256, 256, 4096, 1, 0),
                                              (700, 300, 96, 3, -2), (513, 520, 1056, 1, 1), (40, 24, 32, -1, 5),
                                              (96, 256, 131072, 1, 0), (64, 128, 131072 + 64, 2, 1)])
def test_gemm_i4_bit_exact(m, n, k, alpha, beta):
    """Packed int4 operands, unpacked inside the kernel (no workspace): ragged M / N, K that is a multiple of 32 only,
    alpha / beta with C, and K of 131072 and more, where the kernel sign-extends the nibbles instead of scaling them."""
    assert api.gemm_i4_workspace_bytes(m, n, k) == 0
    a = G.int4_np(G.SEED_A, (m, k)); b = G.int4_np(G.SEED_B, (k, n))
    c = G.int8_np(G.SEED_C, (m, n)).astype(np.int32) * 4321
    bs = np.ascontiguousarray(b.T)
    d = nan_filled((m, n), torch.int32)
    api.gemm_i4(m, n, k, dev(G.pack_int4_np(a)), dev(G.pack_int4_np(bs)), dev(c) if beta else None, d, k // 2, k // 2, n, n,
                alpha, beta, None)
    assert_status_ok()
    ref = oracle_gemm_rows(a, bs, c if beta else None, alpha, beta, np.int32, n, k)
    assert np.array_equal(d.cpu().numpy(), ref)


def test_gemm_i4_extreme_values_and_padded_pitches():
    """Every value -8 (the case in which 256 * sum is largest) at K = 65536, row pitches larger than the rows, and D
    rows that are not 16-byte aligned (element-wise drain)."""
    m, n, k = 130, 70, 65536
    a = np.full((m, k), -8, np.int8); bs = np.full((n, k), -8, np.int8)
    a[::3, ::5] = 7; bs[1::2, ::7] = 7
    lda, ldb, ldd = k // 2 + 32, k // 2 + 16, n + 3
    pad = lambda x, ld: np.concatenate([x, np.full((x.shape[0], ld - x.shape[1]), 0x5A, x.dtype)], axis=1)
    d = torch.full((m, ldd), -7, dtype=torch.int32, device="cuda")
    api.gemm_i4(m, n, k, dev(pad(G.pack_int4_np(a), lda)), dev(pad(G.pack_int4_np(bs), ldb)), None, d, lda, ldb, n, ldd, 1, 0)
    assert_status_ok()
    out = d.cpu().numpy()
    assert np.array_equal(out[:, :n], oracle_gemm_rows(a, bs, None, 1, 0, np.int32, n, k))
    assert (out[:, n:] == -7).all()


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (200, 136, 72), (512, 384, 256)])
def test_gemm_f64(m, n, k):
    a = G.uniform_np(G.SEED_A, (m, k), np.float64); b = G.uniform_np(G.SEED_B, (k, n), np.float64)
    c = G.uniform_np(G.SEED_C, (m, n), np.float64)
    bs = np.ascontiguousarray(b.T)
    d = nan_filled((m, n), torch.float64)
    api.gemm_f64(m, n, k, dev(a), dev(bs), dev(c), d, k, k, n, n, 1.5, 0.5)
    ref = oracle_gemm_rows(a, bs, c, 1.5, 0.5, np.float64, n, k)
    bound = R.gemm_abs_bound(m, n, k, a, b, c, 1.5, 0.5)
    assert gemm_rel_err(d.cpu().numpy(), ref, bound) <= TOL_F64_OUT


@pytest.mark.parametrize("la,lb,lcd", LAYOUTS, ids=["".join("RC"[x] for x in t) for t in LAYOUTS])
@pytest.mark.parametrize("m,n,k", [(256, 128, 64), (301, 202, 100), (64, 390, 34)])
def test_gemm_f64_all_layouts(la, lb, lcd, m, n, k):
    """fp64 GEMM in every combination of row / column-major A, B and C/D (the reference's NN / NT / TN / TT sweep,
    docs/api-reference/api-reference-guide.rst:169-187), odd extents included, against the oracle in the same layouts.
    Leading dimensions are padded to even values where the extent is odd (16-byte async copies)."""
    even = lambda x: x + (x & 1)
    a = G.uniform_np(G.SEED_A, (m, k), np.float64); b = G.uniform_np(G.SEED_B, (k, n), np.float64)
    c = G.uniform_np(G.SEED_C, (m, n), np.float64)
    def store(x, col):   # (storage with an even pitch, pitch)
        t = np.ascontiguousarray(x.T if col else x)
        ld = even(t.shape[1])
        out = np.full((t.shape[0], ld), np.nan)
        out[:, :t.shape[1]] = t
        return out, ld
    (sa, lda), (sb, ldb), (sc, ldc) = store(a, la), store(b, lb), store(c, lcd)
    d = nan_filled(sc.shape, torch.float64)
    api.gemm_f64(m, n, k, dev(sa), dev(sb), dev(sc), d, lda, ldb, ldc, ldc, 1.5, 0.5, la, lb, lcd)
    assert_status_ok()
    nat = lambda x, col: np.ascontiguousarray(x.T if col else x)
    ref = R.gemm(R.port(), m, n, k, nat(a, la).ravel(), nat(b, lb).ravel(), nat(c, lcd).ravel(), 1.5, 0.5, np.float64, la, lb, lcd, lcd)
    ref = ref.reshape(nat(c, lcd).shape)
    bound = nat(R.gemm_abs_bound(m, n, k, a, b, c, 1.5, 0.5), lcd)
    got = d.cpu().numpy()[:, :ref.shape[1]]
    assert gemm_rel_err(got, ref, bound) <= TOL_F64_OUT
    assert np.isnan(d.cpu().numpy()[:, ref.shape[1]:]).all()   # pitch padding untouched


@pytest.mark.parametrize("which", [1, 2], ids=["cp_async", "tma"])
@pytest.mark.parametrize("la,lb", [(0, 1), (1, 0), (0, 0), (1, 1)], ids=["RC", "CR", "RR", "CC"])
def test_gemm_f64_both_kernels(la, lb, which):
    """The fp64 GEMM has a TMA-fed kernel (contiguous extents that are multiples of 4) and a cp.async-fed one (everything
    else); both on one shape that is a multiple of 4 but of no tile size, K spanning several slabs with a ragged last
    one, padded pitches.  `gemm_f64_kernel` = 2 fails instead of falling back, so the TMA-fed kernel provably ran."""
    m, n, k = 300, 204, 100
    a = G.uniform_np(G.SEED_A, (m, k), np.float64); b = G.uniform_np(G.SEED_B, (k, n), np.float64)
    c = G.uniform_np(G.SEED_C, (m, n), np.float64)
    def store(x, col, pad):
        t = np.ascontiguousarray(x.T if col else x)
        out = np.full((t.shape[0], t.shape[1] + pad), np.nan)
        out[:, :t.shape[1]] = t
        return out, t.shape[1] + pad
    (sa, lda), (sb, ldb) = store(a, la, 6), store(b, lb, 2)
    d = nan_filled((m, n), torch.float64)
    api.set_tuning("gemm_f64_kernel", which)
    try:
        api.gemm_f64(m, n, k, dev(sa), dev(sb), dev(c), d, lda, ldb, n, n, 1.5, 0.5, la, lb, 0)
        assert_status_ok()
        if which == 2:   # a shape without the 3-D views is refused, not silently given the other kernel
            with pytest.raises(api.B200WmmaError):
                api.gemm_f64(m, n, 98, dev(sa), dev(sb), dev(c), d, lda, ldb, n, n, 1.5, 0.5, 0, 1, 0)
    finally:
        api.set_tuning("gemm_f64_kernel", 0)
    nat = lambda x, col: np.ascontiguousarray(x.T if col else x)
    ref = R.gemm(R.port(), m, n, k, nat(a, la).ravel(), nat(b, lb).ravel(), c.ravel(), 1.5, 0.5, np.float64, la, lb, 0, 0).reshape(m, n)
    assert gemm_rel_err(d.cpu().numpy(), ref, R.gemm_abs_bound(m, n, k, a, b, c, 1.5, 0.5)) <= TOL_F64_OUT


@pytest.mark.parametrize("k", [64, 128, 320])
def test_gemm_many_tiles_per_sm_pair_short_k(k):
    """More output tiles than SM pairs with only 1-5 K slabs per tile: the persistent kernels walk their operand
    ring across tile boundaries while the epilogue of the previous tile still owns part of it (staging tiles that
    alias an operand stage)."""
    m, n = 4096, 4608
    a = G.uniform_np(1, (m, k), np.float16); b = G.uniform_np(2, (k, n), np.float16); c = G.uniform_np(3, (m, n), np.float16)
    bs = np.ascontiguousarray(b.T)
    d = nan_filled((m, n), torch.float16)
    api.gemm_f16(m, n, k, dev(a), dev(bs), dev(c), d, k, k, n, n, 1.0, 1.0)
    assert_status_ok()
    ref = oracle_gemm_rows(a, bs, c, 1.0, 1.0, np.float16, n, k)
    assert gemm_rel_err(d.cpu().numpy(), ref, R.gemm_abs_bound(m, n, k, a, b, c, 1.0, 1.0)) <= TOL_F16_OUT
    # int8 dense and 2:4 sparse (sparse needs k % 128 == 0)
    ai = G.int8_np(1, (m, k)); bi = np.ascontiguousarray(G.int8_np(2, (k, n)).T)
    ci = G.int8_np(3, (m, n)).astype(np.int32) * 321
    di = nan_filled((m, n), torch.int32)
    api.gemm_i8(m, n, k, dev(ai), dev(bi), dev(ci), di, k, k, n, n, 2, 1)
    assert np.array_equal(di.cpu().numpy(), oracle_gemm_rows(ai, bi, ci, 2, 1, np.int32, n, k))
    if k % 128 == 0:
        vals, meta, densified = G.sparsify_24_np(ai)
        ws = torch.empty(api.gemm_i8_sp24_workspace_bytes(m, n, k), dtype=torch.uint8, device="cuda")
        ds = nan_filled((m, n), torch.int32)
        for w in (ws, None):
            ds.fill_(-1)
            api.gemm_i8_sp24(m, n, k, dev(vals), dev(meta), dev(bi), dev(ci), ds, k // 2, k // 8, k, n, n, 2, 1, w)
            assert np.array_equal(ds.cpu().numpy(), oracle_gemm_rows(densified, bi, ci, 2, 1, np.int32, n, k))
    assert_status_ok()


def _rows_sample(m, count, seed):
    rows = (G.raw_np(seed, count) % np.uint64(m)).astype(np.int64)
    rows[0], rows[-1] = 0, m - 1
    return np.unique(rows)


def test_gemm_f16_full_size_8192_row_sample():
    """Benchmark size (M=N=K=8192, fp16 C/D, alpha=beta=1): all columns of 48 seeded-random rows are
    checked against the oracle (rows are independent), and the whole output must be finite."""
    m = n = k = 8192
    a = G.fill_torch(torch.empty((m, k), dtype=torch.float16, device="cuda"), G.SEED_A, "uniform")
    bs = G.fill_torch(torch.empty((n, k), dtype=torch.float16, device="cuda"), G.SEED_B, "uniform")
    c = G.fill_torch(torch.empty((m, n), dtype=torch.float16, device="cuda"), G.SEED_C, "uniform")
    d = nan_filled((m, n), torch.float16)
    api.gemm_f16(m, n, k, a, bs, c, d, k, k, n, n, 1.0, 1.0)
    assert_status_ok()
    assert bool(torch.isfinite(d).all())
    rows = _rows_sample(m, 48, 99)
    idx = torch.from_numpy(rows).cuda()
    a_r, c_r, d_r = a[idx].cpu().numpy(), c[idx].cpu().numpy(), d[idx].cpu().numpy()
    b_h = bs.cpu().numpy()
    ref = oracle_gemm_rows(a_r, b_h, c_r, 1.0, 1.0, np.float16, n, k)
    bound = R.gemm_abs_bound(len(rows), n, k, a_r, b_h.T, c_r, 1.0, 1.0)
    assert gemm_rel_err(d_r, ref, bound) <= TOL_F16_OUT


def test_gemm_i8_full_size_row_sample():
    """M=N=8192, K=16384 int8 -> int32, alpha=1, beta=0: 32 seeded-random rows bit-exact."""
    m, n, k = 8192, 8192, 16384
    a = G.fill_torch(torch.empty((m, k), dtype=torch.int8, device="cuda"), G.SEED_A, "int8")
    bs = G.fill_torch(torch.empty((n, k), dtype=torch.int8, device="cuda"), G.SEED_B, "int8")
    d = nan_filled((m, n), torch.int32)
    api.gemm_i8(m, n, k, a, bs, None, d, k, k, n, n, 1, 0)
    assert_status_ok()
    rows = _rows_sample(m, 32, 98)
    idx = torch.from_numpy(rows).cuda()
    ref = oracle_gemm_rows(a[idx].cpu().numpy(), bs.cpu().numpy(), None, 1, 0, np.int32, n, k)
    assert np.array_equal(d[idx].cpu().numpy(), ref)
    # a checksum over the whole output that no element can be missing from: column sums of D equal
    # (column sums of A) x B, computed exactly in int64 on the device by torch as plumbing
    col = d.to(torch.int64).sum(dim=0)
    a_sum = a.to(torch.float64).sum(dim=0)          # exact: |sum| < 2^53
    expect = (bs.to(torch.float64) @ a_sum)          # n values, each exact in fp64 (|.| < 2^53)
    assert torch.equal(col.to(torch.float64), expect)


def test_gemm_i4_full_size_row_sample():
    """M=N=8192, K=16384 with both operands int4 in [-8, 7], packed two per byte (low nibble = even k): 32
    seeded-random rows bit-exact against the oracle on the sign-extended operands, and the exact column-sum
    checksum over the whole output (no element can be missing from it)."""
    m, n, k = 8192, 8192, 16384
    a = G.fill_torch(torch.empty((m, k), dtype=torch.int8, device="cuda"), G.SEED_A, "int4")
    bs = G.fill_torch(torch.empty((n, k), dtype=torch.int8, device="cuda"), G.SEED_B, "int4")
    assert int(a.min()) >= -8 and int(a.max()) <= 7
    pack = lambda t: ((t[:, 0::2].to(torch.uint8) & 0xF) | ((t[:, 1::2].to(torch.uint8) & 0xF) << 4)).contiguous()
    ap, bp = pack(a), pack(bs)
    ws_bytes = api.gemm_i4_workspace_bytes(m, n, k)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda") if ws_bytes else None
    d = nan_filled((m, n), torch.int32)
    api.gemm_i4(m, n, k, ap, bp, None, d, k // 2, k // 2, n, n, 1, 0, ws)
    assert_status_ok()
    rows = _rows_sample(m, 32, 96)
    idx = torch.from_numpy(rows).cuda()
    ref = oracle_gemm_rows(a[idx].cpu().numpy(), bs.cpu().numpy(), None, 1, 0, np.int32, n, k)
    assert np.array_equal(d[idx].cpu().numpy(), ref)
    col = d.to(torch.int64).sum(dim=0)
    a_sum = a.to(torch.float64).sum(dim=0)
    expect = bs.to(torch.float64) @ a_sum
    assert torch.equal(col.to(torch.float64), expect)


@pytest.mark.parametrize("size,nrows", [(4096, 64), (7168, 16)], ids=["4096", "7168"])
def test_gemm_f64_bench_size_row_sample(size, nrows):
    """fp64 at M=N=K=4096 (the size bench.py measures) and 7168 (the reference's perf_dgemm size,
    samples/perf_dgemm.cpp:875), alpha=beta=1: all columns of seeded-random rows within 1e-12 of the oracle, and the
    whole output finite."""
    m = n = k = size
    f = lambda shape, seed: G.fill_torch(torch.empty(shape, dtype=torch.float64, device="cuda"), seed, "uniform")
    a, bs, c = f((m, k), G.SEED_A), f((n, k), G.SEED_B), f((m, n), G.SEED_C)
    d = nan_filled((m, n), torch.float64)
    api.gemm_f64(m, n, k, a, bs, c, d, k, k, n, n, 1.0, 1.0)
    assert_status_ok()
    assert bool(torch.isfinite(d).all())
    rows = _rows_sample(m, nrows, 95)
    idx = torch.from_numpy(rows).cuda()
    a_r, c_r, d_r = a[idx].cpu().numpy(), c[idx].cpu().numpy(), d[idx].cpu().numpy()
    b_h = bs.cpu().numpy()
    ref = oracle_gemm_rows(a_r, b_h, c_r, 1.0, 1.0, np.float64, n, k)
    bound = R.gemm_abs_bound(len(rows), n, k, a_r, b_h.T, c_r, 1.0, 1.0)
    assert gemm_rel_err(d_r, ref, bound) <= TOL_F64_OUT


# Shapes whose tile count is not a whole number of rounds over the SM pairs, so that with a workspace the last round is
# split along K (stream-K): a few tiles over many pairs, whole rounds followed by a split round, ragged M / N / K,
# the per-GPU problem of an 8192^3 GEMM sharded 8 ways.
SPLIT_SHAPES = [(1024, 1024, 8192), (2560, 7680, 2048), (1100, 900, 4160), (8192, 1024, 8192), (600, 256, 1024),
                (8192, 2048, 8192), (3584, 3072, 4096), (2048, 4864, 4096)]


@pytest.fixture(autouse=True)
def _split_whenever_possible():
    """The planner only splits when it expects a gain; these tests are about correctness, so they make it split whenever
    the schedule allows (exchange cost counted as one slab)."""
    api.set_tuning("gemm_split_fixup", 1)
    yield
    api.set_tuning("gemm_split_fixup", 0)


@pytest.mark.parametrize("m,n,k", SPLIT_SHAPES)
def test_gemm_split_tail_int8_bit_exact(m, n, k):
    """int8 with the split-K workspace: bit-identical to the unsplit call (integer addition is associative) and to the
    oracle on a row sample; alpha / beta with C included."""
    a = G.fill_torch(torch.empty((m, k), dtype=torch.int8, device="cuda"), G.SEED_A, "int8")
    bs = G.fill_torch(torch.empty((n, k), dtype=torch.int8, device="cuda"), G.SEED_B, "int8")
    c = (G.fill_torch(torch.empty((m, n), dtype=torch.int8, device="cuda"), G.SEED_C, "int8").to(torch.int32) * 1000).contiguous()
    ws = torch.empty(api.gemm_split_workspace_bytes(), dtype=torch.uint8, device="cuda")
    for alpha, beta in ((1, 0), (3, -2)):
        plain, split = nan_filled((m, n), torch.int32), nan_filled((m, n), torch.int32)
        api.gemm_i8(m, n, k, a, bs, c if beta else None, plain, k, k, n, n, alpha, beta)
        for _ in range(2):   # twice: the flags in the workspace are reset by every call
            split.fill_(-5)
            api.gemm_i8(m, n, k, a, bs, c if beta else None, split, k, k, n, n, alpha, beta, workspace=ws)
            assert_status_ok()
            assert torch.equal(plain, split)
        rows = _rows_sample(m, 12, 91)
        idx = torch.from_numpy(rows).cuda()
        ref = oracle_gemm_rows(a[idx].cpu().numpy(), bs.cpu().numpy(), c[idx].cpu().numpy() if beta else None, alpha, beta,
                               np.int32, n, k)
        assert np.array_equal(split[idx].cpu().numpy(), ref)


@pytest.mark.parametrize("m,n,k", SPLIT_SHAPES)
@pytest.mark.parametrize("out_np", [np.float16, np.float32], ids=["f16out", "f32out"])
def test_gemm_split_tail_f16(m, n, k, out_np):
    """fp16 with the split-K workspace against the oracle on a row sample (the partial sums are fp32)."""
    tdt = torch.float16 if out_np == np.float16 else torch.float32
    a = G.fill_torch(torch.empty((m, k), dtype=torch.float16, device="cuda"), G.SEED_A, "uniform")
    bs = G.fill_torch(torch.empty((n, k), dtype=torch.float16, device="cuda"), G.SEED_B, "uniform")
    c = G.fill_torch(torch.empty((m, n), dtype=tdt, device="cuda"), G.SEED_C, "uniform")
    ws = torch.empty(api.gemm_split_workspace_bytes(), dtype=torch.uint8, device="cuda")
    d = nan_filled((m, n), tdt)
    api.gemm_f16(m, n, k, a, bs, c, d, k, k, n, n, 1.0, 1.0, workspace=ws)
    assert_status_ok()
    assert bool(torch.isfinite(d).all())
    rows = _rows_sample(m, 12, 92)
    idx = torch.from_numpy(rows).cuda()
    a_r, c_r, b_h = a[idx].cpu().numpy(), c[idx].cpu().numpy(), bs.cpu().numpy()
    ref = oracle_gemm_rows(a_r, b_h, c_r, 1.0, 1.0, out_np, n, k)
    bound = R.gemm_abs_bound(len(rows), n, k, a_r, b_h.T, c_r, 1.0, 1.0)
    assert gemm_rel_err(d[idx].cpu().numpy(), ref, bound) <= (TOL_F16_OUT if out_np == np.float16 else TOL_F32_OUT)


def test_gemm_split_tail_declined_cases():
    """A workspace that is too small, and C / D rows that are not 16-byte aligned: the unsplit schedule runs, results
    unchanged."""
    m, n, k = 1024, 1024, 2048
    a = G.fill_torch(torch.empty((m, k), dtype=torch.int8, device="cuda"), 1, "int8")
    bs = G.fill_torch(torch.empty((n, k), dtype=torch.int8, device="cuda"), 2, "int8")
    want = nan_filled((m, n), torch.int32)
    api.gemm_i8(m, n, k, a, bs, None, want, k, k, n, n, 1, 0)
    small = torch.empty(4096, dtype=torch.uint8, device="cuda")
    got = nan_filled((m, n), torch.int32)
    api.gemm_i8(m, n, k, a, bs, None, got, k, k, n, n, 1, 0, workspace=small)
    assert torch.equal(got, want)
    ws = torch.empty(api.gemm_split_workspace_bytes(), dtype=torch.uint8, device="cuda")
    odd = torch.full((m, n + 3), -9, dtype=torch.int32, device="cuda")
    api.gemm_i8(m, n, k, a, bs, None, odd, k, k, n, n + 3, 1, 0, workspace=ws)
    assert_status_ok()
    assert torch.equal(odd[:, :n], want) and bool((odd[:, n:] == -9).all())


@pytest.mark.parametrize("variant", [1, 2, 3], ids=["1cta", "2cta", "2cta512"])
def test_gemm_every_tile_variant(variant):
    """Each tile shape of the tcgen05 GEMM (one-CTA 128x256, pair 256x256, pair 512x256), forced through
    b200wmma_set_tuning, on shapes with ragged edges; fp16 within tolerance, int8 exact."""
    api.set_tuning("gemm_tile_variant", variant)
    try:
        for (m, n, k) in [(640, 768, 320), (1100, 300, 144), (128, 256, 64)]:
            run_f16(m, n, k, 1.0, 1.0, np.float16)
            ai = G.int8_np(1, (m, k)); bi = np.ascontiguousarray(G.int8_np(2, (k, n)).T)
            di = nan_filled((m, n), torch.int32)
            api.gemm_i8(m, n, k, dev(ai), dev(bi), None, di, k, k, n, n, 1, 0)
            assert np.array_equal(di.cpu().numpy(), oracle_gemm_rows(ai, bi, None, 1, 0, np.int32, n, k))
        assert_status_ok()
    finally:
        api.set_tuning("gemm_tile_variant", 0)
