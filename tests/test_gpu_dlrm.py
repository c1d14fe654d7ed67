"""GPU parity of the fused DLRM dot-interaction kernels (through the C ABI) against the CPU oracle,
the reference-generated fixtures and the reference's shipped known-answer arrays.
Tolerance: |d - ref| / sum|a||b| <= 2e-3 (fp16 outputs); pass-through copies must be exact."""
import os

import numpy as np
import pytest
import torch

import gen_golden as GG
from conftest import TOL_F16_OUT
from gpu_util import assert_status_ok, dev, nan_filled
from oracle import cpu_ref as R
from rocwmma_b200 import api
from rocwmma_b200 import datagen as G

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def pad_rows(x, m_stride):
    b, m, k = x.shape
    out = np.full((b, m_stride, k), np.float16(7.0))  # padding rows hold junk: they must not be read
    out[:, :m] = x
    return out


def fwd_bound(x):
    x64 = np.abs(x.astype(np.float64))
    m = x.shape[1]
    il, jl = np.tril_indices(m, -1)
    return np.einsum("bik,bjk->bij", x64, x64)[:, il, jl]


def bwd_bound(x, up, k):
    b, m, _ = x.shape
    il, jl = np.tril_indices(m, -1)
    T = np.zeros((b, m, m))
    T[:, il, jl] = np.abs(up[:, k:k + len(il)].astype(np.float64))
    T = T + T.transpose(0, 2, 1)
    return np.einsum("bih,bhj->bij", T, np.abs(x.astype(np.float64)))


def run_fwd(x, m_stride, out_stride):
    b, m, k = x.shape
    out = nan_filled((b, out_stride), torch.float16)
    api.dlrm_dot_fwd(dev(pad_rows(x, m_stride)), out, m, m_stride, k, b, out_stride)
    assert_status_ok()
    return out.cpu().numpy()


def check_fwd(got, x, ref):
    b, m, k = x.shape
    w = k + m * (m - 1) // 2
    assert np.array_equal(got[:, :k], x[:, 0, :])
    if m > 1:
        err = np.abs(got[:, k:w].astype(np.float64) - ref[:, k:].astype(np.float64)) / np.maximum(fwd_bound(x), 1e-30)
        assert err.max() <= TOL_F16_OUT, err.max()
    assert (got[:, w:] == 0).all()  # padding columns are written as zero


def run_bwd(x, up, m_stride, up_stride, fuse, want_mlp=True):
    b, m, k = x.shape
    upp = np.zeros((b, up_stride), np.float16)
    upp[:, :up.shape[1]] = up
    grad = nan_filled((b, m_stride, k), torch.float16)
    mlp = nan_filled((b, k), torch.float16) if want_mlp else None
    api.dlrm_dot_bwd(dev(pad_rows(x, m_stride)), dev(upp), grad, mlp, m, m_stride, k, b, up_stride, fuse)
    assert_status_ok()
    return grad.cpu().numpy(), None if mlp is None else mlp.cpu().numpy()


def check_bwd(grad, mlp, x, up, ref_grad, ref_mlp, fuse):
    b, m, k = x.shape
    expect = ref_grad.astype(np.float64).copy()
    bound = bwd_bound(x, up, k)
    if fuse:
        expect[:, 0, :] += up[:, :k].astype(np.float64)
        bound[:, 0, :] += np.abs(up[:, :k].astype(np.float64))
    err = np.abs(grad[:, :m].astype(np.float64) - expect) / np.maximum(bound, 1e-30)
    # the oracle rounds grad to fp16 before the fused add; allow one extra fp16 rounding in that row
    tol = TOL_F16_OUT * (2 if fuse else 1)
    assert err.max() <= tol, err.max()
    assert np.isnan(grad[:, m:]).all()  # padding rows are not written
    if mlp is not None:
        assert np.array_equal(mlp, ref_mlp)


@pytest.mark.parametrize("case", [c for c in GG.DLRM_CASES if c[4] == np.float16], ids=lambda c: c[0])
def test_dlrm_reference_fixtures(case):
    name, b, m, k, dt = case
    gold = np.load(os.path.join(GOLD, "dlrm_ref.npz"))
    x, g = GG.dlrm_inputs(case)
    w = k + m * (m - 1) // 2
    stride = (w + 7) // 8 * 8
    check_fwd(run_fwd(x, 32, stride), x, gold[name + "_fwd"])
    for fuse in (False, True):
        grad, mlp = run_bwd(x, g, 32, stride, fuse)
        check_bwd(grad, mlp, x, g, gold[name + "_grad"], gold[name + "_mlp"], fuse)


def test_dlrm_known_answer_vectors():
    """The reference's own data set (test/dlrm/data, B=64, m=27, k=128)."""
    kat = np.load(os.path.join(GOLD, "dlrm_kat.npz"))
    B, m, k = 64, 27, 128
    x = kat["input_fp16"].reshape(B, m, k)
    up = kat["input_grad_fp16"].reshape(B, -1)
    check_fwd(run_fwd(x, 27, 480), x, kat["output_fp16"].reshape(B, -1))
    grad, mlp = run_bwd(x, up, 27, 480, False)
    check_bwd(grad, mlp, x, up, kat["output_input_grad_fp16"].reshape(B, m, k),
              kat["output_mlp_input_grad_fp16"].reshape(B, k), False)


@pytest.mark.parametrize("b,m,k,m_stride", [(1, 27, 128, 32), (5, 32, 128, 32), (130, 16, 64, 16), (7, 1, 16, 4),
                                            (33, 17, 256, 20), (1000, 27, 128, 32), (3, 2, 32, 2)])
def test_dlrm_vs_oracle(b, m, k, m_stride):
    x = G.normal_np(G.SEED_X, (b, m, k), 0.25, np.float16)
    w = k + m * (m - 1) // 2
    stride = (w + 7) // 8 * 8 + 8
    up = G.normal_np(G.SEED_G, (b, w), 0.1, np.float16)
    check_fwd(run_fwd(x, m_stride, stride), x, R.dlrm_fwd(R.port(), x, m, k, b))
    rg, rm = R.dlrm_bwd(R.port(), x, up, m, k, b)
    for fuse, want_mlp in ((False, True), (True, False)):
        grad, mlp = run_bwd(x, up, m_stride, stride, fuse, want_mlp)
        check_bwd(grad, mlp, x, up, rg, rm, fuse)


@pytest.mark.parametrize("b,m,k,m_stride", [(64, 128, 128, 128), (4, 1024, 1024, 1024), (9, 100, 48, 112), (6, 40, 512, 48),
                                            (3, 27, 1024, 32), (5, 33, 16, 48)])
def test_dlrm_beyond_one_warp_per_sample(b, m, k, m_stride):
    """Sizes of the reference's own sweep (test/dlrm/test/dlrm_test_params.hpp:55-58: m = 128 / k = 128 and
    m = k = 1024) plus ragged ones: m > 32 or k > 256 run on the block-tiled kernels."""
    x = G.normal_np(G.SEED_X, (b, m, k), 0.25, np.float16)
    w = k + m * (m - 1) // 2
    stride = (w + 7) // 8 * 8 + 8
    up = G.normal_np(G.SEED_G, (b, w), 0.1, np.float16)
    check_fwd(run_fwd(x, m_stride, stride), x, R.dlrm_fwd(R.port(), x, m, k, b))
    rg, rm = R.dlrm_bwd(R.port(), x, up, m, k, b)
    for fuse, want_mlp in ((False, True), (True, False)):
        grad, mlp = run_bwd(x, up, m_stride, stride, fuse, want_mlp)
        check_bwd(grad, mlp, x, up, rg, rm, fuse)


TOL_F32_DATA = 1e-5   # fp32 data: three TF32 products per multiply, fp32 accumulation (the acceptance bound for fp32 outputs is 1e-3)


@pytest.mark.parametrize("b,m,k,m_stride", [(4, 27, 128, 32), (64, 32, 32, 32), (8, 128, 128, 128), (2, 1024, 1024, 1024),
                                            (5, 50, 48, 64)])
def test_dlrm_fp32_data(b, m, k, m_stride):
    """fp32 DLRM data, the second data type of the reference sweep (test/dlrm/test/dlrm_test_params.hpp:51-58): against
    the oracle and, for the fixture case, against the committed output of the reference's own dlrm_*_CPU<float>."""
    x = G.normal_np(G.SEED_X, (b, m, k), 0.25, np.float32)
    w = k + m * (m - 1) // 2
    stride = (w + 7) // 8 * 8 + 8
    up = G.normal_np(G.SEED_G, (b, w), 0.1, np.float32)
    ref_fwd = R.dlrm_fwd(R.port(), x, m, k, b)
    rg, rm = R.dlrm_bwd(R.port(), x, up, m, k, b)
    if (b, m, k) == (4, 27, 128):
        gold = np.load(os.path.join(GOLD, "dlrm_ref.npz"))
        assert np.array_equal(ref_fwd, gold["f32_m27_fwd"]) and np.array_equal(rg, gold["f32_m27_grad"])
    xp = np.full((b, m_stride, k), np.float32(7.0)); xp[:, :m] = x
    out = nan_filled((b, stride), torch.float32)
    api.dlrm_dot_fwd(dev(xp), out, m, m_stride, k, b, stride)
    assert_status_ok()
    got = out.cpu().numpy()
    assert np.array_equal(got[:, :k], x[:, 0, :]) and (got[:, w:] == 0).all()
    if m > 1:
        err = np.abs(got[:, k:w].astype(np.float64) - ref_fwd[:, k:].astype(np.float64)) / np.maximum(fwd_bound(x), 1e-30)
        assert err.max() <= TOL_F32_DATA, err.max()
    upp = np.zeros((b, stride), np.float32); upp[:, :w] = up
    for fuse in (False, True):
        grad = nan_filled((b, m_stride, k), torch.float32)
        mlp = nan_filled((b, k), torch.float32)
        api.dlrm_dot_bwd(dev(xp), dev(upp), grad, mlp, m, m_stride, k, b, stride, fuse)
        assert_status_ok()
        g = grad.cpu().numpy()
        expect = rg.astype(np.float64).copy()
        bound = bwd_bound(x, up, k)
        if fuse:
            expect[:, 0, :] += up[:, :k].astype(np.float64)
            bound[:, 0, :] += np.abs(up[:, :k].astype(np.float64))
        err = np.abs(g[:, :m].astype(np.float64) - expect) / np.maximum(bound, 1e-30)
        assert err.max() <= TOL_F32_DATA * (2 if fuse else 1), err.max()
        assert np.isnan(g[:, m:]).all()
        assert np.array_equal(mlp.cpu().numpy(), rm)


def test_dlrm_full_size_config():
    """B=16384, F=27 padded to 32 rows, D=128, output width 480: sampled rows vs the oracle plus whole-batch
    properties (pass-through exact everywhere; Z symmetric => fwd(x) on a row-permuted sample permutes pairs)."""
    B, m, k, ms, w = 16384, 27, 128, 32, 480
    x = G.fill_torch(torch.zeros((B, ms, k), dtype=torch.float16, device="cuda"), G.SEED_X, "normal", sigma=0.25)
    x[:, m:] = 0
    up = G.fill_torch(torch.zeros((B, w), dtype=torch.float16, device="cuda"), G.SEED_G, "normal", sigma=0.1)
    up[:, w - 1] = 0
    out = nan_filled((B, w), torch.float16)
    api.dlrm_dot_fwd(x, out, m, ms, k, B, w)
    grad = torch.zeros((B, ms, k), dtype=torch.float16, device="cuda")
    api.dlrm_dot_bwd(x, up, grad, None, m, ms, k, B, w, True)
    assert_status_ok()
    assert torch.equal(out[:, :k], x[:, 0, :])
    assert bool(torch.isfinite(out).all()) and bool((out[:, w - 1] == 0).all())
    assert bool((grad[:, m:] == 0).all())
    sel = torch.from_numpy(np.unique((G.raw_np(77, 256) % np.uint64(B)).astype(np.int64))).cuda()
    xs = np.ascontiguousarray(x[sel][:, :m].cpu().numpy())
    ups = up[sel].cpu().numpy()
    check_fwd(out[sel].cpu().numpy(), xs, R.dlrm_fwd(R.port(), xs, m, k, len(sel)))
    rg, rm = R.dlrm_bwd(R.port(), xs, np.ascontiguousarray(ups[:, :w - 1]), m, k, len(sel))
    g = grad[sel].cpu().numpy()
    g[:, m:] = np.nan
    check_bwd(g, None, xs, ups, rg, rm, True)


def test_dlrm_back_to_back_launches_keep_stream_order():
    """The kernels are launched with programmatic stream serialization: a launch may start while its predecessor
    in the stream is finishing, but must not touch global memory before that kernel has completed.  A chain with
    write-after-write (two forwards into one output) and read-after-write (a backward fed by the forward's output,
    a forward fed by the backward's gradient) hazards, issued without any host synchronisation in between and
    repeated, must give what the same calls give one at a time."""
    b, m, k, ms = 4096, 27, 128, 32
    w = k + m * (m - 1) // 2
    stride = 480
    x1 = G.normal_np(11, (b, m, k), 0.25, np.float16)
    x2 = G.normal_np(12, (b, m, k), 0.25, np.float16)
    d1, d2 = dev(pad_rows(x1, ms)), dev(pad_rows(x2, ms))
    out = nan_filled((b, stride), torch.float16)
    grad = torch.zeros((b, ms, k), dtype=torch.float16, device="cuda")
    out2 = nan_filled((b, stride), torch.float16)

    def chain():
        api.dlrm_dot_fwd(d1, out, m, ms, k, b, stride)                       # out = f(x1)
        api.dlrm_dot_fwd(d2, out, m, ms, k, b, stride)                       # WAW: out = f(x2)
        api.dlrm_dot_bwd(d2, out, grad, None, m, ms, k, b, stride, False)    # RAW: upstream = out
        api.dlrm_dot_fwd(grad, out2, m, ms, k, b, stride)                    # RAW: input = grad (pad rows stay zero)

    for _ in range(5):
        chain()
    torch.cuda.synchronize()
    assert_status_ok()
    got_out, got_grad, got_out2 = out.cpu().numpy(), grad.cpu().numpy(), out2.cpu().numpy()
    # the same calls, each followed by a synchronisation
    out_s = nan_filled((b, stride), torch.float16)
    grad_s = torch.zeros((b, ms, k), dtype=torch.float16, device="cuda")
    out2_s = nan_filled((b, stride), torch.float16)
    api.dlrm_dot_fwd(d2, out_s, m, ms, k, b, stride); torch.cuda.synchronize()
    api.dlrm_dot_bwd(d2, out_s, grad_s, None, m, ms, k, b, stride, False); torch.cuda.synchronize()
    api.dlrm_dot_fwd(grad_s, out2_s, m, ms, k, b, stride); torch.cuda.synchronize()
    assert np.array_equal(got_out, out_s.cpu().numpy())
    assert np.array_equal(got_grad, grad_s.cpu().numpy())
    assert np.array_equal(got_out2, out2_s.cpu().numpy(), equal_nan=True)
    check_fwd(got_out, x2, R.dlrm_fwd(R.port(), x2, m, k, b))
