"""b200wmma_gemm_i8_sp24_static: the 2:4-sparse int8 GEMM for callers that cannot supply scratch memory
(they launch through the bare GEMM kernel signature, or live in a process where an arena owns all device
memory and nobody may call the CUDA allocator).  Its scratch is an array inside the library.

The GPU test calls it through the C ABI twice in a row - a larger problem first, then a smaller one with
different data, so anything the first call left in the shared array would show - and requires results
bit-identical to the workspace-taking entry point and to the CPU oracle on the densified operand.  Further
cases: k a multiple of 32 only, padded row pitches, a problem that fills the built-in array exactly, and (where
there is one) a second GPU, whose copy of the array has its own address.  This file sorts last so that a failure
here cannot hide another test's result in a run that stops at the first failure."""
import ctypes as C
import os

import numpy as np
import pytest

from rocwmma_b200 import _lib

MAX_BYTES = 16 << 20


def _vp(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def test_static_variant_refuses_oversized_problems():
    if not os.path.exists(_lib.LIB_PATH):
        pytest.skip("librocwmma_b200.so not built")
    L = _lib.lib()
    m, k = 4096, 8192  # 32 MiB of expanded A: over the built-in 16 MiB
    assert m * k > MAX_BYTES
    rc = L.b200wmma_gemm_i8_sp24_static(m, 256, k, 16, 16, 16, None, 16, k // 2, k // 8, k, 256, 256, 1, 0, None)
    assert rc == 2
    msg = L.b200wmma_last_error_string().decode()
    assert "exceeds the built-in scratch" in msg and "b200wmma_gemm_i8_sp24" in msg


def _case(L, torch, m, n, k, alpha, beta, seed, pad=(0, 0, 0, 0, 0), with_workspace_variant=True):
    """One call of the static entry point checked against the oracle (and the workspace entry point)."""
    from oracle import cpu_ref as R
    from rocwmma_b200 import datagen as G

    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    dense = G.int8_np(G.SEED_A + seed, (m, k))
    vals, meta, densified = G.sparsify_24_np(dense, seed=G.SEED_SPARSITY + seed)
    b = np.ascontiguousarray(G.int8_np(G.SEED_B + seed, (k, n)).T)
    c = G.int8_np(G.SEED_C + seed, (m, n)).astype(np.int32) * 321
    lda, ldm, ldb, ldc, ldd = k // 2 + pad[0], k // 8 + pad[1], k + pad[2], n + pad[3], n + pad[4]
    padto = lambda x, ld, fill: np.concatenate([x, np.full((x.shape[0], ld - x.shape[1]), fill, x.dtype)], axis=1)
    dv, dm, db, dc = dev(padto(vals, lda, 99)), dev(padto(meta, ldm, 0xEE)), dev(padto(b, ldb, 55)), dev(padto(c, ldc, 7))
    got = torch.full((m, ldd), -2, dtype=torch.int32, device="cuda")
    cptr = _vp(dc) if beta else None
    assert L.b200wmma_gemm_i8_sp24_static(m, n, k, _vp(dv), _vp(dm), _vp(db), cptr, _vp(got), lda, ldm, ldb, ldc, ldd,
                                          alpha, beta, stream) == 0, L.b200wmma_last_error_string()
    torch.cuda.synchronize()
    ref = R.gemm(R.port(), m, n, k, densified.ravel(), b.ravel(), c.ravel() if beta else None, alpha, beta, np.int32).reshape(m, n)
    out = got.cpu().numpy()
    assert np.array_equal(out[:, :n], ref), "static-scratch result differs from the CPU oracle on the densified operand"
    assert (out[:, n:] == -2).all()
    if with_workspace_variant:
        want = torch.full((m, ldd), -1, dtype=torch.int32, device="cuda")
        ws = torch.empty(L.b200wmma_gemm_i8_sp24_workspace_bytes(m, n, k), dtype=torch.uint8, device="cuda")
        assert L.b200wmma_gemm_i8_sp24(m, n, k, _vp(dv), _vp(dm), _vp(db), cptr, _vp(want), lda, ldm, ldb, ldc, ldd,
                                       alpha, beta, _vp(ws), ws.numel(), stream) == 0
        torch.cuda.synchronize()
        assert torch.equal(got[:, :n], want[:, :n]), "static-scratch result differs from the workspace result"


@pytest.mark.gpu
def test_static_variant_matches_oracle_and_workspace_variant_two_calls_in_a_row():
    import torch

    L = _lib.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (m, n, k, alpha, beta) in enumerate([(1024, 512, 4096, 1, 0), (200, 136, 512, 3, -2)]):
        _case(L, torch, m, n, k, alpha, beta, seed=call)
    st, detail = C.c_int(0), C.c_uint(0)
    assert L.b200wmma_device_status(stream, C.byref(st), C.byref(detail)) == 0 and st.value == 0


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k,pad", [(300, 200, 96, (0, 0, 0, 0, 0)),            # k a multiple of 32 only
                                       (260, 136, 384, (64, 16, 128, 4, 8)),       # padded pitches everywhere
                                       (2048, 128, 8192, (0, 0, 0, 0, 0))],        # m * k == the built-in array exactly
                         ids=["k96", "padded", "full_array"])
def test_static_variant_edge_shapes(m, n, k, pad):
    import torch

    L = _lib.lib()
    if (m, k) == (2048, 8192):
        assert m * k == MAX_BYTES
    _case(L, torch, m, n, k, 2, 1, seed=5, pad=pad)
    # a smaller problem right after: leftovers of the larger one in the shared array must not matter
    _case(L, torch, 128, 72, 64, 1, 0, seed=6, with_workspace_variant=False)
    st, detail = C.c_int(0), C.c_uint(0)
    assert L.b200wmma_device_status(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(st), C.byref(detail)) == 0
    assert st.value == 0


@pytest.mark.gpu
def test_static_variant_on_a_second_device():
    """Each GPU holds its own copy of the array; the address is looked up per device."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    L = _lib.lib()
    try:
        for d in (1, 0, 1):
            torch.cuda.set_device(d)
            _case(L, torch, 256, 128, 256, 1, 0, seed=7 + d, with_workspace_variant=False)
    finally:
        torch.cuda.set_device(0)
