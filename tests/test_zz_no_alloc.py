"""b200wmma_gemm_i8_sp24_static: the 2:4-sparse int8 GEMM for callers that cannot supply scratch memory
(they launch through the bare GEMM kernel signature, or live in a process where an arena owns all device
memory and nobody may call the CUDA allocator).  Its scratch is an array inside the library.

The GPU test calls it through the C ABI twice in a row - a larger problem first, then a smaller one with
different data, so anything the first call left in the shared array would show - and requires bit-identical
results to the workspace-taking entry point.  This file sorts last so that a failure here cannot hide
another test's result in a run that stops at the first failure."""
import ctypes as C

import numpy as np
import pytest

from rocwmma_b200 import _lib

MAX_BYTES = 16 << 20


def _vp(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def test_static_variant_refuses_oversized_problems():
    L = _lib.lib()
    m, k = 4096, 8192  # 32 MiB of expanded A: over the built-in 16 MiB
    assert m * k > MAX_BYTES
    rc = L.b200wmma_gemm_i8_sp24_static(m, 256, k, 16, 16, 16, None, 16, k // 2, k // 8, k, 256, 256, 1, 0, None)
    assert rc == 2
    msg = L.b200wmma_last_error_string().decode()
    assert "exceeds the built-in scratch" in msg and "b200wmma_gemm_i8_sp24" in msg


@pytest.mark.gpu
def test_static_variant_matches_workspace_variant_two_calls_in_a_row():
    import torch

    from rocwmma_b200 import datagen as G

    L = _lib.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    for call, (m, n, k, alpha, beta) in enumerate([(1024, 512, 4096, 1, 0), (200, 136, 512, 3, -2)]):
        dense = G.int8_np(G.SEED_A + call, (m, k))
        vals, meta, _ = G.sparsify_24_np(dense, seed=G.SEED_SPARSITY + call)
        b = np.ascontiguousarray(G.int8_np(G.SEED_B + call, (k, n)).T)
        c = G.int8_np(G.SEED_C + call, (m, n)).astype(np.int32) * 321
        dv, dm, db, dc = dev(vals), dev(meta), dev(b), dev(c)
        want = torch.full((m, n), -1, dtype=torch.int32, device="cuda")
        got = torch.full((m, n), -2, dtype=torch.int32, device="cuda")
        ws = torch.empty(L.b200wmma_gemm_i8_sp24_workspace_bytes(m, n, k), dtype=torch.uint8, device="cuda")
        cptr = _vp(dc) if beta else None
        assert L.b200wmma_gemm_i8_sp24(m, n, k, _vp(dv), _vp(dm), _vp(db), cptr, _vp(want), k // 2, k // 8, k, n, n,
                                       alpha, beta, _vp(ws), ws.numel(), stream) == 0
        assert L.b200wmma_gemm_i8_sp24_static(m, n, k, _vp(dv), _vp(dm), _vp(db), cptr, _vp(got), k // 2, k // 8, k,
                                              n, n, alpha, beta, stream) == 0, L.b200wmma_last_error_string()
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}: static-scratch result differs from the workspace result"
    st, detail = C.c_int(0), C.c_uint(0)
    assert L.b200wmma_device_status(stream, C.byref(st), C.byref(detail)) == 0 and st.value == 0
