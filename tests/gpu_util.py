"""Helpers shared by the GPU parity tests: upload, guard bands, oracle calls on row subsets."""
import numpy as np
import torch

from oracle import cpu_ref as R
from rocwmma_b200 import api


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def nan_filled(shape, dtype):
    """Output buffer pre-filled with a marker so that unwritten elements are caught
    (the reference harness pre-fills D with signalling NaNs, test/gemm/gemm_kernel_base_impl.hpp:582-585)."""
    if dtype in (torch.int32, torch.int8):
        return torch.full(shape, -77777777 if dtype == torch.int32 else -77, dtype=dtype, device="cuda")
    return torch.full(shape, float("nan"), dtype=dtype, device="cuda")


def assert_status_ok():
    st, detail = api.device_status()
    assert st == 0, f"device status {st}, detail 0x{detail:08x}"


def oracle_gemm_rows(a_rows, b_store, c_rows, alpha, beta, out_dtype, n, k):
    """Reference result for a subset of rows: A rows [r, k] row-major, B stored column-major [n, k],
    C rows [r, n] row-major.  Rows of a GEMM are independent, so this equals those rows of the full result."""
    r = a_rows.shape[0]
    d = R.gemm(R.port(), r, n, k, np.ascontiguousarray(a_rows).ravel(), np.ascontiguousarray(b_store).ravel(),
               None if c_rows is None else np.ascontiguousarray(c_rows).ravel(), alpha, beta, out_dtype)
    return d.reshape(r, n)
