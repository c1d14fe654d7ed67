import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu")


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    # GPU tests are selected with -m gpu; without a device they are skipped, never silently passed.
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# ---- acceptance metrics -----------------------------------------------------------------------
TOL_F32_OUT = 1e-3   # |d - ref| / (|alpha| sum|a||b| + |beta||c|) for fp32 outputs
TOL_F16_OUT = 2e-3   # fp16 outputs
TOL_F64_OUT = 1e-12  # fp64 outputs


def gemm_rel_err(d, ref, bound):
    """max over elements of |d - ref| / bound, where bound = |alpha| sum_h |a||b| + |beta||c| (> 0)."""
    d = np.asarray(d, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert np.isfinite(d).all(), "non-finite values in the result (unwritten or overflowed elements)"
    return float(np.max(np.abs(d - ref) / np.maximum(bound, 1e-300)))


@pytest.fixture(scope="session")
def oracle_port():
    from oracle import cpu_ref
    return cpu_ref.port()
