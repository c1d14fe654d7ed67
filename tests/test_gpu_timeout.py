"""Failure detection without a GPU fault: a bounded device-side wait that nothing satisfies must give up after
its (here 1 ms) limit, report {DEVICE_TIMEOUT, detail} through the status word, let the kernel return, and leave
the CUDA context usable; a satisfied wait must report nothing."""
import ctypes as C
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def unit():
    path = os.path.join(HERE, "libtimeout_unit.so")
    assert os.path.exists(path), "tests/libtimeout_unit.so missing: run __graft_entry__.build()"
    h = C.CDLL(path)
    h.timeout_unit_run.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_ulonglong]
    return h


def test_unsatisfied_wait_times_out_and_reports(unit):
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    result = torch.full((2,), 7, dtype=torch.int32, device="cuda")
    assert unit.timeout_unit_run(status.data_ptr(), result.data_ptr(), 0, 1_000_000) == 0  # kernel returned normally
    st, res = status.cpu().tolist(), result.cpu().tolist()
    assert st[0] == 5                                  # B200WMMA_ERR_DEVICE_TIMEOUT
    assert (st[1] & 0xFFF00000) == 0xABC00000          # who gave up first
    assert res == [0, 1]                               # wait returned false, CTA abort flag raised
    # the context is still usable
    x = torch.arange(1024, device="cuda")
    assert int(x.sum()) == 1023 * 512


def test_satisfied_wait_reports_nothing(unit):
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    result = torch.full((2,), 7, dtype=torch.int32, device="cuda")
    assert unit.timeout_unit_run(status.data_ptr(), result.data_ptr(), 1, 1_000_000) == 0
    assert status.cpu().tolist() == [0, 0, 0, 0]
    assert result.cpu().tolist() == [1, 0]


def test_library_status_word_roundtrip():
    """b200wmma_device_status returns 0 after healthy launches and clears itself."""
    from rocwmma_b200 import api
    assert api.device_status() == (0, 0)
