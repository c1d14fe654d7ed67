"""rocwmma_b200: the rocWMMA GEMM / DLRM / GEMV hot path as hand-written sm_100a kernels.

Layout of the package:
  csrc/        CUDA kernels and the C ABI (built into librocwmma_b200.so by build.py)
  _lib.py      ctypes binding of the C ABI
  api.py       host mirror of the reference entry points on torch CUDA tensors
  datagen.py   seeded synthetic inputs
The device-side template API (rocwmma::fragment, load_matrix_sync, mma_sync, ...) lives in
include/rocwmma/ at the repository root.
"""
from ._lib import B200WmmaError, LIB_PATH, lib  # noqa: F401

__all__ = ["B200WmmaError", "LIB_PATH", "lib"]
