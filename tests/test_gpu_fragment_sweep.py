"""Systematic fragment-shape sweep (tests/csrc/frag_sweep.cu): for every point of the reference unit suites'
parameter space (test/unit/unit_test_params.hpp:86-141: BlockDim 16..256 x BlockK 8..64, plus 128 and 256 of its
extended set, x {i8, f16, f32, f64} x {row, col} major, matrix_a / matrix_b / accumulator) a load -> store round trip must reproduce the block exactly,
leave every padding and guard element untouched (the contamination test), and the cooperative forms with 1, 4 and
6 waves must move the same block collectively."""
import ctypes as C
import os

import numpy as np
import pytest

from gpu_util import dev
from rocwmma_b200 import datagen as G

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))

KINDS = ["matrix_a", "matrix_b", "accumulator"]
TYPES = [np.int8, np.float16, np.float32, np.float64]
DIMS = [16, 32, 64, 128, 256]
KS = [8, 16, 32, 64, 128, 256]
MARK = {np.int8: 99, np.float16: 777.0, np.float32: 777.0, np.float64: 777.0}


@pytest.fixture(scope="module")
def sweep():
    path = os.path.join(HERE, "libfrag_sweep.so")
    assert os.path.exists(path), "tests/libfrag_sweep.so missing: run __graft_entry__.build()"
    h = C.CDLL(path)
    u32, vp = C.c_uint32, C.c_void_p
    h.frag_sweep.restype = C.c_int
    h.frag_sweep.argtypes = [C.c_int, u32, u32, C.c_int, C.c_int, C.c_int, vp, vp, u32, u32, u32, u32, u32, u32, u32,
                             C.POINTER(u32)]
    return h


def offered(kind, bd, bk, dt):
    """Accumulator blocks are at least 16 wide; a block is at most 32 KB (256 registers per lane)."""
    if bd * bk * np.dtype(dt).itemsize > 32768:
        return False
    return bk % 16 == 0 if kind == 2 else True


def rand_matrix(rows, cols, dt, seed):
    if np.issubdtype(dt, np.integer):
        return (G.raw_np(seed, rows * cols) % np.uint64(251)).astype(np.int64).astype(dt).reshape(rows, cols)
    return G.uniform_np(seed, (rows, cols), dt)


def stored(mat, col, ld, dt):
    """`mat` in a padded buffer with leading dimension ld in the given layout, a marker value everywhere else."""
    r, c = mat.shape
    outer, inner = (c, r) if col else (r, c)
    buf = np.full((outer + 3, ld), MARK[dt], dtype=dt)
    buf[:outer, :inner] = mat.T if col else mat
    return buf


@pytest.mark.parametrize("ti", range(4), ids=["i8", "f16", "f32", "f64"])
@pytest.mark.parametrize("bk", KS)
@pytest.mark.parametrize("bd", DIMS)
@pytest.mark.parametrize("kind", range(3), ids=KINDS)
def test_fragment_shape_sweep(sweep, kind, bd, bk, ti):
    dt = TYPES[ti]
    shape = (C.c_uint32 * 4)()
    rc = sweep.frag_sweep(kind, bd, bk, ti, 0, 0, None, None, 0, 0, 0, 0, 1, 1, 1, shape)
    if not offered(kind, bd, bk, dt):
        assert rc == -3  # documented limits
        return
    assert rc == 0
    bh, bw, eb, ne = list(shape)
    assert (bh, bw) == ((bk, bd) if kind == 1 else (bd, bk))
    assert eb == np.dtype(dt).itemsize and ne == bh * bw // 32
    for col in (0, 1):
        # one block per wave over a 2 x 3 grid of blocks, 2 x 2 waves per thread block
        rows, cols = bh * 2, bw * 3
        mat = rand_matrix(rows, cols, dt, 1000 + 97 * kind + bd + bk + ti)
        inner = rows if col else cols
        ld_src, ld_dst = inner + 8, inner + 24
        src = stored(mat, col, ld_src, dt)
        dst = dev(np.full(((cols if col else rows) + 3, ld_dst), MARK[dt], dtype=dt))
        assert sweep.frag_sweep(kind, bd, bk, ti, col, 1, dev(src).data_ptr(), dst.data_ptr(), rows, cols, ld_src, ld_dst,
                                2, 2, 1, shape) == 0
        assert np.array_equal(dst.cpu().numpy(), stored(mat, col, ld_dst, dt))
        # cooperative: 3 blocks side by side, each moved by all waves of a thread block together
        rows, cols = bh, bw * 3
        mat = rand_matrix(rows, cols, dt, 2000 + 97 * kind + bd + bk + ti)
        inner = rows if col else cols
        ld_src, ld_dst = inner + 8, inner + 16
        src = dev(stored(mat, col, ld_src, dt))
        for waves in ((1, 1), (2, 2), (3, 2)):
            dst = dev(np.full(((cols if col else rows) + 3, ld_dst), MARK[dt], dtype=dt))
            assert sweep.frag_sweep(kind, bd, bk, ti, col, 2, src.data_ptr(), dst.data_ptr(), rows, cols, ld_src, ld_dst,
                                    *waves, 3, shape) == 0
            assert np.array_equal(dst.cpu().numpy(), stored(mat, col, ld_dst, dt))
