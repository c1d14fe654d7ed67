"""Generates the committed parity fixtures.  Run where the rocWMMA reference tree is mounted:

    make -C oracle && python tests/golden/gen_golden.py [--ref-root <rocWMMA checkout>]

Writes into tests/golden/:
  gemm_ref.npz    outputs of the reference's OWN gemm_CPU (test/reference_impl.hpp:36-81, compiled
                  unmodified into oracle/_ref/libref.so) on small seeded inputs, for every dtype /
                  layout combination the hot path uses.  Inputs are regenerated from the seeds by
                  the tests, only the outputs are stored.
  dlrm_ref.npz    outputs of the reference's dlrm_fwd_CPU / dlrm_bwd_CPU (:83-179) on seeded inputs.
  gemv_ref.npz    reference gemm_CPU with n = 1 (the reference has no CPU gemv) on seeded inputs.
  dlrm_kat.npz    the reference's shipped DLRM known-answer arrays (test/dlrm/data/*_fp16: B=64,
                  m=27, k=128), copied verbatim as data fixtures.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import cpu_ref as R  # noqa: E402
from rocwmma_b200 import datagen as G  # noqa: E402

# (name, m, n, k, in dtype, out dtype, alpha, beta, la, lb, lc, ld)
GEMM_CASES = [
    ("f16_f32_tn", 48, 80, 96, np.float16, np.float32, 2.0, 2.0, 0, 1, 0, 0),
    ("f16_f16_tn", 64, 64, 128, np.float16, np.float16, 1.0, 1.0, 0, 1, 0, 0),
    ("f16_f16_nt", 32, 48, 64, np.float16, np.float16, 2.0, 2.0, 1, 0, 0, 0),
    ("f16_f32_nn_colout", 32, 16, 48, np.float16, np.float32, 0.5, -1.5, 0, 0, 1, 1),
    ("i8_i32_tn", 48, 64, 160, np.int8, np.int32, 1, 0, 0, 1, 0, 0),
    ("i8_i32_tn_ab", 32, 32, 64, np.int8, np.int32, 3, -2, 0, 1, 0, 0),
    ("i8_i8_tn", 48, 64, 160, np.int8, np.int8, 1, 1, 0, 1, 0, 0),      # int8 outputs: the int32 result cast (wraps)
    ("i8_i8_nt_ab", 32, 48, 64, np.int8, np.int8, 3, -2, 1, 0, 0, 0),
    ("f64_tn", 40, 56, 72, np.float64, np.float64, 1.5, 0.5, 0, 1, 0, 0),
    ("f32_tn", 24, 40, 56, np.float32, np.float32, 1.5, 0.5, 0, 1, 0, 0),
]


def gemm_inputs(case):
    """Seeded logical (row-major) A, B, C and their storage-layout flattenings."""
    name, m, n, k, it, ot, alpha, beta, la, lb, lc, ld = case
    if it == np.int8:
        a = G.int8_np(G.SEED_A, (m, k)); b = G.int8_np(G.SEED_B, (k, n))
        c = G.int8_np(G.SEED_C, (m, n)) if ot == np.int8 else (G.int8_np(G.SEED_C, (m, n)).astype(np.int32) * 1000)
    else:
        a = G.uniform_np(G.SEED_A, (m, k), it); b = G.uniform_np(G.SEED_B, (k, n), it)
        c = G.uniform_np(G.SEED_C, (m, n), ot)
    store = lambda x, col: np.ascontiguousarray(x.T if col else x).ravel()
    return a, b, c, store(a, la), store(b, lb), store(c, lc)


# (name, batch, m, k, dtype)
DLRM_CASES = [("f16_m27", 8, 27, 128, np.float16), ("f16_m32", 4, 32, 64, np.float16),
              ("f16_m5", 3, 5, 32, np.float16), ("f32_m27", 4, 27, 128, np.float32)]


def dlrm_inputs(case):
    name, batch, m, k, dt = case
    x = G.normal_np(G.SEED_X, (batch, m, k), 0.25, dt)
    g = G.normal_np(G.SEED_G, (batch, k + m * (m - 1) // 2), 0.1, dt)
    return x, g


# (name, m, n, dtype, col_major)
GEMV_CASES = [("f32_row", 37, 200, np.float32, False), ("f64_row", 19, 130, np.float64, False),
              ("f32_col", 48, 64, np.float32, True), ("f64_col", 32, 40, np.float64, True)]


def gemv_inputs(case):
    name, m, n, dt, col = case
    a = G.uniform_np(G.SEED_GEMV_A, (m, n), dt)
    x = G.uniform_np(G.SEED_GEMV_X, (n,), dt)
    y = G.uniform_np(G.SEED_GEMV_Y, (m,), dt)
    return a, x, y, np.ascontiguousarray(a.T if col else a).ravel()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-root", default=os.environ.get("ROCWMMA_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference"),
                    help="rocWMMA checkout (default: $ROCWMMA_REFERENCE_ROOT, else a directory `reference` beside this repository)")
    args = ap.parse_args()
    ref = R.reference()

    out = {}
    for case in GEMM_CASES:
        name, m, n, k, it, ot, alpha, beta, la, lb, lc, ld = case
        _, _, _, sa, sb, sc = gemm_inputs(case)
        out[name] = R.gemm(ref, m, n, k, sa, sb, sc, alpha, beta, ot, la, lb, lc, ld)
    np.savez_compressed(os.path.join(HERE, "gemm_ref.npz"), **out)

    out = {}
    for case in DLRM_CASES:
        name, batch, m, k, dt = case
        x, g = dlrm_inputs(case)
        out[name + "_fwd"] = R.dlrm_fwd(ref, x, m, k, batch)
        grad, mlp = R.dlrm_bwd(ref, x, g, m, k, batch)
        out[name + "_grad"] = grad
        out[name + "_mlp"] = mlp
    np.savez_compressed(os.path.join(HERE, "dlrm_ref.npz"), **out)

    out = {}
    for case in GEMV_CASES:
        name, m, n, dt, col = case
        a, x, y, sa = gemv_inputs(case)
        out[name] = R.gemv(ref, m, n, sa, x, y, dt(1.5), dt(0.5), col)
    np.savez_compressed(os.path.join(HERE, "gemv_ref.npz"), **out)

    data = os.path.join(args.ref_root, "test", "dlrm", "data")
    kat = {}
    for f in ("input_fp16", "output_fp16", "input_grad_fp16", "output_input_grad_fp16", "output_mlp_input_grad_fp16"):
        kat[f] = np.fromfile(os.path.join(data, f), dtype=np.float16)
    np.savez_compressed(os.path.join(HERE, "dlrm_kat.npz"), **kat)
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
