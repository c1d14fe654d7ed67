"""bench.py's workload registry is consistent (no GPU needed): every `also` workload exists, names are unique, and each
workload states the fields the JSON line is built from."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_also_workloads_are_registered():
    assert len(set(bench.ALSO)) == len(bench.ALSO)
    missing = [name for name in bench.ALSO if name not in bench.WORKLOADS]
    assert not missing, missing
    assert "gemm_f16" in bench.WORKLOADS and "gemm_f16" not in bench.ALSO   # the headline is measured first, not twice


def test_every_workload_states_its_line_fields():
    for name, cls in bench.WORKLOADS.items():
        wl = cls()
        assert wl.name == name
        assert wl.bound in ("tensor", "hbm"), name
        assert isinstance(wl.metric, str) and wl.metric, name
        assert wl.unit in ("TFLOP/s", "TOP/s", "GB/s", "samples/s"), name
        assert wl.dtype in ("f16", "bf16", "fp8", "f32", "f64", "i8", "i4"), (name, wl.dtype)
        cfg = wl.config(1)
        assert "workload" in cfg and "model" not in cfg, name
