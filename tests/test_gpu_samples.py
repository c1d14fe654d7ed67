"""Runs the C++ sample hosts (samples/*.cpp, the mirrors of the reference samples' main()) on the GPU:
each fills seeded data, calls the C ABI, times it and validates a row sample on the host; exit code 0
and a PASSED line are required."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
BIN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "samples", "bin")


@pytest.mark.parametrize("name,args", [
    ("perf_hgemm", ["1024", "2048", "512", "2", "2"]),
    ("perf_hgemm", []),                       # the shipped default: 8192^3
    ("perf_hgemm", ["1536", "1024", "768", "2", "2", "nt"]),  # the reference sample's own layouts
    ("perf_sgemm", ["1024", "1536", "512", "2", "0.5"]),      # fp32 GEMM sample (3 x TF32)
    ("simple_hgemm", ["256", "512", "128"]),
    ("simple_sgemm", ["256", "512", "128"]),
    ("simple_dgemm", ["256", "384", "128"]),
    ("perf_dgemm", ["1024", "768", "512", "2", "0.5"]),
    ("simple_dlrm", ["27", "128", "2048"]),
    ("simple_sgemv", ["2048", "4096"]),
    ("simple_dgemv", ["1024", "4096"]),
])
def test_sample_host(name, args):
    exe = os.path.join(BIN, name)
    assert os.path.exists(exe), f"{exe} missing: run __graft_entry__.build()"
    res = subprocess.run([exe, *args], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "PASSED" in res.stdout and "FAILED" not in res.stdout, res.stdout
