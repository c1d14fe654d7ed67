"""Multi-GPU path through the C ABI's own plumbing (b200wmma_mg_unique_id / _create / _broadcast / _destroy and
b200wmma_shard_range): two ranks, one process per GPU; skipped on a single-GPU machine.  The sharding arithmetic and
the host logic around it are covered on CPU by tests/test_multi_gloo.py."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_two_ranks_broadcast_and_column_sharded_gemm():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(HERE, "workers", "mg_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "MG_OK world=2" in res.stdout


def test_cpp_multi_gpu_sample(tmp_path):
    """samples/multi_gpu_hgemm.cpp: two processes, one per GPU, exchanging the NCCL id through a file."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    exe = os.path.join(os.path.dirname(HERE), "samples", "bin", "multi_gpu_hgemm")
    assert os.path.exists(exe), "samples/bin/multi_gpu_hgemm missing: run __graft_entry__.build()"
    idfile = str(tmp_path / "nccl_id")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([exe, str(r), "2", idfile], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
             for r in range(2)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r}:\n{out[-1500:]}"
        assert "PASS" in out.upper() or "passed" in out.lower(), out[-500:]
