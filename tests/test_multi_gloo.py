"""The N > 1 host path on CPU: two gloo ranks shard each workload the way bench.py does on GPUs
(GEMM by column blocks with one broadcast of A, DLRM by batch, GEMV by rows), compute their shard,
gather, and the assembled result must equal the unsharded one bit for bit.  The per-shard compute
is the CPU oracle here (there is no GPU in this test); what is under test is the partitioning,
the broadcast and the assembly."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rocwmma_b200.sharding import gemm_column_shard, shard_range


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import cpu_ref as R
    from rocwmma_b200 import datagen as G

    # ---- GEMM: column blocks, A broadcast from rank 0 --------------------------------------
    m, n, k = 48, 64, 96
    col0, ncols, boff = gemm_column_shard(n, k, world, rank)
    a = torch.zeros((m, k), dtype=torch.float16)
    if rank == 0:
        a = torch.from_numpy(G.uniform_np(G.SEED_A, (m, k), np.float16))
    dist.broadcast(a, src=0)
    b_full = G.uniform_np(G.SEED_B, (n, k), np.float16)           # column-major storage: n rows of k
    c_full = G.uniform_np(G.SEED_C, (m, n), np.float32)
    b_loc = b_full.ravel()[boff:boff + ncols * k]
    c_loc = np.ascontiguousarray(c_full[:, col0:col0 + ncols])
    d_loc = R.gemm(R.port(), m, ncols, k, a.numpy().ravel(), b_loc, c_loc.ravel(), 2.0, 2.0, np.float32).reshape(m, ncols)
    parts = [torch.zeros((m, ncols), dtype=torch.float32) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(d_loc))
    d = torch.cat(parts, dim=1).numpy()
    # ---- DLRM: batch shards ---------------------------------------------------------------
    B, mm, kk = 8, 27, 32
    b0, bl = shard_range(B, world, rank)
    x = G.normal_np(G.SEED_X, (B, mm, kk), 0.25, np.float16)
    f_loc = R.dlrm_fwd(R.port(), np.ascontiguousarray(x[b0:b0 + bl]), mm, kk, bl)
    fparts = [torch.zeros(f_loc.shape, dtype=torch.float16) for _ in range(world)]
    dist.all_gather(fparts, torch.from_numpy(f_loc))
    f = torch.cat(fparts, dim=0).numpy()
    # ---- GEMV: row shards, x replicated by broadcast ------------------------------------------
    M, N = 32, 40
    r0, rl = shard_range(M, world, rank)
    A = G.uniform_np(G.SEED_GEMV_A, (M, N), np.float64)
    xv = torch.zeros(N, dtype=torch.float64)
    if rank == 0:
        xv = torch.from_numpy(G.uniform_np(G.SEED_GEMV_X, (N,), np.float64))
    dist.broadcast(xv, src=0)
    y0 = G.uniform_np(G.SEED_GEMV_Y, (M,), np.float64)
    y_loc = R.gemv(R.port(), rl, N, np.ascontiguousarray(A[r0:r0 + rl]).ravel(), xv.numpy(), y0[r0:r0 + rl].copy(), 1.5, 0.5)
    yparts = [torch.zeros(rl, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(yparts, torch.from_numpy(y_loc))
    y = torch.cat(yparts).numpy()
    # timing reduction used by bench.py: max over ranks
    t = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        np.savez(os.path.join(out_dir, "out.npz"), d=d, f=f, y=y, tmax=t.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_matches_unsharded(tmp_path):
    world = 2
    mp.start_processes(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True, start_method="spawn")
    out = np.load(os.path.join(tmp_path, "out.npz"))
    from oracle import cpu_ref as R
    from rocwmma_b200 import datagen as G
    m, n, k = 48, 64, 96
    a = G.uniform_np(G.SEED_A, (m, k), np.float16); b = G.uniform_np(G.SEED_B, (n, k), np.float16)
    c = G.uniform_np(G.SEED_C, (m, n), np.float32)
    assert np.array_equal(out["d"], R.gemm(R.port(), m, n, k, a.ravel(), b.ravel(), c.ravel(), 2.0, 2.0, np.float32).reshape(m, n))
    x = G.normal_np(G.SEED_X, (8, 27, 32), 0.25, np.float16)
    assert np.array_equal(out["f"], R.dlrm_fwd(R.port(), x, 27, 32, 8))
    A = G.uniform_np(G.SEED_GEMV_A, (32, 40), np.float64)
    y = R.gemv(R.port(), 32, 40, A.ravel(), G.uniform_np(G.SEED_GEMV_X, (40,), np.float64),
               G.uniform_np(G.SEED_GEMV_Y, (32,), np.float64), 1.5, 0.5)
    assert np.array_equal(out["y"], y)
    assert out["tmax"][0] == 2.0


def test_shard_range_rejects_bad_splits():
    assert shard_range(8192, 8, 3) == (3072, 1024)
    assert gemm_column_shard(8192, 8192, 4, 1) == (2048, 2048, 2048 * 8192)
    with pytest.raises(ValueError):
        shard_range(10, 4, 0)
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)
