"""One rank of the multi-GPU C-ABI check (launched by tests/test_gpu_multi.py through torch.distributed.run):
the library's own NCCL plumbing (b200wmma_mg_*) ships A to every rank, each rank multiplies its block of N columns
with the tcgen05 GEMM, and the blocks put side by side must equal the unsharded product of the oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import cpu_ref as R  # noqa: E402
from rocwmma_b200 import api  # noqa: E402
from rocwmma_b200 import datagen as G  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("gloo")  # only carries the 128-byte id and the final gather: plain host traffic
    ident = [api.MultiGpu.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ident, src=0)
    mg = api.MultiGpu(ident[0], rank, world)

    m, n, k = 512, 1024, 256
    col0, ncols = api.shard_range(n, world, rank, 16)
    a = G.uniform_np(G.SEED_A, (m, k), np.float16)
    b = G.uniform_np(G.SEED_B, (k, n), np.float16)
    c = G.uniform_np(G.SEED_C, (m, n), np.float16)
    # A lives on rank 0 only; the others receive it through the library's broadcast
    da = torch.from_numpy(a).cuda() if rank == 0 else torch.zeros(m, k, dtype=torch.float16, device="cuda")
    mg.broadcast(da, root=0)
    torch.cuda.synchronize()
    assert np.array_equal(da.cpu().numpy(), a), "broadcast of A differs"
    bs = torch.from_numpy(np.ascontiguousarray(b.T[col0:col0 + ncols])).cuda()  # column-major B: this rank's columns
    cs = torch.from_numpy(np.ascontiguousarray(c[:, col0:col0 + ncols])).cuda()
    ds = torch.empty(m, ncols, dtype=torch.float16, device="cuda")
    api.gemm_f16(m, ncols, k, da, bs, cs, ds, k, k, ncols, ncols, 1.0, 1.0)
    torch.cuda.synchronize()
    st, detail = api.device_status()
    assert st == 0, (st, detail)
    # the host-buffer driver of the same shard: only rank 0 hands over A, the library ships it inside its pipeline
    ctx = api.HostContext()
    hb = np.ascontiguousarray(b.T[col0:col0 + ncols]); hc = np.ascontiguousarray(c[:, col0:col0 + ncols])
    hd = np.full((m, ncols), np.float16(np.nan))
    for _ in range(2):  # twice: the cached device buffers and events are reused
        ctx.gemm_f16_mg(mg, 0, m, ncols, k, a if rank == 0 else None, hb, hc, hd, k, k, ncols, ncols, 1.0, 1.0, 0)
    assert np.array_equal(hd, ds.cpu().numpy()), "host-buffer multi-GPU driver differs from the device-pointer call"
    # rotating root: every rank holds A; with 2048 rows there are two row blocks, one uploaded by each rank
    m2 = 2048
    a2 = G.uniform_np(21, (m2, k), np.float16); c2 = G.uniform_np(23, (m2, n), np.float16)
    hc2 = np.ascontiguousarray(c2[:, col0:col0 + ncols]); hd2 = np.full((m2, ncols), np.float16(np.nan))
    ctx.gemm_f16_mg(mg, -1, m2, ncols, k, a2, hb, hc2, hd2, k, k, ncols, ncols, 1.0, 1.0, 0)
    ref2 = R.gemm(R.port(), m2, ncols, k, a2.ravel(), hb.ravel(), hc2.ravel(), 1.0, 1.0, np.float16).reshape(m2, ncols)
    bound2 = R.gemm_abs_bound(m2, ncols, k, a2, b[:, col0:col0 + ncols], hc2, 1.0, 1.0)
    err2 = float(np.max(np.abs(hd2.astype(np.float64) - ref2.astype(np.float64)) / bound2))
    assert err2 <= 2e-3, err2
    # int8 form, bit-exact
    a8 = G.int8_np(31, (m2, k)); b8 = G.int8_np(32, (k, n))
    hb8 = np.ascontiguousarray(b8.T[col0:col0 + ncols]); hd8 = np.zeros((m2, ncols), np.int32)
    ctx.gemm_i8_mg(mg, -1, m2, ncols, k, a8, hb8, None, hd8, k, k, ncols, ncols, 1, 0)
    assert np.array_equal(hd8, a8.astype(np.int32) @ b8[:, col0:col0 + ncols].astype(np.int32)), "int8 multi-GPU driver"
    ctx.close()
    parts = [None] * world
    dist.all_gather_object(parts, (col0, ds.cpu().numpy()))
    if rank == 0:
        full = np.concatenate([p for _, p in sorted(parts, key=lambda t: t[0])], axis=1)
        ref = R.gemm(R.port(), m, n, k, a.ravel(), np.ascontiguousarray(b.T).ravel(), c.ravel(), 1.0, 1.0, np.float16).reshape(m, n)
        bound = R.gemm_abs_bound(m, n, k, a, b, c, 1.0, 1.0)
        err = float(np.max(np.abs(full.astype(np.float64) - ref.astype(np.float64)) / bound))
        assert err <= 2e-3, err
        print(f"MG_OK world={world} err={err:.3e}", flush=True)
    mg.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
