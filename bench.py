"""Benchmark of the hot path.  One JSON line on stdout (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Default workload (the one the headline metric is quoted on): dense fp16 GEMM in the perf_hgemm form,
D = alpha*(A x B) + beta*C, M=N=K=8192, A row-major fp16, B column-major fp16, C/D row-major fp16,
fp32 accumulate, alpha=beta=1, seeded uniform[-1,1) inputs.  A "step" is one GEMM.

N > 1: one process per GPU.  The problem is sharded by N-column blocks (B, C, D split; A broadcast once
over NCCL before the timed region and reported separately as `a_broadcast_ms`); there is no collective in
the data path, total work is fixed (strong scaling), value = 2*M*N*K / max-over-ranks time.

The line also carries `"also"`: every other component of the metric (int8 / 2:4-sparse / int4 / bf16 / fp8 / fp32 / fp64 GEMM,
DLRM forward and backward, sgemv / dgemv, the fragment-API GEMMs) measured in the same process the same way, each with
its own ms_per_step, roofline, clocks, parity_check and (where a host driver exists) e2e; at N > 1 each is sharded its own
way (GEMM by N-column blocks, DLRM by batch, GEMV by rows).  `--no-also` skips them, `--workload NAME` makes one of
them the headline instead (`gemm_bf16 | gemm_fp8 | gemm_f32 | gemm_i8 | gemm_i8_sp24 | gemm_i4 | gemm_f64 | dlrm_fwd |
dlrm_bwd | sgemv | dgemv | frag_simple_hgemm | frag_perf_hgemm`).

`"parity_check"`: after the timed region and outside it, every rank compares a seeded sample of rows / samples of its own
result (device-pointer path, and the host-driver result where there is one) with the CPU oracle; the run exits non-zero
when a check fails.

`--impl reference` times the reference's own CPU implementation (oracle/_ref/libref.so, compiled from
rocWMMA's test/reference_impl.hpp; the port oracle/libref_port.so if that is absent) on the host cores,
each step a bounded row sub-block of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under profiles/
# (None where no capture exists yet).
NCU_TRAFFIC_BYTES = {
    "gemm_f16": 1.108e9,      # profiles/gemm_tc05_f16_8192.md: 986.6 MB read + 121.5 MB written (512x256 pair kernel)
    "gemm_i8": 1.072e9,       # profiles/gemm_tc05_i8_8192x8192x16384.md: 833.4 + 238.2 MB (512x256 pair kernel)
    "gemm_i8_sp24": 8.591e8,  # profiles/gemm_tc05_sp24_8192x8192x16384.md (GEMM kernel; the re-tiling pre-pass adds ~33 MB)
    "gemm_i4": 6.234e8,       # profiles/gemm_tc05_i4_8192x8192x16384.md: 386.0 + 237.3 MB
    "gemm_fp8": 9.165e8,      # profiles/gemm_tc05_fp8_8192.md: 676.4 + 240.1 MB
    "gemm_f64": 1.354e9,      # profiles/gemm_f64_4096.md: 1233 + 120.4 MB
    "frag_perf_hgemm": 2.300e9,  # profiles/frag_perf_hgemm_8192.md: 2169 + 131 MB
    "dlrm_fwd": 119.1e6,      # profiles/dlrm_dot_B16384.md
    "dlrm_bwd": 192.4e6,      # profiles/dlrm_dot_B16384.md
    "sgemv": 4.299e9,         # profiles/gemv_32768.md: 4.295 GB read + 3.6 MB written
    "dgemv": 8.595e9,         # profiles/gemv_32768.md (the four-rows-per-CTA capture; the fp64 matrix is read once either way)
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                p = json.load(f)
            p["_source"] = "measured"
            return p
        except Exception:
            pass
    p = dict(FALLBACK_PEAKS)
    p["_source"] = "fallback"
    return p


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and clock-event reasons through NVML (read-only) while the timed region runs."""

    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
        0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, index: int, period_s: float = 0.01):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _once(self):
        nv = self._nv
        try:
            self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
            try:
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
            except Exception:
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
            for bit, name in self.REASONS.items():
                if mask & bit and name != "gpu_idle":
                    self.reasons.add(name)
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self._once()
            self._stop.wait(self._period)

    def start(self):
        if self._nv is None:
            return
        self._stop.clear()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# --------------------------------------------------------------------------------------- workloads
class Workload:
    """name, algorithmic work, device step, host (end-to-end) step and CPU-reference sample for one config."""

    name = ""
    metric = ""
    unit = ""
    dtype = ""
    bound = "tensor"
    scaling = "strong"

    def describe(self, world):
        raise NotImplementedError


def _shard(n, world, rank):
    from rocwmma_b200.sharding import shard_range
    return shard_range(n, world, rank)


def _timed_broadcast(torch, dist, t):
    """A is needed whole by every rank: one NCCL broadcast from rank 0 before the timed region.  Returns
    (ms of that first call, which includes NCCL's channel set-up; ms of a second, warmed call of the same size)."""
    out = []
    for _ in range(2):
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dist.broadcast(t, src=0)
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1))
    return out[0], out[1]


def _sample_rows(total, count, seed):
    """Seeded sample of row / sample indices, always with the first and the last one."""
    import numpy as np
    from rocwmma_b200 import datagen as G
    rows = (G.raw_np(seed, count) % np.uint64(total)).astype(np.int64)
    rows[0], rows[-1] = 0, total - 1
    return np.unique(rows)


def _parity_result(rows, err, tol, exact=None, what=""):
    """`err`: max |got - ref| / bound (floating point); `exact`: number of mismatching elements (integer paths)."""
    if exact is not None:
        return {"rows": int(rows), "max_rel_err": 0.0 if exact == 0 else float("inf"), "mismatches": int(exact),
                "tol": 0.0, "ok": exact == 0, "what": what}
    ok = bool(err == err and err <= tol)
    return {"rows": int(rows), "max_rel_err": float(err), "tol": tol, "ok": ok, "what": what}


def _gemm_rows_parity(wl, torch, a_rows, b_store, c_rows, got, alpha, beta, out_np, tol, what):
    """Rows of D = alpha*A*B + beta*C against the oracle.  a_rows [r, k] and b_store [n, k] (column-major B) are
    numpy arrays in the oracle's input type; the error bound |alpha| sum|a||b| + |beta||c| is formed on the device
    in fp64 (plumbing for the tolerance only)."""
    import numpy as np
    from oracle import cpu_ref as R
    r, k = a_rows.shape
    n = b_store.shape[0]
    ref = R.gemm(R.port(), r, n, k, np.ascontiguousarray(a_rows).ravel(), np.ascontiguousarray(b_store).ravel(),
                 None if c_rows is None else np.ascontiguousarray(c_rows).ravel(), alpha, beta, out_np).reshape(r, n)
    if np.issubdtype(np.dtype(out_np), np.integer):
        return _parity_result(r, 0.0, 0.0, exact=int(np.count_nonzero(got != ref)), what=what)
    # the error bound's denominator sum|a||b|, on the host (no device kernel of any library takes part in the check)
    ta = np.abs(a_rows.astype(np.float64))
    bound = np.zeros((r, n), dtype=np.float64)
    for c0 in range(0, n, 2048):   # column chunks keep the fp64 copy of B small
        bound[:, c0:c0 + 2048] = abs(alpha) * (ta @ np.abs(b_store[c0:c0 + 2048].astype(np.float64)).T)
    if c_rows is not None:
        bound += abs(beta) * np.abs(c_rows.astype(np.float64))
    g64 = got.astype(np.float64)
    if not np.isfinite(g64).all():
        return _parity_result(r, float("nan"), tol, what=what)
    err = float(np.max(np.abs(g64 - ref.astype(np.float64)) / np.maximum(bound, 1e-300)))
    return _parity_result(r, err, tol, what=what)


class GemmF16(Workload):
    name, metric, unit, dtype, bound = "gemm_f16", "fp16 GEMM TFLOP/s at 8192^3", "TFLOP/s", "f16", "tensor"
    M = N = K = 8192
    alpha = beta = 1.0

    def setup(self, torch, rank, world, dist):
        from rocwmma_b200 import datagen as G
        self.torch, self.rank, self.world = torch, rank, world
        M, N, K = self.M, self.N, self.K
        col0, self.nloc = _shard(N, world, rank)
        f16 = torch.float16
        # B column-major = N rows of K; C/D: this rank's column block stored compactly (ld = nloc)
        self.b = torch.empty((self.nloc, K), dtype=f16, device="cuda")
        G.fill_torch(self.b, G.SEED_B, "uniform", start=col0 * K)  # logical index of B^T storage rows
        self.c = torch.empty((M, self.nloc), dtype=f16, device="cuda")
        # C logical index = i*N + j: generate row by row block (seeded, independent of sharding)
        idx = (torch.arange(M, device="cuda", dtype=torch.int64)[:, None] * N
               + torch.arange(col0, col0 + self.nloc, device="cuda", dtype=torch.int64)[None, :])
        z, lsr = G._mix_torch(G.SEED_C, idx)
        self.c.copy_((2.0 * (lsr(z, 40).to(torch.float64) * 2.0 ** -24) - 1.0).to(f16))
        del idx, z
        self.d = torch.empty_like(self.c)
        self.a = torch.empty((M, K), dtype=f16, device="cuda")
        self.a_broadcast_ms = 0.0
        if rank == 0:
            G.fill_torch(self.a, G.SEED_A, "uniform")
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier()
            self.a_broadcast_ms, self.a_broadcast_warm_ms = _timed_broadcast(torch, dist, self.a)
        self.work_total = 2.0 * M * N * K
        self.work_local = 2.0 * M * self.nloc * K

    def step(self):
        from rocwmma_b200 import api
        api.gemm_f16(self.M, self.nloc, self.K, self.a, self.b, self.c, self.d,
                     self.K, self.K, self.nloc, self.nloc, self.alpha, self.beta, workspace=self._split_ws())

    def _split_ws(self):
        """Caller-owned scratch of the split-K tail (b200wmma_gemm_*_ws): lets a shard whose tiles do not fill a whole
        number of rounds (64 tiles on 74 SM pairs at 8 GPUs) use every pair; the library itself allocates nothing."""
        if not hasattr(self, "_ws"):
            from rocwmma_b200 import api
            self._ws = self.torch.empty(api.gemm_split_workspace_bytes(), dtype=self.torch.uint8, device="cuda")
        return self._ws

    def setup_host(self):
        from rocwmma_b200 import api
        t = self.torch
        self.h_a = self.a.cpu().pin_memory()
        self.h_b = self.b.cpu().pin_memory()
        self.h_c = self.c.cpu().pin_memory()
        self.h_d = t.empty(self.c.shape, dtype=self.c.dtype).pin_memory()
        self.ctx = api.HostContext()
        self.h2d = self.h_a.numel() * 2 + self.h_b.numel() * 2 + self.h_c.numel() * 2
        self.d2h = self.h_d.numel() * 2
        self.mg = None
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            # several ranks: each row block of A is uploaded by one rank and travels to the others over NVLink (the
            # library's NCCL plumbing, inside the timed call) instead of one PCIe upload of all of A per rank
            ident = [api.MultiGpu.unique_id() if dist.get_rank() == 0 else None]
            dist.broadcast_object_list(ident, src=0)
            self.mg = api.MultiGpu(ident[0], dist.get_rank(), dist.get_world_size())
            # every rank holds A on the host: row block i is uploaded and broadcast by rank i mod world
            blocks = (self.M + 1023) // 1024
            mine = len(range(dist.get_rank(), blocks, dist.get_world_size()))
            self.h2d -= (blocks - mine) * 1024 * self.K * 2

    def step_host(self):
        if self.mg is not None:
            self.ctx.gemm_f16_mg(self.mg, -1, self.M, self.nloc, self.K, self.h_a, self.h_b,
                                 self.h_c, self.h_d, self.K, self.K, self.nloc, self.nloc, self.alpha, self.beta, 0)
            return
        self.ctx.gemm_f16(self.M, self.nloc, self.K, self.h_a, self.h_b, self.h_c, self.h_d,
                          self.K, self.K, self.nloc, self.nloc, self.alpha, self.beta, 0)

    def host_stage_ms(self):
        """Device times of the stages of the last host-driver call (upload span, exchange of A, GEMM, download, total)."""
        return self.ctx.last_stage_ms()

    def config(self, world):
        return {"workload": "perf_hgemm-form dense fp16 GEMM, M=N=K=8192, A row-major fp16, B col-major fp16, "
                            "C/D row-major fp16, fp32 accumulate, alpha=beta=1",
                "M": self.M, "N": self.N, "K": self.K,
                "sharding": "single GPU" if world == 1 else f"N split into {world} column blocks, A broadcast once (NCCL)",
                "l2": "inputs larger than L2 (A+B+C+D = 512 MiB)"}

    # CPU reference: first `rows` rows of the same problem (rows are independent in gemm_CPU)
    def cpu_sample(self, impl, rows):
        import numpy as np
        from oracle import cpu_ref as R
        from rocwmma_b200 import datagen as G
        K, N = self.K, self.N
        if not hasattr(self, "_cpu"):
            a = G.uniform_np(G.SEED_A, (rows, K), np.float16)
            b = G.uniform_np(G.SEED_B, (N, K), np.float16)
            c = G.uniform_np(G.SEED_C, (rows, N), np.float16)
            self._cpu = (a, b, c)
        a, b, c = self._cpu
        t0 = time.perf_counter()
        R.gemm(impl, rows, N, K, a[:rows].ravel(), b.ravel(), c[:rows].ravel(), 1.0, 1.0, np.float16)
        dt = time.perf_counter() - t0
        return 2.0 * rows * N * K, dt

    def value(self, work, seconds):
        return work / seconds / 1e12

    cpu_rows = 64
    parity_rows = 16
    parity_tol = 2e-3     # fp16 outputs: |d - ref| / (|alpha| sum|a||b| + |beta||c|)

    def _oracle_np(self, t):
        """Device tensor -> numpy array in the oracle's input type (exact widening for bf16 / fp8)."""
        torch = self.torch
        if t.dtype in (torch.float16, torch.float32, torch.float64, torch.int8, torch.int32):
            return t.cpu().numpy()
        return t.to(torch.float32).cpu().numpy()

    def parity(self, host=False):
        """Seeded rows of this rank's block of D (device path: self.d after the last step; host path: h_d)."""
        import numpy as np
        torch = self.torch
        rows = _sample_rows(self.M, self.parity_rows, 4321 + self.rank)
        idx = torch.from_numpy(rows).cuda()
        out_np = {torch.float16: np.float16, torch.float32: np.float32, torch.int32: np.int32,
                  torch.float64: np.float64}[self.d.dtype]
        got = self.h_d[torch.from_numpy(rows)].numpy() if host else self.d[idx].cpu().numpy()
        c = getattr(self, "c", None)
        beta = getattr(self, "beta", 0)
        return _gemm_rows_parity(self, torch, self._oracle_np(self._a_for_oracle()[idx]), self._oracle_np(self.b),
                                 None if (c is None or not beta) else c[idx].cpu().numpy(), got,
                                 getattr(self, "alpha", 1), beta, out_np, self.parity_tol,
                                 f"{len(rows)} seeded rows x this rank's {self.nloc} columns vs the CPU oracle"
                                 + (" (host-buffer driver result)" if host else ""))

    def _a_for_oracle(self):
        return self.a


class GemmBF16(GemmF16):
    """bfloat16 (or fp8) inputs, fp32 C / D: the same problem as gemm_f16 with the inputs rounded to the type."""
    name, metric, dtype = "gemm_bf16", "bf16 GEMM TFLOP/s at 8192^3 (fp32 C/D)", "bf16"
    has_host = False
    parity_tol = 1e-3     # fp32 outputs

    def _in_dtype(self, torch):
        return torch.bfloat16

    def setup(self, torch, rank, world, dist):
        super().setup(torch, rank, world, dist)
        t = self._in_dtype(torch)
        self.a, self.b = self.a.to(t), self.b.to(t)
        self.c = self.c.to(torch.float32)
        self.d = torch.empty_like(self.c)

    def step(self):
        from rocwmma_b200 import api
        fn = api.gemm_bf16 if self.dtype == "bf16" else api.gemm_fp8
        fn(self.M, self.nloc, self.K, self.a, self.b, self.c, self.d, self.K, self.K, self.nloc, self.nloc,
           self.alpha, self.beta)

    def config(self, world):
        cfg = super().config(world)
        cfg["workload"] = (f"dense {self.dtype} GEMM, M=N=K=8192, A row-major, B col-major, C/D row-major fp32, "
                           "fp32 accumulate, alpha=beta=1")
        cfg["l2"] = "inputs larger than L2"
        return cfg

    def cpu_sample(self, impl, rows):
        import numpy as np
        import torch
        from oracle import cpu_ref as R
        from rocwmma_b200 import datagen as G
        K, N = self.K, self.N
        if not hasattr(self, "_cpu"):
            t = self._in_dtype(torch)
            widen = lambda x: torch.from_numpy(x).to(t).to(torch.float32).numpy()
            self._cpu = (widen(G.uniform_np(G.SEED_A, (rows, K), np.float32)), widen(G.uniform_np(G.SEED_B, (N, K), np.float32)),
                         G.uniform_np(G.SEED_C, (rows, N), np.float32))
        a, b, c = self._cpu
        t0 = time.perf_counter()
        R.gemm(impl, rows, N, K, a[:rows].ravel(), b.ravel(), c[:rows].ravel(), 1.0, 1.0, np.float32)
        return 2.0 * rows * N * K, time.perf_counter() - t0


class GemmF32(GemmBF16):
    name, metric, dtype = "gemm_f32", "fp32 GEMM (3 x TF32) TFLOP/s at 8192^3", "f32"
    launches_per_step = 3   # split A, split B, GEMM

    def _in_dtype(self, torch):
        return torch.float32

    def setup(self, torch, rank, world, dist):
        super().setup(torch, rank, world, dist)
        from rocwmma_b200 import api
        from rocwmma_b200 import datagen as G
        # full 24-bit mantissas (the inherited tensors hold fp16-rounded values, whose low TF32 terms would be zero)
        col0, _ = _shard(self.N, world, rank)
        G.fill_torch(self.a, G.SEED_A, "uniform")
        G.fill_torch(self.b, G.SEED_B, "uniform", start=col0 * self.K)
        self.ws = torch.empty(api.gemm_f32_workspace_bytes(self.M, self.nloc, self.K), dtype=torch.uint8, device="cuda")

    def step(self):
        from rocwmma_b200 import api
        api.gemm_f32(self.M, self.nloc, self.K, self.a, self.b, self.c, self.d, self.K, self.K, self.nloc, self.nloc,
                     self.alpha, self.beta, self.ws)


class GemmFP8(GemmBF16):
    name, metric, dtype = "gemm_fp8", "fp8 (e4m3) GEMM TFLOP/s at 8192^3 (fp32 C/D)", "fp8"

    def _in_dtype(self, torch):
        return torch.float8_e4m3fn


class GemmI8(GemmF16):
    name, metric, unit, dtype = "gemm_i8", "int8 GEMM TOP/s at 8192x8192x16384", "TOP/s", "i8"
    M, N, K = 8192, 8192, 16384
    variant = "dense"

    def setup(self, torch, rank, world, dist):
        from rocwmma_b200 import api
        from rocwmma_b200 import datagen as G
        self.torch, self.rank, self.world = torch, rank, world
        M, N, K = self.M, self.N, self.K
        col0, self.nloc = _shard(N, world, rank)
        kind = "int4" if self.variant == "i4" else "int8"
        self.b = G.fill_torch(torch.empty((self.nloc, K), dtype=torch.int8, device="cuda"), G.SEED_B, kind, start=col0 * K)
        self.a = torch.empty((M, K), dtype=torch.int8, device="cuda")
        if rank == 0:
            G.fill_torch(self.a, G.SEED_A, kind)
        self.a_broadcast_ms = 0.0
        if world > 1:
            torch.cuda.synchronize(); dist.barrier()
            self.a_broadcast_ms, self.a_broadcast_warm_ms = _timed_broadcast(torch, dist, self.a)
        self.d = torch.empty((M, self.nloc), dtype=torch.int32, device="cuda")
        if self.variant == "sp24":
            import numpy as np
            # compress on the host in row chunks (format definition lives in datagen.sparsify_24_np)
            vals = torch.empty((M, K // 2), dtype=torch.int8, device="cuda")
            meta = torch.empty((M, K // 8), dtype=torch.uint8, device="cuda")
            self.a_dense = torch.empty_like(self.a)   # the densified operand, kept for the parity check only
            for r0 in range(0, M, 1024):
                v, md, dn = G.sparsify_24_np(self.a[r0:r0 + 1024].cpu().numpy(), row_start=r0)
                vals[r0:r0 + 1024] = torch.from_numpy(v).cuda()
                meta[r0:r0 + 1024] = torch.from_numpy(md).cuda()
                self.a_dense[r0:r0 + 1024] = torch.from_numpy(dn).cuda()
            self.vals, self.meta = vals, meta
            self.ws = torch.empty(api.gemm_i8_sp24_workspace_bytes(M, self.nloc, K), dtype=torch.uint8, device="cuda")
        elif self.variant == "i4":
            pack = lambda t: ((t[:, 0::2].to(torch.uint8) & 0xF) | ((t[:, 1::2].to(torch.uint8) & 0xF) << 4)).contiguous()
            self.ap, self.bp = pack(self.a), pack(self.b)
            nws = api.gemm_i4_workspace_bytes(M, self.nloc, K)
            self.ws = torch.empty(nws, dtype=torch.uint8, device="cuda") if nws else None
        self.work_total = 2.0 * M * N * K
        self.work_local = 2.0 * M * self.nloc * K

    def step(self):
        from rocwmma_b200 import api
        M, K, n = self.M, self.K, self.nloc
        if self.variant == "dense":
            api.gemm_i8(M, n, K, self.a, self.b, None, self.d, K, K, n, n, 1, 0, workspace=self._split_ws())
        elif self.variant == "sp24":
            api.gemm_i8_sp24(M, n, K, self.vals, self.meta, self.b, None, self.d, K // 2, K // 8, K, n, n, 1, 0, self.ws)
        else:
            api.gemm_i4(M, n, K, self.ap, self.bp, None, self.d, K // 2, K // 2, n, n, 1, 0, self.ws)

    def setup_host(self):
        from rocwmma_b200 import api
        t = self.torch
        self.h_a = self.a.cpu().pin_memory(); self.h_b = self.b.cpu().pin_memory()
        self.h_d = t.empty(self.d.shape, dtype=t.int32).pin_memory()
        self.ctx = api.HostContext()
        self.h2d = self.h_a.numel() + self.h_b.numel()
        self.d2h = self.h_d.numel() * 4
        self.mg = None
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            # as for the fp16 GEMM: each row block of A is uploaded by one rank and broadcast inside the timed call
            ident = [api.MultiGpu.unique_id() if dist.get_rank() == 0 else None]
            dist.broadcast_object_list(ident, src=0)
            self.mg = api.MultiGpu(ident[0], dist.get_rank(), dist.get_world_size())
            blocks = (self.M + 1023) // 1024
            mine = len(range(dist.get_rank(), blocks, dist.get_world_size()))
            self.h2d -= (blocks - mine) * 1024 * self.K

    def step_host(self):
        n = self.nloc
        if self.mg is not None:
            self.ctx.gemm_i8_mg(self.mg, -1, self.M, n, self.K, self.h_a, self.h_b, None, self.h_d, self.K, self.K, n, n, 1, 0)
            return
        self.ctx.gemm_i8(self.M, n, self.K, self.h_a, self.h_b, None, self.h_d, self.K, self.K, n, n, 1, 0)

    def config(self, world):
        return {"workload": f"int8 GEMM ({self.variant}), M=N=8192, K=16384, A row-major, B col-major, C/D int32 row-major, "
                            "alpha=1, beta=0", "M": self.M, "N": self.N, "K": self.K,
                "sharding": "single GPU" if world == 1 else f"N split into {world} column blocks, A broadcast once (NCCL)",
                "l2": "inputs larger than L2"}

    def cpu_sample(self, impl, rows):
        import numpy as np
        from oracle import cpu_ref as R
        from rocwmma_b200 import datagen as G
        K, N = self.K, self.N
        if not hasattr(self, "_cpu"):
            self._cpu = (G.int8_np(G.SEED_A, (rows, K)), G.int8_np(G.SEED_B, (N, K)))
        a, b = self._cpu
        t0 = time.perf_counter()
        R.gemm(impl, rows, N, K, a[:rows].ravel(), b.ravel(), None, 1, 0, np.int32)
        return 2.0 * rows * N * K, time.perf_counter() - t0

    cpu_rows = 64
    alpha, beta = 1, 0

    def _a_for_oracle(self):
        return self.a_dense if self.variant == "sp24" else self.a


class GemmI8Sp24(GemmI8):
    name, variant = "gemm_i8_sp24", "sp24"
    has_host = False   # the host-buffer driver exists for the dense int8 form only
    launches_per_step = 2   # metadata re-tiling + sparse tensor-core GEMM
    metric = "2:4-sparse int8 GEMM dense-equivalent TOP/s at 8192x8192x16384"


class GemmI4(GemmI8):
    name, variant = "gemm_i4", "i4"
    has_host = False
    launches_per_step = 1   # one kernel: the nibbles are sign-extended between the TMA load and the MMA
    metric = "int4-unpacked GEMM TOP/s at 8192x8192x16384"


class GemmF64(Workload):
    name, metric, unit, dtype, bound = "gemm_f64", "fp64 GEMM TFLOP/s at 4096^3", "TFLOP/s", "f64", "tensor"
    M = N = K = 4096

    def setup(self, torch, rank, world, dist):
        from rocwmma_b200 import datagen as G
        self.torch, self.rank = torch, rank
        col0, self.nloc = _shard(self.N, world, rank)
        f = lambda shape, seed, start=0: G.fill_torch(torch.empty(shape, dtype=torch.float64, device="cuda"), seed, "uniform", start=start)
        self.a, self.b = f((self.M, self.K), 1), f((self.nloc, self.K), 2, col0 * self.K)
        self.c = f((self.M, self.nloc), 3 + 10 * rank)
        self.d = torch.empty_like(self.c)
        self.a_broadcast_ms = 0.0
        self.work_total = 2.0 * self.M * self.N * self.K
        self.work_local = 2.0 * self.M * self.nloc * self.K

    def step(self):
        from rocwmma_b200 import api
        api.gemm_f64(self.M, self.nloc, self.K, self.a, self.b, self.c, self.d, self.K, self.K, self.nloc, self.nloc, 1.0, 1.0)

    def config(self, world):
        return {"workload": "fp64 GEMM (DMMA), M=N=K=4096, A row-major, B col-major, alpha=beta=1", "l2": "inputs larger than L2"}

    alpha = beta = 1.0
    parity_rows, parity_tol = 32, 1e-12
    _oracle_np = GemmF16._oracle_np
    _a_for_oracle = GemmF16._a_for_oracle
    parity = GemmF16.parity

    def value(self, work, seconds):
        return work / seconds / 1e12

    def cpu_sample(self, impl, rows):
        import numpy as np
        from oracle import cpu_ref as R
        from rocwmma_b200 import datagen as G
        if not hasattr(self, "_cpu"):
            self._cpu = (G.uniform_np(1, (rows, self.K), np.float64), G.uniform_np(2, (self.N, self.K), np.float64),
                         G.uniform_np(3, (rows, self.N), np.float64))
        a, b, c = self._cpu
        t0 = time.perf_counter()
        R.gemm(impl, rows, self.N, self.K, a.ravel(), b.ravel(), c.ravel(), 1.0, 1.0, np.float64)
        return 2.0 * rows * self.N * self.K, time.perf_counter() - t0

    cpu_rows = 128


class Dlrm(Workload):
    bound, unit, dtype, scaling = "hbm", "samples/s", "f16", "strong"
    graph_replay = True   # short launches: time them as one replayed CUDA graph (Harness.timed_graph)
    B, m, m_stride, k, width = 16384, 27, 32, 128, 480
    backward = False

    @property
    def name(self):
        return "dlrm_bwd" if self.backward else "dlrm_fwd"

    @property
    def metric(self):
        return f"DLRM dot-interaction {'backward' if self.backward else 'forward'} samples/s at B=16384"

    def setup(self, torch, rank, world, dist):
        from rocwmma_b200 import datagen as G
        self.torch, self.rank = torch, rank
        b0, self.bloc = _shard(self.B, world, rank)
        ms, k, w = self.m_stride, self.k, self.width
        # L2 is 126 MB and one full batch is ~134 MB of X: rotate over independent batches holding at least 300 MB
        # together (4 of them on one GPU, more when the batch is split over ranks) so no step finds its input cached
        self.nbuf = max(4, int((300 << 20) // (self.bloc * ms * k * 2)) + 1)
        self.x = [torch.zeros((self.bloc, ms, k), dtype=torch.float16, device="cuda") for _ in range(self.nbuf)]
        self.up = [torch.zeros((self.bloc, w), dtype=torch.float16, device="cuda") for _ in range(self.nbuf)]
        for i in range(self.nbuf):
            G.fill_torch(self.x[i], G.SEED_X + 100 * i, "normal", sigma=0.25, start=b0 * ms * k)
            self.x[i][:, self.m:] = 0
            G.fill_torch(self.up[i], G.SEED_G + 100 * i, "normal", sigma=0.1, start=b0 * w)
            self.up[i][:, w - 1] = 0
        self.out = torch.empty((self.bloc, w), dtype=torch.float16, device="cuda")
        self.grad = torch.zeros((self.bloc, ms, k), dtype=torch.float16, device="cuda")
        self.i = 0
        self.a_broadcast_ms = 0.0
        self.work_total, self.work_local = float(self.B), float(self.bloc)
        real = self.m * k * 2
        self.bytes_per_sample = (real + w * 2 + real) if self.backward else (real + w * 2)

    def step(self):
        from rocwmma_b200 import api
        i = self.i = (self.i + 1) % self.nbuf
        if self.backward:
            api.dlrm_dot_bwd(self.x[i], self.up[i], self.grad, None, self.m, self.m_stride, self.k, self.bloc, self.width, True)
        else:
            api.dlrm_dot_fwd(self.x[i], self.out, self.m, self.m_stride, self.k, self.bloc, self.width)

    def setup_host(self):
        from rocwmma_b200 import api
        t = self.torch
        self.h_x = self.x[0].cpu().pin_memory(); self.h_up = self.up[0].cpu().pin_memory()
        self.h_out = t.empty(self.out.shape, dtype=t.float16).pin_memory()
        self.h_grad = t.zeros(self.grad.shape, dtype=t.float16).pin_memory()
        self.ctx = api.HostContext()
        if self.backward:
            self.h2d = (self.h_x.numel() + self.h_up.numel() + self.h_grad.numel()) * 2
            self.d2h = self.h_grad.numel() * 2
        else:
            self.h2d, self.d2h = self.h_x.numel() * 2, self.h_out.numel() * 2

    def step_host(self):
        if self.backward:
            self.ctx.dlrm_bwd(self.h_x, self.h_up, self.h_grad, None, self.m, self.m_stride, self.k, self.bloc, self.width, True)
        else:
            self.ctx.dlrm_fwd(self.h_x, self.h_out, self.m, self.m_stride, self.k, self.bloc, self.width)

    def config(self, world):
        return {"workload": f"DLRM dot interaction {'backward' if self.backward else 'forward'}, B=16384, 27 feature rows padded "
                            "to 32 x 128 fp16, output / upstream width 480",
                "sharding": "single GPU" if world == 1 else f"batch split over {world} ranks",
                "l2": "independent input batches (4 or more, at least 300 MB together) rotated so that no step re-reads a "
                      "cached input",
                "launch": getattr(self, "launch_mode", None) or
                          "the K timed launches are captured once in a CUDA graph and replayed between the events (a "
                          "launch lasts 10-50 us, a launch from Python about 12 us)"}

    def value(self, work, seconds):
        return work / seconds

    def parity(self, host=False):
        """64 seeded samples of this rank's shard against the oracle: pass-through columns exact, the packed triangle /
        the gradient within 2e-3 of sum|a||b| (fp16 outputs; twice that on the fused row 0, which is rounded once
        more in the oracle), padding columns zero."""
        import numpy as np
        from oracle import cpu_ref as R
        from rocwmma_b200 import api
        torch, m, k, w = self.torch, self.m, self.k, self.width
        rows = _sample_rows(self.bloc, 64, 977 + self.rank)
        idx = torch.from_numpy(rows).cuda()
        if not host:
            if self.backward:
                api.dlrm_dot_bwd(self.x[0], self.up[0], self.grad, None, m, self.m_stride, k, self.bloc, w, True)
            else:
                api.dlrm_dot_fwd(self.x[0], self.out, m, self.m_stride, k, self.bloc, w)
            torch.cuda.synchronize()
        x = np.ascontiguousarray(self.x[0][idx][:, :m].cpu().numpy())
        x64 = np.abs(x.astype(np.float64))
        il, jl = np.tril_indices(m, -1)
        what = f"{len(rows)} seeded samples of this rank's shard vs the CPU oracle" + (" (host-buffer driver result)" if host else "")
        if not self.backward:
            got = (self.h_out[torch.from_numpy(rows)] if host else self.out[idx].cpu()).numpy()
            ref = R.dlrm_fwd(R.port(), x, m, k, len(rows))
            wreal = k + len(il)
            bound = np.einsum("bik,bjk->bij", x64, x64)[:, il, jl]
            err = float(np.max(np.abs(got[:, k:wreal].astype(np.float64) - ref[:, k:].astype(np.float64)) / np.maximum(bound, 1e-30)))
            exact = np.array_equal(got[:, :k], x[:, 0, :]) and bool((got[:, wreal:] == 0).all())
            res = _parity_result(len(rows), err if exact else float("inf"), 2e-3, what=what)
            return res
        up = self.up[0][idx].cpu().numpy()
        got = (self.h_grad[torch.from_numpy(rows)] if host else self.grad[idx].cpu()).numpy()[:, :m]
        ref_grad, _ = R.dlrm_bwd(R.port(), x, np.ascontiguousarray(up[:, :k + len(il)]), m, k, len(rows))
        expect = ref_grad.astype(np.float64)
        expect[:, 0, :] += up[:, :k].astype(np.float64)
        T = np.zeros((len(rows), m, m))
        T[:, il, jl] = np.abs(up[:, k:k + len(il)].astype(np.float64))
        T = T + T.transpose(0, 2, 1)
        bound = np.einsum("bih,bhj->bij", T, x64)
        bound[:, 0, :] += np.abs(up[:, :k].astype(np.float64))
        err = float(np.max(np.abs(got.astype(np.float64) - expect) / np.maximum(bound, 1e-30)))
        return _parity_result(len(rows), err, 4e-3, what=what)

    def cpu_sample(self, impl, rows):
        import numpy as np
        from oracle import cpu_ref as R
        from rocwmma_b200 import datagen as G
        if not hasattr(self, "_cpu"):
            self._cpu = (G.normal_np(G.SEED_X, (rows, self.m, self.k), 0.25, np.float16),
                         G.normal_np(G.SEED_G, (rows, self.k + self.m * (self.m - 1) // 2), 0.1, np.float16))
        x, g = self._cpu
        t0 = time.perf_counter()
        if self.backward:
            R.dlrm_bwd(impl, x, g, self.m, self.k, rows)
        else:
            R.dlrm_fwd(impl, x, self.m, self.k, rows)
        return float(rows), time.perf_counter() - t0

    cpu_rows = 16384


class DlrmBwd(Dlrm):
    backward = True


class Gemv(Workload):
    bound, unit, scaling = "hbm", "GB/s", "strong"
    M = N = 32768
    double = False

    @property
    def name(self):
        return "dgemv" if self.double else "sgemv"

    @property
    def dtype(self):
        return "f64" if self.double else "f32"

    @property
    def metric(self):
        return f"{'dgemv' if self.double else 'sgemv'} achieved GB/s at 32768^2"

    def setup(self, torch, rank, world, dist):
        from rocwmma_b200 import datagen as G
        self.torch, self.rank = torch, rank
        dt = torch.float64 if self.double else torch.float32
        r0, self.mloc = _shard(self.M, world, rank)
        self.a = G.fill_torch(torch.empty((self.mloc, self.N), dtype=dt, device="cuda"), G.SEED_GEMV_A, "uniform", start=r0 * self.N)
        self.x = G.fill_torch(torch.empty(self.N, dtype=dt, device="cuda"), G.SEED_GEMV_X, "uniform")
        self.y = G.fill_torch(torch.empty(self.mloc, dtype=dt, device="cuda"), G.SEED_GEMV_Y, "uniform", start=r0)
        self.y0 = self.y.clone()   # y is updated in place by every step; the parity check starts from this copy
        es = 8 if self.double else 4
        self.a_broadcast_ms = 0.0
        self.work_total = float(es * (self.M * self.N + self.N + 2 * self.M))
        self.work_local = float(es * (self.mloc * self.N + self.N + 2 * self.mloc))

    def step(self):
        from rocwmma_b200 import api
        api.gemv(self.mloc, self.N, self.a, self.N, self.x, self.y, 1.5, 0.5)

    def setup_host(self):
        from rocwmma_b200 import api
        self.h_a = self.a.cpu().pin_memory(); self.h_x = self.x.cpu().pin_memory(); self.h_y = self.y0.cpu().pin_memory()
        self.h_y0 = self.y0.cpu()
        self.ctx = api.HostContext()
        es = 8 if self.double else 4
        self.h2d = (self.h_a.numel() + self.h_x.numel() + self.h_y.numel()) * es
        self.d2h = self.h_y.numel() * es

    def step_host(self):
        self.ctx.gemv(self.mloc, self.N, self.h_a, self.N, self.h_x, self.h_y, 1.5, 0.5, double=self.double)

    def host_parity_prepare(self):
        self.h_y.copy_(self.h_y0)   # y is updated in place: one call on the original vector
        self.step_host()

    def config(self, world):
        return {"workload": f"{'dgemv' if self.double else 'sgemv'} y = 1.5*A*x + 0.5*y, A row-major 32768 x 32768",
                "sharding": "single GPU" if world == 1 else f"rows split over {world} ranks, x replicated",
                "l2": "matrix (4 / 8 GiB) larger than L2"}

    def value(self, work, seconds):
        return work / seconds / 1e9

    def parity(self, host=False):
        """64 seeded rows of this rank's shard, one call on a fresh copy of y, against the oracle:
        |y - ref| / (|alpha| sum|a||x| + |beta||y0|) <= 1e-3 (fp32) / 1e-12 (fp64)."""
        import numpy as np
        from oracle import cpu_ref as R
        from rocwmma_b200 import api
        torch = self.torch
        dt = np.float64 if self.double else np.float32
        rows = _sample_rows(self.mloc, 64, 611 + self.rank)
        idx = torch.from_numpy(rows).cuda()
        if host:
            y0, got = self.h_y0[torch.from_numpy(rows)].numpy(), self.h_y[torch.from_numpy(rows)].numpy()
        else:
            y = self.y0.clone()
            api.gemv(self.mloc, self.N, self.a, self.N, self.x, y, 1.5, 0.5)
            torch.cuda.synchronize()
            y0, got = self.y0[idx].cpu().numpy(), y[idx].cpu().numpy()
        ah, xh = self.a[idx].cpu().numpy(), self.x.cpu().numpy()
        ref = R.gemv(R.port(), len(rows), self.N, np.ascontiguousarray(ah).ravel(), xh, y0, dt(1.5), dt(0.5))
        bound = 1.5 * (np.abs(ah.astype(np.float64)) @ np.abs(xh.astype(np.float64))) + 0.5 * np.abs(y0.astype(np.float64))
        err = float(np.max(np.abs(got.astype(np.float64) - ref.astype(np.float64)) / np.maximum(bound, 1e-300)))
        return _parity_result(len(rows), err, 1e-12 if self.double else 1e-3,
                              what=f"{len(rows)} seeded rows of this rank's shard vs the CPU oracle" + (" (host-buffer driver result)" if host else ""))

    def cpu_sample(self, impl, rows):
        import numpy as np
        from oracle import cpu_ref as R
        from rocwmma_b200 import datagen as G
        dt = np.float64 if self.double else np.float32
        if not hasattr(self, "_cpu"):
            self._cpu = (G.uniform_np(6, (rows, self.N), dt), G.uniform_np(7, (self.N,), dt), G.uniform_np(8, (rows,), dt))
        a, x, y = self._cpu
        t0 = time.perf_counter()
        R.gemv(impl, rows, self.N, a.ravel(), x, y, dt(1.5), dt(0.5))
        es = 8 if self.double else 4
        return float(es * (rows * self.N + self.N + 2 * rows)), time.perf_counter() - t0

    cpu_rows = 8192


class Dgemv(Gemv):
    double = True


class FragSimpleHgemm(GemmF16):
    """hgemm_rocwmma_d of samples/simple_hgemm.cpp on this repository's fragment headers: the 1024^3 correctness-gate
    configuration (A row-major, B column-major fp16, C / D fp32, alpha = beta = 2), one 16x16 block per warp."""
    name, metric, dtype = "frag_simple_hgemm", "fragment-API simple_hgemm TFLOP/s at 1024^3 (fp32 C/D, alpha=beta=2)", "f16"
    M = N = K = 1024
    alpha = beta = 2.0
    has_host = False
    legacy_mma = True
    parity_rows, parity_tol = 64, 1e-3

    def setup(self, torch, rank, world, dist):
        from rocwmma_b200 import datagen as G
        self.torch, self.rank, self.world = torch, rank, world
        M, N, K = self.M, self.N, self.K
        col0, self.nloc = _shard(N, world, rank)
        self.a = G.fill_torch(torch.empty((M, K), dtype=torch.float16, device="cuda"), G.SEED_A, "uniform")
        self.b = G.fill_torch(torch.empty((self.nloc, K), dtype=torch.float16, device="cuda"), G.SEED_B, "uniform", start=col0 * K)
        self.c = G.fill_torch(torch.empty((M, self.nloc), dtype=torch.float32, device="cuda"), G.SEED_C + 10 * rank, "uniform")
        self.d = torch.empty_like(self.c)
        self.a_broadcast_ms = 0.0
        self.work_total, self.work_local = 2.0 * M * N * K, 2.0 * M * self.nloc * K

    def step(self):
        from rocwmma_b200 import api
        api.simple_hgemm(self.M, self.nloc, self.K, self.a, self.b, self.c, self.d, self.K, self.K, self.nloc, self.nloc,
                         self.alpha, self.beta)

    def config(self, world):
        return {"workload": "simple_hgemm on the fragment API (mma.sync), M=N=K=1024, A row-major / B col-major fp16, C/D fp32, "
                            "alpha=beta=2", "M": self.M, "N": self.N, "K": self.K,
                "sharding": "single GPU" if world == 1 else f"N split into {world} column blocks",
                "l2": "problem fits L2 (correctness-gate size)"}


class FragPerfHgemm(FragSimpleHgemm):
    """perf_hgemm's kernel pattern (cooperative global reads, shared-memory double buffer, fragment transforms) on the
    fragment headers, in the layouts the sample ships with: A column-major, B row-major, C / D row-major fp16."""
    name, metric = "frag_perf_hgemm", "fragment-API perf_hgemm TFLOP/s at 8192^3 (A col-major, B row-major, fp16 C/D)"
    M = N = K = 8192
    alpha = beta = 1.0
    parity_rows, parity_tol = 16, 2e-3

    def setup(self, torch, rank, world, dist):
        from rocwmma_b200 import datagen as G
        self.torch, self.rank, self.world = torch, rank, world
        M, N, K = self.M, self.N, self.K
        col0, self.nloc = _shard(N, world, rank)
        f16 = torch.float16
        self.a_t = G.fill_torch(torch.empty((K, M), dtype=f16, device="cuda"), G.SEED_A, "uniform")            # A column-major
        self.b_kn = G.fill_torch(torch.empty((K, self.nloc), dtype=f16, device="cuda"), G.SEED_B + 10 * rank, "uniform")  # B row-major
        self.c = G.fill_torch(torch.empty((M, self.nloc), dtype=f16, device="cuda"), G.SEED_C + 10 * rank, "uniform")
        self.d = torch.empty_like(self.c)
        self.a_broadcast_ms = 0.0
        self.work_total, self.work_local = 2.0 * M * N * K, 2.0 * M * self.nloc * K

    def step(self):
        from rocwmma_b200 import api
        api.perf_hgemm_fragment(self.M, self.nloc, self.K, self.a_t, self.b_kn, self.c, self.d, self.M, self.nloc,
                                self.nloc, self.nloc, self.alpha, self.beta)

    def parity(self, host=False):
        import numpy as np
        torch = self.torch
        rows = _sample_rows(self.M, self.parity_rows, 4321 + self.rank)
        idx = torch.from_numpy(rows).cuda()
        a_rows = self.a_t[:, idx].t().contiguous().cpu().numpy()
        b_store = self.b_kn.t().contiguous().cpu().numpy()   # [n, k]: the oracle helper takes column-major B
        return _gemm_rows_parity(self, torch, a_rows, b_store, self.c[idx].cpu().numpy(), self.d[idx].cpu().numpy(),
                                 self.alpha, self.beta, np.float16, self.parity_tol,
                                 f"{len(rows)} seeded rows x this rank's {self.nloc} columns vs the CPU oracle")

    def config(self, world):
        return {"workload": "perf_hgemm kernel pattern on the fragment API (mma.sync), M=N=K=8192, A col-major / B row-major fp16, "
                            "C/D row-major fp16, alpha=beta=1", "M": self.M, "N": self.N, "K": self.K,
                "sharding": "single GPU" if world == 1 else f"N split into {world} column blocks",
                "l2": "inputs larger than L2"}


WORKLOADS = {w().name: w for w in (FragSimpleHgemm, FragPerfHgemm, GemmF16, GemmBF16, GemmFP8, GemmF32, GemmI8, GemmI8Sp24, GemmI4, GemmF64, Dlrm, DlrmBwd, Gemv, Dgemv)}


# ---------------------------------------------------------------------------------------- CPU arm
def cpu_impl():
    from oracle import cpu_ref as R
    impl, kind = (R.reference(), "reference") if R.have_reference() else (R.port(), "port")
    R.use_all_host_threads(impl)  # torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every host thread
    return impl, kind


def cpu_baseline(wl, budget_s=12.0):
    """Times the CPU reference on a bounded sample of the workload; returns the cpu_baseline object."""
    from oracle import cpu_ref as R
    impl, kind = cpu_impl()
    rows = wl.cpu_rows
    work, dt = wl.cpu_sample(impl, rows)  # also warms caches / first-touch
    work, dt = wl.cpu_sample(impl, rows)
    reps = 1
    while dt < budget_s and reps < 256:  # about budget_s seconds of wall time on all host threads
        w2, d2 = wl.cpu_sample(impl, rows)
        work, dt, reps = work + w2, dt + d2, reps + 1
    return {"value": wl.value(work, dt), "unit": wl.unit, "cores": R.num_threads(impl), "kind": kind,
            "sample": f"{reps} x first {rows} rows/samples of the same seeded workload ({dt:.2f} s timed)"}


def run_reference_arm(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import cpu_ref as R
    impl, kind = cpu_impl()
    rows = wl.cpu_rows
    for _ in range(max(1, min(args.warmup, 2))):
        wl.cpu_sample(impl, rows)
    work, secs = 0.0, 0.0
    for _ in range(args.steps):
        w, d = wl.cpu_sample(impl, rows)
        work, secs = work + w, secs + d
    v = wl.value(work, secs)
    line = {
        "impl": "reference", "metric": wl.metric, "value": v, "unit": wl.unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True, "scaling": wl.scaling,
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic (seeded)", "config": wl.config(1),
        "cpu_baseline": {"value": v, "unit": wl.unit, "cores": R.num_threads(impl), "kind": kind,
                         "sample": f"each step = first {rows} rows/samples of the workload; rows are independent in the reference loop"},
        "e2e": {"value": v, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------- GPU arm
_MMA_SYNC_RATE = {}


def mma_sync_rate(kind):
    """Measured issue rate (TFLOP/s) of mma.sync m16n8k16 f16->f32 (kind 0) / m16n8k8 f64 (kind 1) on this GPU; cached."""
    if kind not in _MMA_SYNC_RATE:
        try:
            from rocwmma_b200 import api
            _MMA_SYNC_RATE[kind] = api.measure_mma_sync_rate(kind)
        except Exception:
            _MMA_SYNC_RATE[kind] = None
    return _MMA_SYNC_RATE[kind]


def roofline_of(wl, ms_step, peaks, copy_same):
    """roofline object of one workload from its measured step time (this rank's share of the work / this GPU's peak)."""
    if wl.bound == "tensor":
        peak = peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"])
        variant = getattr(wl, "variant", "")
        if wl.dtype == "f32":
            peak /= 6.0  # TF32 runs at half the 16-bit rate and every product takes three MMAs
            peak_note = "cuBLAS bf16 8192^3 burst / 6: TF32 rate over three products"
        elif wl.dtype == "fp8":
            peak *= 2.0  # the fp8 tensor rate is twice the 16-bit rate; no fp8 figure is measured
            peak_note = "2 x cuBLAS bf16 8192^3 burst, standing in for the dense fp8 rate"
        elif wl.dtype == "i8" and variant == "sp24":
            peak *= 4.0  # sparse int8: twice the dense int8 rate (measured: 112 clocks per 256x224x64 pair MMA)
            peak_note = "4 x cuBLAS bf16 8192^3 burst, standing in for the 2:4-sparse int8 rate"
        elif wl.dtype == "i8":
            peak *= 2.0  # the dense int8 tensor rate is twice the 16-bit rate; no int8 figure is measured
            peak_note = "2 x cuBLAS bf16 8192^3 burst, standing in for the dense int8 rate"
        elif wl.dtype == "f64":
            peak = 40.0
            peak_note = "nominal B200 fp64 tensor rate"
        elif getattr(wl, "legacy_mma", False):
            peak_note = "cuBLAS bf16 8192^3 burst (tcgen05); this workload runs on the warp-level mma.sync path of the fragment API"
        else:
            peak_note = "cuBLAS bf16 8192^3 burst"
        achieved = wl.work_local / (ms_step * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s" if wl.dtype != "i8" else "TOP/s",
                "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(wl.name),
                "peak_source": f"{peaks['_source']} ({peak_note})"}
        # the vendor's dense figures, for context: 2250 TFLOP/s 16-bit, 4500 fp8 / int8, 9000 for 2:4-sparse int8,
        # 1125 / 3 for fp32 through three TF32 products, 40 fp64
        nominal = {"f16": 2250.0, "bf16": 2250.0, "fp8": 4500.0, "f32": 375.0, "f64": 40.0}.get(wl.dtype)
        if wl.dtype == "i8":
            nominal = 9000.0 if variant == "sp24" else 4500.0
        if nominal:
            roof["nominal_peak"] = nominal
            roof["frac_of_nominal"] = achieved / nominal
        # kernels built on warp-level mma.sync: the rate at which this GPU issues that instruction from registers,
        # measured just now (b200wmma_measure_mma_sync_rate), is the bound that applies to them
        kind = 1 if wl.dtype == "f64" else (0 if getattr(wl, "legacy_mma", False) else None)
        if kind is not None:
            rate = mma_sync_rate(kind)
            if rate:
                roof["mma_sync_rate"] = rate
                roof["frac_of_mma_sync_rate"] = achieved / rate
        return roof
    peak = peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"])
    nbytes = wl.bytes_per_sample * wl.work_local if hasattr(wl, "bytes_per_sample") else wl.work_local
    achieved = nbytes / (ms_step * 1e-3) / 1e9
    roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": NCU_TRAFFIC_BYTES.get(wl.name), "peak_source": f"{peaks['_source']} (copy bandwidth)"}
    if copy_same:
        roof["copy_same_bytes"] = copy_same  # GB/s of torch copy_ moving the same bytes per launch
        roof["frac_of_copy_same_bytes"] = achieved / copy_same
    roof["nominal_peak"] = 8000.0  # GB/s, the vendor's HBM3e figure
    roof["frac_of_nominal"] = achieved / 8000.0
    return roof


class Harness:
    """Device timing shared by the headline workload and the `also` workloads of one process."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; rocwmma_b200 has no CPU fallback (use --impl reference for the CPU arm)")
        torch.cuda.set_device(self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
        assert self.world == args.gpus or self.world == 1, f"--gpus {args.gpus} but WORLD_SIZE={self.world}"
        self.peaks = measured_peaks()

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def reduce_max(self, x):
        if self.world == 1:
            return float(x)
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, fn, steps, sampler=None):
        """K back-to-back calls between two CUDA events on the launching stream, barrier + synchronize on both sides;
        returns (device ms, max over ranks; host wall seconds of this rank)."""
        torch = self.torch
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler:
            sampler.start()
        t0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        if sampler:
            sampler.stop()
        self.barrier()
        return self.reduce_max(e0.elapsed_time(e1)), wall

    def timed_graph(self, fn, steps, sampler=None, wl=None):
        """As `timed`, for launches shorter than the host can issue them: the K calls are captured once into a CUDA graph
        on a side stream (nothing runs during capture), the graph is replayed once untimed, then once between the
        events.  Same K kernels, same buffers, same order as K direct calls.  A rank whose capture fails times direct
        launches instead and says so in `config.launch`."""
        torch = self.torch
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.stream(side):
                # thread_local: a CUDA call from another thread of the process (NCCL's watchdog) must not end the capture
                with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                    for _ in range(steps):
                        fn()
            torch.cuda.current_stream().wait_stream(side)
            graph.replay()
            torch.cuda.synchronize()
        except RuntimeError as exc:
            if wl is not None:
                wl.launch_mode = f"direct launches (graph capture failed: {str(exc)[:80]})"
            torch.cuda.synchronize()
            return self.timed(fn, steps, sampler)
        out = self.timed(graph.replay, 1, sampler)
        del graph
        return out

    def merge_parity(self, res):
        """Combine the per-rank parity results: rows summed, error maximised, ok only if every rank is ok."""
        if self.world == 1:
            return res
        torch, dist = self.torch, self.dist
        err = res["max_rel_err"] if res["max_rel_err"] == res["max_rel_err"] else float("inf")
        t = torch.tensor([err, 0.0 if res["ok"] else 1.0], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        r = torch.tensor([res["rows"]], dtype=torch.int64, device="cuda")
        dist.all_reduce(r)
        out = dict(res)
        out.update(rows=int(r.item()), max_rel_err=float(t[0].item()), ok=bool(t[1].item() == 0.0), ranks=self.world)
        return out

    def measure(self, wl, steps, warmup, headline):
        """Times one workload; returns its part of the JSON line (rank 0 uses it; every rank must call)."""
        torch, args, world = self.torch, self.args, self.world
        from rocwmma_b200 import api
        wl.setup(torch, self.rank, world, self.dist)
        for _ in range(max(warmup, 3)):
            wl.step()
        sampler = ClockSampler(self.local_rank)
        timed = self.timed
        if getattr(wl, "graph_replay", False):
            def timed(fn, k, smp=None):
                return self.timed_graph(fn, k, smp, wl)
        ms_total, _ = timed(wl.step, steps, sampler)
        if len(sampler.samples) < 5:
            # the timed region was too short for the sampling period: extend the same loop (untimed) under the sampler
            sampler.start()
            t_end = time.perf_counter() + 0.4
            while time.perf_counter() < t_end:
                for _ in range(20):
                    wl.step()
                torch.cuda.synchronize()
            sampler.stop()
        st, detail = api.device_status()
        assert st == 0, f"device status {st} (detail {detail:#x})"
        ms_step = ms_total / steps
        value = wl.value(wl.work_total, ms_step * 1e-3)
        parity = self.merge_parity(wl.parity())   # outside the timed region, every rank on its own block

        # Tensor-bound workloads: the same step repeated for a few seconds.  The timed K steps above are a burst (the part
        # has not settled under its power cap yet); this is the rate it holds, to set beside the sustained library figure.
        sustained = None
        if headline and wl.bound == "tensor" and args.sustained_seconds > 0:
            per_batch = max(10, int(0.25 / max(ms_step * 1e-3, 1e-6)))
            done, ms_acc = 0, 0.0
            # the batch count comes from the (rank-reduced) step time, so every rank runs the same number of batches
            batches = max(1, int(args.sustained_seconds / (per_batch * ms_step * 1e-3) + 0.5))
            for _ in range(batches):
                ms_b, _ = self.timed(wl.step, per_batch)
                ms_acc += ms_b
                done += per_batch
            sustained = {"value": wl.value(wl.work_total, ms_acc / done * 1e-3), "unit": wl.unit, "launches": done,
                         "seconds": ms_acc * 1e-3}
            ref = self.peaks.get("bf16_tflops_sustained")
            if ref and wl.dtype == "f16":
                # the aggregate over all ranks against as many GPUs' worth of the measured one-GPU cuBLAS bf16 loop
                sustained["frac_of_sustained_peak"] = sustained["value"] / (ref * world)

        # HBM-bound workloads: a plain device-to-device copy moving the same number of bytes per launch, timed the same
        # way (sources and destinations rotate through sets larger than L2).  The measured copy peak is a large-transfer
        # figure; at these launch sizes a copy does not reach it either, and this figure says what does.
        copy_same = None
        if wl.bound == "hbm" and not args.no_copy_ref:
            nbytes_launch = wl.bytes_per_sample * wl.work_local if hasattr(wl, "bytes_per_sample") else wl.work_local
            half = max(int(nbytes_launch) // 2 // 4 * 4, 4)
            if half <= (6 << 30):
                nbuf = max(2, int((300 << 20) // half) + 1)
                srcs = [torch.empty(half, dtype=torch.uint8, device="cuda") for _ in range(nbuf)]
                dsts = [torch.empty(half, dtype=torch.uint8, device="cuda") for _ in range(nbuf)]
                state = {"i": 0}

                def copy_step():
                    i = state["i"]
                    dsts[i % nbuf].copy_(srcs[i % nbuf])
                    state["i"] = i + 1

                for _ in range(3):
                    copy_step()
                ms_copy, _ = timed(copy_step, steps)
                copy_same = 2.0 * half / (ms_copy / steps * 1e-3) / 1e9
                del srcs, dsts

        # end to end: host buffers through the C ABI host drivers, copies inside the timed region
        e2e = None
        if hasattr(wl, "setup_host") and getattr(wl, "has_host", True) and not args.no_e2e:
            wl.setup_host()
            for _ in range(2):
                wl.step_host()
            e2e_steps = max(2, min(steps, 5)) if headline else 3
            _, wall = self.timed(wl.step_host, e2e_steps)
            wall = self.reduce_max(wall)
            e2e = {"value": wl.value(wl.work_total, wall / e2e_steps), "unit": wl.unit,
                   "h2d_bytes_per_step": int(wl.h2d), "d2h_bytes_per_step": int(wl.d2h), "steps": e2e_steps,
                   "timing": "host wall clock around synchronous C-ABI host calls (pinned host buffers), max over ranks"}
            if hasattr(wl, "host_parity_prepare"):
                wl.host_parity_prepare()
            e2e["parity_check"] = self.merge_parity(wl.parity(host=True))
            stages = getattr(wl, "host_stage_ms", None)
            if stages:
                e2e["stage_ms"] = stages()

        out = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "steps": steps, "warmup": max(warmup, 3),
            "ms_per_step": ms_step, "dtype": wl.dtype, "config": wl.config(world),
            "roofline": roofline_of(wl, ms_step, self.peaks, copy_same), "clocks": sampler.summary(),
            "gpu_launches": steps * getattr(wl, "launches_per_step", 1), "parity_check": parity,
        }
        if getattr(wl, "a_broadcast_ms", 0.0):
            out["a_broadcast_ms"] = wl.a_broadcast_ms
            if getattr(wl, "a_broadcast_warm_ms", None) is not None:
                out["a_broadcast_warm_ms"] = wl.a_broadcast_warm_ms
        if e2e:
            out["e2e"] = e2e
        if sustained:
            out["sustained"] = sustained
        return out


# the other components of the metric, measured after the headline workload in the same process
ALSO = ["gemm_i8", "gemm_i8_sp24", "gemm_i4", "gemm_bf16", "gemm_fp8", "gemm_f32", "gemm_f64", "dlrm_fwd", "dlrm_bwd", "sgemv", "dgemv",
        "frag_simple_hgemm", "frag_perf_hgemm"]


def run_gpu_arm(args, wl):
    import gc
    H = Harness(args)
    torch = H.torch
    main = H.measure(wl, args.steps, args.warmup, headline=True)
    failed = [] if main["parity_check"]["ok"] else [wl.name]
    if "e2e" in main and not main["e2e"]["parity_check"]["ok"]:
        failed.append(wl.name + " (host driver)")
    cpu = cpu_baseline(wl) if (H.rank == 0 and H.world == 1 and not args.no_cpu) else None
    also = {}
    if not args.no_also:
        for name in ALSO:
            if name == wl.name:
                continue
            del wl
            gc.collect()
            torch.cuda.empty_cache()
            wl = WORKLOADS[name]()
            r = H.measure(wl, max(args.also_steps, 20), 3, headline=False)
            if not r["parity_check"]["ok"]:
                failed.append(name)
            if "e2e" in r and not r["e2e"]["parity_check"]["ok"]:
                failed.append(name + " (host driver)")
            also[name] = r
    if H.rank == 0:
        line = {
            "metric": main["metric"], "value": main["value"], "unit": main["unit"], "n_gpus": H.world, "steps": args.steps,
            "warmup": main["warmup"], "ms_per_step": main["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": main["dtype"],
            "data": "synthetic (seeded counter-based generator)", "config": main["config"],
            "roofline": main["roofline"], "clocks": main["clocks"], "gpu_launches": main["gpu_launches"],
            "a_broadcast_ms": main.get("a_broadcast_ms", 0.0), "parity_check": main["parity_check"],
        }
        for key in ("a_broadcast_warm_ms", "e2e", "sustained"):
            if key in main:
                line[key] = main[key]
        if cpu:
            line["cpu_baseline"] = cpu
        if also:
            line["also"] = also
        print(json.dumps(line), flush=True)
    if H.world > 1:
        H.dist.barrier()
        H.dist.destroy_process_group()
    if failed:
        raise SystemExit(f"bench.py: parity check failed for {failed}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm_f16", choices=sorted(WORKLOADS))
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end measurement")
    ap.add_argument("--sustained-seconds", type=float, default=3.0,
                    help="tensor-bound workloads: also report the rate held over this many seconds of back-to-back steps (0 = skip)")
    ap.add_argument("--no-copy-ref", action="store_true",
                    help="HBM-bound workloads: skip timing a plain device copy of the same byte count")
    ap.add_argument("--no-cpu", action="store_true", help="skip the timed CPU baseline")
    ap.add_argument("--no-also", action="store_true", help="measure the headline workload only")
    ap.add_argument("--also-steps", type=int, default=20, help="timed steps of each `also` workload (at least 20)")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]()
    if args.impl == "reference":
        run_reference_arm(args, wl)
    else:
        run_gpu_arm(args, wl)


if __name__ == "__main__":
    main()
