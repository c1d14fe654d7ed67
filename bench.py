"""Benchmark of the hot path.  One JSON line on stdout (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Default workload (the one the headline metric is quoted on): dense fp16 GEMM in the perf_hgemm form,
D = alpha*(A x B) + beta*C, M=N=K=8192, A row-major fp16, B column-major fp16, C/D row-major fp16,
fp32 accumulate, alpha=beta=1, seeded uniform[-1,1) inputs.  A "step" is one GEMM.

N > 1: one process per GPU.  The problem is sharded by N-column blocks (B, C, D split; A broadcast once
over NCCL before the timed region and reported separately as `a_broadcast_ms`); there is no collective in
the data path, total work is fixed (strong scaling), value = 2*M*N*K / max-over-ranks time.

Other workloads (`--workload gemm_bf16 | gemm_fp8 | gemm_f32 | gemm_i8 | gemm_i8_sp24 | gemm_i4 | gemm_f64 | dlrm_fwd | dlrm_bwd | sgemv | dgemv`)
print the same line for the other configurations; they are not the default.

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
    "gemm_f16": 1.144e9,   # profiles/gemm_tc05_f16_8192.md: 1.022 GB read + 122.4 MB written (512x256 pair kernel)
    "gemm_i8": 1.416e9,    # profiles/gemm_tc05_i8_8192x8192x16384.md (256x256 pair kernel capture)
    "gemm_i8_sp24": 8.595e8,  # profiles/gemm_tc05_sp24_8192x8192x16384.md (GEMM kernel; the re-tiling pre-pass adds ~33 MB)
    "dlrm_fwd": 119.5e6,   # profiles/dlrm_dot_B16384.md
    "dlrm_bwd": 195.8e6,   # profiles/dlrm_dot_B16384.md
    "sgemv": 4.299e9,      # profiles/gemv_32768.md
    "dgemv": 8.595e9,      # profiles/gemv_32768.md
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
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            dist.broadcast(self.a, src=0)  # A is needed whole by every rank: one NCCL broadcast, untimed
            e1.record()
            torch.cuda.synchronize()
            self.a_broadcast_ms = e0.elapsed_time(e1)
        self.work_total = 2.0 * M * N * K
        self.work_local = 2.0 * M * self.nloc * K

    def step(self):
        from rocwmma_b200 import api
        api.gemm_f16(self.M, self.nloc, self.K, self.a, self.b, self.c, self.d,
                     self.K, self.K, self.nloc, self.nloc, self.alpha, self.beta)

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


class GemmBF16(GemmF16):
    """bfloat16 (or fp8) inputs, fp32 C / D: the same problem as gemm_f16 with the inputs rounded to the type."""
    name, metric, dtype = "gemm_bf16", "bf16 GEMM TFLOP/s at 8192^3 (fp32 C/D)", "bf16"
    has_host = False

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
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); dist.broadcast(self.a, src=0); e1.record(); torch.cuda.synchronize()
            self.a_broadcast_ms = e0.elapsed_time(e1)
        self.d = torch.empty((M, self.nloc), dtype=torch.int32, device="cuda")
        if self.variant == "sp24":
            import numpy as np
            # compress on the host in row chunks (format definition lives in datagen.sparsify_24_np)
            vals = torch.empty((M, K // 2), dtype=torch.int8, device="cuda")
            meta = torch.empty((M, K // 8), dtype=torch.uint8, device="cuda")
            for r0 in range(0, M, 1024):
                v, md, _ = G.sparsify_24_np(self.a[r0:r0 + 1024].cpu().numpy(), row_start=r0)
                vals[r0:r0 + 1024] = torch.from_numpy(v).cuda()
                meta[r0:r0 + 1024] = torch.from_numpy(md).cuda()
            self.vals, self.meta = vals, meta
            self.ws = torch.empty(api.gemm_i8_sp24_workspace_bytes(M, self.nloc, K), dtype=torch.uint8, device="cuda")
        elif self.variant == "i4":
            pack = lambda t: ((t[:, 0::2].to(torch.uint8) & 0xF) | ((t[:, 1::2].to(torch.uint8) & 0xF) << 4)).contiguous()
            self.ap, self.bp = pack(self.a), pack(self.b)
            self.ws = torch.empty(api.gemm_i4_workspace_bytes(M, self.nloc, K), dtype=torch.uint8, device="cuda")
        self.work_total = 2.0 * M * N * K
        self.work_local = 2.0 * M * self.nloc * K

    def step(self):
        from rocwmma_b200 import api
        M, K, n = self.M, self.K, self.nloc
        if self.variant == "dense":
            api.gemm_i8(M, n, K, self.a, self.b, None, self.d, K, K, n, n, 1, 0)
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


class GemmI8Sp24(GemmI8):
    name, variant = "gemm_i8_sp24", "sp24"
    launches_per_step = 2   # metadata re-tiling + sparse tensor-core GEMM
    metric = "2:4-sparse int8 GEMM dense-equivalent TOP/s at 8192x8192x16384"


class GemmI4(GemmI8):
    name, variant = "gemm_i4", "i4"
    launches_per_step = 3   # unpack A, unpack B, dense int8 GEMM
    metric = "int4-unpacked GEMM TOP/s at 8192x8192x16384"


class GemmF64(Workload):
    name, metric, unit, dtype, bound = "gemm_f64", "fp64 GEMM TFLOP/s at 4096^3", "TFLOP/s", "f64", "tensor"
    M = N = K = 4096

    def setup(self, torch, rank, world, dist):
        from rocwmma_b200 import datagen as G
        self.torch = torch
        col0, self.nloc = _shard(self.N, world, rank)
        f = lambda shape, seed: G.fill_torch(torch.empty(shape, dtype=torch.float64, device="cuda"), seed, "uniform")
        self.a, self.b, self.c = f((self.M, self.K), 1), f((self.nloc, self.K), 2), f((self.M, self.nloc), 3)
        self.d = torch.empty_like(self.c)
        self.a_broadcast_ms = 0.0
        self.work_total = 2.0 * self.M * self.N * self.K
        self.work_local = 2.0 * self.M * self.nloc * self.K

    def step(self):
        from rocwmma_b200 import api
        api.gemm_f64(self.M, self.nloc, self.K, self.a, self.b, self.c, self.d, self.K, self.K, self.nloc, self.nloc, 1.0, 1.0)

    def config(self, world):
        return {"workload": "fp64 GEMM (DMMA), M=N=K=4096, A row-major, B col-major, alpha=beta=1", "l2": "inputs larger than L2"}

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
        self.torch = torch
        b0, self.bloc = _shard(self.B, world, rank)
        ms, k, w = self.m_stride, self.k, self.width
        # L2 is 126 MB and one batch is ~134 MB of X: rotate over 4 independent batches so no step finds its input cached
        self.nbuf = 4
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
                "l2": "4 independent input batches rotated so that no step re-reads a cached input"}

    def value(self, work, seconds):
        return work / seconds

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
        self.torch = torch
        dt = torch.float64 if self.double else torch.float32
        r0, self.mloc = _shard(self.M, world, rank)
        self.a = G.fill_torch(torch.empty((self.mloc, self.N), dtype=dt, device="cuda"), G.SEED_GEMV_A, "uniform", start=r0 * self.N)
        self.x = G.fill_torch(torch.empty(self.N, dtype=dt, device="cuda"), G.SEED_GEMV_X, "uniform")
        self.y = G.fill_torch(torch.empty(self.mloc, dtype=dt, device="cuda"), G.SEED_GEMV_Y, "uniform", start=r0)
        es = 8 if self.double else 4
        self.a_broadcast_ms = 0.0
        self.work_total = float(es * (self.M * self.N + self.N + 2 * self.M))
        self.work_local = float(es * (self.mloc * self.N + self.N + 2 * self.mloc))

    def step(self):
        from rocwmma_b200 import api
        api.gemv(self.mloc, self.N, self.a, self.N, self.x, self.y, 1.5, 0.5)

    def setup_host(self):
        from rocwmma_b200 import api
        self.h_a = self.a.cpu().pin_memory(); self.h_x = self.x.cpu().pin_memory(); self.h_y = self.y.cpu().pin_memory()
        self.ctx = api.HostContext()
        es = 8 if self.double else 4
        self.h2d = (self.h_a.numel() + self.h_x.numel() + self.h_y.numel()) * es
        self.d2h = self.h_y.numel() * es

    def step_host(self):
        self.ctx.gemv(self.mloc, self.N, self.h_a, self.N, self.h_x, self.h_y, 1.5, 0.5, double=self.double)

    def config(self, world):
        return {"workload": f"{'dgemv' if self.double else 'sgemv'} y = 1.5*A*x + 0.5*y, A row-major 32768 x 32768",
                "sharding": "single GPU" if world == 1 else f"rows split over {world} ranks, x replicated",
                "l2": "matrix (4 / 8 GiB) larger than L2"}

    def value(self, work, seconds):
        return work / seconds / 1e9

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


WORKLOADS = {w().name: w for w in (GemmF16, GemmBF16, GemmFP8, GemmF32, GemmI8, GemmI8Sp24, GemmI4, GemmF64, Dlrm, DlrmBwd, Gemv, Dgemv)}


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
def run_gpu_arm(args, wl):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; rocwmma_b200 has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    assert world == args.gpus or world == 1, f"--gpus {args.gpus} but WORLD_SIZE={world}"

    from rocwmma_b200 import api
    wl.setup(torch, rank, world, dist)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps, sampler=None):
        barrier()
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
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, wall

    for _ in range(max(args.warmup, 3)):
        wl.step()
    sampler = ClockSampler(local_rank)
    ms_total, _ = timed(wl.step, args.steps, sampler)
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
    ms_step = ms_total / args.steps
    value = wl.value(wl.work_total, ms_step * 1e-3)

    # Tensor-bound workloads: the same step repeated for a few seconds.  The timed K steps above are a burst (the part
    # has not settled under its power cap yet); this is the rate it holds, to set beside the sustained library figure.
    sustained = None
    if wl.bound == "tensor" and args.sustained_seconds > 0:
        per_batch = max(10, int(0.25 / max(ms_step * 1e-3, 1e-6)))
        done, ms_acc = 0, 0.0
        # the batch count comes from the (rank-reduced) step time, so every rank runs the same number of batches
        batches = max(1, int(args.sustained_seconds / (per_batch * ms_step * 1e-3) + 0.5))
        for _ in range(batches):
            ms_b, _ = timed(wl.step, per_batch)
            ms_acc += ms_b
            done += per_batch
        sustained = {"value": wl.value(wl.work_total, ms_acc / done * 1e-3), "unit": wl.unit, "launches": done,
                     "seconds": ms_acc * 1e-3}

    # HBM-bound workloads: a plain device-to-device copy moving the same number of bytes per launch, timed the same
    # way (sources and destinations rotate through sets larger than L2).  The measured copy peak is a large-transfer figure; at these launch
    # sizes a copy does not reach it either, and this figure says what does.
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
            ms_copy, _ = timed(copy_step, args.steps)
            copy_same = 2.0 * half / (ms_copy / args.steps * 1e-3) / 1e9
            del srcs, dsts

    # end to end: host buffers through the C ABI host drivers, copies inside the timed region
    e2e = None
    if hasattr(wl, "setup_host") and getattr(wl, "has_host", True) and not args.no_e2e:
        wl.setup_host()
        for _ in range(2):
            wl.step_host()
        e2e_steps = max(2, min(args.steps, 5))
        _, wall = timed(wl.step_host, e2e_steps)
        if world > 1:
            t = torch.tensor([wall], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            wall = float(t.item())
        e2e = {"value": wl.value(wl.work_total, wall / e2e_steps), "unit": wl.unit,
               "h2d_bytes_per_step": int(wl.h2d), "d2h_bytes_per_step": int(wl.d2h), "steps": e2e_steps,
               "timing": "host wall clock around synchronous C-ABI host calls (pinned host buffers), max over ranks"}

    if rank == 0:
        peaks = measured_peaks()
        if wl.bound == "tensor":
            peak = peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"])
            if wl.dtype == "f32":
                peak /= 6.0  # TF32 runs at half the 16-bit rate and every product takes three MMAs
                peak_note = "cuBLAS bf16 8192^3 burst / 6: TF32 rate over three products"
            elif wl.dtype == "fp8":
                peak *= 2.0  # the fp8 tensor rate is twice the 16-bit rate; no fp8 figure is measured
                peak_note = "2 x cuBLAS bf16 8192^3 burst, standing in for the dense fp8 rate"
            elif wl.dtype == "i8" and getattr(wl, "variant", "") == "sp24":
                peak *= 4.0  # sparse int8: twice the dense int8 rate (measured: 112 clocks per 256x224x64 pair MMA)
                peak_note = "4 x cuBLAS bf16 8192^3 burst, standing in for the 2:4-sparse int8 rate"
            elif wl.dtype == "i8":
                peak *= 2.0  # the dense int8 tensor rate is twice the 16-bit rate; no int8 figure is measured
                peak_note = "2 x cuBLAS bf16 8192^3 burst, standing in for the dense int8 rate"
            elif wl.dtype == "f64":
                peak = 40.0
                peak_note = "nominal B200 fp64 tensor rate; no measured figure"
            else:
                peak_note = "cuBLAS bf16 8192^3 burst"
            achieved = wl.work_local / (ms_step * 1e-3) / 1e12
            roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s" if wl.dtype != "i8" else "TOP/s",
                    "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(wl.name),
                    "peak_source": f"{peaks['_source']} ({peak_note})"}
            # the vendor's dense figures, for context: 2250 TFLOP/s 16-bit, 4500 fp8 / int8, 9000 for 2:4-sparse int8,
            # 1125 / 3 for fp32 through three TF32 products, 40 fp64
            nominal = {"f16": 2250.0, "bf16": 2250.0, "fp8": 4500.0, "i4": 4500.0, "f32": 375.0, "f64": 40.0}.get(wl.dtype)
            if wl.dtype == "i8":
                nominal = 9000.0 if getattr(wl, "variant", "") == "sp24" else 4500.0
            if nominal:
                roof["nominal_peak"] = nominal
                roof["frac_of_nominal"] = achieved / nominal
        else:
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
        line = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": wl.scaling,
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic (seeded counter-based generator)",
            "config": wl.config(world), "roofline": roof, "clocks": sampler.summary(),
            "gpu_launches": args.steps * getattr(wl, "launches_per_step", 1),
            "a_broadcast_ms": wl.a_broadcast_ms,
        }
        if e2e:
            line["e2e"] = e2e
        if sustained:
            ref = peaks.get("bf16_tflops_sustained")
            if ref and wl.dtype == "f16":
                sustained["frac_of_sustained_peak"] = sustained["value"] / ref  # measured cuBLAS bf16 sustained loop
            line["sustained"] = sustained
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(wl)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]()
    if args.impl == "reference":
        run_reference_arm(args, wl)
    else:
        run_gpu_arm(args, wl)


if __name__ == "__main__":
    main()
