"""Seeded synthetic inputs for the GEMM / DLRM / GEMV workloads.

One counter-based generator, identical in numpy (host) and torch (device):
    z = splitmix64_finalise(seed * 0x9E3779B97F4A7C15 + idx)        (64-bit wrap-around)
    u = (z >> 40) * 2**-24 in [0, 1)
`idx` is the row-major logical index of the element, whatever the memory layout.
uniform[-1,1) = 2u - 1; normal = Box-Muller on draws 2*idx and 2*idx+1;
int8 = (z >> 56) - 128; int4 = (z >> 60) - 8.

These stand in for the reference's host fills (samples/common.hpp:180-224: rand()-based,
unseeded) with the value distributions the benchmark configurations name.
"""
from __future__ import annotations

import numpy as np

GAMMA = 0x9E3779B97F4A7C15
M1 = 0xBF58476D1CE4E5B9
M2 = 0x94D049BB133111EB

SEED_A, SEED_B, SEED_C, SEED_X, SEED_G, SEED_GEMV_A, SEED_GEMV_X, SEED_GEMV_Y, SEED_SPARSITY = range(1, 10)

# kept positions (i0 < i1) of a 2:4 group, indexed by z % 6
PAIRS = np.array([(0, 1), (0, 2), (0, 3), (1, 2), (1, 3), (2, 3)], dtype=np.uint8)


# ------------------------------------------------------------------------------------- numpy
def _mix_np(seed: int, idx: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = idx.astype(np.uint64) + np.uint64((seed * GAMMA) & 0xFFFFFFFFFFFFFFFF)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(M1)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(M2)
        z = z ^ (z >> np.uint64(31))
    return z


def raw_np(seed: int, count: int, start: int = 0) -> np.ndarray:
    return _mix_np(seed, np.arange(start, start + count, dtype=np.uint64))


def uniform_np(seed: int, shape, dtype=np.float32, start: int = 0) -> np.ndarray:
    n = int(np.prod(shape))
    u = (raw_np(seed, n, start) >> np.uint64(40)).astype(np.float64) * 2.0 ** -24
    return (2.0 * u - 1.0).astype(dtype).reshape(shape)


def normal_np(seed: int, shape, sigma: float, dtype=np.float16, start: int = 0) -> np.ndarray:
    n = int(np.prod(shape))
    z = raw_np(seed, 2 * n, 2 * start)
    j = (z >> np.uint64(40)).astype(np.float64)
    u1 = (j[0::2] + 0.5) * 2.0 ** -24  # in (0, 1): log is finite
    u2 = j[1::2] * 2.0 ** -24
    v = sigma * np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return v.astype(dtype).reshape(shape)


def int8_np(seed: int, shape, start: int = 0) -> np.ndarray:
    n = int(np.prod(shape))
    return ((raw_np(seed, n, start) >> np.uint64(56)).astype(np.int16) - 128).astype(np.int8).reshape(shape)


def int4_np(seed: int, shape, start: int = 0) -> np.ndarray:
    """int4 values in [-8, 7], one per int8 element (unpacked)."""
    n = int(np.prod(shape))
    return ((raw_np(seed, n, start) >> np.uint64(60)).astype(np.int16) - 8).astype(np.int8).reshape(shape)


def pack_int4_np(vals: np.ndarray) -> np.ndarray:
    """[rows, k] int8 in [-8,7] -> [rows, k/2] bytes, low nibble = even k."""
    v = vals.astype(np.uint8) & 0xF
    return (v[:, 0::2] | (v[:, 1::2] << 4)).astype(np.uint8)


def unpack_int4_np(packed: np.ndarray) -> np.ndarray:
    lo = (packed & 0xF).astype(np.int8)
    hi = (packed >> 4).astype(np.int8)
    lo = np.where(lo > 7, lo - 16, lo).astype(np.int8)
    hi = np.where(hi > 7, hi - 16, hi).astype(np.int8)
    out = np.empty((packed.shape[0], packed.shape[1] * 2), dtype=np.int8)
    out[:, 0::2] = lo
    out[:, 1::2] = hi
    return out


def sparsify_24_np(dense: np.ndarray, seed: int = SEED_SPARSITY, row_start: int = 0):
    """2:4-compress [m, k] int8 along k.

    Returns (vals [m, k/2] int8, meta [m, k/8] uint8, densified [m, k] int8): per aligned group
    of 4 the two kept positions are PAIRS[z(seed, group index) % 6]; metadata nibble =
    i0 | (i1 << 2), two groups per byte, low nibble = even group."""
    m, k = dense.shape
    groups = k // 4
    z = raw_np(seed, m * groups, row_start * groups).reshape(m, groups)
    sel = (z % np.uint64(6)).astype(np.int64)
    i0 = PAIRS[sel, 0].astype(np.int64)
    i1 = PAIRS[sel, 1].astype(np.int64)
    g = dense.reshape(m, groups, 4)
    v0 = np.take_along_axis(g, i0[..., None], axis=2)[..., 0]
    v1 = np.take_along_axis(g, i1[..., None], axis=2)[..., 0]
    vals = np.stack([v0, v1], axis=2).reshape(m, k // 2).astype(np.int8)
    nib = (i0 | (i1 << 2)).astype(np.uint8)
    meta = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    return vals, meta, densify_24_np(vals, meta)


def densify_24_np(vals: np.ndarray, meta: np.ndarray) -> np.ndarray:
    m, half_k = vals.shape
    groups = half_k // 2
    nib = np.empty((m, groups), dtype=np.uint8)
    nib[:, 0::2] = meta & 0xF
    nib[:, 1::2] = meta >> 4
    i0 = (nib & 3).astype(np.int64)
    i1 = (nib >> 2).astype(np.int64)
    out = np.zeros((m, groups, 4), dtype=np.int8)
    v = vals.reshape(m, groups, 2)
    np.put_along_axis(out, i0[..., None], v[..., 0:1], axis=2)
    np.put_along_axis(out, i1[..., None], v[..., 1:2], axis=2)
    return out.reshape(m, groups * 4)


# ------------------------------------------------------------------------------------- torch
def _mix_torch(seed: int, idx):
    """idx: int64 tensor (any device).  64-bit wrap-around arithmetic in int64."""
    import torch

    def s64(x):  # python int -> signed 64-bit
        x &= 0xFFFFFFFFFFFFFFFF
        return x - (1 << 64) if x >= (1 << 63) else x

    def lsr(x, s):  # logical shift right on int64
        return (x >> s) & ((1 << (64 - s)) - 1)

    z = idx + s64(seed * GAMMA)
    z = (z ^ lsr(z, 30)) * s64(M1)
    z = (z ^ lsr(z, 27)) * s64(M2)
    z = z ^ lsr(z, 31)
    return z, lsr


def fill_torch(out, seed: int, kind: str, sigma: float = 1.0, chunk: int = 1 << 25, start: int = 0):
    """Fill the contiguous tensor `out` (viewed flat, logical index = flat index + start) on its device.

    kind: 'uniform' | 'normal' | 'int8' | 'int4' (int4: one value per int8 element)."""
    import math
    import torch

    flat = out.view(-1)
    n = flat.numel()
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        idx = torch.arange(start + lo, start + hi, dtype=torch.int64, device=out.device)
        if kind == "normal":
            z1, lsr = _mix_torch(seed, idx * 2)
            z2, _ = _mix_torch(seed, idx * 2 + 1)
            u1 = (lsr(z1, 40).to(torch.float64) + 0.5) * 2.0 ** -24
            u2 = lsr(z2, 40).to(torch.float64) * 2.0 ** -24
            v = sigma * torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2.0 * math.pi * u2)
            flat[lo:hi] = v.to(out.dtype)
            continue
        z, lsr = _mix_torch(seed, idx)
        if kind == "uniform":
            u = lsr(z, 40).to(torch.float64) * 2.0 ** -24
            flat[lo:hi] = (2.0 * u - 1.0).to(out.dtype)
        elif kind == "int8":
            flat[lo:hi] = (lsr(z, 56) - 128).to(out.dtype)
        elif kind == "int4":
            flat[lo:hi] = (lsr(z, 60) - 8).to(out.dtype)
        else:
            raise ValueError(kind)
    return out
