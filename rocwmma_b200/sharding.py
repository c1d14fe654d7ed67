"""Work partitioning for multi-GPU runs (one process per GPU).

All three paths shard without any exchange after the kernel:
  GEMM  by blocks of N columns  - B (column-major) and C / D (row-major) are split by column block,
                                  A is needed whole by every rank (one broadcast before the kernel);
  DLRM  by batch;
  GEMV  by rows of A (row-major) - x is replicated, each rank owns a slice of y.
The reference has no multi-GPU path; these helpers are new here.
"""
from __future__ import annotations


def shard_range(total: int, world: int, rank: int):
    """Contiguous, equally sized slice [start, start + count) of `total` units for `rank`."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}")
    if total % world != 0:
        raise ValueError(f"{total} units do not split evenly over {world} ranks")
    count = total // world
    return rank * count, count


def gemm_column_shard(n: int, k: int, world: int, rank: int):
    """Column block of a GEMM for `rank`: (col0, ncols, offset of the block inside column-major B in elements)."""
    col0, ncols = shard_range(n, world, rank)
    return col0, ncols, col0 * k
