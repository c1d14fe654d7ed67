// Process-wide tuning overrides of the kernel selection, set through b200wmma_set_tuning() (capi.cu).  They exist for
// A/B comparisons and for tests that must reach every kernel; 0 always means "the library's own choice".
#pragma once
#include <atomic>

namespace b200wmma
{
    namespace tuning
    {
        enum Key : int
        {
            GEMM_TILE_VARIANT = 0, // dense tcgen05 GEMM tile shape: 1 = 128x256 per SM, 2 = 256x256 per SM pair, 3 = 512x256 per pair
            GEMM_GROUP_M      = 1, // rasterisation band height in row tiles
            SP24_FORCE_EXPAND = 2, // 1: the 2:4-sparse GEMM always densifies A into the workspace and runs the dense kernel
            GEMM_SPLIT_TAIL   = 4, // 512x256 kernel given a workspace: 1 = split the last partial round along K when it pays, 2 = never
            GEMM_SPLIT_FIXUP  = 5, // cost of the split-K exchange the planner assumes, in K slabs (0 = built-in)
            GEMM_MMA_ORDER    = 3, // 512x256 kernel, first / last K slabs of a tile: 1 = by accumulator, 2 = by slab
            DLRM_BWD_STAGES   = 6, // one-warp-per-sample DLRM backward kernel: ring depth 2 or 3
            DLRM_BWD_WARPS    = 7, // ... and warps per CTA (1..12, clipped to what fits in shared memory)
            DLRM_FWD_STAGES   = 8, // the same two for the forward kernel
            DLRM_FWD_WARPS    = 9,
            GEMM_F64_KERNEL   = 10, // fp64 GEMM: 1 = the cp.async kernel, 2 = the TMA-fed kernel or an error where it cannot run
            FRAG_PERF_SLAB_K  = 11, // b200wmma_perf_hgemm_fragment: K depth of a shared-memory slab, 16 / 32 / 64
            GEMV_ROWS         = 12, // row-major GEMV: 4 = four rows of A per CTA with two loads in flight (default: one row, eight loads)
            GEMV_COL_VN       = 13, // column-major GEMV: rows per lane, 2 or 4 (default: 1)
            NUM_KEYS
        };
        int  get(Key k);
        void set(Key k, int value);
    } // namespace tuning
} // namespace b200wmma
