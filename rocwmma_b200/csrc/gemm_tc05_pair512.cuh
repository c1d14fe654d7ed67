// Two-CTA tcgen05 GEMM with 256 x 256 outputs per CTA (512 x 256 per SM pair).
//
// Why a second pair kernel: the 256 x 256-per-pair kernel (gemm_tc05_pair.cuh) moves 32 KiB of
// operands per CTA per 64-wide K slab for 128 x 256 x 64 of work.  Here a CTA keeps 256 rows of A
// (two 128-row sub-tiles) against the same half B slab: 48 KiB per slab for twice the work, i.e. a
// quarter less L2 -> SM traffic and fewer DRAM re-reads per flop.  On a power-capped part that is
// clock speed.  The price: the two 128 x 256 fp32 accumulators fill all 512 tensor-memory columns,
// so the accumulators are not double-buffered and the epilogue has to be short.  It is made short
// by (a) sixteen epilogue warps - two per lane quadrant of each accumulator, taking alternate 64-byte column
// steps, (b) moving C and D through small swizzled shared-memory tiles with TMA - a thread-per-row global
// access touches 32 different cache lines per warp instruction, which costs ~32 LSU cycles each and dominated
// the drain - and (c) releasing each accumulator to the MMA issuer separately.  Every warp has two staging
// tiles: a dedicated one, whose C tile is requested while the tile is still being multiplied, and one inside the
// A region of the last operand stage, which the producer refills only after a counter says every epilogue warp
// has finished with the tile (bounded wait).
//
// Roles (576 threads): warp 0 TMA producer (one lane), warp 1 tensor-memory owner / MMA issuer
// (one lane, leader CTA only), warps 2-17 epilogue.  Barrier protocol as in gemm_tc05_pair.cuh
// (loads of both CTAs counted on the leader's full[s]; commits signal both CTAs), with one
// tmem_full barrier per tile and one tmem_empty barrier per accumulator.
#pragma once
#include "gemm_tc05_common.cuh"

namespace b200wmma
{
    namespace tc05q
    {
        using namespace tc05;

        constexpr uint32_t SUB_M         = 128; // rows per MMA per CTA
        constexpr uint32_t CTA_M         = 256; // rows of A / D per CTA (two accumulators)
        constexpr uint32_t PAIR_M        = 512;
        constexpr uint32_t TILE_N        = 256;
        constexpr uint32_t HALF_N        = 128;
        constexpr uint32_t STAGES        = 4;
        constexpr uint32_t A_STAGE_BYTES = CTA_M * BLOCK_K_BYTES; // 32 KiB
        constexpr uint32_t B_STAGE_BYTES = HALF_N * BLOCK_K_BYTES; // 16 KiB
        constexpr uint32_t STAGE_BYTES   = A_STAGE_BYTES + B_STAGE_BYTES;
        constexpr uint32_t EPI_WARPS     = 16; // two per TMEM lane quadrant of each accumulator (alternate 64-byte column steps)
        constexpr uint32_t NUM_THREADS   = 64 + EPI_WARPS * 32;
        constexpr uint32_t TMEM_COLS     = 512;
        constexpr uint32_t GROUP_M       = 8; // rasterisation band: 8 pair-row tiles = 4096 rows
        constexpr uint32_t EPI_BUF_BYTES = 2048; // 32 rows x 64 bytes, TMA SWIZZLE_64B
        constexpr uint32_t EPI_BYTES     = EPI_WARPS * EPI_BUF_BYTES; // dedicated staging tiles: the first of each epilogue warp's two
        constexpr uint32_t EPI_STAGE     = STAGES - 1; // operand stage whose A region holds every epilogue warp's second staging tile
        constexpr uint32_t MISC_BYTES    = 512; // barriers, tensor-memory slot, abort flag, epilogue counter
        constexpr uint32_t SMEM_BYTES    = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + MISC_BYTES;

        // ---- work schedule ------------------------------------------------------------------------------------------
        // A persistent pair walks "units".  Without a split-K tail every unit is a whole tile: pair p takes tiles
        // p, p + P, ...  With one (stream-K over the last, partial round): the first `dp_rounds` units of every pair are
        // whole tiles as before, and the remaining `sk_tiles` tiles, seen as sk_tiles * num_kb K slabs in a row, are cut
        // into `sk_pairs` equal ranges, one per pair.  A range covers at most two tiles: the tail of one and the head of
        // the next.  A unit that does not end its tile (PARTIAL) writes its raw accumulators to the pair's slot of a
        // workspace and raises the slot's flag; the unit that ends a tile (FINISH) adds the other units' partials to its
        // own accumulators and runs the alpha / beta epilogue.  Every pair works its PARTIAL unit first and its FINISH
        // unit last, so a FINISH unit never waits for work that has not been started before it.
        struct SplitPlan
        {
            uint32_t dp_rounds; // whole-tile units per pair (split mode); unused otherwise
            uint32_t sk_tiles; // tiles of the split round (0 = no split round)
            uint32_t sk_pairs; // pairs that take part in it
        };
        enum UnitKind : uint32_t
        {
            UNIT_FULL    = 0,
            UNIT_PARTIAL = 1,
            UNIT_FINISH  = 2
        };
        struct Unit
        {
            uint32_t tile, kb0, kb1, kind;
        };
        constexpr uint32_t SLOT_WORDS = 2u * 2u * TILE_N * SUB_M; // one pair's accumulators: [CTA][accumulator][column][row]

        // slab range [u0, u1) of pair q in the split round
        __device__ __forceinline__ void split_range(uint32_t q, const SplitPlan& plan, uint32_t num_kb, uint32_t& u0, uint32_t& u1)
        {
            const uint64_t total = static_cast<uint64_t>(plan.sk_tiles) * num_kb;
            u0 = static_cast<uint32_t>(total * q / plan.sk_pairs);
            u1 = static_cast<uint32_t>(total * (q + 1u) / plan.sk_pairs);
        }
        // the idx-th unit of `pair`; false when the pair has no more units
        __device__ __forceinline__ bool unit_at(uint32_t idx, uint32_t pair, uint32_t num_pairs, uint32_t num_tiles,
                                                uint32_t num_kb, const SplitPlan& plan, Unit& u)
        {
            if(plan.sk_tiles == 0u)
            {
                u.tile = pair + idx * num_pairs;
                u.kb0 = 0u, u.kb1 = num_kb, u.kind = UNIT_FULL;
                return u.tile < num_tiles;
            }
            if(idx < plan.dp_rounds)
            {
                u.tile = pair + idx * num_pairs;
                u.kb0 = 0u, u.kb1 = num_kb, u.kind = UNIT_FULL;
                return true;
            }
            const uint32_t sidx = idx - plan.dp_rounds;
            if(pair >= plan.sk_pairs || sidx > 1u)
                return false;
            uint32_t u0, u1;
            split_range(pair, plan, num_kb, u0, u1);
            if(u0 >= u1)
                return false;
            const uint32_t first_tile = plan.dp_rounds * num_pairs;
            const uint32_t ta = u0 / num_kb, tb = (u1 - 1u) / num_kb;
            if(ta == tb)
            {
                if(sidx != 0u)
                    return false;
                u.tile = first_tile + ta, u.kb0 = u0 - ta * num_kb, u.kb1 = u1 - ta * num_kb;
            }
            else if(sidx == 0u) // the head of the later tile first: it only produces a partial
                u.tile = first_tile + tb, u.kb0 = 0u, u.kb1 = u1 - tb * num_kb;
            else
                u.tile = first_tile + ta, u.kb0 = u0 - ta * num_kb, u.kb1 = num_kb;
            u.kind = (u.kb1 == num_kb) ? (u.kb0 == 0u ? UNIT_FULL : UNIT_FINISH) : UNIT_PARTIAL;
            return true;
        }
        // How many pairs before `pair` hold partials of the tile whose FINISH unit starts at slab kb0 (they are the pairs
        // pair-1, pair-2, ...: ranges are laid out in pair order).
        __device__ __forceinline__ uint32_t finish_contributors(uint32_t pair, uint32_t tile, uint32_t num_pairs, uint32_t num_kb,
                                                                const SplitPlan& plan)
        {
            const uint32_t tile_first_unit = (tile - plan.dp_rounds * num_pairs) * num_kb;
            uint32_t       count           = 0;
            for(uint32_t q = pair; q-- > 0u;)
            {
                uint32_t u0, u1;
                split_range(q, plan, num_kb, u0, u1);
                if(u1 <= tile_first_unit)
                    break;
                if(u0 < u1)
                    ++count;
                else
                    break; // (an empty range cannot lie between non-empty ones of equal size; defensive)
            }
            return count;
        }
        __device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p)
        {
            uint32_t v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
            return v;
        }
        __device__ __forceinline__ void red_release_gpu_add_u32(uint32_t* p, uint32_t v)
        {
            asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
        }

        // Epilogue of one warp through shared-memory staging tiles.
        // A step covers 64 bytes of each of the warp's 32 rows (32 columns of 2-byte outputs, 16
        // columns of 4-byte outputs).  Per step: tcgen05.ld the accumulator columns, wait for the C
        // tile of the step (TMA, requested two steps earlier), combine in place (each lane owns one
        // row of the tile; the 64-byte swizzle keeps the 16-byte accesses conflict-free), hand the
        // tile to a TMA store and request the C tile two steps ahead into the same buffer once the
        // store has read it.  TMA clips rows / columns outside the matrix, so ragged edges need no
        // special case.  All 32 lanes execute every step.
        // TN: columns of the accumulator being drained.  STRIDE > 1 lets several warps share one lane quadrant of an
        // accumulator: warp `first` (0 .. STRIDE-1) takes the steps first, first + STRIDE, ...
        // ROW_BYTES: bytes per row of a staging tile, 64 (TMA SWIZZLE_64B) or, for 32-bit outputs, 128 (SWIZZLE_128B:
        // half as many row requests per byte moved).
        // ACC_SHIFT (integer accumulators): the accumulator is shifted right by that many bits (arithmetic) before alpha /
        // beta are applied, for kernels whose operands carry a power-of-two scale.
        template <typename OutT, typename ScalarT, uint32_t TN = TILE_N, uint32_t STRIDE = 1, uint32_t ROW_BYTES = 64,
                  int ACC_SHIFT = 0>
        struct StagedDrain
        {
            static_assert(ACC_SHIFT == 0 || std::is_same<ScalarT, int32_t>::value, "accumulator shift: integer paths only");
            static constexpr uint32_t BUF_BYTES = 32 * ROW_BYTES; // one staging tile: 32 rows
            static constexpr uint32_t CELLS     = ROW_BYTES / 16; // 16-byte cells per row
            static_assert(ROW_BYTES == 64 || (ROW_BYTES == 128 && sizeof(OutT) == 4), "staging rows: 64 bytes, or 128 for 32-bit outputs");
            static_assert(sizeof(OutT) >= 2, "one-byte outputs are drained element-wise, not through staging tiles");
            static constexpr uint32_t STEP_COLS = ROW_BYTES / sizeof(OutT);
            static constexpr uint32_t STEPS     = TN / STEP_COLS; // of the whole accumulator
            static constexpr uint32_t MY_STEPS  = STEPS / STRIDE; // of one warp
            static_assert(STEPS % STRIDE == 0, "steps must divide evenly among the warps of a quadrant");

            // requests the C tiles of steps 0 and 1 (called while the tile is still being multiplied)
            // ls_begin / ls_end: which of the warp's first two steps to request (both by default); buf1: address of the
            // second staging tile when it does not follow the first one
            __device__ static __forceinline__ void prefetch_c(const CUtensorMap* tmap_c, uint32_t buf0, uint32_t cbar0,
                                                             uint32_t col_base, uint32_t row0, uint32_t n, uint32_t first = 0,
                                                             uint32_t ls_begin = 0, uint32_t ls_end = 2, uint32_t buf1 = 0)
            {
                if(buf1 == 0u)
                    buf1 = buf0 + BUF_BYTES;
                ptx::bulk_wait_group_read<0>(); // the previous tile's last stores have read both buffers
#pragma unroll
                for(uint32_t ls = ls_begin; ls < ls_end && ls < MY_STEPS; ++ls)
                {
                    const uint32_t s = first + ls * STRIDE;
                    if(col_base + s * STEP_COLS >= n)
                        break; // steps that start right of the matrix are skipped everywhere
                    ptx::mbar_arrive_expect_tx(cbar0 + 8 * ls, BUF_BYTES);
                    ptx::tma_load_2d(ls == 0u ? buf0 : buf1, tmap_c, static_cast<int32_t>(col_base + s * STEP_COLS),
                                     static_cast<int32_t>(row0), cbar0 + 8 * ls);
                }
            }

            __device__ static __forceinline__ bool run(uint32_t tmem_acc, uint32_t quad, uint32_t lane, uint8_t* smem,
                                                       uint32_t buf_off, uint32_t buf0, uint32_t cbar0,
                                                       const CUtensorMap* tmap_c, const CUtensorMap* tmap_d,
                                                       uint32_t col_base, uint32_t row0, uint32_t n, ScalarT alpha,
                                                       ScalarT beta, bool read_c, uint32_t& cpar,
                                                       volatile uint32_t* cta_abort, unsigned* status, uint32_t who,
                                                       uint32_t first = 0, uint32_t buf1_off = 0, uint32_t buf1 = 0,
                                                       const uint32_t* partials = nullptr, uint32_t npartials = 0)
            {
                // partials: this thread's row in the accumulator copy that the nearest contributing pair left in the split-K
                // workspace ([column][row] words); further contributors lie SLOT_WORDS lower each.  Their sum is added to
                // the accumulator before alpha / beta.
                if(buf1 == 0u)
                {
                    buf1_off = buf_off + BUF_BYTES;
                    buf1     = buf0 + BUF_BYTES;
                }
                // cpar: bit b = parity of the next completed C load into staging buffer b (kept across tiles)
                // swizzle phase of this lane's row: 16-byte cell index XOR (128-byte line index mod 4 or 8)
                const uint32_t row_sw = ROW_BYTES == 64 ? ((lane >> 1) & 3u) : (lane & 7u);
#pragma unroll 2
                for(uint32_t ls = 0; ls < MY_STEPS; ++ls)
                {
                    const uint32_t s  = first + ls * STRIDE;
                    const uint32_t bi = ls & 1u;
                    uint32_t       v[STEP_COLS];
                    static_assert(STEP_COLS == 32 || STEP_COLS == 16, "one tensor-memory load per step");
                    if constexpr(STEP_COLS == 32)
                        ptx::tmem_ld_32x32b_x32(tmem_acc + ((quad * 32u) << 16) + s * STEP_COLS, v);
                    else
                        ptx::tmem_ld_32x32b_x16(tmem_acc + ((quad * 32u) << 16) + s * STEP_COLS, v);
                    if(col_base + s * STEP_COLS >= n)
                    {
                        // this step lies right of the matrix (ragged N): nothing to load, combine or store
                        ptx::tmem_ld_wait();
                        continue;
                    }
                    if(read_c)
                    {
                        bool ok = ptx::mbar_wait_bounded(cbar0 + 8 * bi, (cpar >> bi) & 1u, cta_abort, status, who,
                                                         WAIT_TIMEOUT_NS);
                        if(!__all_sync(0xFFFFFFFFu, ok))
                        {
                            ptx::tmem_ld_wait();
                            return false;
                        }
                        cpar ^= 1u << bi;
                    }
                    else
                    {
                        if(lane == 0)
                            ptx::bulk_wait_group_read<1>(); // the store issued two steps ago has read this buffer
                        __syncwarp();
                    }
                    ptx::tmem_ld_wait();
                    for(uint32_t pi = 0; pi < npartials; ++pi)
                    {
                        const uint32_t* src = partials - static_cast<size_t>(pi) * SLOT_WORDS + (s * STEP_COLS) * SUB_M;
                        // sixteen loads in flight at a time (each a coalesced 128-byte row of the warp), then the adds
#pragma unroll
                        for(uint32_t h = 0; h < STEP_COLS; h += 16)
                        {
                            uint32_t w[16];
#pragma unroll
                            for(uint32_t i = 0; i < 16; ++i)
                                asm volatile("ld.global.cg.u32 %0, [%1];" // written by another SM: read through L2
                                             : "=r"(w[i])
                                             : "l"(src + (h + i) * SUB_M));
#pragma unroll
                            for(uint32_t i = 0; i < 16; ++i)
                            {
                                if constexpr(std::is_same<ScalarT, float>::value)
                                    v[h + i] = __float_as_uint(__uint_as_float(v[h + i]) + __uint_as_float(w[i]));
                                else
                                    v[h + i] += w[i];
                            }
                        }
                    }
                    uint8_t* rowp = smem + (bi == 0u ? buf_off : buf1_off) + lane * ROW_BYTES;
                    // The epilogue warps share four issue ports, so the drain's length is close to its instruction count:
                    // the common scalars get their own code (alpha == 1: one fused multiply-add per element; no C: none).
                    const auto combine = [&](auto mode_tag) {
                        constexpr int MODE = decltype(mode_tag)::value; // 0 general, 1 alpha == 1 with C, 2 alpha == 1 without C
                        const auto one = [&](uint32_t accbits, auto cval) {
                            if constexpr(std::is_same<ScalarT, float>::value)
                            {
                                const float acc = __uint_as_float(accbits);
                                if constexpr(MODE == 2)
                                    return acc;
                                else if constexpr(MODE == 1)
                                    return fmaf(beta, static_cast<float>(cval), acc);
                                else
                                    return epi(acc, static_cast<float>(cval), alpha, beta);
                            }
                            else
                            {
                                const int32_t acc = static_cast<int32_t>(accbits) >> ACC_SHIFT;
                                if constexpr(MODE == 2)
                                    return acc;
                                else
                                    return epi(acc, static_cast<int32_t>(cval), MODE == 1 ? ScalarT(1) : alpha, beta);
                            }
                        };
#pragma unroll
                        for(uint32_t q = 0; q < CELLS; ++q)
                        {
                            uint4* cell = reinterpret_cast<uint4*>(rowp + ((q ^ row_sw) << 4));
                            uint4  cv   = make_uint4(0, 0, 0, 0);
                            if(MODE != 2 && read_c)
                                cv = *cell;
                            const uint32_t cwv[4] = {cv.x, cv.y, cv.z, cv.w};
                            uint32_t       ow[4];
#pragma unroll
                            for(uint32_t w = 0; w < 4; ++w)
                            {
                                if constexpr(sizeof(OutT) == 2)
                                {
                                    const float2 cf = Pack16<OutT>::widen(cwv[w]);
                                    ow[w] = Pack16<OutT>::narrow(one(v[8 * q + 2 * w], cf.x), one(v[8 * q + 2 * w + 1], cf.y));
                                }
                                else if constexpr(std::is_same<OutT, float>::value)
                                    ow[w] = __float_as_uint(one(v[4 * q + w], __uint_as_float(cwv[w])));
                                else
                                    ow[w] = static_cast<uint32_t>(one(v[4 * q + w], static_cast<int32_t>(cwv[w])));
                            }
                            *cell = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                        }
                    };
                    if(alpha == ScalarT(1) && !read_c)
                        combine(std::integral_constant<int, 2>{});
                    else if(alpha == ScalarT(1))
                        combine(std::integral_constant<int, 1>{});
                    else
                        combine(std::integral_constant<int, 0>{});
                    ptx::fence_proxy_async_smem(); // the tile written above -> visible to the TMA store
                    __syncwarp();
                    if(lane == 0)
                    {
                        ptx::tma_store_2d(tmap_d, static_cast<int32_t>(col_base + s * STEP_COLS), static_cast<int32_t>(row0),
                                          bi == 0u ? buf0 : buf1);
                        ptx::bulk_commit_group();
                        if(read_c && ls + 2 < MY_STEPS && col_base + (s + 2 * STRIDE) * STEP_COLS < n)
                        {
                            ptx::bulk_wait_group_read<0>(); // the store has read the buffer: refill it with C
                            ptx::mbar_arrive_expect_tx(cbar0 + 8 * bi, BUF_BYTES);
                            ptx::tma_load_2d(bi == 0u ? buf0 : buf1, tmap_c,
                                             static_cast<int32_t>(col_base + (s + 2 * STRIDE) * STEP_COLS),
                                             static_cast<int32_t>(row0), cbar0 + 8 * bi);
                        }
                    }
                }
                return true;
            }

            // A unit that does not end its tile: the warp's share of the raw accumulator goes to the workspace
            // (dst: this thread's row of the pair's slot, [column][row] words - consecutive lanes, consecutive addresses).
            __device__ static __forceinline__ void store_partial(uint32_t tmem_acc, uint32_t quad, uint32_t* dst, uint32_t first)
            {
#pragma unroll 2
                for(uint32_t ls = 0; ls < MY_STEPS; ++ls)
                {
                    const uint32_t s = first + ls * STRIDE;
                    uint32_t       v[STEP_COLS];
                    if constexpr(STEP_COLS == 32)
                        ptx::tmem_ld_32x32b_x32(tmem_acc + ((quad * 32u) << 16) + s * STEP_COLS, v);
                    else
                        ptx::tmem_ld_32x32b_x16(tmem_acc + ((quad * 32u) << 16) + s * STEP_COLS, v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for(uint32_t i = 0; i < STEP_COLS; ++i)
                        __stcg(dst + (s * STEP_COLS + i) * SUB_M, v[i]);
                }
            }
        };

        // A_MN / B_MN: the operand is MN-major (column-major A / row-major B) instead of K-major.
        // SPLIT: order the MMAs of a tile's first HEAD_KB and last TAIL_KB K slabs by accumulator instead of by slab
        // (accumulator 0 over those slabs, then accumulator 1), with one tmem_full barrier per accumulator.  The two
        // accumulators fill tensor memory, so a tile's drain cannot overlap the next tile's MMAs on the same accumulator;
        // ordered this way accumulator 0 is drained while accumulator 1 still multiplies the tile's last slabs, and
        // accumulator 1 while accumulator 0 already multiplies the next tile's first slabs.
        constexpr uint32_t HEAD_KB = STAGES - 1; // the next tile's slab in the stage that holds staging tiles is not among them
        constexpr uint32_t TAIL_KB = STAGES; // every stage: all slabs of the block are resident at once
        template <int KIND, typename OutT, typename ScalarT, bool A_MN = false, bool B_MN = false, bool SPLIT = false>
        __global__ void __launch_bounds__(NUM_THREADS, 1)
            gemm_tc05_pair512_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                     const __grid_constant__ CUtensorMap tmap_b,
                                     const __grid_constant__ CUtensorMap tmap_c, // 32-row x 64-byte boxes of C
                                     const __grid_constant__ CUtensorMap tmap_d, // ... and of D (both unused if vec_ok == 0)
                                     const OutT* __restrict__ c,
                                     OutT* __restrict__ d,
                                     uint32_t  m,
                                     uint32_t  n,
                                     uint32_t  k_bytes,
                                     uint32_t  ldc,
                                     uint32_t  ldd,
                                     ScalarT   alpha,
                                     ScalarT   beta,
                                     uint32_t  tiles_m, // pair tiles along M (512 rows each)
                                     uint32_t  tiles_n,
                                     int       vec_ok,
                                     uint32_t  group_m,
                                     unsigned* status,
                                     SplitPlan plan, // sk_tiles == 0: every unit is a whole tile
                                     uint32_t* split_ws) // split round: num_pairs slots of SLOT_WORDS words, then one flag per pair
        {
            extern __shared__ uint8_t smem_raw[];
            const uint32_t            raw_addr = ptx::smem_u32(smem_raw);
            const uint32_t            base     = (raw_addr + 1023u) & ~1023u;
            uint8_t*                  smem     = smem_raw + (base - raw_addr);

            // [A stages][B stages][epilogue staging tiles][barriers, tensor-memory slot, abort flag]
            const uint32_t     smem_a     = base;
            const uint32_t     smem_b     = base + STAGES * A_STAGE_BYTES;
            const uint32_t     epi_off    = STAGES * STAGE_BYTES;
            const uint32_t     misc_off   = epi_off + EPI_BYTES;
            const uint32_t     bar_base   = base + misc_off;
            const uint32_t     full_bar   = bar_base; // STAGES x 8 (leader's copy in use)
            const uint32_t     empty_bar  = bar_base + 32;
            const uint32_t     tfull_bar  = bar_base + 64; // 2 x 8, one per accumulator
            const uint32_t     tempty_bar = bar_base + 80; // 2 x 8, one per accumulator (leader's copy in use)
            const uint32_t     cbar_base  = bar_base + 96; // EPI_WARPS x 2 x 8: C tiles of the epilogue warps
            uint32_t*          tmem_slot  = reinterpret_cast<uint32_t*>(smem + misc_off + 96 + EPI_WARPS * 16);
            volatile uint32_t* cta_abort  = tmem_slot + 1;
            const uint32_t     drained_bar = bar_base + 96 + EPI_WARPS * 16 + 16; // every epilogue warp is done with a tile's staging tiles
            // the A region of the last stage holds the second staging tile of every epilogue warp while a tile is drained
            const uint32_t     alias_base_off = EPI_STAGE * A_STAGE_BYTES;

            const uint32_t warp      = threadIdx.x >> 5;
            const uint32_t lane      = threadIdx.x & 31u;
            const uint32_t rank      = ptx::cluster_ctarank();
            const uint32_t pair      = blockIdx.x >> 1;
            const uint32_t num_pairs = gridDim.x >> 1;
            const uint32_t num_tiles = tiles_m * tiles_n;
            const uint32_t num_kb    = (k_bytes + BLOCK_K_BYTES - 1) / BLOCK_K_BYTES;

            if(threadIdx.x == 0)
            {
                ptx::prefetch_tensormap(&tmap_a);
                ptx::prefetch_tensormap(&tmap_b);
                ptx::prefetch_tensormap(&tmap_c);
                ptx::prefetch_tensormap(&tmap_d);
                for(uint32_t s = 0; s < STAGES; ++s)
                {
                    ptx::mbar_init(full_bar + 8 * s, 1);
                    ptx::mbar_init(empty_bar + 8 * s, 1);
                }
                ptx::mbar_init(tfull_bar, 1);
                ptx::mbar_init(tfull_bar + 8, 1);
                ptx::mbar_init(drained_bar, EPI_WARPS);
                ptx::mbar_init(tempty_bar, 16); // accumulator 0: 8 warps x 2 CTAs
                ptx::mbar_init(tempty_bar + 8, 16); // accumulator 1
                for(uint32_t i = 0; i < EPI_WARPS * 2; ++i)
                    ptx::mbar_init(cbar_base + 8 * i, 1);
                *cta_abort = 0u;
                ptx::fence_barrier_init();
                ptx::fence_proxy_async_smem();
            }
            if(warp == 1)
            {
                ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), TMEM_COLS);
                ptx::tmem_relinquish_pair();
            }
            ptx::tc_fence_before_sync();
            ptx::cluster_sync();
            ptx::tc_fence_after_sync();
            const uint32_t tmem_base = *tmem_slot;

            if(warp == 0)
            {
                // ------------------------------ TMA producer (both CTAs) ------------------------------
                if(lane == 0)
                {
                    uint32_t stage = 0, phase = 0, iter = 0, drained_seen = 0;
                    bool     ok = true;
                    Unit     unit;
                    for(; ok && unit_at(iter, pair, num_pairs, num_tiles, num_kb, plan, unit); ++iter)
                    {
                        uint32_t m_idx, n_idx;
                        tile_coords(unit.tile, tiles_m, tiles_n, group_m, m_idx, n_idx);
                        const int32_t row_a = static_cast<int32_t>(m_idx * PAIR_M + rank * CTA_M);
                        const int32_t row_b = static_cast<int32_t>(n_idx * TILE_N + rank * HALF_N);
                        for(uint32_t kb = unit.kb0; kb < unit.kb1; ++kb)
                        {
                            ok = ptx::mbar_wait_bounded(empty_bar + 8 * stage, phase ^ 1u, cta_abort, status,
                                                        (ROLE_PRODUCER << 24) | blockIdx.x, WAIT_TIMEOUT_NS);
                            if(!ok)
                                break;
                            if(stage == EPI_STAGE && iter != 0u)
                            {
                                // this stage's A region doubles as staging tiles of the epilogue: every epilogue
                                // warp must have finished with them for all earlier units (bounded wait).  The phases of
                                // the barrier are consumed one by one: a unit with fewer slabs than stages may never come
                                // here, and a parity wait that skipped a phase would be satisfied by the wrong one.
                                while(ok && drained_seen < iter)
                                {
                                    ok = ptx::mbar_wait_bounded(drained_bar, drained_seen & 1u, cta_abort, status,
                                                                (ROLE_PRODUCER << 24) | (2u << 20) | blockIdx.x, WAIT_TIMEOUT_NS);
                                    ++drained_seen;
                                }
                                if(!ok)
                                    break;
                                ptx::fence_proxy_async_smem(); // generic writes of the staging tiles before the TMA overwrite
                            }
                            if(rank == 0)
                                ptx::mbar_arrive_expect_tx(full_bar + 8 * stage, 2u * STAGE_BYTES);
                            const uint32_t leader_full = ptx::mapa(full_bar + 8 * stage, 0u);
                            constexpr uint32_t ES       = elem_bytes<KIND>();
                            constexpr uint32_t SLAB_K   = BLOCK_K_BYTES / ES; // K elements per slab
                            constexpr uint32_t MN_GROUP = 128u / ES; // MN elements per 128-byte line
                            constexpr uint32_t GROUP_B  = SLAB_K * 128u; // bytes of one MN group over a slab
                            const int32_t      kc       = static_cast<int32_t>(kb * SLAB_K);
                            if constexpr(A_MN)
                            {
#pragma unroll
                                for(uint32_t gq = 0; gq < CTA_M / MN_GROUP; ++gq)
                                    ptx::tma_load_2d_pair(smem_a + stage * A_STAGE_BYTES + gq * GROUP_B, &tmap_a,
                                                          row_a + static_cast<int32_t>(gq * MN_GROUP), kc, leader_full);
                            }
                            else
                                ptx::tma_load_2d_pair(smem_a + stage * A_STAGE_BYTES, &tmap_a, kc, row_a, leader_full);
                            if constexpr(B_MN)
                            {
#pragma unroll
                                for(uint32_t gq = 0; gq < HALF_N / MN_GROUP; ++gq)
                                    ptx::tma_load_2d_pair(smem_b + stage * B_STAGE_BYTES + gq * GROUP_B, &tmap_b,
                                                          row_b + static_cast<int32_t>(gq * MN_GROUP), kc, leader_full);
                            }
                            else
                                ptx::tma_load_2d_pair(smem_b + stage * B_STAGE_BYTES, &tmap_b, kc, row_b, leader_full);
                            if(++stage == STAGES)
                            {
                                stage = 0;
                                phase ^= 1u;
                            }
                        }
                    }
                }
                __syncwarp();
            }
            else if(warp == 1)
            {
                // ------------------------------- MMA issuer (leader only) -------------------------------
                if(lane == 0 && rank == 0)
                {
                    constexpr uint32_t idesc = make_idesc<KIND, 2 * SUB_M, TILE_N, A_MN, B_MN>();
                    constexpr uint32_t ES      = elem_bytes<KIND>();
                    constexpr uint32_t GROUP_B = (BLOCK_K_BYTES / ES) * 128u; // one MN group over a slab
                    // descriptor start-address step per MMA (32 bytes of K): 32 bytes inside the K-major line,
                    // or (32 / ES) K rows of 128 bytes for an MN-major tile
                    constexpr uint32_t A_STEP = A_MN ? ((32u / ES) * 128u) >> 4 : 2u;
                    constexpr uint32_t B_STEP = B_MN ? ((32u / ES) * 128u) >> 4 : 2u;
                    uint32_t           stage = 0, phase = 0, iter = 0;
                    bool               ok = true;
                    const auto advance = [](uint32_t& st, uint32_t& ph) {
                        if(++st == STAGES)
                        {
                            st = 0;
                            ph ^= 1u;
                        }
                    };
                    // the slab in stage `st` has arrived (both CTAs' loads are counted on this barrier)
                    const auto wait_slab = [&](uint32_t st, uint32_t ph) {
                        const bool got = ptx::mbar_wait_bounded(full_bar + 8 * st, ph, cta_abort, status,
                                                                (ROLE_MMA << 24) | (1u << 20) | blockIdx.x, WAIT_TIMEOUT_NS);
                        ptx::tc_fence_after_sync();
                        return got;
                    };
                    // accumulator j of the previous tile has been drained by both CTAs
                    const auto wait_drained = [&](uint32_t j, uint32_t tphase) {
                        const bool got = ptx::mbar_wait_bounded(tempty_bar + 8 * j, tphase ^ 1u, cta_abort, status,
                                                                (ROLE_MMA << 24) | blockIdx.x, WAIT_TIMEOUT_NS);
                        ptx::tc_fence_after_sync();
                        return got;
                    };
                    // the MMAs of one K slab (stage st) into accumulator j; `fresh`: the slab is the tile's first
                    const auto mma_slab = [&](uint32_t j, uint32_t st, bool fresh) {
                        const uint64_t b_desc = B_MN ? ptx::make_mnmajor_sw128_desc(smem_b + st * B_STAGE_BYTES, GROUP_B)
                                                     : ptx::make_kmajor_sw128_desc(smem_b + st * B_STAGE_BYTES);
                        const uint32_t a_addr = smem_a + st * A_STAGE_BYTES + j * (SUB_M * BLOCK_K_BYTES);
                        const uint64_t a_desc = A_MN ? ptx::make_mnmajor_sw128_desc(a_addr, GROUP_B)
                                                     : ptx::make_kmajor_sw128_desc(a_addr);
#pragma unroll
                        for(uint32_t ks = 0; ks < BLOCK_K_BYTES / 32; ++ks)
                        {
                            const uint32_t acc = (fresh && ks == 0u) ? 0u : 1u;
                            if constexpr(KIND == KIND_F16 || KIND == KIND_BF16)
                                ptx::mma_f16_ss_pair(tmem_base + j * TILE_N, a_desc + A_STEP * ks, b_desc + B_STEP * ks, idesc, acc);
                            else if constexpr(KIND == KIND_I8)
                                ptx::mma_i8_ss_pair(tmem_base + j * TILE_N, a_desc + A_STEP * ks, b_desc + B_STEP * ks, idesc, acc);
                            else
                                ptx::mma_f8_ss_pair(tmem_base + j * TILE_N, a_desc + A_STEP * ks, b_desc + B_STEP * ks, idesc, acc);
                        }
                    };
                    Unit unit;
                    for(; ok && unit_at(iter, pair, num_pairs, num_tiles, num_kb, plan, unit); ++iter)
                    {
                        const uint32_t tphase = iter & 1u;
                        const uint32_t nslab  = unit.kb1 - unit.kb0; // slabs of this unit; kb counts them from 0
                        const bool     split  = SPLIT && nslab >= HEAD_KB + TAIL_KB;
                        uint32_t       kb     = 0;
                        if(split)
                        {
                            // head: accumulator 0 over the first slabs (accumulator 1 of the previous tile may still be
                            // draining), then accumulator 1 over the same slabs, releasing each stage
                            uint32_t st = stage, ph = phase;
                            ok = wait_drained(0, tphase);
                            for(uint32_t i = 0; ok && i < HEAD_KB; ++i)
                            {
                                ok = wait_slab(st, ph);
                                if(ok)
                                    mma_slab(0, st, i == 0u);
                                advance(st, ph);
                            }
                            if(ok)
                                ok = wait_drained(1, tphase);
                            for(uint32_t i = 0; ok && i < HEAD_KB; ++i)
                            {
                                mma_slab(1, stage, i == 0u);
                                ptx::tc_commit_pair(empty_bar + 8 * stage, 0x3);
                                advance(stage, phase);
                            }
                            kb = HEAD_KB;
                        }
                        const uint32_t mid_end = split ? nslab - TAIL_KB : nslab;
                        for(; ok && kb < mid_end; ++kb)
                        {
                            ok = wait_slab(stage, phase);
#pragma unroll
                            for(uint32_t j = 0; j < 2; ++j)
                            {
                                if(ok && kb == 0u)
                                    ok = wait_drained(j, tphase);
                                if(ok)
                                    mma_slab(j, stage, kb == 0u);
                            }
                            if(!ok)
                                break;
                            ptx::tc_commit_pair(empty_bar + 8 * stage, 0x3);
                            advance(stage, phase);
                        }
                        if(split && ok)
                        {
                            // tail: accumulator 0 over the last slabs and its tmem_full, then accumulator 1
                            uint32_t st = stage, ph = phase;
                            for(uint32_t i = 0; ok && i < TAIL_KB; ++i)
                            {
                                ok = wait_slab(st, ph);
                                if(ok)
                                    mma_slab(0, st, false);
                                advance(st, ph);
                            }
                            if(ok)
                                ptx::tc_commit_pair(tfull_bar, 0x3);
                            for(uint32_t i = 0; ok && i < TAIL_KB; ++i)
                            {
                                mma_slab(1, stage, false);
                                ptx::tc_commit_pair(empty_bar + 8 * stage, 0x3);
                                advance(stage, phase);
                            }
                            if(ok)
                                ptx::tc_commit_pair(tfull_bar + 8, 0x3);
                        }
                        else if(ok)
                        {
                            ptx::tc_commit_pair(tfull_bar, 0x3);
                            ptx::tc_commit_pair(tfull_bar + 8, 0x3);
                        }
                    }
                }
                __syncwarp();
            }
            else
            {
                // -------------------------------- epilogue (both CTAs) --------------------------------
                const uint32_t e      = warp - 2u; // 0..15
                const uint32_t quad   = warp & 3u; // lane quadrant this warp may read
                const uint32_t j      = (e >> 2) & 1u; // accumulator: warps 2-5, 10-13 -> 0; warps 6-9, 14-17 -> 1
                const uint32_t first  = e >> 3; // 0: even 64-byte column steps, 1: odd steps
                const bool     read_c = (beta != ScalarT(0)) && (c != nullptr);
                const uint32_t buf_off  = epi_off + e * EPI_BUF_BYTES; // first tile: dedicated
                const uint32_t buf0     = base + buf_off;
                // second tile: inside the A region of the last operand stage, accumulator 0's warps in the half that holds
                // rows 0-127 (which only accumulator 0's MMAs read), accumulator 1's in the other half
                const uint32_t buf1_off = alias_base_off + (j * 8u + (e & 3u) + 4u * first) * EPI_BUF_BYTES;
                const uint32_t buf1     = base + buf1_off;
                const uint32_t cbar0   = cbar_base + e * 16u;
                // one-byte outputs have no staged path (the host passes vec_ok == 0 for them)
                using StageT           = typename std::conditional<sizeof(OutT) >= 2, OutT, int32_t>::type;
                using Drain            = StagedDrain<StageT, ScalarT, TILE_N, 2>;
                // The eight warps of an accumulator wait for it together: one of them (the leader) watches the tmem_full
                // barrier, the others park on a named hardware barrier and issue nothing meanwhile - sixteen warps polling
                // through every tile's main loop were most of the kernel's instructions.  A warp that gives up (a bounded
                // wait ran out, the CTA is aborting) keeps going round the loop without working, so that the named
                // barrier always sees all of its warps.
                const bool leader = (e & 11u) == 0u; // e == 0 (accumulator 0), e == 4 (accumulator 1)
                uint32_t   iter = 0, cpar = 0;
                bool       dead = false;
                // split round: this thread's row in its pair's workspace slot, and the flags
                uint32_t* const slot_row = split_ws + static_cast<size_t>(pair) * SLOT_WORDS
                                           + static_cast<size_t>(rank * 2u + j) * (TILE_N * SUB_M) + quad * 32u + lane;
                uint32_t* const flags = split_ws + static_cast<size_t>(num_pairs) * SLOT_WORDS;
                Unit            unit;
                for(; unit_at(iter, pair, num_pairs, num_tiles, num_kb, plan, unit); ++iter)
                {
                    uint32_t m_idx, n_idx;
                    tile_coords(unit.tile, tiles_m, tiles_n, group_m, m_idx, n_idx);
                    const uint32_t row_base = m_idx * PAIR_M + rank * CTA_M + j * SUB_M; // this accumulator's first row
                    const uint32_t row0     = row_base + quad * 32u; // this warp's first row
                    const uint32_t col_base = n_idx * TILE_N;
                    // staged path: needs 16-byte aligned rows (TMA) and a tile that starts inside the matrix
                    const bool partial = unit.kind == UNIT_PARTIAL; // no C, no D: the raw accumulators go to the workspace
                    const bool staged  = !partial && vec_ok != 0 && row0 < m && col_base < n;
                    // C does not depend on the accumulators: the tile of the warp's first step is requested now
                    if(!dead && staged && read_c && lane == 0)
                        Drain::prefetch_c(&tmap_c, buf0, cbar0, col_base, row0, n, first, 0, 1, buf1);
                    if(leader && !dead)
                        dead = !ptx::mbar_wait_bounded_warp(tfull_bar + 8 * j, iter & 1u, cta_abort, status,
                                                            (ROLE_EPILOGUE << 24) | blockIdx.x, WAIT_TIMEOUT_NS, lane);
                    ptx::named_bar_sync(1u + j, 8u * 32u);
                    if(!dead && !leader)
                        // the leader saw the phase complete (or gave up and raised the abort flag): confirm it here
                        dead = (*cta_abort != 0u) || !ptx::mbar_try_wait(tfull_bar + 8 * j, iter & 1u);
                    if(dead)
                        continue;
                    ptx::tc_fence_after_sync();
                    // every MMA of the tile into this accumulator has retired: its half of the aliased staging tiles may be
                    // written now
                    if(staged && read_c && lane == 0)
                        Drain::prefetch_c(&tmap_c, buf0, cbar0, col_base, row0, n, first, 1, 2, buf1);
                    const uint32_t tmem_acc = tmem_base + j * TILE_N;
                    if(partial)
                    {
                        Drain::store_partial(tmem_acc, quad, slot_row, first);
                        __threadfence(); // this thread's partial sums before the flag
                        __syncwarp();
                        if(lane == 0)
                            red_release_gpu_add_u32(flags + pair, 1u); // complete at 2 CTAs x EPI_WARPS
                    }
                    else if(staged)
                    {
                        uint32_t npart = 0;
                        if(unit.kind == UNIT_FINISH)
                        {
                            // the pairs before this one hold the rest of the tile's K range: wait for their partials
                            npart = finish_contributors(pair, unit.tile, num_pairs, num_kb, plan);
                            const uint64_t t0 = ptx::globaltimer_ns();
                            for(uint32_t pi = 0; pi < npart && !dead; ++pi)
                            {
                                uint32_t spins = 0;
                                while(ld_acquire_gpu_u32(flags + pair - 1u - pi) < 2u * EPI_WARPS)
                                {
                                    __nanosleep(64);
                                    if((++spins & 0x3Fu) == 0u && (*cta_abort || ptx::globaltimer_ns() - t0 > WAIT_TIMEOUT_NS))
                                    {
                                        if(!*cta_abort)
                                        {
                                            *cta_abort = 1u;
                                            if(atomicCAS(status, 0u, ptx::STATUS_TIMEOUT_CODE) == 0u)
                                                status[1] = (ROLE_EPILOGUE << 24) | (6u << 20) | blockIdx.x;
                                        }
                                        dead = true;
                                        break;
                                    }
                                }
                            }
                            dead = __any_sync(0xFFFFFFFFu, dead);
                        }
                        if(!dead)
                            dead = !Drain::run(tmem_acc, quad, lane, smem, buf_off, buf0, cbar0, &tmap_c, &tmap_d, col_base, row0,
                                               n, alpha, beta, read_c, cpar, cta_abort, status,
                                               (ROLE_EPILOGUE << 24) | (1u << 20) | blockIdx.x, first, buf1_off, buf1,
                                               slot_row - SLOT_WORDS, npart);
                    }
                    else if(vec_ok == 0 && first == 0u)
                    {
                        // one-byte outputs have no staged path: with aligned rows they still move 16 or 32 bytes at a time
                        int vec = 0;
                        if constexpr(sizeof(OutT) == 1)
                        {
                            const uintptr_t bits = reinterpret_cast<uintptr_t>(d) | ldd | (read_c ? (reinterpret_cast<uintptr_t>(c) | ldc) : 0u);
                            vec = (bits % 32u) == 0u ? 2 : ((bits % 16u) == 0u ? 1 : 0);
                        }
                        drain_accumulator<OutT, ScalarT, TILE_N>(tmem_acc, quad, lane, row_base, col_base, m, n, c, d, ldc,
                                                                 ldd, alpha, beta, read_c, vec);
                    }
                    // (an aligned tile that lies wholly outside the matrix has nothing to store)
                    if(dead)
                        continue;
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if(lane == 0)
                    {
                        ptx::mbar_arrive_cluster(ptx::mapa(tempty_bar + 8 * j, 0u));
                        // hand the aliased staging tiles back to the producer once this warp's stores have read them
                        ptx::bulk_wait_group_read<0>();
                        ptx::mbar_arrive(drained_bar);
                    }
                }
                if(lane == 0)
                    ptx::bulk_wait_group<0>(); // the staging tiles must outlive the stores that read them
                __syncwarp();
            }

            // ---------------------------------- teardown ----------------------------------
            ptx::tc_fence_before_sync();
            ptx::cluster_sync();
            {
                const uint32_t peer_abort = ptx::ld_shared_cluster_u32(
                    ptx::mapa(ptx::smem_u32(const_cast<uint32_t*>(cta_abort)), rank ^ 1u));
                if(*cta_abort || peer_abort)
                {
                    const uint64_t t0 = ptx::globaltimer_ns();
                    while(ptx::globaltimer_ns() - t0 < 2000000ull)
                        __nanosleep(1000);
                }
            }
            ptx::cluster_sync();
            if(warp == 1)
            {
                ptx::tc_fence_after_sync();
                ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
            }
        }
    } // namespace tc05q
} // namespace b200wmma
