// Thin inline-PTX wrappers for the sm_100a features the tensor-core GEMM uses:
// mbarrier (with bounded waits), TMA tiled loads, tcgen05 alloc / mma / commit / ld.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace b200wmma
{
    namespace ptx
    {
        __device__ __forceinline__ uint32_t smem_u32(const void* p)
        {
            return static_cast<uint32_t>(__cvta_generic_to_shared(p));
        }
        __device__ __forceinline__ uint64_t globaltimer_ns()
        {
            uint64_t t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            return t;
        }

        // ---- mbarrier -----------------------------------------------------------------
        __device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
        {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)
                         : "memory");
        }
        __device__ __forceinline__ void fence_barrier_init()
        {
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __device__ __forceinline__ void fence_proxy_async_smem()
        {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
        {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                         "r"(bytes)
                         : "memory");
        }
        __device__ __forceinline__ void mbar_arrive(uint32_t bar)
        {
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
        }
        // Programmatic dependent launch.  launch_dependents: the next kernel of the stream, if it was launched with
        // programmatic stream serialization, may start its CTAs once every CTA of this grid has passed this point
        // (or exited).  grid_dep_wait: returns when the preceding grid has completed and its memory operations are
        // visible; a no-op when the kernel was launched the ordinary way.  Everything a kernel does before
        // grid_dep_wait overlaps the tail of its predecessor, so it must touch no global memory there.
        __device__ __forceinline__ void grid_dep_launch_dependents()
        {
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        }
        __device__ __forceinline__ void grid_dep_wait()
        {
            asm volatile("griddepcontrol.wait;" ::: "memory");
        }

        __device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
        {
            uint32_t ok;
            asm volatile("{\n"
                         ".reg .pred p;\n"
                         "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                         "selp.u32 %0, 1, 0, p;\n"
                         "}"
                         : "=r"(ok)
                         : "r"(bar), "r"(parity)
                         : "memory");
            return ok != 0;
        }

        // try_wait that lets the hardware park the thread for up to `hint_ns` while the phase is
        // incomplete (it returns as soon as the phase completes): no instructions issue meanwhile.
        __device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns)
        {
            uint32_t ok;
            asm volatile("{\n"
                         ".reg .pred p;\n"
                         "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
                         "selp.u32 %0, 1, 0, p;\n"
                         "}"
                         : "=r"(ok)
                         : "r"(bar), "r"(parity), "r"(hint_ns)
                         : "memory");
            return ok != 0;
        }

        // Bounded wait.  Returns false when the wait was abandoned: either this thread ran
        // past `timeout_ns` (it then raises the CTA-wide abort flag and records `who` in the
        // device status word {code, detail}) or another thread of the CTA already aborted.
        // No trap, no unbounded loop: the caller unwinds to the kernel's common exit.
        constexpr unsigned STATUS_TIMEOUT_CODE = 5u; // == B200WMMA_ERR_DEVICE_TIMEOUT
        // Suspend-time hint (ns) of the waits below; 0 = poll with plain try_wait.
#ifndef B200WMMA_WAIT_HINT_NS
#define B200WMMA_WAIT_HINT_NS 4000
#endif
        __device__ __forceinline__ bool mbar_wait_bounded(uint32_t           bar,
                                                          uint32_t           parity,
                                                          volatile uint32_t* cta_abort,
                                                          unsigned*          status,
                                                          uint32_t           who,
                                                          uint64_t           timeout_ns)
        {
            if(mbar_try_wait(bar, parity))
                return true;
            const uint64_t t0    = globaltimer_ns();
            uint32_t       spins = 0;
            while(true)
            {
#if B200WMMA_WAIT_HINT_NS > 0
                // parked in hardware until the phase completes or the hint runs out: a waiting thread issues a
                // handful of instructions per wake-up instead of polling
                if(mbar_try_wait_hint(bar, parity, B200WMMA_WAIT_HINT_NS))
                    return true;
                if((++spins & 0x7u) == 0u)
#else
                if(mbar_try_wait(bar, parity))
                    return true;
                if((++spins & 0xFFu) == 0u)
#endif
                {
                    if(*cta_abort)
                        return false;
                    if(globaltimer_ns() - t0 > timeout_ns)
                    {
                        *cta_abort = 1u;
                        if(atomicCAS(status, 0u, STATUS_TIMEOUT_CODE) == 0u)
                            status[1] = who;
                        return false;
                    }
                }
            }
        }

        // Warp-wide bounded wait for waits that last a whole tile: lane 0 waits with the hardware
        // suspend hint (31 lanes stop issuing instructions), then every lane confirms the completed
        // phase itself so that each has observed the barrier.  All 32 lanes must call it.
        __device__ __forceinline__ bool mbar_wait_bounded_warp(uint32_t           bar,
                                                               uint32_t           parity,
                                                               volatile uint32_t* cta_abort,
                                                               unsigned*          status,
                                                               uint32_t           who,
                                                               uint64_t           timeout_ns,
                                                               uint32_t           lane)
        {
            bool ok = true;
            if(lane == 0 && !mbar_try_wait(bar, parity))
            {
                const uint64_t t0    = globaltimer_ns();
                uint32_t       spins = 0;
                while(true)
                {
                    if(mbar_try_wait_hint(bar, parity, 20000u)) // parked in hardware, woken by the completion
                        break;
                    if((++spins & 0x3u) == 0u)
                    {
                        if(*cta_abort)
                        {
                            ok = false;
                            break;
                        }
                        if(globaltimer_ns() - t0 > timeout_ns)
                        {
                            *cta_abort = 1u;
                            if(atomicCAS(status, 0u, STATUS_TIMEOUT_CODE) == 0u)
                                status[1] = who;
                            ok = false;
                            break;
                        }
                    }
                }
            }
            ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
            if(ok)
            {
                // the phase lane 0 saw complete cannot advance again before this warp releases the
                // resource it guards, so this returns at once; the bound is a formality
                uint32_t tries = 0;
                while(!mbar_try_wait(bar, parity))
                    if(++tries > (1u << 20))
                    {
                        ok = false;
                        break;
                    }
                ok = __all_sync(0xFFFFFFFFu, ok);
            }
            return ok;
        }

        // Named hardware barrier `id` (1..15) over `threads` threads (a multiple of 32): the waiting warps issue no
        // instructions until the last one arrives.
        __device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t threads)
        {
            asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
        }

        // ---- counters in shared memory (release / acquire at CTA scope) ---------------------------
        __device__ __forceinline__ uint32_t ld_acquire_shared_u32(const uint32_t* p)
        {
            uint32_t v;
            asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
            return v;
        }
        __device__ __forceinline__ void red_release_shared_add_u32(uint32_t* p, uint32_t v)
        {
            asm volatile("red.release.cta.shared::cta.add.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
        }

        // ---- TMA ------------------------------------------------------------------------
        __device__ __forceinline__ void prefetch_tensormap(const void* tmap)
        {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap))
                         : "memory");
        }
        // 2-D tiled load global -> shared (this CTA), completion counted on `bar`.
        // c0 is the innermost coordinate: c0 * element size must be a multiple of 16 bytes.
        __device__ __forceinline__ void
            tma_load_2d(uint32_t dst_smem, const void* tmap, int32_t c0, int32_t c1, uint32_t bar)
        {
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
                         " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
                         "l"(reinterpret_cast<uint64_t>(tmap)),
                         "r"(c0),
                         "r"(c1),
                         "r"(bar)
                         : "memory");
        }

        __device__ __forceinline__ void
            tma_load_3d(uint32_t dst_smem, const void* tmap, int32_t c0, int32_t c1, int32_t c2, uint32_t bar)
        {
            asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
                         " [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst_smem),
                         "l"(reinterpret_cast<uint64_t>(tmap)),
                         "r"(c0),
                         "r"(c1),
                         "r"(c2),
                         "r"(bar)
                         : "memory");
        }

        // 1-D bulk copy global -> shared (this CTA); both addresses 16-byte aligned, size a multiple of 16.
        __device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar)
        {
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             dst_smem),
                         "l"(src),
                         "r"(bytes),
                         "r"(bar)
                         : "memory");
        }
        // 1-D bulk copy shared -> global, tracked by the issuing thread's bulk async-group.
        __device__ __forceinline__ void bulk_store_1d(void* dst, uint32_t src_smem, uint32_t bytes)
        {
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem),
                         "r"(bytes)
                         : "memory");
        }
        // 2-D tiled store shared -> global.  c0 * element size must be a multiple of 16 bytes and
        // neither coordinate may be negative.
        __device__ __forceinline__ void tma_store_2d(const void* tmap, int32_t c0, int32_t c1, uint32_t src_smem)
        {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                             reinterpret_cast<uint64_t>(tmap)),
                         "r"(c0),
                         "r"(c1),
                         "r"(src_smem)
                         : "memory");
        }
        __device__ __forceinline__ void bulk_commit_group()
        {
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        // Wait until at most N of this thread's bulk groups still have to READ their shared-memory source.
        template <int N>
        __device__ __forceinline__ void bulk_wait_group_read()
        {
            asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
        }
        // Wait until at most N of this thread's bulk groups are still incomplete (writes performed).
        template <int N>
        __device__ __forceinline__ void bulk_wait_group()
        {
            asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
        }

        // ---- tcgen05 / tensor memory ----------------------------------------------------
        __device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols)
        {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             dst_smem),
                         "r"(ncols)
                         : "memory");
        }
        __device__ __forceinline__ void tmem_relinquish()
        {
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::
                             : "memory");
        }
        __device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
        {
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr),
                         "r"(ncols)
                         : "memory");
        }
        __device__ __forceinline__ void tc_fence_before_sync()
        {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
        __device__ __forceinline__ void tc_fence_after_sync()
        {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        // D[tmem] (+)= A[smem] * B[smem]; one thread issues for the whole CTA.
        __device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem,
                                                   uint64_t a_desc,
                                                   uint64_t b_desc,
                                                   uint32_t idesc,
                                                   uint32_t accumulate)
        {
            asm volatile("{\n"
                         ".reg .pred p;\n"
                         "setp.ne.b32 p, %4, 0;\n"
                         "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
                         "}" ::"r"(d_tmem),
                         "l"(a_desc),
                         "l"(b_desc),
                         "r"(idesc),
                         "r"(accumulate)
                         : "memory");
        }
        __device__ __forceinline__ void mma_i8_ss(uint32_t d_tmem,
                                                  uint64_t a_desc,
                                                  uint64_t b_desc,
                                                  uint32_t idesc,
                                                  uint32_t accumulate)
        {
            asm volatile("{\n"
                         ".reg .pred p;\n"
                         "setp.ne.b32 p, %4, 0;\n"
                         "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
                         "}" ::"r"(d_tmem),
                         "l"(a_desc),
                         "l"(b_desc),
                         "r"(idesc),
                         "r"(accumulate)
                         : "memory");
        }
        // mbarrier arrive once every MMA issued so far by this thread has completed.
        __device__ __forceinline__ void tc_commit(uint32_t bar)
        {
            asm volatile(
                "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                    bar)
                : "memory");
        }
        // 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets lane
        // (taddr.lane + i), registers j = columns taddr.col + j.
        __device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
        {
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, "
                "[%32];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                  "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                  "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
                  "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                  "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
                  "=r"(r[30]), "=r"(r[31])
                : "r"(taddr)
                : "memory");
        }
        // 32 lanes x 16 consecutive 32-bit columns.
        __device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16])
        {
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                         "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                         : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                           "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
                           "=r"(r[14]), "=r"(r[15])
                         : "r"(taddr)
                         : "memory");
        }
        __device__ __forceinline__ void tmem_ld_wait()
        {
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        }


        // ---- thread-block clusters and the two-CTA (cta_group::2) forms ------------------------
        __device__ __forceinline__ uint32_t cluster_ctarank()
        {
            uint32_t r;
            asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
            return r;
        }
        // Full cluster barrier with release / acquire ordering; every thread of every CTA calls it.
        __device__ __forceinline__ void cluster_sync()
        {
            asm volatile("barrier.cluster.arrive.release.aligned;\n"
                         "barrier.cluster.wait.acquire.aligned;" ::
                             : "memory");
        }
        // shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
        __device__ __forceinline__ uint32_t mapa(uint32_t smem_addr, uint32_t rank)
        {
            uint32_t r;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
            return r;
        }
        // Arrive on a barrier that may live in the peer CTA (`cluster_addr` from mapa).  Default semantics (release at
        // CTA scope): what the arrival publishes has already been made visible to its consumer by other means - tensor
        // memory reads by tcgen05.wait::ld + tcgen05.fence, shared-memory tiles for the tensor core by
        // fence.proxy.async - so the cluster-scope release, a fence that costs ~1000 cycles per arrival, is not needed.
        __device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
        {
            asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
        }
        __device__ __forceinline__ uint32_t ld_shared_cluster_u32(uint32_t cluster_addr)
        {
            uint32_t v;
            asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
            return v;
        }
        // 2-D tiled load into THIS CTA's shared memory whose completion bytes are counted on a
        // barrier that may live in the peer CTA of the pair (`bar_cluster_addr` from mapa).
        // No multicast: each CTA fetches its own boxes.
        __device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const void* tmap, int32_t c0,
                                                         int32_t c1, uint32_t bar_cluster_addr)
        {
            asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
                         " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
                         "l"(reinterpret_cast<uint64_t>(tmap)),
                         "r"(c0),
                         "r"(c1),
                         "r"(bar_cluster_addr)
                         : "memory");
        }
        __device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols)
        {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                         "r"(ncols)
                         : "memory");
        }
        __device__ __forceinline__ void tmem_relinquish_pair()
        {
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        }
        __device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
        {
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                         : "memory");
        }
        // One MMA spanning both CTAs of the pair: M = 256 (128 rows of A and of D per CTA),
        // each CTA supplies half of B's N extent from the same shared-memory offset.
        __device__ __forceinline__ void mma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                        uint32_t idesc, uint32_t accumulate)
        {
            asm volatile("{\n"
                         ".reg .pred p;\n"
                         "setp.ne.b32 p, %4, 0;\n"
                         "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
                         "}" ::"r"(d_tmem),
                         "l"(a_desc),
                         "l"(b_desc),
                         "r"(idesc),
                         "r"(accumulate)
                         : "memory");
        }
        __device__ __forceinline__ void mma_i8_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                       uint32_t idesc, uint32_t accumulate)
        {
            asm volatile("{\n"
                         ".reg .pred p;\n"
                         "setp.ne.b32 p, %4, 0;\n"
                         "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n"
                         "}" ::"r"(d_tmem),
                         "l"(a_desc),
                         "l"(b_desc),
                         "r"(idesc),
                         "r"(accumulate)
                         : "memory");
        }
        // 8-bit floating point inputs (e4m3 / e5m2 chosen in the instruction descriptor), fp32 accumulate;
        // 32 bytes of K per instruction like the int8 form.
        __device__ __forceinline__ void mma_f8_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                       uint32_t idesc, uint32_t accumulate)
        {
            asm volatile("{\n"
                         ".reg .pred p;\n"
                         "setp.ne.b32 p, %4, 0;\n"
                         "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
                         "}" ::"r"(d_tmem),
                         "l"(a_desc),
                         "l"(b_desc),
                         "r"(idesc),
                         "r"(accumulate)
                         : "memory");
        }
        // Once every MMA issued so far by this thread has completed, arrive on the barrier at this
        // shared-memory offset in each CTA of the pair named by `cta_mask` (bit r = CTA rank r).
        // This is a barrier signal, not a data transfer: no operand is multicast.
        __device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask)
        {
            asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
                         "[%0], %1;" ::"r"(bar),
                         "h"(cta_mask)
                         : "memory");
        }

        // ---- 2:4 structured-sparse int8 MMA ---------------------------------------------------
        // D[tmem] (+)= A[smem, compressed] * B[smem] with A's position metadata in tensor memory.
        // One instruction covers 64 logical K: 32 bytes per row of compressed A, 64 bytes per row of
        // B, and 128 lanes x 2 columns of metadata at `e_tmem` (one bit per logical element: a byte
        // holds the two 4-bit position codes of 8 consecutive K positions).
        __device__ __forceinline__ void mma_i8_sp_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                          uint32_t e_tmem, uint32_t idesc, uint32_t accumulate)
        {
            asm volatile("{\n"
                         ".reg .pred p;\n"
                         "setp.ne.b32 p, %5, 0;\n"
                         "tcgen05.mma.sp.cta_group::2.kind::i8 [%0], %1, %2, [%3], %4, p;\n"
                         "}" ::"r"(d_tmem),
                         "l"(a_desc), "l"(b_desc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
                         : "memory");
        }
        // Shared memory -> tensor memory: 128 rows of 32 bytes become 128 lanes x 8 columns in each CTA of the
        // pair (each copies from its own shared memory).  The source is two 16-byte-wide column blocks
        // (make_rows16_desc with the distance between the blocks as `lbo_bytes`).  Issued by the MMA thread;
        // it executes in order with that thread's MMAs and is covered by its commits.
        __device__ __forceinline__ void tmem_cp_128x256b_pair(uint32_t taddr, uint64_t smem_desc)
        {
            asm volatile("tcgen05.cp.cta_group::2.128x256b [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
        }
        // Unswizzled tile of 16-byte rows stored back to back (row r at r * 16 bytes): 8-row core
        // matrices of 128 bytes, 128 bytes apart (SBO).  A second 16-byte-wide column block, if the
        // instruction reads one, lies `lbo_bytes` after the first (LBO).
        __device__ __forceinline__ uint64_t make_rows16_desc(uint32_t smem_addr, uint32_t lbo_bytes = 128u)
        {
            uint64_t desc = 0;
            desc |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
            desc |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16; // LBO
            desc |= static_cast<uint64_t>(128u >> 4) << 32; // SBO
            desc |= static_cast<uint64_t>(1u) << 46; // descriptor version; layout type 0 = no swizzle
            return desc;
        }

        // Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128
        // bytes with the 128-byte swizzle (what a TMA SWIZZLE_128B box load produces):
        // 8-row groups are 1024 bytes apart (SBO), the leading-dimension offset is unused for
        // swizzled K-major layouts, descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B).
        // The tile base must be 1024-byte aligned; stepping along K inside the 128-byte row
        // adds the byte offset (>>4) to the start-address field.
        __device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr)
        {
            uint64_t desc = 0;
            desc |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
            desc |= static_cast<uint64_t>(1u) << 16; // LBO (ignored for swizzled K-major)
            desc |= static_cast<uint64_t>(1024u >> 4) << 32; // SBO
            desc |= static_cast<uint64_t>(1u) << 46; // descriptor version
            desc |= static_cast<uint64_t>(2u) << 61; // SWIZZLE_128B
            return desc;
        }
        // Descriptor for an MN-major operand tile (the M or N index is contiguous in memory, as in a
        // column-major A or a row-major B).  The tile is stored as TMA SWIZZLE_128B boxes: each box
        // holds one group of 128 bytes of MN (64 fp16 / 128 int8) for all K rows of the slab, one K row
        // per 128-byte line.  8-K-row groups are 1024 bytes apart (SBO); consecutive MN groups are
        // `group_bytes` apart (LBO).  Stepping along K adds (rows x 128 bytes) >> 4 to the start address.
        __device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr, uint32_t group_bytes)
        {
            uint64_t desc = 0;
            desc |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
            desc |= static_cast<uint64_t>((group_bytes >> 4) & 0x3FFFu) << 16; // LBO
            desc |= static_cast<uint64_t>(1024u >> 4) << 32; // SBO
            desc |= static_cast<uint64_t>(1u) << 46; // descriptor version
            desc |= static_cast<uint64_t>(2u) << 61; // SWIZZLE_128B
            return desc;
        }
    } // namespace ptx
} // namespace b200wmma
