// Flow-control wrappers with the names of rocWMMA's internal/flow_control.hpp:103-118
// (Barrier, SchedBarrier, SetPrio, Waitcnt, WaitVmcnt, WaitLgkmcnt), each with a static exec().
//
// The reference's wrappers issue AMD scalar instructions (s_barrier, s_setprio, s_waitcnt with
// vector-memory / LDS counters, a scheduling fence for the compiler).  CUDA has no per-warp priority
// and no user-visible memory counters: loads and stores of a thread are ordered by the hardware
// scoreboard.  What remains meaningful is kept:
//   Barrier      -> __syncthreads()
//   Waitcnt<..>  -> a compiler-level memory fence (asm volatile with a "memory" clobber), so that code
//                   which placed a wait to order its own shared-memory traffic keeps that order
//   SchedBarrier -> the same compiler fence (instructions are not moved across it)
//   SetPrio      -> nothing
#ifndef ROCWMMA_B200_FLOW_CONTROL_HPP
#define ROCWMMA_B200_FLOW_CONTROL_HPP

#include "config.hpp"

namespace rocwmma
{
    namespace detail
    {
        struct cuda_barrier
        {
            ROCWMMA_DEVICE static inline void exec()
            {
                __syncthreads();
            }
        };
        struct compiler_fence
        {
            ROCWMMA_DEVICE static inline void exec()
            {
                asm volatile("" ::: "memory");
            }
        };
        template <int32_t mask = 0>
        struct sched_barrier : compiler_fence
        {
        };
        template <int32_t priority = 0>
        struct setprio
        {
            ROCWMMA_DEVICE static inline void exec()
            {
                static_assert(priority >= 0 && priority <= 3, "Priority must be from 0 to 3");
            }
        };
        template <int32_t vmcnt, int32_t lgkmcnt>
        struct waitcnt : compiler_fence
        {
            static_assert(vmcnt >= 0 && vmcnt < 64, "Vector memory operations allocated a maximum of 6 bits");
            static_assert(lgkmcnt >= 0 && lgkmcnt < 16, "Scalar mem/LDS/GDS allocated a maximum of 4 bits");
        };
    } // namespace detail

    using Barrier = detail::cuda_barrier;
    template <int32_t mask>
    using SchedBarrier = detail::sched_barrier<mask>;
    template <int32_t priority>
    using SetPrio = detail::setprio<priority>;
    template <int32_t vmcnt, int32_t lgkmcnt>
    using Waitcnt = detail::waitcnt<vmcnt, lgkmcnt>;
    template <int32_t vmcnt>
    using WaitVmcnt = detail::waitcnt<vmcnt, 0>;
    template <int32_t lgkmcnt>
    using WaitLgkmcnt = detail::waitcnt<0, lgkmcnt>;
} // namespace rocwmma

#endif
