// Warp-level mma.sync wrappers, one per supported (input type, compute type) pair.
// Each takes the per-lane registers of one A atom, one B atom and one 16x16 accumulator atom
// in the register orders defined in layout.hpp and accumulates acc += A x B.
#ifndef ROCWMMA_B200_MMA_ATOMS_HPP
#define ROCWMMA_B200_MMA_ATOMS_HPP

#include "types.hpp"

namespace rocwmma
{
    namespace detail
    {
        // fp16 x fp16 -> fp32: a = 4 x b32 (8 halfs), b = 4 x b32 ordered
        // [n-half 0 k-lo, n-half 1 k-lo, n-half 0 k-hi, n-half 1 k-hi], acc = 8 floats (two m16n8 tiles).
        ROCWMMA_DEVICE inline void mma_atom_f16_f32(float (&acc)[8], const uint32_t (&a)[4],
                                                    const uint32_t (&b)[4])
        {
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[2]));
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(acc[4]), "+f"(acc[5]), "+f"(acc[6]), "+f"(acc[7])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[1]), "r"(b[3]));
        }

        // fp16, 8 deep (m16n8k8): a = 2 x b32, b = 2 x b32 [n-half 0, n-half 1]
        ROCWMMA_DEVICE inline void mma_atom_f16_f32_k8(float (&acc)[8], const uint32_t (&a)[2], const uint32_t (&b)[2])
        {
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
                         : "r"(a[0]), "r"(a[1]), "r"(b[0]));
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+f"(acc[4]), "+f"(acc[5]), "+f"(acc[6]), "+f"(acc[7])
                         : "r"(a[0]), "r"(a[1]), "r"(b[1]));
        }

        // bf16 x bf16 -> fp32, same register orders as fp16
        ROCWMMA_DEVICE inline void mma_atom_bf16_f32(float (&acc)[8], const uint32_t (&a)[4], const uint32_t (&b)[4])
        {
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[2]));
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(acc[4]), "+f"(acc[5]), "+f"(acc[6]), "+f"(acc[7])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[1]), "r"(b[3]));
        }
        ROCWMMA_DEVICE inline void mma_atom_bf16_f32_k8(float (&acc)[8], const uint32_t (&a)[2], const uint32_t (&b)[2])
        {
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
                         : "r"(a[0]), "r"(a[1]), "r"(b[0]));
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+f"(acc[4]), "+f"(acc[5]), "+f"(acc[6]), "+f"(acc[7])
                         : "r"(a[0]), "r"(a[1]), "r"(b[1]));
        }

        // int8 x int8 -> int32 (m16n8k16): a = 2 x b32, b = 2 x b32 [n-half 0, n-half 1]
        ROCWMMA_DEVICE inline void mma_atom_i8_i32(int32_t (&acc)[8], const uint32_t (&a)[2],
                                                   const uint32_t (&b)[2])
        {
            asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+r"(acc[0]), "+r"(acc[1]), "+r"(acc[2]), "+r"(acc[3])
                         : "r"(a[0]), "r"(a[1]), "r"(b[0]));
            asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+r"(acc[4]), "+r"(acc[5]), "+r"(acc[6]), "+r"(acc[7])
                         : "r"(a[0]), "r"(a[1]), "r"(b[1]));
        }

        // int8, 8 deep: no such integer mma.sync shape.  The products are formed on m16n8k8 with exact fp16 copies of the
        // operands (|v| <= 128) and fp32 accumulation from zero - eight products of at most 2^14 each, exact - and added
        // to the int32 accumulator as integers.  a = 4 int8 (one register), b = 4 int8 [n-half 0 pair, n-half 1 pair].
        ROCWMMA_DEVICE inline uint32_t i8pair_to_half2(uint32_t word, uint32_t shift)
        {
            const int     lo = static_cast<int8_t>((word >> shift) & 0xFFu), hi = static_cast<int8_t>((word >> (shift + 8u)) & 0xFFu);
            const __half2 h  = __halves2half2(__int2half_rn(lo), __int2half_rn(hi));
            return *reinterpret_cast<const uint32_t*>(&h);
        }
        ROCWMMA_DEVICE inline void mma_atom_i8_i32_k8(int32_t (&acc)[8], uint32_t a, uint32_t b)
        {
            const uint32_t ah[2] = {i8pair_to_half2(a, 0), i8pair_to_half2(a, 16)};
            const uint32_t bh[2] = {i8pair_to_half2(b, 0), i8pair_to_half2(b, 16)};
            float          p[8]  = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+f"(p[0]), "+f"(p[1]), "+f"(p[2]), "+f"(p[3])
                         : "r"(ah[0]), "r"(ah[1]), "r"(bh[0]));
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+f"(p[4]), "+f"(p[5]), "+f"(p[6]), "+f"(p[7])
                         : "r"(ah[0]), "r"(ah[1]), "r"(bh[1]));
#pragma unroll
            for(int e = 0; e < 8; ++e)
                acc[e] += __float2int_rn(p[e]);
        }

        // OCP fp8 x fp8 -> fp32 (m16n8k16), same register orders as int8
        ROCWMMA_DEVICE inline void mma_atom_e4m3_f32(float (&acc)[8], const uint32_t (&a)[2], const uint32_t (&b)[2])
        {
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.e4m3.e4m3.f32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
                         : "r"(a[0]), "r"(a[1]), "r"(b[0]));
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.e4m3.e4m3.f32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+f"(acc[4]), "+f"(acc[5]), "+f"(acc[6]), "+f"(acc[7])
                         : "r"(a[0]), "r"(a[1]), "r"(b[1]));
        }
        ROCWMMA_DEVICE inline void mma_atom_e5m2_f32(float (&acc)[8], const uint32_t (&a)[2], const uint32_t (&b)[2])
        {
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.e5m2.e5m2.f32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
                         : "r"(a[0]), "r"(a[1]), "r"(b[0]));
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.e5m2.e5m2.f32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+f"(acc[4]), "+f"(acc[5]), "+f"(acc[6]), "+f"(acc[7])
                         : "r"(a[0]), "r"(a[1]), "r"(b[1]));
        }

        // fp64 (m16n8k4): a = 2 doubles, b = 2 doubles [n-half 0, n-half 1]
        ROCWMMA_DEVICE inline void mma_atom_f64(double (&acc)[8], const double (&a)[2], const double (&b)[2])
        {
            asm volatile("mma.sync.aligned.m16n8k4.row.col.f64.f64.f64.f64 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+d"(acc[0]), "+d"(acc[1]), "+d"(acc[2]), "+d"(acc[3])
                         : "d"(a[0]), "d"(a[1]), "d"(b[0]));
            asm volatile("mma.sync.aligned.m16n8k4.row.col.f64.f64.f64.f64 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+d"(acc[4]), "+d"(acc[5]), "+d"(acc[6]), "+d"(acc[7])
                         : "d"(a[0]), "d"(a[1]), "d"(b[1]));
        }

        // fp32 x fp32 -> fp32 on the tf32 tensor path with error compensation (3xTF32):
        // x = hi + lo with hi = tf32(x); acc += lo_a*hi_b + hi_a*lo_b + hi_a*hi_b.
        // The dropped lo*lo term is below 2^-22 relative, so results track an fp32 FMA chain.
        ROCWMMA_DEVICE inline uint32_t to_tf32(float x)
        {
            uint32_t r;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
            return r;
        }
        ROCWMMA_DEVICE inline void mma_tf32_1688(float* acc, const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
        {
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 "
                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
        }
        // a = 4 floats (16x8 atom), b = 4 floats ordered [k-lo n-half0, k-lo n-half1, k-hi n-half0, k-hi n-half1]
        ROCWMMA_DEVICE inline void mma_atom_f32(float (&acc)[8], const float (&a)[4], const float (&b)[4])
        {
            uint32_t ah[4], al[4], bh[4], bl[4];
#pragma unroll
            for(int i = 0; i < 4; ++i)
            {
                ah[i] = to_tf32(a[i]);
                al[i] = to_tf32(a[i] - __uint_as_float(ah[i]));
                bh[i] = to_tf32(b[i]);
                bl[i] = to_tf32(b[i] - __uint_as_float(bh[i]));
            }
            mma_tf32_1688(acc, al, bh[0], bh[2]);
            mma_tf32_1688(acc, ah, bl[0], bl[2]);
            mma_tf32_1688(acc, ah, bh[0], bh[2]);
            mma_tf32_1688(acc + 4, al, bh[1], bh[3]);
            mma_tf32_1688(acc + 4, ah, bl[1], bl[3]);
            mma_tf32_1688(acc + 4, ah, bh[1], bh[3]);
        }
        // xfloat32: one TF32 product per atom (inputs rounded to TF32, fp32 accumulate)
        ROCWMMA_DEVICE inline void mma_atom_xf32(float (&acc)[8], const float (&a)[4], const float (&b)[4])
        {
            uint32_t ah[4], bh[4];
#pragma unroll
            for(int i = 0; i < 4; ++i)
            {
                ah[i] = to_tf32(a[i]);
                bh[i] = to_tf32(b[i]);
            }
            mma_tf32_1688(acc, ah, bh[0], bh[2]);
            mma_tf32_1688(acc + 4, ah, bh[1], bh[3]);
        }

        // 4 deep (m16n8k4): a = 2 floats (rows g, g + 8 at k = t), b = 2 floats [n-half 0, n-half 1]
        ROCWMMA_DEVICE inline void mma_tf32_1684(float* acc, const uint32_t (&a)[2], uint32_t b0)
        {
            asm volatile("mma.sync.aligned.m16n8k4.row.col.f32.tf32.tf32.f32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
                         : "r"(a[0]), "r"(a[1]), "r"(b0));
        }
        ROCWMMA_DEVICE inline void mma_atom_f32_k4(float (&acc)[8], const float (&a)[2], const float (&b)[2])
        {
            uint32_t ah[2], al[2], bh[2], bl[2];
#pragma unroll
            for(int i = 0; i < 2; ++i)
            {
                ah[i] = to_tf32(a[i]);
                al[i] = to_tf32(a[i] - __uint_as_float(ah[i]));
                bh[i] = to_tf32(b[i]);
                bl[i] = to_tf32(b[i] - __uint_as_float(bh[i]));
            }
            mma_tf32_1684(acc, al, bh[0]);
            mma_tf32_1684(acc, ah, bl[0]);
            mma_tf32_1684(acc, ah, bh[0]);
            mma_tf32_1684(acc + 4, al, bh[1]);
            mma_tf32_1684(acc + 4, ah, bl[1]);
            mma_tf32_1684(acc + 4, ah, bh[1]);
        }
        // fp32, 2 deep: no such mma.sync shape.  A atom 16 x 2 and B atom 2 x 16 hold one element per lane (lane l: block
        // index l / 2, k = l % 2); every accumulator element fetches its two products' operands by shuffle and adds them
        // with FMAs in ascending k.  ROUND_TF32: the xfloat32_t form (inputs rounded to TF32 first).
        template <bool ROUND_TF32>
        ROCWMMA_DEVICE inline void mma_atom_f32_k2(float (&acc)[8], float a, float b)
        {
            if constexpr(ROUND_TF32)
            {
                a = __uint_as_float(to_tf32(a));
                b = __uint_as_float(to_tf32(b));
            }
            const uint32_t lane = threadIdx.x & 31u, g = lane >> 2, t = lane & 3u;
#pragma unroll
            for(uint32_t e = 0; e < 8; ++e)
            {
                const uint32_t row = g + 8u * ((e >> 1) & 1u), col = 2u * t + (e & 1u) + 8u * (e >> 2);
                const float    a0 = __shfl_sync(0xFFFFFFFFu, a, 2u * row), a1 = __shfl_sync(0xFFFFFFFFu, a, 2u * row + 1u);
                const float    b0 = __shfl_sync(0xFFFFFFFFu, b, 2u * col), b1 = __shfl_sync(0xFFFFFFFFu, b, 2u * col + 1u);
                acc[e]            = fmaf(a1, b1, fmaf(a0, b0, acc[e]));
            }
        }
        ROCWMMA_DEVICE inline void mma_atom_xf32_k4(float (&acc)[8], const float (&a)[2], const float (&b)[2])
        {
            const uint32_t ah[2] = {to_tf32(a[0]), to_tf32(a[1])};
            mma_tf32_1684(acc, ah, to_tf32(b[0]));
            mma_tf32_1684(acc + 4, ah, to_tf32(b[1]));
        }
    } // namespace detail
} // namespace rocwmma

#endif
