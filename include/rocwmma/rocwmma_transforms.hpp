// Fragment transforms: applyTranspose and applyDataLayout
// (reference: rocwmma_transforms.hpp:36-66, rocwmma_transforms_impl.hpp:54-306).
//
// applyTranspose(frag<matrix_a, BM, BN, BK, T, L>) is frag<matrix_b, BN, BM, BK, T, orthogonal(L)>
// and vice versa: the same registers seen as the transposed operand.  applyDataLayout changes
// only the memory layout tag.  Both are re-interpretations here because a fragment's register
// layout is independent of its data layout and matrix_b is laid out as the transpose of matrix_a
// (internal/layout.hpp); the WaveCount template argument of applyDataLayout is accepted for
// source compatibility and has no effect.  ApplyRegisterFile_t is the one transform that changes the shape: it
// names the raw register file of a fragment as a matrix of its own.
#ifndef ROCWMMA_B200_TRANSFORMS_API_HPP
#define ROCWMMA_B200_TRANSFORMS_API_HPP

#include "rocwmma.hpp"

namespace rocwmma
{
    namespace detail
    {
        template <typename FragT>
        struct TransposeOf;
        template <uint32_t BM, uint32_t BN, uint32_t BK, typename DataT, typename L>
        struct TransposeOf<fragment<matrix_a, BM, BN, BK, DataT, L>>
        {
            using type = fragment<matrix_b, BN, BM, BK, DataT, typename OrthoLayout<L>::type>;
        };
        template <uint32_t BM, uint32_t BN, uint32_t BK, typename DataT, typename L>
        struct TransposeOf<fragment<matrix_b, BM, BN, BK, DataT, L>>
        {
            using type = fragment<matrix_a, BN, BM, BK, DataT, typename OrthoLayout<L>::type>;
        };

        template <typename FragT, typename NewLayout>
        struct WithLayout;
        template <typename MatrixT, uint32_t BM, uint32_t BN, uint32_t BK, typename DataT, typename L,
                  typename NewLayout>
        struct WithLayout<fragment<MatrixT, BM, BN, BK, DataT, L>, NewLayout>
        {
            using type = fragment<MatrixT, BM, BN, BK, DataT, NewLayout>;
        };
    }

    template <typename FragT>
    using ApplyTranspose_t = typename detail::TransposeOf<std::decay_t<FragT>>::type;
    template <typename FragT, typename DataLayoutT>
    using ApplyDataLayout_t = typename detail::WithLayout<std::decay_t<FragT>, DataLayoutT>::type;
    // Register-file view of a fragment: its registers as a (registers per lane) x (warp size) matrix_b block, for
    // parking them in shared memory as they are (reference: rocwmma_transforms_impl.hpp:272-289).  Obtained by
    // reinterpret_cast of the fragment, as the reference's users do (test/gemm/gemm_local_mapping.hpp:417-434).
    template <typename FragT>
    using ApplyRegisterFile_t
        = fragment<matrix_b, 1u, Constants::AMDGCN_WAVE_SIZE, std::decay_t<FragT>::num_elements,
                   typename detail::FragInfo<std::decay_t<FragT>>::Data, typename detail::FragInfo<std::decay_t<FragT>>::Layout>;

    template <typename FragT>
    ROCWMMA_DEVICE inline ApplyTranspose_t<FragT> const& applyTranspose(FragT const& frag)
    {
        using Out = ApplyTranspose_t<FragT>;
        static_assert(sizeof(Out) == sizeof(FragT), "transpose must preserve the register footprint");
        return reinterpret_cast<Out const&>(frag);
    }
    template <typename FragT>
    ROCWMMA_DEVICE inline ApplyTranspose_t<FragT>& applyTranspose(FragT& frag)
    {
        using Out = ApplyTranspose_t<FragT>;
        return reinterpret_cast<Out&>(frag);
    }

    template <typename DataLayoutT, uint32_t WaveCount = 1, typename FragT>
    ROCWMMA_DEVICE inline ApplyDataLayout_t<FragT, DataLayoutT> const& applyDataLayout(FragT const& frag)
    {
        using Out = ApplyDataLayout_t<FragT, DataLayoutT>;
        static_assert(sizeof(Out) == sizeof(FragT), "data layout change must preserve the register footprint");
        return reinterpret_cast<Out const&>(frag);
    }
    template <typename DataLayoutT, uint32_t WaveCount = 1, typename FragT>
    ROCWMMA_DEVICE inline ApplyDataLayout_t<FragT, DataLayoutT>& applyDataLayout(FragT& frag)
    {
        using Out = ApplyDataLayout_t<FragT, DataLayoutT>;
        return reinterpret_cast<Out&>(frag);
    }
} // namespace rocwmma

#endif
