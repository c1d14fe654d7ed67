// rocWMMA-compatible device API on NVIDIA warps (32 threads, mma.sync tensor-core instructions).
//
// Same names, template parameters and semantics as rocWMMA's public header
// (library/include/rocwmma/rocwmma.hpp:74-316): tags, layout_t, fragment, fill_fragment,
// load_matrix_sync, store_matrix_sync, mma_sync, synchronize_workgroup.  A kernel written against
// that header compiles against this one with nvcc for sm_100a; the "wave" is the CUDA warp
// (Constants::AMDGCN_WAVE_SIZE == 32) and blockDim.x must be a multiple of 32.
//
// Supported block shapes: BlockM, BlockN multiples of 16; BlockK a multiple of 8 for 8- and 16-bit
// inputs (OCP fp8: 16), 2 for fp32, 4 for fp64 - the reference's minimum K per type.  Supported mma_sync type pairs (input -> compute):
// float16_t/hfloat16_t -> float32_t or the input type, bfloat16_t -> float32_t or bfloat16_t,
// float8_t / bfloat8_t (OCP e4m3 / e5m2) -> float32_t, int8_t -> int32_t, xfloat32_t -> float32_t (one TF32
// product), float32_t -> float32_t (3xTF32), float64_t -> float64_t.
#ifndef ROCWMMA_B200_API_HPP
#define ROCWMMA_B200_API_HPP

#include "internal/config.hpp"
#include "internal/flow_control.hpp"
#include "internal/layout.hpp"
#include "internal/mapping_util.hpp"
#include "internal/mma_atoms.hpp"
#include "internal/types.hpp"
#include "internal/utils.hpp"

namespace rocwmma
{
    // ------------------------------------------------------------------------------------------
    // fragment  (reference: rocwmma.hpp:127-202)
    // ------------------------------------------------------------------------------------------
    template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT,
              typename DataLayoutT = void>
    class alignas(alignof(DataT) > 4 ? alignof(DataT) : 4) fragment
    {
    public:
        using Geometry = detail::FragGeometry<MatrixT, BlockM, BlockN, BlockK, DataT>;

        struct Traits
        {
            constexpr static uint32_t Size = Geometry::Size;
            using AccessT  = VecT<DataT, Size>;
            using StorageT = VecT<DataT, Size>;
            static_assert(Size * sizeof(DataT) >= 4, "Fragments must occupy at least one 32-bit register");
        };

        fragment() = default;

        ROCWMMA_DEVICE inline DataT& operator[](uint32_t index)
        {
            return x[index];
        }
        ROCWMMA_DEVICE inline DataT const& operator[](uint32_t index) const
        {
            return x[index];
        }
        ROCWMMA_DEVICE inline typename Traits::StorageT& operator*()
        {
            return mStorage;
        }
        ROCWMMA_DEVICE inline typename Traits::StorageT const& operator*() const
        {
            return mStorage;
        }

        ROCWMMA_HOST_DEVICE constexpr static inline uint32_t height()
        {
            return Geometry::BlockHeight;
        }
        ROCWMMA_HOST_DEVICE constexpr static inline uint32_t width()
        {
            return Geometry::BlockWidth;
        }
        ROCWMMA_HOST_DEVICE constexpr static inline uint32_t blockDim()
        {
            return Geometry::BlockDim;
        }
        ROCWMMA_HOST_DEVICE constexpr static inline uint32_t kDim()
        {
            return Geometry::KDim;
        }
        ROCWMMA_HOST_DEVICE constexpr static inline uint32_t size()
        {
            return Traits::Size;
        }

        union
        {
            typename Traits::StorageT mStorage;
            typename Traits::AccessT  mAccess;
            DataT                     x[Traits::Size];
        };

        constexpr static uint32_t num_elements = Traits::Size;
        using element_type                     = DataT;
    };

    // ---- fragment introspection used by kernels (reference: internal/api_fwd.hpp, io_shape.hpp) ----
    namespace detail
    {
        template <typename FragT>
        struct FragInfo;
        template <typename MatrixT, uint32_t BM, uint32_t BN, uint32_t BK, typename DataT, typename LayoutT>
        struct FragInfo<fragment<MatrixT, BM, BN, BK, DataT, LayoutT>>
        {
            using Matrix   = MatrixT;
            using Data     = DataT;
            using Layout   = LayoutT;
            using Geometry = FragGeometry<MatrixT, BM, BN, BK, DataT>;
            static constexpr uint32_t BlockM = BM, BlockN = BN, BlockK = BK;
        };

        template <typename Geometry_>
        struct IOShape
        {
            enum : uint32_t
            {
                BlockHeight = Geometry_::BlockHeight,
                BlockWidth  = Geometry_::BlockWidth,
                BlockDim    = Geometry_::BlockDim,
                KDim        = Geometry_::KDim
            };
        };
    }
    template <typename FragT>
    using GetIOShape_t = detail::IOShape<typename detail::FragInfo<std::decay_t<FragT>>::Geometry>;
    template <typename FragT>
    using GetDataLayout_t = detail::DataSpace<typename detail::FragInfo<std::decay_t<FragT>>::Layout>;
    template <typename FragT>
    using GetDataType_t = typename detail::FragInfo<std::decay_t<FragT>>::Data;
    // MappingUtil of a fragment's block shape, data type and data layout (reference: internal/accessors.hpp:89)
    template <typename FragT>
    using GetMappingUtil_t = MappingUtil<GetIOShape_t<FragT>::BlockHeight, GetIOShape_t<FragT>::BlockWidth,
                                         GetDataType_t<FragT>, typename detail::FragInfo<std::decay_t<FragT>>::Layout>;

    // Cooperative IO configuration of a fragment shared by WaveCount warps (reference: internal/accessors.hpp:59,
    // internal/io_traits.hpp:61).  IOTraits::IOCount is the number of independent IO steps the whole fragment
    // takes: here the number of 32-bit register units per lane, the unit the cooperative loads and stores deal out
    // to the warps.  It depends only on the fragment's size and element type, so the IOCounts of a global-read
    // fragment and of its shared-memory-write view (transposed, re-laid-out or as a register file) are equal and
    // always have a common divisor (what user code asserts on).
    namespace detail
    {
        template <typename FragT, uint32_t WaveCount>
        struct CoopIOConfig
        {
            struct IOTraits
            {
                enum : uint32_t
                {
                    IOCount = FragInfo<FragT>::Geometry::Size / CoopUnit<typename FragInfo<FragT>::Data>::value
                };
            };
        };
    }
    template <typename FragT, uint32_t WaveCount = 1u>
    using GetCoopIOConfig_t = detail::CoopIOConfig<std::decay_t<FragT>, WaveCount>;

    // ------------------------------------------------------------------------------------------
    // fill_fragment  (reference: rocwmma.hpp:217-219, rocwmma_impl.hpp:204-217)
    // ------------------------------------------------------------------------------------------
    template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void fill_fragment(fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>& frag,
                                             DataT value)
    {
#pragma unroll
        for(uint32_t i = 0; i < frag.num_elements; ++i)
            frag.x[i] = value;
    }

    namespace detail
    {
        template <uint32_t Bytes>
        struct RawVec;
        template <>
        struct RawVec<2>
        {
            using type = unsigned short;
        };
        template <>
        struct RawVec<4>
        {
            using type = uint32_t;
        };
        template <>
        struct RawVec<8>
        {
            using type = uint2;
        };
        template <>
        struct RawVec<16>
        {
            using type = uint4;
        };

        // ---- whole-matrix moves of 16-bit atoms ------------------------------------------------
        // A 16-bit atom is two (16 x 8) or four (16 x 16, accumulators included) 8 x 8 matrices in exactly the
        // register order of ldmatrix / stmatrix: matrix j is the atom's elements 2j, 2j + 1 of every lane, thread
        // (g, t) holding its entries (g, 2t) and (g, 2t + 1) with rows along the atom's block dimension and columns
        // along k.  So an atom moves to or from SHARED memory in one instruction: plain when memory is contiguous
        // along k, .trans when it is contiguous along the block dimension (the stored 8 x 8 tiles then have their
        // rows along k).  In GLOBAL memory the second case is the expensive one for per-lane accesses (eight
        // 2-byte accesses per atom); there each lane moves the 32-bit word it would own in the transposed tile
        // and movmatrix swaps the tile across the warp.
        template <typename Geometry, typename DataT>
        struct MatrixAtoms
        {
            static constexpr uint32_t Mats = (sizeof(DataT) == 2 && Geometry::Run == 2)
                                                 ? (Geometry::AtomElems == 8 ? 4u : (Geometry::AtomElems == 4 ? 2u : 0u))
                                                 : 0u;
        };
        ROCWMMA_DEVICE inline uint32_t movmatrix_trans(uint32_t w)
        {
            uint32_t r;
            asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(w));
            return r;
        }
        template <uint32_t Mats, bool Trans>
        ROCWMMA_DEVICE inline void ldmatrix_atom(uint32_t* r, uint32_t saddr)
        {
            if constexpr(Mats == 4 && !Trans)
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr) : "memory");
            else if constexpr(Mats == 4)
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr) : "memory");
            else if constexpr(!Trans)
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];"
                             : "=r"(r[0]), "=r"(r[1]) : "r"(saddr) : "memory");
            else
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                             : "=r"(r[0]), "=r"(r[1]) : "r"(saddr) : "memory");
        }
        template <uint32_t Mats, bool Trans>
        ROCWMMA_DEVICE inline void stmatrix_atom(const uint32_t* r, uint32_t saddr)
        {
            if constexpr(Mats == 4 && !Trans)
                asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%4], {%0,%1,%2,%3};" ::"r"(r[0]), "r"(r[1]), "r"(r[2]),
                             "r"(r[3]), "r"(saddr) : "memory");
            else if constexpr(Mats == 4)
                asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%4], {%0,%1,%2,%3};" ::"r"(r[0]), "r"(r[1]),
                             "r"(r[2]), "r"(r[3]), "r"(saddr) : "memory");
            else if constexpr(!Trans)
                asm volatile("stmatrix.sync.aligned.m8n8.x2.shared.b16 [%2], {%0,%1};" ::"r"(r[0]), "r"(r[1]), "r"(saddr) : "memory");
            else
                asm volatile("stmatrix.sync.aligned.m8n8.x2.trans.shared.b16 [%2], {%0,%1};" ::"r"(r[0]), "r"(r[1]), "r"(saddr)
                             : "memory");
        }

        // One whole 16-bit atom between registers and memory through the instructions above.  Returns false (and moves
        // nothing) when the addresses do not allow it; every lane of the warp takes the same branch (mem, ldm are
        // warp-uniform arguments of the *_sync functions).
        template <bool IsLoad, bool ColMajorMem, typename Geometry, typename DataT>
        ROCWMMA_DEVICE inline bool move_matrix_atom(DataT* atom_regs, DataT* mem, uint32_t ldm, uint32_t atom, uint32_t lane)
        {
            // atom_regs: the AtomElems registers that hold (or receive) atom `atom` of the fragment
            constexpr uint32_t Mats  = MatrixAtoms<Geometry, DataT>::Mats;
            constexpr bool     Trans = Geometry::RunAlongCol == ColMajorMem; // memory is contiguous along the block dimension
            const uintptr_t    base  = reinterpret_cast<uintptr_t>(mem);
            const uintptr_t    pitch = static_cast<uintptr_t>(ldm) * sizeof(DataT);
            uint32_t*          r32   = reinterpret_cast<uint32_t*>(atom_regs);
            const auto offset_of = [&](uint32_t syn_lane, uint32_t syn_elem) {
                uint32_t row, col;
                Geometry::coord(syn_lane, atom, syn_elem, row, col);
                return ColMajorMem ? static_cast<size_t>(col) * ldm + row : static_cast<size_t>(row) * ldm + col;
            };
            if(__isShared(mem) && ((base | pitch) & 15u) == 0u)
            {
                // lane l gives the address of row (l % 8) of matrix (l / 8); lanes beyond the last matrix repeat valid ones
                const uint32_t j = (lane >> 3) % Mats, rr = lane & 7u;
                // plain: row rr = (block-dimension index rr, k 0..7) of the matrix; .trans: stored row rr = (k index rr)
                const size_t off = Trans ? offset_of(rr >> 1, 2u * j + (rr & 1u)) : offset_of(rr << 2, 2u * j);
                const uint32_t saddr = static_cast<uint32_t>(__cvta_generic_to_shared(mem + off));
                if constexpr(IsLoad)
                    ldmatrix_atom<Mats, Trans>(r32, saddr);
                else
                    stmatrix_atom<Mats, Trans>(r32, saddr);
                return true;
            }
            if constexpr(Trans)
            {
                if(((base | pitch) & 3u) == 0u)
                {
                    // the word this lane owns in the transposed tile: (k index g, block-dimension indices 2t, 2t + 1)
                    const uint32_t g = lane >> 2, t = lane & 3u;
#pragma unroll
                    for(uint32_t j = 0; j < Mats; ++j)
                    {
                        uint32_t* word = reinterpret_cast<uint32_t*>(mem + offset_of(((2u * t) << 2) | (g >> 1), 2u * j + (g & 1u)));
                        if constexpr(IsLoad)
                            r32[j] = movmatrix_trans(*word);
                        else
                            *word = movmatrix_trans(r32[j]);
                    }
                    return true;
                }
            }
            return false;
        }

        // Moves the elements [elemBegin, elemBegin + count) of a fragment between memory and the registers
        // regs[0 .. count): register r holds element elemBegin + r.  A whole-fragment move has elemBegin = 0 and
        // count = Size (constants: the loops below then fold to straight-line code with constant register numbers and
        // atom coordinates); a cooperative move passes the warp's slice, which therefore always sits in the FIRST
        // registers of the warp's fragment whatever the wave index - only addresses depend on it.
        // ColMajorMem selects the memory layout.  When consecutive register elements are adjacent in memory (Run > 1
        // and the run direction is the contiguous memory direction) and the addresses are suitably aligned, a run
        // moves as one 2..16-byte access; 16-bit atoms that lie wholly inside the range move as 8 x 8 matrices.
        // RunAligned: elemBegin and count are multiples of the run length.  Cooperative slices are whole 32-bit register
        // units, which is a whole run for 8- and 16-bit types; a slice of a 32- or 64-bit accumulator (runs of two) may
        // start or end inside a run, and is then moved element by element.
        template <bool IsLoad, bool ColMajorMem, typename Geometry, typename DataT, bool RunAligned = true>
        ROCWMMA_DEVICE inline void move_atoms(DataT* regs, DataT* mem, uint32_t ldm, uint32_t elemBegin, uint32_t count)
        {
            const uint32_t     lane       = threadIdx.x & 31u;
            constexpr uint32_t Run        = RunAligned ? Geometry::Run : 1u;
            constexpr uint32_t AE         = Geometry::AtomElems;
            constexpr bool     contiguous = (Run > 1) && (Geometry::RunAlongCol != ColMajorMem);
            constexpr uint32_t VecBytes   = contiguous ? Run * sizeof(DataT) : sizeof(DataT);
            bool               vec_ok     = false;
            if constexpr(contiguous)
                vec_ok = ((reinterpret_cast<uintptr_t>(mem) | (static_cast<uintptr_t>(ldm) * sizeof(DataT)))
                          % VecBytes)
                         == 0;
#pragma unroll
            for(uint32_t chunk = 0; chunk < Geometry::Atoms; ++chunk) // registers [chunk * AE, (chunk + 1) * AE)
            {
                const uint32_t r0 = chunk * AE;
                if(r0 >= count)
                    continue; // (no early exit: the loops must stay fully unrolled for the registers to stay registers)
                if constexpr(MatrixAtoms<Geometry, DataT>::Mats != 0)
                {
                    // a 16-bit atom wholly inside the range: one matrix instruction (or word moves + movmatrix)
                    const uint32_t e0 = elemBegin + r0;
                    if(e0 % AE == 0u && r0 + AE <= count)
                        if(move_matrix_atom<IsLoad, ColMajorMem, Geometry, DataT>(regs + r0, mem, ldm, e0 / AE, lane))
                            continue;
                }
#pragma unroll
                for(uint32_t ri = 0; ri < AE; ri += Run)
                {
                    const uint32_t r = r0 + ri; // first register of this run
                    if(r >= count)
                        continue;
                    const uint32_t e = elemBegin + r, atom = e / AE, i = e % AE;
                    DataT*         rp = regs + r;
                    if constexpr(contiguous)
                    {
                        uint32_t row, col;
                        Geometry::coord(lane, atom, i, row, col);
                        const size_t off = ColMajorMem ? static_cast<size_t>(col) * ldm + row
                                                       : static_cast<size_t>(row) * ldm + col;
                        if(vec_ok)
                        {
                            // staged through a correctly aligned temporary: the fragment itself is
                            // only 4-byte aligned
                            using V = typename RawVec<VecBytes>::type;
                            V      tmp;
                            DataT* tp = reinterpret_cast<DataT*>(&tmp);
                            if constexpr(IsLoad)
                            {
                                tmp = *reinterpret_cast<const V*>(mem + off);
#pragma unroll
                                for(uint32_t j = 0; j < Run; ++j)
                                    rp[j] = tp[j];
                            }
                            else
                            {
#pragma unroll
                                for(uint32_t j = 0; j < Run; ++j)
                                    tp[j] = rp[j];
                                *reinterpret_cast<V*>(mem + off) = tmp;
                            }
                        }
                        else
                        {
#pragma unroll
                            for(uint32_t j = 0; j < Run; ++j)
                            {
                                if constexpr(IsLoad)
                                    rp[j] = mem[off + j];
                                else
                                    mem[off + j] = rp[j];
                            }
                        }
                    }
                    else
                    {
#pragma unroll
                        for(uint32_t j = 0; j < Run; ++j)
                        {
                            uint32_t rr, cc;
                            Geometry::coord(lane, atom, i + j, rr, cc);
                            const size_t off = ColMajorMem ? static_cast<size_t>(cc) * ldm + rr
                                                           : static_cast<size_t>(rr) * ldm + cc;
                            if constexpr(IsLoad)
                                rp[j] = mem[off];
                            else
                                mem[off] = rp[j];
                        }
                    }
                }
            }
        }
    } // namespace detail

    // ------------------------------------------------------------------------------------------
    // load_matrix_sync  (reference: rocwmma.hpp:235-253, rocwmma_impl.hpp:225-264)
    // ------------------------------------------------------------------------------------------
    template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void load_matrix_sync(fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>& frag,
                                                const DataT* data, uint32_t ldm)
    {
        static_assert(!std::is_same<DataLayoutT, void>::value,
                      "Must provide layout information. Either statically assign data layout in "
                      "fragment declaration or use the run-time function overload.");
        using G = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>::Geometry;
        detail::move_atoms<true, std::is_same<DataLayoutT, col_major>::value, G, DataT>(
            frag.x, const_cast<DataT*>(data), ldm, 0u, G::Size);
    }

    template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT>
    ROCWMMA_DEVICE inline void load_matrix_sync(fragment<MatrixT, BlockM, BlockN, BlockK, DataT>& frag,
                                                const DataT* data, uint32_t ldm, layout_t layout)
    {
        using G = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT>::Geometry;
        if(layout == layout_t::mem_row_major)
            detail::move_atoms<true, false, G, DataT>(frag.x, const_cast<DataT*>(data), ldm, 0u, G::Size);
        else
            detail::move_atoms<true, true, G, DataT>(frag.x, const_cast<DataT*>(data), ldm, 0u, G::Size);
    }

    // ------------------------------------------------------------------------------------------
    // store_matrix_sync  (reference: rocwmma.hpp:269-288, rocwmma_impl.hpp:272-312)
    // Writes exactly the BlockHeight x BlockWidth block and nothing around it.
    // ------------------------------------------------------------------------------------------
    template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void
        store_matrix_sync(DataT* data, fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT> const& frag,
                          uint32_t ldm)
    {
        static_assert(!std::is_same<DataLayoutT, void>::value,
                      "Must provide data layout. Either statically assign data layout in "
                      "fragment declaration or use the run-time function overload.");
        using G = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>::Geometry;
        detail::move_atoms<false, std::is_same<DataLayoutT, col_major>::value, G, DataT>(
            const_cast<DataT*>(frag.x), data, ldm, 0u, G::Size);
    }

    template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT>
    ROCWMMA_DEVICE inline void store_matrix_sync(DataT* data,
                                                 fragment<MatrixT, BlockM, BlockN, BlockK, DataT> const& frag,
                                                 uint32_t ldm, layout_t layout)
    {
        using G = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT>::Geometry;
        if(layout == layout_t::mem_row_major)
            detail::move_atoms<false, false, G, DataT>(const_cast<DataT*>(frag.x), data, ldm, 0u, G::Size);
        else
            detail::move_atoms<false, true, G, DataT>(const_cast<DataT*>(frag.x), data, ldm, 0u, G::Size);
    }

    // ------------------------------------------------------------------------------------------
    // mma_sync  (reference: rocwmma.hpp:309-313, rocwmma_impl.hpp:323-364)
    // d = a x b + c over the whole BlockK; c may alias d.  fp16 compute (ComputeT = float16_t)
    // accumulates in fp32 and rounds to fp16 once per call, as the reference's MFMA path does
    // (internal/mfma_impl.hpp:82-114).
    // ------------------------------------------------------------------------------------------
    namespace detail
    {
        template <typename InputT, typename ComputeT>
        struct MmaAtomOp;

        // exec<KA>: one input atom of depth KA (the fragment geometry's choice for its BlockK)
        template <typename InputT>
        struct MmaF16Common
        {
            using AccT = float;
            template <uint32_t KA>
            ROCWMMA_DEVICE static inline void exec(float (&acc)[8], const InputT* a, const InputT* b)
            {
                if constexpr(KA == 16)
                    mma_atom_f16_f32(acc, *reinterpret_cast<const uint32_t(*)[4]>(a),
                                     *reinterpret_cast<const uint32_t(*)[4]>(b));
                else
                    mma_atom_f16_f32_k8(acc, *reinterpret_cast<const uint32_t(*)[2]>(a),
                                        *reinterpret_cast<const uint32_t(*)[2]>(b));
            }
        };
        template <>
        struct MmaAtomOp<float16_t, float32_t> : MmaF16Common<float16_t>
        {
        };
        template <>
        struct MmaAtomOp<float16_t, float16_t> : MmaF16Common<float16_t>
        {
        };
        template <>
        struct MmaAtomOp<hfloat16_t, float32_t> : MmaF16Common<hfloat16_t>
        {
        };
        template <>
        struct MmaAtomOp<hfloat16_t, hfloat16_t> : MmaF16Common<hfloat16_t>
        {
        };
        struct MmaBf16Common
        {
            using AccT = float;
            template <uint32_t KA>
            ROCWMMA_DEVICE static inline void exec(float (&acc)[8], const bfloat16_t* a, const bfloat16_t* b)
            {
                if constexpr(KA == 16)
                    mma_atom_bf16_f32(acc, *reinterpret_cast<const uint32_t(*)[4]>(a),
                                      *reinterpret_cast<const uint32_t(*)[4]>(b));
                else
                    mma_atom_bf16_f32_k8(acc, *reinterpret_cast<const uint32_t(*)[2]>(a),
                                         *reinterpret_cast<const uint32_t(*)[2]>(b));
            }
        };
        template <>
        struct MmaAtomOp<bfloat16_t, float32_t> : MmaBf16Common
        {
        };
        template <>
        struct MmaAtomOp<bfloat16_t, bfloat16_t> : MmaBf16Common
        {
        };
        template <>
        struct MmaAtomOp<int8_t, int32_t>
        {
            using AccT = int32_t;
            template <uint32_t KA>
            ROCWMMA_DEVICE static inline void exec(int32_t (&acc)[8], const int8_t* a, const int8_t* b)
            {
                if constexpr(KA == 16)
                    mma_atom_i8_i32(acc, *reinterpret_cast<const uint32_t(*)[2]>(a),
                                    *reinterpret_cast<const uint32_t(*)[2]>(b));
                else
                    mma_atom_i8_i32_k8(acc, *reinterpret_cast<const uint32_t*>(a), *reinterpret_cast<const uint32_t*>(b));
            }
        };
        template <>
        struct MmaAtomOp<float8_t, float32_t>
        {
            using AccT = float;
            template <uint32_t KA>
            ROCWMMA_DEVICE static inline void exec(float (&acc)[8], const float8_t* a, const float8_t* b)
            {
                mma_atom_e4m3_f32(acc, *reinterpret_cast<const uint32_t(*)[2]>(a),
                                  *reinterpret_cast<const uint32_t(*)[2]>(b));
            }
        };
        template <>
        struct MmaAtomOp<bfloat8_t, float32_t>
        {
            using AccT = float;
            template <uint32_t KA>
            ROCWMMA_DEVICE static inline void exec(float (&acc)[8], const bfloat8_t* a, const bfloat8_t* b)
            {
                mma_atom_e5m2_f32(acc, *reinterpret_cast<const uint32_t(*)[2]>(a),
                                  *reinterpret_cast<const uint32_t(*)[2]>(b));
            }
        };
        template <>
        struct MmaAtomOp<xfloat32_t, float32_t>
        {
            using AccT = float;
            template <uint32_t KA>
            ROCWMMA_DEVICE static inline void exec(float (&acc)[8], const xfloat32_t* a, const xfloat32_t* b)
            {
                if constexpr(KA == 8)
                    mma_atom_xf32(acc, *reinterpret_cast<const float(*)[4]>(a), *reinterpret_cast<const float(*)[4]>(b));
                else if constexpr(KA == 4)
                    mma_atom_xf32_k4(acc, *reinterpret_cast<const float(*)[2]>(a),
                                     *reinterpret_cast<const float(*)[2]>(b));
                else
                    mma_atom_f32_k2<true>(acc, *reinterpret_cast<const float*>(a), *reinterpret_cast<const float*>(b));
            }
        };
        template <>
        struct MmaAtomOp<float64_t, float64_t>
        {
            using AccT = double;
            template <uint32_t KA>
            ROCWMMA_DEVICE static inline void exec(double (&acc)[8], const double* a, const double* b)
            {
                mma_atom_f64(acc, *reinterpret_cast<const double(*)[2]>(a),
                             *reinterpret_cast<const double(*)[2]>(b));
            }
        };
        template <>
        struct MmaAtomOp<float32_t, float32_t>
        {
            using AccT = float;
            template <uint32_t KA>
            ROCWMMA_DEVICE static inline void exec(float (&acc)[8], const float* a, const float* b)
            {
                if constexpr(KA == 8)
                    mma_atom_f32(acc, *reinterpret_cast<const float(*)[4]>(a),
                                 *reinterpret_cast<const float(*)[4]>(b));
                else if constexpr(KA == 4)
                    mma_atom_f32_k4(acc, *reinterpret_cast<const float(*)[2]>(a),
                                    *reinterpret_cast<const float(*)[2]>(b));
                else
                    mma_atom_f32_k2<false>(acc, *a, *b);
            }
        };
    } // namespace detail

    template <uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename InputT, typename ComputeT,
              typename LayoutA, typename LayoutB, typename LayoutC, typename LayoutD>
    ROCWMMA_DEVICE inline void mma_sync(fragment<accumulator, BlockM, BlockN, BlockK, ComputeT, LayoutD>&       d,
                                        fragment<matrix_a, BlockM, BlockN, BlockK, InputT, LayoutA> const&      a,
                                        fragment<matrix_b, BlockM, BlockN, BlockK, InputT, LayoutB> const&      b,
                                        fragment<accumulator, BlockM, BlockN, BlockK, ComputeT, LayoutC> const& c)
    {
        using Op = detail::MmaAtomOp<InputT, ComputeT>;
        using AccT = typename Op::AccT;
        using GA = detail::FragGeometry<matrix_a, BlockM, BlockN, BlockK, InputT>;
        using GB = detail::FragGeometry<matrix_b, BlockM, BlockN, BlockK, InputT>;
        using GC = detail::FragGeometry<accumulator, BlockM, BlockN, BlockK, ComputeT>;
        static_assert(GA::AtomsK == GB::AtomsK, "A and B K dimensions must match");

#pragma unroll
        for(uint32_t mi = 0; mi < GC::AtomsM; ++mi)
        {
#pragma unroll
            for(uint32_t ni = 0; ni < GC::AtomsN; ++ni)
            {
                const uint32_t cbase = (mi * GC::AtomsN + ni) * 8u;
                AccT           acc[8];
#pragma unroll
                for(uint32_t e = 0; e < 8; ++e)
                    acc[e] = static_cast<AccT>(c.x[cbase + e]);
#pragma unroll
                for(uint32_t ki = 0; ki < GA::AtomsK; ++ki)
                    Op::template exec<GA::KA>(acc, a.x + (mi * GA::AtomsK + ki) * GA::AtomElems,
                             b.x + (ni * GB::AtomsK + ki) * GB::AtomElems);
#pragma unroll
                for(uint32_t e = 0; e < 8; ++e)
                    d.x[cbase + e] = static_cast<ComputeT>(acc[e]);
            }
        }
    }

    // ------------------------------------------------------------------------------------------
    // synchronize_workgroup  (reference: rocwmma.hpp:316, rocwmma_impl.hpp:366-369)
    // ------------------------------------------------------------------------------------------
    ROCWMMA_DEVICE inline void synchronize_workgroup()
    {
        __syncthreads();
    }
} // namespace rocwmma

#endif // ROCWMMA_B200_API_HPP
