// Register layouts of fragments on 32-thread warps, and the 1-D data-space mappers.
//
// rocWMMA leaves the order of fragment elements unspecified ("vector elements have no
// guaranteed order or locality", library/include/rocwmma/rocwmma.hpp:126).  What user code
// relies on, and what holds here:
//   * accumulator fragments of one shape map element i to the same matrix coordinate for
//     every data type (so `d.x[i] = alpha * acc.x[i] + beta * c.x[i]` is element-wise);
//   * a fragment's register layout does not depend on its memory data layout, so
//     applyDataLayout is a re-interpretation;
//   * matrix_b<BN,BK> is the register-for-register transpose of matrix_a<BM=BN,BK>, so
//     applyTranspose is a re-interpretation as well;
//   * num_elements = BlockDim * BlockK / 32.
//
// A fragment is a grid of 16-row "atoms" shaped after the operands of NVIDIA's warp-level
// mma.sync instructions, so that mma_sync needs no shuffles:
//   element size   A atom (M x K)   instruction            per-lane elements
//   1 byte         16 x 16          m16n8k16 (s8)          (row g + 8*(i>>2),      col 4t + (i&3))
//                  16 x 8           m16n8k8 on fp16 copies (row g + 8*(i>>1),      col 2t + (i&1))   [int8, BlockK = 8]
//   2 bytes        16 x 16          m16n8k16 (f16, bf16)   (row g + 8*((i>>1)&1),  col 2t + (i&1) + 8*(i>>2))
//                  16 x 8           m16n8k8  (f16, bf16)   (row g + 8*(i>>1),      col 2t + (i&1))
//   4 bytes        16 x 8           m16n8k8  (tf32)        (row g + 8*(i&1),       col t + 4*(i>>1))
//                  16 x 4           m16n8k4  (tf32)        (row g + 8*i,           col t)
//                  16 x 2           shuffles + FMA         (row lane / 2,          col lane % 2)     [fp32, BlockK = 2]
//   8 bytes        16 x 4           m16n8k4  (f64)         (row g + 8*i,           col t)
// with g = lane / 4, t = lane % 4.  The deeper atom is used when BlockK is a multiple of it, the
// shallower one otherwise (BlockK = 8 for 8- and 16-bit types, 4 and 2 for fp32: the reference's minimum K of 32 x 32
// blocks, docs/api-reference/api-reference-guide.rst:100-146; there is no 8-deep int8 or 2-deep fp32 mma.sync shape, so
// those two multiply through exact fp16 copies on m16n8k8 resp. through shuffles and FMAs).  B atoms are the transposes (k takes the role of col, n of
// row).  Accumulator atoms are 16 x 16 = two m16n8 result tiles:
//   (row g + 8*((i>>1)&1), col 2t + (i&1) + 8*(i>>2)).
#ifndef ROCWMMA_B200_LAYOUT_HPP
#define ROCWMMA_B200_LAYOUT_HPP

#include "types.hpp"
#include "utils.hpp"

namespace rocwmma
{
    struct row_major
    {
    };
    struct col_major
    {
    };
    struct matrix_a
    {
    };
    struct matrix_b
    {
    };
    struct accumulator
    {
    };

    enum layout_t : uint32_t
    {
        mem_row_major,
        mem_col_major
    };

    // BLAS-style names of the data layouts (reference: internal/utils.hpp:312-323)
    template <>
    constexpr const char* dataTypeToString<row_major>()
    {
        return "T";
    }
    template <>
    constexpr const char* dataTypeToString<col_major>()
    {
        return "N";
    }

    namespace detail
    {
        // ---- 1-D data space (rocWMMA internal/mapping_util.hpp DataSpace) ---------------------
        template <typename DataOrientation>
        struct DataSpace
        {
            enum : uint32_t
            {
                MajorIndex = std::is_same<DataOrientation, row_major>::value ? 0 : 1,
                MinorIndex = std::is_same<DataOrientation, row_major>::value ? 1 : 0
            };
            using Orientation = DataOrientation;
            ROCWMMA_HOST_DEVICE constexpr static inline uint32_t leadingDim(Coord2d const& matrixSize)
            {
                return get<MinorIndex>(matrixSize);
            }
            ROCWMMA_HOST_DEVICE constexpr static inline uint32_t fromMatrixCoord(Coord2d const& c,
                                                                                 uint32_t       ld)
            {
                return get<MajorIndex>(c) * ld + get<MinorIndex>(c);
            }
        };
        template <>
        struct DataSpace<void>;
    } // namespace detail

    // 1-D array layouts by name (reference: internal/layout.hpp:36-44)
    namespace DataLayout
    {
        template <typename DataLayoutT>
        using Array1d = detail::DataSpace<DataLayoutT>;
        using RowMajor = Array1d<row_major>;
        using ColMajor = Array1d<col_major>;
    } // namespace DataLayout

    namespace detail
    {

        template <typename L>
        struct OrthoLayout;
        template <>
        struct OrthoLayout<row_major>
        {
            using type = col_major;
        };
        template <>
        struct OrthoLayout<col_major>
        {
            using type = row_major;
        };
        template <>
        struct OrthoLayout<void>
        {
            using type = void;
        };

        // ---- atom geometry by element size and BlockK -----------------------------------------
        // Depth of one input atom: the deepest mma.sync K that divides BlockK (0: shape not offered).
        template <uint32_t ElemBytes, uint32_t BK>
        struct AtomK;
        template <uint32_t BK>
        struct AtomK<1, BK>
        {
            static constexpr uint32_t value = BK % 16 == 0 ? 16 : (BK % 8 == 0 ? 8 : 0);
        };
        template <uint32_t BK>
        struct AtomK<2, BK>
        {
            static constexpr uint32_t value = BK % 16 == 0 ? 16 : (BK % 8 == 0 ? 8 : 0);
        };
        template <uint32_t BK>
        struct AtomK<4, BK>
        {
            static constexpr uint32_t value = BK % 8 == 0 ? 8 : (BK % 4 == 0 ? 4 : (BK % 2 == 0 ? 2 : 0));
        };
        template <uint32_t BK>
        struct AtomK<8, BK>
        {
            static constexpr uint32_t value = BK % 4 == 0 ? 4 : 0;
        };

        // Coordinates (dim, k) of element `i` of one input atom for lane (g, t); `dim` runs along
        // the 16-wide block dimension (rows of A / columns of B), `k` along the reduction.
        // `Run` = number of consecutive elements that are adjacent along k.
        template <uint32_t ElemBytes, uint32_t KA>
        struct InputAtom;
        template <>
        struct InputAtom<1, 16>
        {
            static constexpr uint32_t Elems = 8, Run = 4;
            ROCWMMA_DEVICE static inline void coord(uint32_t g, uint32_t t, uint32_t i, uint32_t& dim,
                                                    uint32_t& k)
            {
                dim = g + 8u * (i >> 2);
                k   = 4u * t + (i & 3u);
            }
        };
        template <>
        struct InputAtom<1, 8>
        {
            static constexpr uint32_t Elems = 4, Run = 2;
            ROCWMMA_DEVICE static inline void coord(uint32_t g, uint32_t t, uint32_t i, uint32_t& dim,
                                                    uint32_t& k)
            {
                dim = g + 8u * (i >> 1);
                k   = 2u * t + (i & 1u);
            }
        };
        template <>
        struct InputAtom<2, 16>
        {
            static constexpr uint32_t Elems = 8, Run = 2;
            ROCWMMA_DEVICE static inline void coord(uint32_t g, uint32_t t, uint32_t i, uint32_t& dim,
                                                    uint32_t& k)
            {
                dim = g + 8u * ((i >> 1) & 1u);
                k   = 2u * t + (i & 1u) + 8u * (i >> 2);
            }
        };
        template <>
        struct InputAtom<2, 8>
        {
            static constexpr uint32_t Elems = 4, Run = 2;
            ROCWMMA_DEVICE static inline void coord(uint32_t g, uint32_t t, uint32_t i, uint32_t& dim,
                                                    uint32_t& k)
            {
                dim = g + 8u * (i >> 1);
                k   = 2u * t + (i & 1u);
            }
        };
        template <>
        struct InputAtom<4, 8>
        {
            static constexpr uint32_t Elems = 4, Run = 1;
            ROCWMMA_DEVICE static inline void coord(uint32_t g, uint32_t t, uint32_t i, uint32_t& dim,
                                                    uint32_t& k)
            {
                dim = g + 8u * (i & 1u);
                k   = t + 4u * (i >> 1);
            }
        };
        template <>
        struct InputAtom<4, 4>
        {
            static constexpr uint32_t Elems = 2, Run = 1;
            ROCWMMA_DEVICE static inline void coord(uint32_t g, uint32_t t, uint32_t i, uint32_t& dim,
                                                    uint32_t& k)
            {
                dim = g + 8u * i;
                k   = t;
            }
        };
        template <>
        struct InputAtom<4, 2>
        {
            static constexpr uint32_t Elems = 1, Run = 1;
            ROCWMMA_DEVICE static inline void coord(uint32_t g, uint32_t t, uint32_t, uint32_t& dim, uint32_t& k)
            {
                const uint32_t lane = 4u * g + t;
                dim = lane >> 1;
                k   = lane & 1u;
            }
        };
        template <>
        struct InputAtom<8, 4>
        {
            static constexpr uint32_t Elems = 2, Run = 1;
            ROCWMMA_DEVICE static inline void coord(uint32_t g, uint32_t t, uint32_t i, uint32_t& dim,
                                                    uint32_t& k)
            {
                dim = g + 8u * i;
                k   = t;
            }
        };

        struct AccAtom
        {
            static constexpr uint32_t Elems = 8, Run = 2;
            ROCWMMA_DEVICE static inline void coord(uint32_t g, uint32_t t, uint32_t i, uint32_t& row,
                                                    uint32_t& col)
            {
                row = g + 8u * ((i >> 1) & 1u);
                col = 2u * t + (i & 1u) + 8u * (i >> 2);
            }
        };

        // Unit of a cooperative split: one 32-bit register's worth of elements (4 x 8-bit, 2 x 16-bit, 1 otherwise).
        // Warps sharing a fragment each move a contiguous range of its elements, a whole number of these units;
        // the rule depends only on the fragment's size and element type, so a fragment and any re-interpretation
        // of its registers (transpose, data layout, register file) are split identically.
        template <typename DataT>
        struct CoopUnit
        {
            static constexpr uint32_t value = sizeof(DataT) >= 4 ? 1u : 4u / sizeof(DataT);
        };

        // ---- whole-fragment geometry -----------------------------------------------------------
        // Gives, for each fragment kind: block height / width in matrix space, the atom grid and
        // the map  element index -> (row, col)  inside the block.  `RunAlongCol` says whether
        // consecutive elements of a run are adjacent along the column (true) or the row (false).
        template <typename MatrixT, uint32_t BM, uint32_t BN, uint32_t BK, typename DataT>
        struct FragGeometry;

        template <uint32_t BM, uint32_t BN, uint32_t BK, typename DataT>
        struct FragGeometry<matrix_a, BM, BN, BK, DataT>
        {
            static constexpr uint32_t KA = AtomK<sizeof(DataT), BK>::value;
            static_assert(KA != 0, "BlockK must be a multiple of the smallest atom depth "
                                   "(8 for 8- and 16-bit types, 2 for 32-bit, 4 for 64-bit)");
            using Atom = InputAtom<sizeof(DataT), KA>;
            static constexpr uint32_t BlockHeight = BM, BlockWidth = BK, BlockDim = BM, KDim = BK;
            static_assert(BM % 16 == 0, "matrix_a fragments need BlockM to be a multiple of 16");
            static constexpr uint32_t AtomsDim = BM / 16, AtomsK = BK / KA;
            static constexpr uint32_t Atoms = AtomsDim * AtomsK, AtomElems = Atom::Elems, Run = Atom::Run;
            static constexpr uint32_t Size = Atoms * AtomElems;
            static constexpr bool RunAlongCol = true;
            ROCWMMA_DEVICE static inline void coord(uint32_t lane, uint32_t atom, uint32_t i, uint32_t& row,
                                                    uint32_t& col)
            {
                uint32_t d, k;
                Atom::coord(lane >> 2, lane & 3u, i, d, k);
                row = (atom / AtomsK) * 16u + d;
                col = (atom % AtomsK) * KA + k;
            }
        };

        template <uint32_t BM, uint32_t BN, uint32_t BK, typename DataT>
        struct FragGeometry<matrix_b, BM, BN, BK, DataT>
        {
            static constexpr uint32_t KA = AtomK<sizeof(DataT), BK>::value;
            static_assert(KA != 0, "BlockK must be a multiple of the smallest atom depth "
                                   "(8 for 8- and 16-bit types, 2 for 32-bit, 4 for 64-bit)");
            using Atom = InputAtom<sizeof(DataT), KA>;
            static constexpr uint32_t BlockHeight = BK, BlockWidth = BN, BlockDim = BN, KDim = BK;
            static_assert(BN % 16 == 0, "matrix_b fragments need BlockN to be a multiple of 16");
            static constexpr uint32_t AtomsDim = BN / 16, AtomsK = BK / KA;
            static constexpr uint32_t Atoms = AtomsDim * AtomsK, AtomElems = Atom::Elems, Run = Atom::Run;
            static constexpr uint32_t Size = Atoms * AtomElems;
            static constexpr bool RunAlongCol = false; // runs are adjacent along k = along rows of B
            ROCWMMA_DEVICE static inline void coord(uint32_t lane, uint32_t atom, uint32_t i, uint32_t& row,
                                                    uint32_t& col)
            {
                uint32_t d, k;
                Atom::coord(lane >> 2, lane & 3u, i, d, k);
                row = (atom % AtomsK) * KA + k;
                col = (atom / AtomsK) * 16u + d;
            }
        };

        // Register-file view: fragment<matrix_b, 1, warp size, R, DataT> is R registers of one warp seen as an
        // R x 32 matrix, element i of lane l at (row i, col l) - the type ApplyRegisterFile_t produces
        // (reference: rocwmma_transforms_impl.hpp:272-289).  It exists to park any fragment's registers in
        // shared memory and to read them back into the same registers; BlockM = 1 marks it and it is not an
        // mma_sync operand.  One "atom" is one register row.
        template <uint32_t BN, uint32_t BK, typename DataT>
        struct FragGeometry<matrix_b, 1u, BN, BK, DataT>
        {
            static_assert(BN == Constants::AMDGCN_WAVE_SIZE, "A register file is as wide as the warp");
            static constexpr uint32_t BlockHeight = BK, BlockWidth = BN, BlockDim = BN, KDim = BK;
            static constexpr uint32_t Atoms = BK, AtomElems = 1, Run = 1, Size = BK;
            static constexpr bool     RunAlongCol = true;
            ROCWMMA_DEVICE static inline void coord(uint32_t lane, uint32_t atom, uint32_t, uint32_t& row,
                                                    uint32_t& col)
            {
                row = atom;
                col = lane;
            }
        };

        template <uint32_t BM, uint32_t BN, uint32_t BK, typename DataT>
        struct FragGeometry<accumulator, BM, BN, BK, DataT>
        {
            static constexpr uint32_t BlockHeight = BM, BlockWidth = BN, BlockDim = BM, KDim = BN;
            static_assert(BM % 16 == 0 && BN % 16 == 0,
                          "accumulator fragments need BlockM and BlockN to be multiples of 16");
            static constexpr uint32_t AtomsM = BM / 16, AtomsN = BN / 16;
            static constexpr uint32_t Atoms = AtomsM * AtomsN, AtomElems = AccAtom::Elems, Run = AccAtom::Run;
            static constexpr uint32_t Size = Atoms * AtomElems;
            static constexpr bool RunAlongCol = true;
            ROCWMMA_DEVICE static inline void coord(uint32_t lane, uint32_t atom, uint32_t i, uint32_t& row,
                                                    uint32_t& col)
            {
                uint32_t r, c;
                AccAtom::coord(lane >> 2, lane & 3u, i, r, c);
                row = (atom / AtomsN) * 16u + r;
                col = (atom % AtomsN) * 16u + c;
            }
        };
    } // namespace detail
} // namespace rocwmma

#endif
