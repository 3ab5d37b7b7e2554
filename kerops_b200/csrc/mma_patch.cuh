// Device helpers shared by the tensor-core (mma.sync) kernels in patch form: dwconv_fprop_mma.cu (forward) and
// dwconv_wgrad_mma.cu (weight gradient).
//
// Geometry common to both.  A warp works on a UNIT of 16 BLOCKS x 8 channels; a block is 2 x 2 output voxels
// (w, d), the blocks of a unit are 2 along w x 8 along d (4 x 16 voxels).  The outputs of a block depend on a PATCH
// of 4 x 4 input voxels of the same plane (patch row pw = 0..3 along w, column pd = 0..3 along d; output (ow, od)
// reads patch voxel (ow + b, od + t) through tap (b, t)).  With g = lane / 4 and t = lane % 4 the fragments of an
// m16n8k16 mma are laid out as: matrix row g <-> block (bw = 0, bd = g), row g + 8 <-> block (bw = 1, bd = g);
// a k pair (2t, 2t+1) <-> the two channels of one 32-bit word of patch voxel (pw, pd = t).
#pragma once
#include "kdw_common.cuh"

namespace kdw {

// Byte offset inside a 1024-byte aligned tile written by TMA with a swizzle span of SWZ bytes: the 16-byte chunk
// index within the span (address bits 4..) is XORed with the address bits from bit 7 up - 3 bits for 128, 2 for
// 64, 1 for 32.  With one voxel per span, the same chunk of 8 (and more) consecutive voxels lands in distinct
// banks, which is what makes the 16-byte loads of a quarter-warp conflict-free.
template <int SWZ>
KDW_HD uint32_t swz(uint32_t off) {
    return SWZ == 0 ? off : off ^ (((off >> 7) & (uint32_t)(SWZ / 16 - 1)) << 4);
}

// How a tile of the volume is staged in shared memory and which TMA boxes fill it.
//   MODE 0: 5-D tensor map (C, D, W, H, N), one box per tile and plane, rows of one voxel (2*CS bytes) with the
//           swizzle whose span is one voxel (none for 16-byte voxels).
//   MODE 1: C == CS == 8: tensor map with the d and c axes merged, (D*C, W, H, N), so that a box row is a run of
//           up to 32 voxels instead of 16 bytes - the TMA unit handles a fixed number of box rows per clock, and
//           16-byte rows cap a kernel at less than half the HBM rate.  The d range of a tile is cut into NBX boxes
//           staged one after the other: [box][w][KD][c].  16-byte voxels need no swizzle.
//   MODE 2: C == CS == 16 and D even: 5-D map whose innermost axis is a PAIR of voxels, (2*16, D/2, W, H, N):
//           64-byte rows with the 64-byte swizzle (conflict-free like MODE 0).  A tile then starts at an even d, one
//           voxel earlier than the stencil needs.
// "in" is the halo'd input tile of a plane ((WT+2) x DIN voxels, the tile's first voxel at (1, DPAD)), "out" the
// WT x DT tile of outputs (or of grad in the weight gradient).
template <int CS_, int WT_, int DT_, int MODE_>
struct TileGeo {
    static constexpr int CS = CS_, WT = WT_, DT = DT_, MODE = MODE_;
    static constexpr int VOXB = CS * 2;
    static constexpr int SWZ = MODE == 1 ? 0 : (MODE == 2 ? 64 : (CS == 8 ? 0 : VOXB));
    static constexpr int DPAD = MODE == 2 ? 2 : 1;
    static constexpr int DIN = DT + 2 * DPAD;  // MODE 2 stages one voxel more than needed at either end (whole pairs)
    static constexpr int NBX = MODE == 1 ? (DIN + 31) / 32 : 1;
    static constexpr int KD = (DIN + NBX - 1) / NBX;
    static constexpr int IN_BOX = ((WT + 2) * KD * VOXB + 127) / 128 * 128;  // bytes from one box to the next
    static constexpr int IN_BYTES = NBX * (WT + 2) * KD * VOXB;              // bytes the copies of a plane deliver
    static constexpr int IN_STRIDE = (NBX * IN_BOX + 1023) / 1024 * 1024;
    static constexpr int NBO = MODE == 1 ? (DT + 31) / 32 : 1;
    static constexpr int KDO = DT / NBO;
    static constexpr int OUT_BOX = WT * KDO * VOXB;
    static constexpr int OUT_BYTES = WT * DT * VOXB;
    static constexpr int OUT_STRIDE = (OUT_BYTES + 1023) / 1024 * 1024;
    static_assert(MODE == 0 || (MODE == 1 && CS == 8) || (MODE == 2 && CS == 16), "merged maps need CS == C");
    static_assert(DT % NBO == 0 && OUT_BOX % 128 == 0, "output boxes");
    static_assert(MODE != 1 || (KD * CS <= 256 && KDO * CS <= 256), "a box row holds at most 256 elements");
    static_assert(MODE != 2 || (DIN % 2 == 0 && DT % 2 == 0), "pairs of voxels");
    // byte offset (before the swizzle) of input voxel (row wr, column dd of the staged tile) / output voxel (wr, dd)
    KDW_HD static constexpr uint32_t in_off(int wr, int dd) {
        return (uint32_t)((dd / KD) * IN_BOX + (wr * KD + dd % KD) * VOXB);
    }
    KDW_HD static constexpr uint32_t out_off(int wr, int dd) {
        return (uint32_t)((dd / KDO) * OUT_BOX + (wr * KDO + dd % KDO) * VOXB);
    }
    // rows four apart in the input tile / two apart in the output tile differ by a constant that preserves the
    // swizzle phase
    static constexpr uint32_t IN_ROW4 = 4 * KD * VOXB, OUT_ROW2 = 2 * KDO * VOXB;
    static constexpr uint32_t SWZ_PERIOD = 8 * (SWZ ? SWZ : 1);
    static_assert(SWZ == 0 || (IN_ROW4 % SWZ_PERIOD == 0 && OUT_ROW2 % SWZ_PERIOD == 0), "row steps and swizzle phase");
};

// The copies of one input tile (plane q of sample n, tile origin (w0, d0), channel slice c0) into `dst`, all
// completing on `bar`; and the store of / the copy of one output-shaped tile.
template <class Geo>
__device__ __forceinline__ void tile_load_in(int* status, uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int d0,
                                             int w0, int q, int n) {
    if (Geo::MODE == 1) {
#pragma unroll
        for (int k = 0; k < Geo::NBX; ++k)
            tma_load_5d(status, dst + k * Geo::IN_BOX, tm, bar, (d0 - Geo::DPAD + k * Geo::KD) * Geo::CS, w0 - 1, q, n, 0);
    } else if (Geo::MODE == 2) {
        tma_load_5d(status, dst, tm, bar, 0, (d0 - Geo::DPAD) / 2, w0 - 1, q, n);
    } else {
        tma_load_5d(status, dst, tm, bar, c0, d0 - Geo::DPAD, w0 - 1, q, n);
    }
}
template <class Geo>
__device__ __forceinline__ void tile_load_out(int* status, uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0,
                                              int d0, int w0, int h, int n) {
    if (Geo::MODE == 1) {
#pragma unroll
        for (int k = 0; k < Geo::NBO; ++k)
            tma_load_5d(status, dst + k * Geo::OUT_BOX, tm, bar, (d0 + k * Geo::KDO) * Geo::CS, w0, h, n, 0);
    } else if (Geo::MODE == 2) {
        tma_load_5d(status, dst, tm, bar, 0, d0 / 2, w0, h, n);
    } else {
        tma_load_5d(status, dst, tm, bar, c0, d0, w0, h, n);
    }
}
template <class Geo>
__device__ __forceinline__ void tile_store_out(int* status, const CUtensorMap* tm, uint32_t src, int c0, int d0, int w0,
                                               int h, int n) {
    if (Geo::MODE == 1) {
#pragma unroll
        for (int k = 0; k < Geo::NBO; ++k)
            tma_store_5d(status, tm, src + k * Geo::OUT_BOX, (d0 + k * Geo::KDO) * Geo::CS, w0, h, n, 0);
    } else if (Geo::MODE == 2) {
        tma_store_5d(status, tm, src, 0, d0 / 2, w0, h, n);
    } else {
        tma_store_5d(status, tm, src, c0, d0, w0, h, n);
    }
}

// d = a * b + c (m16n8k16, fp16 operands, fp32 accumulate); ZERO: c = 0.  The four A registers and the four
// accumulator registers of an mma are register QUADS (consecutive registers) in the machine instruction, the two
// B registers a pair; Quad / the arrays below are laid out accordingly.
struct Quad {
    uint32_t r[4];
};
template <bool ZERO>
__device__ __forceinline__ void mma16816(float (&d)[4], const Quad& a, uint32_t b0, uint32_t b1) {
    if (ZERO) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
            "{%10, %10, %10, %10};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a.r[0]), "r"(a.r[1]), "r"(a.r[2]), "r"(a.r[3]), "r"(b0), "r"(b1), "f"(0.f));
    } else {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
            "{%0, %1, %2, %3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a.r[0]), "r"(a.r[1]), "r"(a.r[2]), "r"(a.r[3]), "r"(b0), "r"(b1));
    }
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ void st_shared_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_shared_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
// A register copy the assembler cannot remove: x ^ zero with `zero` a kernel argument that is always 0.  A 16-byte
// load delivers the four channel pairs of ONE voxel in a register quad, an mma wants the words of FOUR voxels for
// one channel pair in a quad: the 4 x 4 transpose between the two is 16 register copies per quad set, made ONCE
// per plane step - each copy is then used, in the same position of the same quad, by the three mma (a = 2, 1, 0)
// that read it.  (A plain move is folded away and the quads are then gathered again before every mma.)
__device__ __forceinline__ uint32_t reg_copy(uint32_t x, uint32_t zero) {
    uint32_t y;
    asm("xor.b32 %0, %1, %2;" : "=r"(y) : "r"(x), "r"(zero));
    return y;
}

// Two halves of two words in one register (PRMT with a constant selector): pair_lo(a, b) = (a.lo, b.lo) with a in
// the low half of the result, pair_hi(a, b) = (a.hi, b.hi) - the same channel of two voxels, out of channel-pair words.
__device__ __forceinline__ uint32_t pair_lo(uint32_t a, uint32_t b) {
    uint32_t y;
    asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(y) : "r"(a), "r"(b));
    return y;
}
__device__ __forceinline__ uint32_t pair_hi(uint32_t a, uint32_t b) {
    uint32_t y;
    asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(y) : "r"(a), "r"(b));
    return y;
}

// Transpose of an 8 x 8 matrix of 16-bit elements held one row per four lanes (lane (g, t): row g, columns 2t, 2t+1),
// the layout in which raw channels-last words arrive: rows = blocks, columns = (voxel t, channel of the pair).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}

// State of the thread that issues the copies, kept in shared memory so that it costs the consumer warps no registers.
struct ProdState {
    StepIter it;
    uint32_t pi;   // copies issued so far
    int done;      // end marker written, test hook reached, or a wait ran out
};

// Host: the tensor maps of a TileGeo over volume `base` (H planes); `in` selects the halo'd input box.
template <class Geo>
int encode_tile_map(CUtensorMap* map, const void* base, int64_t N, int64_t C, int64_t H, int64_t W, int64_t D,
                    int64_t sN, int64_t sH, int64_t sW, bool in, bool nan_fill = false) {
    if (Geo::MODE == 1) {
        if (C != Geo::CS) {
            set_error("this kernel variant needs C == %d", Geo::CS);
            return KDW_ERR_TUNE;
        }
        return encode_merged_map(map, base, N, C, H, W, D, sN, sH, sW, (in ? Geo::KD : Geo::KDO) * Geo::CS,
                                 in ? Geo::WT + 2 : Geo::WT, nan_fill);
    }
    if (Geo::MODE == 2) {
        if (C != Geo::CS || (D & 1)) {
            set_error("this kernel variant needs C == %d and an even D", Geo::CS);
            return KDW_ERR_TUNE;
        }
        return encode_paired_map(map, base, N, C, H, W, D, sN, sH, sW, (in ? Geo::DIN : Geo::DT) / 2,
                                 in ? Geo::WT + 2 : Geo::WT, nan_fill);
    }
    return encode_volume_map(map, base, N, C, H, W, D, sN, sH, sW, Geo::CS, in ? Geo::DIN : Geo::DT,
                             in ? Geo::WT + 2 : Geo::WT, nan_fill, Geo::SWZ);
}
}  // namespace kdw
