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

}  // namespace kdw
