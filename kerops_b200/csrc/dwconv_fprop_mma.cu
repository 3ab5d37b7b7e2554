// Depthwise 3x3x3 forward pass on the tensor cores (warp-level mma.sync.m16n8k16), fp32 accumulation.
//
// Replaces kerops/kernels/dw_conv.py:5-142 (_DWConv_cl3d_impl), like fprop_tma_kernel (dwconv_fprop.cu), whose
// column march, TMA input ring and plane-by-plane accumulation it shares.  Only the arithmetic differs: the 27
// multiply-adds per output leave the FMA pipe, which caps every CUDA-core formulation of this operator at 0.84 of
// the HBM roofline on B200, and become small matrix products.
//
// Patch formulation.  Outputs are grouped in BLOCKS of 2 x 2 voxels (w, d); with one input plane, the outputs of
// a block depend on a PATCH of 4 x 4 input voxels.  For one pair of channels (c0, c1) - one 32-bit word of a
// channels-last voxel - and one of the three output planes an input plane feeds (a = 0, 1, 2):
//     D[block, (out, cc')] += sum_{slot, cc}  A[block, (slot, cc)] * B[(slot, cc), (out, cc')]
//     A[block, (slot, cc)]  = x[patch voxel `slot` of the block, channel c_cc]     a raw word of the staged tile
//     B[(slot, cc), (out, cc')] = weight[a][b][t][c_cc'] if cc == cc' and slot - out is the tap (b, t), else 0
// i.e. M = 16 blocks, K = 16 slots x 2 channels (two k16 steps), N = 4 outputs x 2 channels.  The A fragment of a
// thread is a word it loads itself (one 16-byte load per voxel serves four channel pairs), the B fragments depend
// only on the weights and stay in registers, and the D fragment of a thread is (block, out, both channels) - a
// half2 of the output voxel - so nothing is shuffled or transposed.  27 of 96 multiply-adds are useful, against 1/8
// for a block-diagonal formulation over 8 channels; with the tensor pipe at about 1000 multiply-adds per clock per
// SM that leaves room for the full HBM rate.  fp16 x fp16 products are exact and sums are fp32 (KDW_ACC_F32).
//
// Per-channel form (PCfg::PERCH, used by the 64-channel-slice tiles).  The same patches with K = the 16 slots of ONE
// channel and N = 4 outputs x 2 LANES, the two lanes of an accumulator being two output planes: one mma per channel
// adds the a = 2 taps to the lane that finishes with this step and the a = 1 taps to the other lane; the finished
// lane is rounded, staged and cleared, and a second mma starts the next plane in it with the a = 0 taps (the other
// lane's columns of that B are zero).  From step to step the lanes swap roles; the B fragments exist for both
// assignments and the step is instantiated twice.  16 instead of 24 mma per unit and plane (27 of 64 products
// useful); the A fragment wants two SLOTS of one channel in a word, which is one PRMT from the words of two voxels -
// the same count as the register copies of the channel-pair form.  Measured in one call on one GPU: equal within
// 1 % in bursts of five launches, 4 % faster at C = 64 and 128 in runs of 300 launches, where the kernels sit at
// the board's power limit and the saved tensor-pipe work buys SM clock; equal or slower on the narrower tiles.
//
// A warp owns a UNIT: 16 blocks (2 along w x 8 along d, i.e. 4 x 16 voxels) x 8 channels.  Per input plane it
// reads 6 voxel rows with 16-byte loads (shared memory is laid out with the TMA swizzle whose span is one voxel, which makes
// the loads of a quarter-warp hit distinct banks) and issues 24 mma on two sets of fp32 accumulators that swap roles
// from step to step (finishing plane / middle plane), as in fprop_step_f32 - or, in the per-channel form, 16 mma on
// one set whose lanes swap roles.  Finished planes are staged in shared
// memory and leave through ONE TMA store per CTA and plane, issued by a dedicated warp; all hand-overs are
// mbarriers with bounded waits.
#include "../../include/kdw.h"
#include "kdw_common.cuh"
#include "mma_patch.cuh"

namespace kdw {

template <int CS_, int WW_, int WD_, int UPW_, int ST_, int MODE_ = 0, int PERCH_ = 0, int PRO_ = 0, int EPI_ = 0>
struct PCfg {
    static constexpr int CS = CS_;    // channels per CTA slice (8 .. 64)
    static constexpr int WW = WW_;    // units along w
    static constexpr int WD = WD_;    // units along d
    static constexpr int UPW = UPW_;  // units (along w) per warp; they share the weight fragments
    static constexpr int ST = ST_;    // input pipeline stages
    static constexpr int PERCH = PERCH_;  // 1: per-channel form (16 mma per unit and plane), 0: channel-pair form (24)
    // 1: fused prologue y = conv(relu(x * scale[c] + shift[c])) with scale / shift rounded to fp16 (one packed-half
    // fused multiply-add and a maximum per channel-pair word as it arrives from shared memory).  The input tensor map
    // then fills out-of-bounds elements with NaN, NaN survives the multiply-add, and max(NaN, 0) = 0 restores the zero
    // padding of the ACTIVATED tensor without masks.
    static constexpr int PRO = PRO_;  // 2: the same prologue in fp32 (the reference operator's own arithmetic: fp32
                                      // multiply-add from the fp32 scale / shift, maximum, one rounding to fp16)
    // 1: fused epilogue out = fp16(conv) + residual with per-channel sums of out and out^2 (kdw_fprop_addstats_f16).
    // A stage then also carries the residual tile of the plane the step finishes; the consumer threads add it to the
    // rounded outputs before staging them and accumulate the stored values in fp32; the sums leave the CTA through one
    // workspace row per (CTA, consumer warp), added by a second pass in a fixed order (no atomics).
    static constexpr int EPI = EPI_;
    // Rows 4 and 5 of a warp's first unit are rows 0 and 1 of its second: kept in registers instead of loaded twice
    // where that measured faster (+3.5 % at C = 32, +1 % at C = 8; not with the per-channel form, whose registers are
    // all taken, nor on the paired-voxel tiles).
    static constexpr bool SHARE_ROWS = PERCH_ == 0 && MODE_ != 2;
    static constexpr int NG = CS / 8;  // channel groups of 8 (one 16-byte chunk of a voxel)
    static constexpr int NCW = NG * (WW / UPW) * WD;  // consumer warps
    static constexpr int NT = NCW * 32;
    // Warps 0-3 form the helper warpgroup (warp 0 loads, warp 1 stores, 2 and 3 leave at once), the consumer warps
    // follow.  The kernel is compiled for 168 registers per thread (12 warps); the helper warpgroup then hands
    // registers back (setmaxnreg) and the two consumer warpgroups take them, which this kernel needs: with 168 the
    // weight fragments and accumulators spill and every mma drags register moves along.
    static constexpr int NHELP = 4;
    static constexpr int NTHREADS = NT + NHELP * 32;
    static constexpr int REGS_HELPER = 40, REGS_CONSUMER = 232;
    static constexpr int WT = 4 * WW;
    static constexpr int DT = 16 * WD;
    using Geo = TileGeo<CS, WT, DT, MODE_>;  // staging of the tiles in shared memory and their TMA boxes
    static constexpr int VOXB = Geo::VOXB;
    static constexpr int SWZ = Geo::SWZ;
    static constexpr int IN_BYTES = Geo::IN_BYTES, IN_STRIDE = Geo::IN_STRIDE;
    static constexpr int OUT_BYTES = Geo::OUT_BYTES, OUT_STRIDE = Geo::OUT_STRIDE;
    static constexpr int SMEM =
        ST * IN_STRIDE + 2 * OUT_STRIDE + (EPI_ ? ST * OUT_STRIDE + 8 * ST + 16 : 0) + 16 * ST + 32 + 4 * ST + 256 + 1024;
    static_assert(CS == 8 || CS == 16 || CS == 32 || CS == 64, "a voxel must be one swizzle span (or 16 bytes)");
    static_assert(WW % UPW == 0, "units per warp");
    static_assert(NCW == 8, "register hand-over is laid out for two consumer warpgroups");
    static_assert(NTHREADS <= 1024, "thread count");
    static_assert(DT + 4 <= 256 && WT + 2 <= 256, "TMA box limits");
};

// One input plane of one unit.  X[r] = the thread's voxel of input row r (r = 0..5: rows w-1 .. w+4 of the unit),
// four channel-pair words each.  FIN completes plane q-1 with the a=2 taps (written to the staging tile when
// `store`), MID takes plane q's a=1 taps, then FIN restarts as plane q+1 with the a=0 taps.
// Fragment roles (g = lane / 4, t = lane % 4): A rows g / g+8 are the blocks (bw = 0 / 1, bd = g); the k16 step ks
// covers the patch rows pw = 2ks (k 0-7: slot t) and 2ks+1 (k 8-15), patch column pd = t, i.e. the A quad of
// (ks, channel pair) is the word of input rows 2ks, 2ks+2, 2ks+1, 2ks+3.
// Consecutive mma never touch the same accumulator, so they issue back to back.
template <class Cfg, class Emit>
__device__ __forceinline__ void pg_step(const uint4 (&X)[6], const uint32_t (&Bf)[4][3][2][2], float (&FIN)[4][4],
                                        float (&MID)[4][4], bool store, Emit&& emit, uint32_t zero) {
    Quad Q[2][4];
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
        Q[ks][0].r[0] = reg_copy(X[2 * ks].x, zero), Q[ks][0].r[1] = reg_copy(X[2 * ks + 2].x, zero);
        Q[ks][0].r[2] = reg_copy(X[2 * ks + 1].x, zero), Q[ks][0].r[3] = reg_copy(X[2 * ks + 3].x, zero);
        Q[ks][1].r[0] = reg_copy(X[2 * ks].y, zero), Q[ks][1].r[1] = reg_copy(X[2 * ks + 2].y, zero);
        Q[ks][1].r[2] = reg_copy(X[2 * ks + 1].y, zero), Q[ks][1].r[3] = reg_copy(X[2 * ks + 3].y, zero);
        Q[ks][2].r[0] = reg_copy(X[2 * ks].z, zero), Q[ks][2].r[1] = reg_copy(X[2 * ks + 2].z, zero);
        Q[ks][2].r[2] = reg_copy(X[2 * ks + 1].z, zero), Q[ks][2].r[3] = reg_copy(X[2 * ks + 3].z, zero);
        Q[ks][3].r[0] = reg_copy(X[2 * ks].w, zero), Q[ks][3].r[1] = reg_copy(X[2 * ks + 2].w, zero);
        Q[ks][3].r[2] = reg_copy(X[2 * ks + 1].w, zero), Q[ks][3].r[3] = reg_copy(X[2 * ks + 3].w, zero);
    }
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
#pragma unroll
        for (int cp = 0; cp < 4; ++cp) mma16816<false>(FIN[cp], Q[ks][cp], Bf[cp][2][ks][0], Bf[cp][2][ks][1]);
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
#pragma unroll
        for (int cp = 0; cp < 4; ++cp) mma16816<false>(MID[cp], Q[ks][cp], Bf[cp][1][ks][0], Bf[cp][1][ks][1]);
    if (store) {
        uint4 o0, o1;  // block row g: outputs (t>>1, t&1) of block (bw=0); row g+8: the same of block (bw=1)
        o0.x = pack_h2(FIN[0][0], FIN[0][1]);
        o0.y = pack_h2(FIN[1][0], FIN[1][1]);
        o0.z = pack_h2(FIN[2][0], FIN[2][1]);
        o0.w = pack_h2(FIN[3][0], FIN[3][1]);
        o1.x = pack_h2(FIN[0][2], FIN[0][3]);
        o1.y = pack_h2(FIN[1][2], FIN[1][3]);
        o1.z = pack_h2(FIN[2][2], FIN[2][3]);
        o1.w = pack_h2(FIN[3][2], FIN[3][3]);
        emit(o0, o1);
    }
#pragma unroll
    for (int cp = 0; cp < 4; ++cp) mma16816<true>(FIN[cp], Q[0][cp], Bf[cp][0][0][0], Bf[cp][0][0][1]);
#pragma unroll
    for (int cp = 0; cp < 4; ++cp) mma16816<false>(FIN[cp], Q[1][cp], Bf[cp][0][1][0], Bf[cp][0][1][1]);
}

// The per-channel form of the same step.  Q[c] = the accumulators of channel c: elements 0 / 1 are the two lanes of
// block row g (bw = 0), elements 2 / 3 those of block row g+8 (bw = 1); FL = the lane that finishes with this step.
// k = 2t + j + 8h is the slot (patch row pw = j + 2h, patch column pd = t), so the A quad of a channel is (rows 0,1),
// (rows 2,3), (rows 2,3), (rows 4,5) of the thread's voxel column; B column n = 2 out + lane; D element
// (g, 2t + lane) is output out = t (ow = t >> 1, od = t & 1) of block (bw, g), as in the channel-pair form.
template <int FL, class Emit>
__device__ __forceinline__ void pg_step_ch(const uint4 (&X)[6], const uint32_t (&B21)[2][8][2],
                                           const uint32_t (&B0)[2][8][2], float (&Q)[8][4], bool store, Emit&& emit) {
    Quad A[8];
#pragma unroll
    for (int cp = 0; cp < 4; ++cp) {
        const uint32_t x0 = (&X[0].x)[cp], x1 = (&X[1].x)[cp], x2 = (&X[2].x)[cp];
        const uint32_t x3 = (&X[3].x)[cp], x4 = (&X[4].x)[cp], x5 = (&X[5].x)[cp];
        A[2 * cp].r[0] = pair_lo(x0, x1), A[2 * cp].r[1] = pair_lo(x2, x3);
        A[2 * cp].r[2] = pair_lo(x2, x3), A[2 * cp].r[3] = pair_lo(x4, x5);
        A[2 * cp + 1].r[0] = pair_hi(x0, x1), A[2 * cp + 1].r[1] = pair_hi(x2, x3);
        A[2 * cp + 1].r[2] = pair_hi(x2, x3), A[2 * cp + 1].r[3] = pair_hi(x4, x5);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) mma16816<false>(Q[c], A[c], B21[FL][c][0], B21[FL][c][1]);
    if (store) {
        uint4 o0, o1;  // the finished lane: block (bw=0) in elements 0/1, block (bw=1) in elements 2/3
        o0.x = pack_h2(Q[0][FL], Q[1][FL]);
        o0.y = pack_h2(Q[2][FL], Q[3][FL]);
        o0.z = pack_h2(Q[4][FL], Q[5][FL]);
        o0.w = pack_h2(Q[6][FL], Q[7][FL]);
        o1.x = pack_h2(Q[0][2 + FL], Q[1][2 + FL]);
        o1.y = pack_h2(Q[2][2 + FL], Q[3][2 + FL]);
        o1.z = pack_h2(Q[4][2 + FL], Q[5][2 + FL]);
        o1.w = pack_h2(Q[6][2 + FL], Q[7][2 + FL]);
        emit(o0, o1);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        Q[c][FL] = 0.f, Q[c][2 + FL] = 0.f;  // the lane starts its next plane
        mma16816<false>(Q[c], A[c], B0[FL][c][0], B0[FL][c][1]);
    }
}

// Schedule position of the store warp, kept in shared memory like ProdState (the helper warps run on 40 registers).
struct StoreState {
    StepIter it;
};

// Issues the copy of the next input plane (or the end marker) into the next stage, waiting for the stage to be
// free.  The position in the schedule lives in shared memory (ProdState).
template <class Cfg>
__device__ __forceinline__ void pg_produce(ProdState* ps, const Sched& s, const CUtensorMap& tmx, const CUtensorMap& tmr,
                                           uint32_t in0, uint32_t res0, uint32_t full0, uint32_t empty0, uint32_t desc0,
                                           uint32_t lim0, int W, int D, int* status, const WaitTest& wt) {
    constexpr int ST = Cfg::ST;
    const uint32_t pi = ps->pi;
    if (wt.stop_after >= 0 && (int)pi >= wt.stop_after) {  // test hook: the consumers' wait runs out
        ps->done = 1;
        return;
    }
    const uint32_t st = pi % ST;
    if (pi >= ST && !mbar_wait_bounded(empty0 + 8 * st, ((pi / ST) & 1u) ^ 1u, wt.limit_ns)) {
        atomicExch(status, (int)KDW_STATUS_TMA_TIMEOUT);
        const uint32_t first = pi > ST ? pi - ST : 0;  // copies in flight still target this CTA's shared memory
        for (uint32_t k = first; k < pi; ++k) (void)mbar_wait_bounded(full0 + 8 * (k % ST), (k / ST) & 1u, wt.limit_ns);
        ps->done = 1;
        return;
    }
    StepIter it = ps->it;
    if (!it.active) {  // end marker: completes the stage's barrier without a copy
        st_shared_u32(desc0 + 4 * st, 0xffffffffu);
        mbar_arrive(full0 + 8 * st);
        ps->done = 1;
        return;
    }
    const bool fin = it.q - 1 >= it.g.hb;  // the step finishes a plane the segment owns
    st_shared_u32(desc0 + 4 * st, ((uint32_t)it.g.c0 << 8) | (fin ? 1u : 0u));
    if (Cfg::EPI) {  // how much of the tile lies inside the volume (the statistics skip the rest)
        st_shared_u32(lim0 + 8 * st, (uint32_t)(W - it.g.w0));
        st_shared_u32(lim0 + 8 * st + 4, (uint32_t)(D - it.g.d0));
    }
    mbar_expect_tx(full0 + 8 * st, Cfg::IN_BYTES + (Cfg::EPI && fin ? Cfg::OUT_BYTES : 0));
    tile_load_in<typename Cfg::Geo>(status, in0 + st * Cfg::IN_STRIDE, &tmx, full0 + 8 * st, it.g.c0, it.g.d0, it.g.w0, it.q,
                                    it.g.n);
    if (Cfg::EPI && fin)
        tile_load_out<typename Cfg::Geo>(status, res0 + st * Cfg::OUT_STRIDE, &tmr, full0 + 8 * st, it.g.c0, it.g.d0,
                                         it.g.w0, it.q - 1, it.g.n);
    it.next(s);
    ps->it = it;
    ps->pi = pi + 1;
}

// Stores every finished plane of the CTA's range: waits until all consumer warps have staged it, issues the TMA
// store, and hands the staging tile back once the store has read it.
template <class Cfg>
__device__ __forceinline__ void pg_store(StoreState* ss, const Sched& s, const CUtensorMap& tmy, uint32_t out0,
                                         uint32_t staged0, uint32_t ofree0, int y_h0, int* status, const WaitTest& wt) {
    StepIter it = ss->it;
    uint32_t oc = 0;
    while (it.active) {
        if (it.q - 1 >= it.g.hb) {
            const uint32_t b = oc & 1u;
            if (!mbar_wait_bounded(staged0 + 8 * b, (oc >> 1) & 1u, wt.limit_ns)) {
                atomicExch(status, (int)KDW_STATUS_TMA_TIMEOUT);
                break;
            }
            tile_store_out<typename Cfg::Geo>(status, &tmy, out0 + b * Cfg::OUT_STRIDE, it.g.c0, it.g.d0, it.g.w0,
                                              it.q - 1 - y_h0, it.g.n);
            tma_commit();
            tma_wait_read_all();  // the store has read the tile: the consumers may overwrite it
            mbar_arrive(ofree0 + 8 * b);
            ++oc;
        }
        it.next(s);
    }
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NTHREADS, 1)
    fprop_pg_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmy,
                    const __grid_constant__ CUtensorMap tmr, float* __restrict__ stats_ws, const int W, const int D,
                    const __half* __restrict__ weight, const float* __restrict__ bn_scale,
                    const float* __restrict__ bn_shift, const Sched s, const int C, const int y_h0, int* status,
                    const WaitTest wt) {
    constexpr int ST = Cfg::ST, NCW = Cfg::NCW, UPW = Cfg::UPW;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
    const uint32_t in0 = base;
    const uint32_t out0 = base + ST * Cfg::IN_STRIDE;
    const uint32_t res0 = out0 + 2 * Cfg::OUT_STRIDE;   // epilogue only: the residual tile of each stage
    const uint32_t full0 = res0 + (Cfg::EPI ? ST * Cfg::OUT_STRIDE : 0);  // full[ST], empty[ST], staged[2], ofree[2]
    const uint32_t empty0 = full0 + 8 * ST;
    const uint32_t staged0 = empty0 + 8 * ST;
    const uint32_t ofree0 = staged0 + 16;
    // desc[ST]: what the consumers need to know about the plane in a stage, written by the load warp before the
    // copy is issued: bit 0 = this step finishes an owned plane (store it), bits 8.. = first channel of the slice;
    // -1 = no more planes.  The consumer warps so never decode the schedule themselves.
    const uint32_t desc0 = ofree0 + 16;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        prefetch_tmap(&tmx);
        prefetch_tmap(&tmy);
        if (Cfg::EPI) prefetch_tmap(&tmr);
        for (int k = 0; k < ST; ++k) {
            mbar_init(full0 + 8 * k, 1);
            mbar_init(empty0 + 8 * k, NCW);
        }
        for (int k = 0; k < 2; ++k) {
            mbar_init(staged0 + 8 * k, NCW);
            mbar_init(ofree0 + 8 * k, 1);
        }
        mbar_fence_init();
    }
    __syncthreads();  // the only CTA-wide barrier

    const uint32_t lim0 = (desc0 + 4 * ST + 15) / 16 * 16;  // epilogue only: (w, d) extent of the tile inside the volume
    ProdState* ps = reinterpret_cast<ProdState*>(smem_raw + ((lim0 + (Cfg::EPI ? 8 * ST : 0) + 15) / 16 * 16 - smem_u32(smem_raw)));
    StoreState* ss = reinterpret_cast<StoreState*>(reinterpret_cast<unsigned char*>(ps) + 128);
    if (warp == 0 && lane == 0) {
        ps->it.init(s, (int)blockIdx.x, (int)gridDim.x);
        ps->pi = 0;
        ps->done = 0;
    }
    if (warp == 1 && lane == 0) {
        ss->it.init(s, (int)blockIdx.x, (int)gridDim.x);
    }
    __syncwarp();
    if (warp < Cfg::NHELP) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Cfg::REGS_HELPER));
        if (lane != 0) return;
        if (warp == 0) {
            // ---------------- load warp: one lane streams the input planes of the CTA's range ----------------
            while (!ps->done) pg_produce<Cfg>(ps, s, tmx, tmr, in0, res0, full0, empty0, desc0, lim0, W, D, status, wt);
        } else if (warp == 1) {
            // ---------------- store warp: one TMA store per finished plane of the tile ----------------
            pg_store<Cfg>(ss, s, tmy, out0, staged0, ofree0, y_h0, status, wt);
            tma_wait_all();
        }
        return;
    }
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Cfg::REGS_CONSUMER));

    // ---------------- consumer warps ----------------
    const int cw = warp - Cfg::NHELP;
    const int ng = cw % Cfg::NG;                // channel group
    const int uwg = (cw / Cfg::NG) % (Cfg::WW / UPW);  // group of UPW units along w
    const int ud = cw / (Cfg::NG * (Cfg::WW / UPW));
    const int g = lane >> 2, t = lane & 3;
    // Shared-memory offsets of this thread's voxels.  Input row r of unit u: w index 4*(uwg*UPW+u) + r, d index
    // 16*ud + 2g + t; output voxel k of unit u: w index 4*(uwg*UPW+u) + 2k + (t>>1), d index 16*ud + 2g + (t&1).
    // Rows four apart (and units, and the two output rows) differ by a whole number of swizzle periods, so their
    // offsets differ by a constant: four input offsets and one output offset are kept in registers.
    using Geo = typename Cfg::Geo;
    constexpr uint32_t IN_ROW4 = Geo::IN_ROW4, OUT_ROW2 = Geo::OUT_ROW2;
    uint32_t in_off[4], out_off;
#pragma unroll
    for (int r = 0; r < 4; ++r)
        in_off[r] = swz<Cfg::SWZ>(Geo::in_off(4 * uwg * UPW + r, Geo::DPAD - 1 + 16 * ud + 2 * g + t) + 16 * ng);
    out_off = swz<Cfg::SWZ>(Geo::out_off(4 * uwg * UPW + (t >> 1), 16 * ud + 2 * g + (t & 1)) + 16 * ng);

    uint32_t ci = 0, oc = 0;
    int cur_c0 = -1;
    __half2 sc16[4], sh16[4];  // prologue only: scale / shift of the thread's four channel pairs,
    float2 sc32[4], sh32[4];   // rounded to fp16 (PRO == 1) or as given (PRO == 2); the unused set costs no registers
    // epilogue only: sums of the stored values and of their squares, per channel pair of the thread; the warp's own
    // workspace row [2][C] (sums, sums of squares), zeroed here and added to when the channel slice changes / at the end
    float2 ssum[4], ssq[4];
    float* const srow = Cfg::EPI ? stats_ws + (size_t)((int)blockIdx.x * NCW + cw) * 2 * C : nullptr;
    const int w_t = 4 * uwg * UPW + (t >> 1), d_t = 16 * ud + 2 * g + (t & 1);  // the thread's first output voxel
    if (Cfg::EPI) {
        for (int k = lane; k < 2 * C; k += 32) srow[k] = 0.f;
#pragma unroll
        for (int cp = 0; cp < 4; ++cp) ssum[cp] = ssq[cp] = make_float2(0.f, 0.f);
        __syncwarp();
    }
    auto flush_stats = [&](int c0) {  // all lanes of a warp hold the same eight channels
#pragma unroll
        for (int cp = 0; cp < 4; ++cp) {
            float v[4] = {ssum[cp].x, ssum[cp].y, ssq[cp].x, ssq[cp].y};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v[i] += __shfl_xor_sync(0xffffffffu, v[i], off);
            }
            if (lane == 0) {
                const int c = c0 + 8 * ng + 2 * cp;
                srow[c] += v[0], srow[c + 1] += v[1], srow[C + c] += v[2], srow[C + c + 1] += v[3];
            }
            ssum[cp] = ssq[cp] = make_float2(0.f, 0.f);
        }
    };
    // One plane step, common to both forms: `rebuild(c0)` loads the weight fragments of a new channel slice,
    // `unit(u, X, store, emit)` applies the plane to unit u and, when `store`, hands the two finished, rounded voxels of
    // the thread to `emit`, which (adds the residual and counts them, then) stages them.  Returns false when the warp is done (no more planes, or a wait ran out).
    auto plane_step = [&](auto&& rebuild, auto&& unit) -> bool {
        const uint32_t st = ci % ST;
        const bool ok = mbar_wait_bounded(full0 + 8 * st, (ci / ST) & 1u, wt.limit_ns);
        if (__any_sync(0xffffffffu, !ok)) {
            if (lane == 0) atomicExch(status, (int)KDW_STATUS_TMA_TIMEOUT);
            return false;
        }
        const uint32_t dsc = ld_shared_u32(desc0 + 4 * st);
        if (dsc == 0xffffffffu) return false;  // the load warp has no more planes
        const int c0 = (int)(dsc >> 8);
        if (c0 != cur_c0) {
            if (Cfg::EPI && cur_c0 >= 0) flush_stats(cur_c0);
            cur_c0 = c0;
            rebuild(c0);
            if (Cfg::PRO) {
#pragma unroll
                for (int cp = 0; cp < 4; ++cp) {
                    const int c = c0 + 8 * ng + 2 * cp;
                    sc32[cp] = make_float2(bn_scale[c], bn_scale[c + 1]);
                    sh32[cp] = make_float2(bn_shift[c], bn_shift[c + 1]);
                    sc16[cp] = __float22half2_rn(sc32[cp]);
                    sh16[cp] = __float22half2_rn(sh32[cp]);
                }
            }
        }
        const bool store = (dsc & 1u) != 0;  // this step finishes a plane the segment owns
        const uint32_t stage = in0 + st * Cfg::IN_STRIDE;
        int w_lim = 0, d_lim = 0;
        if (Cfg::EPI) w_lim = (int)ld_shared_u32(lim0 + 8 * st), d_lim = (int)ld_shared_u32(lim0 + 8 * st + 4);
        const uint32_t ob = out0 + (oc & 1u) * Cfg::OUT_STRIDE;
        if (store && oc >= 2) {  // the store that last read this staging tile must have finished
            const bool free_ok = mbar_wait_bounded(ofree0 + 8 * (oc & 1u), ((oc >> 1) - 1u) & 1u, wt.limit_ns);
            if (__any_sync(0xffffffffu, !free_ok)) {
                if (lane == 0) atomicExch(status, (int)KDW_STATUS_TMA_TIMEOUT);
                return false;
            }
        }
        uint4 XN[2];  // SHARE_ROWS: rows 4 and 5 of a unit = rows 0 and 1 of the next one, loaded (and activated) once
#pragma unroll
        for (int u = 0; u < UPW; ++u) {
            uint4 X[6];
            const int r0 = (u == 0 || !Cfg::SHARE_ROWS) ? 0 : 2;  // first row this unit loads itself
            if (r0) X[0] = XN[0], X[1] = XN[1];
#pragma unroll
            for (int r = 0; r < 6; ++r)
                if (r >= r0) X[r] = lds128(stage + in_off[r & 3] + (uint32_t)((r >> 2) + u) * IN_ROW4);
            if (u == UPW - 1) {
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * st);  // the values are in registers: the stage can be refilled
            }
            if (Cfg::PRO) {
#pragma unroll
                for (int r = 0; r < 6; ++r) {
                    if (r < r0) continue;
                    __half2* xw = reinterpret_cast<__half2*>(&X[r]);
#pragma unroll
                    for (int cp = 0; cp < 4; ++cp) {
                        if (Cfg::PRO == 2) {
                            float2 f = __half22float2(xw[cp]);
                            f.x = fmaxf(fmaf(f.x, sc32[cp].x, sh32[cp].x), 0.f);  // fmaxf(NaN, 0) = 0
                            f.y = fmaxf(fmaf(f.y, sc32[cp].y, sh32[cp].y), 0.f);
                            xw[cp] = __float22half2_rn(f);
                        } else {
                            xw[cp] = h2_relu_nan0(h2_fma(xw[cp], sc16[cp], sh16[cp]));
                        }
                    }
                }
            }
            if (Cfg::SHARE_ROWS && u + 1 < UPW) XN[0] = X[4], XN[1] = X[5];
            unit(u, X, store, [&](uint4 o0, uint4 o1) {
                const uint32_t a0 = out_off + u * 2 * OUT_ROW2, a1 = out_off + (u * 2 + 1) * OUT_ROW2;
                if (Cfg::EPI) {
                    const uint32_t rs = res0 + st * Cfg::OUT_STRIDE;
                    const uint4 r0 = lds128(rs + a0), r1 = lds128(rs + a1);
                    __half2* h0 = reinterpret_cast<__half2*>(&o0);
                    __half2* h1 = reinterpret_cast<__half2*>(&o1);
                    const __half2* q0 = reinterpret_cast<const __half2*>(&r0);
                    const __half2* q1 = reinterpret_cast<const __half2*>(&r1);
                    // voxels of the tile that lie outside the volume are not stored (the TMA store clips them) and
                    // must not be counted
                    const bool in0 = d_t < d_lim && w_t + 4 * u < w_lim, in1 = d_t < d_lim && w_t + 4 * u + 2 < w_lim;
                    const __half2 one = __float2half2_rn(1.f);
#pragma unroll
                    for (int cp = 0; cp < 4; ++cp) {
                        h0[cp] = __hadd2(h0[cp], q0[cp]);
                        h1[cp] = __hadd2(h1[cp], q1[cp]);
                        if (in0) ssum[cp] = fma_h2_f2(h0[cp], one, ssum[cp]), ssq[cp] = fma_h2_f2(h0[cp], h0[cp], ssq[cp]);
                        if (in1) ssum[cp] = fma_h2_f2(h1[cp], one, ssum[cp]), ssq[cp] = fma_h2_f2(h1[cp], h1[cp], ssq[cp]);
                    }
                }
                sts128(ob + a0, o0);
                sts128(ob + a1, o1);
            });
        }
        if (store) {
            fence_proxy_async_smem();  // the tile must be visible to the TMA store
            __syncwarp();
            if (lane == 0) mbar_arrive(staged0 + 8 * (oc & 1u));
            ++oc;
        }
        ++ci;
        return true;
    };
    // This thread's B column is n = g.  Its taps: output (ow, od) against patch slot (pw, pd = t) is the tap
    // (b, tt) = (pw - ow, t - od), zero outside 0..2.
    const int tt = t - ((g >> 1) & 1), ow = g >> 2;
    if constexpr (Cfg::PERCH) {
        // column n = 2 out + lane: out = g >> 1, lane = g & 1.  Fragments for both lane assignments (index = the
        // finishing lane): B21 = a=2 taps to the finishing lane, a=1 taps to the other; B0 = a=0 taps to the (cleared)
        // finishing lane, zero columns for the other.  A register holds the slots (pw = 0, 1) or (pw = 2, 3).
        uint32_t B21[2][8][2], B0[2][8][2];
        float Q[UPW][8][4];  // no initialisation: nothing is stored before a lane was cleared and got its three planes
        auto rebuild = [&](int c0) {
            const unsigned short* wp = reinterpret_cast<const unsigned short*>(weight) + c0 + 8 * ng;
            const int ln = g & 1;
            auto taps = [&](int a, int pw, int c) -> uint32_t {  // slots (pw, pw + 1) of plane tap a, channel c
                uint32_t v = 0;
                if (tt >= 0 && tt <= 2) {
                    const int b0 = pw - ow, b1 = pw + 1 - ow;
                    if (b0 >= 0 && b0 <= 2) v = wp[(size_t)((a * 3 + b0) * 3 + tt) * C + c];
                    if (b1 >= 0 && b1 <= 2) v |= (uint32_t)wp[(size_t)((a * 3 + b1) * 3 + tt) * C + c] << 16;
                }
                return v;
            };
#pragma unroll
            for (int fl = 0; fl < 2; ++fl)
#pragma unroll
                for (int c = 0; c < 8; ++c)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        B21[fl][c][h] = taps(ln == fl ? 2 : 1, 2 * h, c);
                        B0[fl][c][h] = ln == fl ? taps(0, 2 * h, c) : 0u;
                    }
        };
        // The two instantiations alternate, so the role change of the lanes costs neither a branch nor a move.
        while (plane_step(rebuild,
                          [&](int u, const uint4(&X)[6], bool store, auto&& emit) {
                              pg_step_ch<0>(X, B21, B0, Q[u], store, emit);
                          }) &&
               plane_step(rebuild, [&](int u, const uint4(&X)[6], bool store, auto&& emit) {
                   pg_step_ch<1>(X, B21, B0, Q[u], store, emit);
               })) {
        }
    } else {
        // column n = g: out = g >> 1, cc' = g & 1; rows k = (slot t of patch row 2ks + j, cc)
        uint32_t Bf[4][3][2][2];             // weight fragments [channel pair][a][k16 step][k half]
        float S0[UPW][4][4], S1[UPW][4][4];  // no initialisation: a plane's sum starts with an mma that ignores them
        auto rebuild = [&](int c0) {
            const unsigned short* wp = reinterpret_cast<const unsigned short*>(weight) + c0 + 8 * ng + (g & 1);
#pragma unroll
            for (int cp = 0; cp < 4; ++cp)
#pragma unroll
                for (int a = 0; a < 3; ++a)
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks)
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const int b = 2 * ks + j - ow;
                            uint32_t v = 0;
                            if (b >= 0 && b <= 2 && tt >= 0 && tt <= 2) v = wp[(size_t)((a * 3 + b) * 3 + tt) * C + 2 * cp];
                            Bf[cp][a][ks][j] = (g & 1) ? (v << 16) : v;
                        }
        };
        // The two accumulator sets swap roles (finishing / middle plane) every step: the step is called with the
        // sets exchanged, which costs neither a branch nor a register move.
        while (plane_step(rebuild,
                          [&](int u, const uint4(&X)[6], bool store, auto&& emit) {
                              pg_step<Cfg>(X, Bf, S0[u], S1[u], store, emit, wt.zero);
                          }) &&
               plane_step(rebuild, [&](int u, const uint4(&X)[6], bool store, auto&& emit) {
                   pg_step<Cfg>(X, Bf, S1[u], S0[u], store, emit, wt.zero);
               })) {
        }
    }
    if (Cfg::EPI && cur_c0 >= 0) flush_stats(cur_c0);
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
struct PgArgs {
    const void* x;
    const void* w;
    void* y;
    const float *scale, *shift;  // prologue variants only
    const void* res;             // epilogue variants only: residual (strides rsN, rsH, rsW), statistics workspace
    int64_t rsN, rsH, rsW;
    float* stats_ws;
    int64_t stats_rows;
    int* rows_used;
    int64_t N, C, Hx, W, D, xsN, xsH, xsW, Hy, ysN, ysH, ysW;
    int h_begin, h_end, y_h0;
    cudaStream_t stream;
};

template <class Cfg>
static int launch_fprop_pg(const PgArgs& a) {
    CUtensorMap tmx, tmy;
    int rc = encode_tile_map<typename Cfg::Geo>(&tmx, a.x, a.N, a.C, a.Hx, a.W, a.D, a.xsN, a.xsH, a.xsW, true, Cfg::PRO != 0);
    if (rc) return rc;
    rc = encode_tile_map<typename Cfg::Geo>(&tmy, a.y, a.N, a.C, a.Hy, a.W, a.D, a.ysN, a.ysH, a.ysW, false);
    if (rc) return rc;
    CUtensorMap tmr = tmy;  // unused without the epilogue
    if (Cfg::EPI) {
        rc = encode_tile_map<typename Cfg::Geo>(&tmr, a.res, a.N, a.C, a.Hx, a.W, a.D, a.rsN, a.rsH, a.rsW, false);
        if (rc) return rc;
    }
    if (((uintptr_t)a.w & 1) != 0) {
        set_error("weight pointer must be 2-byte aligned");
        return KDW_ERR_ALIGN;
    }
    static KernelSetup setup;  // one per kernel instantiation
    auto kern = fprop_pg_kernel<Cfg>;
    int sms = 0, occ = 0;
    rc = setup.get((const void*)kern, Cfg::NTHREADS, Cfg::SMEM, &sms, &occ);
    if (rc) return rc;
    int* status = nullptr;
    rc = status_ptr(&status);
    if (rc) return rc;
    Sched s;
    long long target = (long long)sms * occ;
    if (Cfg::EPI) {  // one statistics row per (CTA, consumer warp)
        if (target * Cfg::NCW > a.stats_rows) target = a.stats_rows / Cfg::NCW;
        if (target < 1) {
            set_error("fprop_addstats: workspace has %lld rows, the tensor-core kernel needs %d per CTA", (long long)a.stats_rows,
                      Cfg::NCW);
            return KDW_ERR_WORKSPACE;
        }
    }
    const int grid = make_sched(&s, a.N, a.C, a.W, a.D, a.h_begin, a.h_end, Cfg::WT, Cfg::DT, Cfg::CS, (int)target);
    if (Cfg::EPI && a.rows_used) *a.rows_used = grid * Cfg::NCW;
    kern<<<grid, Cfg::NTHREADS, Cfg::SMEM, a.stream>>>(tmx, tmy, tmr, a.stats_ws, (int)a.W, (int)a.D, (const __half*)a.w, a.scale, a.shift, s, (int)a.C, a.y_h0, status,
                                                       wait_test());
    KDW_CUDA(cudaGetLastError());
    return 0;
}

typedef int (*PgLaunch)(const PgArgs&);
struct PgVariant {
    int cs, dt, wt, mode;
    PgLaunch f;
};
// PCfg<CS, WW, WD, UPW, ST, MODE>: tile 4*WW x 16*WD voxels (w, d), CS channels; 8 consumer warps, two units each;
// MODE: how the tiles are staged (TileGeo): 0 any C that is a multiple of CS, 1 C == 8, 2 C == 16 and D even
#define KDW_PG(CS, WW, WD, UPW, ST, MODE) {CS, 16 * WD, 4 * WW, MODE, &launch_fprop_pg<PCfg<CS, WW, WD, UPW, ST, MODE>>}
#define KDW_PGC(CS, WW, WD, UPW, ST, MODE) {CS, 16 * WD, 4 * WW, MODE, &launch_fprop_pg<PCfg<CS, WW, WD, UPW, ST, MODE, 1>>}
static const PgVariant g_pg_variants[] = {
    KDW_PGC(64, 2, 1, 2, 4, 0),  // 0: tile 8 x 16, per-channel form
    KDW_PG(32, 4, 1, 2, 4, 0),  // 1: tile 16 x 16
    KDW_PG(16, 4, 2, 2, 4, 0),  // 2: tile 16 x 32
    KDW_PG(8, 4, 4, 2, 4, 0),   // 3: tile 16 x 64
    KDW_PG(32, 2, 2, 2, 4, 0),  // 4: tile 8 x 32
    KDW_PG(64, 2, 1, 2, 5, 0),  // 5: five stages, channel-pair form
    KDW_PG(8, 4, 4, 2, 4, 1),   // 6: C == 8, tile 16 x 64, long box rows
    KDW_PG(16, 4, 2, 2, 4, 2),  // 7: C == 16, D even, tile 16 x 32, 64-byte box rows
    KDW_PG(16, 8, 1, 2, 4, 2),  // 8: C == 16, D even, tile 32 x 16
    KDW_PG(64, 2, 1, 2, 4, 0),  // 9: as 0, channel-pair form
};
#undef KDW_PG
#undef KDW_PGC
static const int g_n_pg_variants = (int)(sizeof(g_pg_variants) / sizeof(g_pg_variants[0]));

int fprop_mma_variants() { return g_n_pg_variants; }

int fprop_mma_variant_channels(int which) {
    if (which < 0 || which >= g_n_pg_variants) return KDW_ERR_TUNE;
    return g_pg_variants[which].cs;
}

void fprop_mma_variant_tile(int which, int* wt, int* dt) {
    *wt = g_pg_variants[which].wt;
    *dt = g_pg_variants[which].dt;
}

// whether variant `which` can run this (C, D): the merged-map variants need C equal to their slice (and an even D)
bool fprop_mma_variant_fits(int which, int64_t C, int64_t D) {
    const PgVariant& v = g_pg_variants[which];
    return C % v.cs == 0 && (v.mode == 0 || C == v.cs) && (v.mode != 2 || (D & 1) == 0);
}

int launch_fprop_mma_variant(int which, const void* x, const void* w, void* y, int64_t N, int64_t C, int64_t Hx,
                             int64_t W, int64_t D, int64_t xsN, int64_t xsH, int64_t xsW, int64_t Hy, int64_t ysN,
                             int64_t ysH, int64_t ysW, int h_begin, int h_end, int y_h0, cudaStream_t stream) {
    if (which < 0 || which >= g_n_pg_variants) {
        set_error("fprop: no such tensor-core variant");
        return KDW_ERR_TUNE;
    }
    const PgVariant& v = g_pg_variants[which];
    if (C % v.cs != 0 || (v.mode != 0 && C != v.cs) || (v.mode == 2 && (D & 1))) {
        set_error("fprop: tensor-core variant %d needs C %s %d%s (C=%lld, D=%lld)", which, v.mode ? "==" : "a multiple of",
                  v.cs, v.mode == 2 ? " and an even D" : "", (long long)C, (long long)D);
        return KDW_ERR_TUNE;
    }
    PgArgs a{x, w, y, nullptr, nullptr, nullptr, 0, 0, 0, nullptr, 0, nullptr, N, C, Hx, W, D, xsN, xsH, xsW, Hy, ysN, ysH, ysW,
             h_begin, h_end, y_h0, stream};
    return v.f(a);
}

// Fused epilogue (kdw_fprop_addstats_f16): the built-in tile of each channel count with PCfg::EPI.  *rows_used = the
// statistics rows the launch writes (all of them: each warp zeroes its own).
bool fprop_addstats_mma_fits(int64_t C, int64_t D) { return C >= 32 || C == 8 || (C == 16 && (D & 1) == 0); }

int launch_fprop_addstats_mma(const void* x, const void* w, const void* res, void* y, float* stats_ws, int64_t stats_rows,
                              int64_t N, int64_t C, int64_t H, int64_t W, int64_t D, int64_t xsN, int64_t xsH, int64_t xsW,
                              int64_t rsN, int64_t rsH, int64_t rsW, int64_t ysN, int64_t ysH, int64_t ysW,
                              cudaStream_t stream, int* rows_used) {
    PgArgs a{x, w, y, nullptr, nullptr, res, rsN, rsH, rsW, stats_ws, stats_rows, rows_used, N, C, H, W, D, xsN, xsH, xsW, H,
             ysN, ysH, ysW, 0, (int)H, 0, stream};
    if (C == 8) return launch_fprop_pg<PCfg<8, 4, 4, 2, 4, 1, 0, 0, 1>>(a);
    if (C == 16) return launch_fprop_pg<PCfg<16, 4, 2, 2, 4, 2, 0, 0, 1>>(a);
    if (C == 32) return launch_fprop_pg<PCfg<32, 2, 2, 2, 4, 0, 0, 0, 1>>(a);
    return launch_fprop_pg<PCfg<64, 2, 1, 2, 4, 0, 0, 0, 1>>(a);
}

// Fused prologue (kdw_fprop_bnrelu_f16): the built-in tile of each channel count with PCfg::PRO = 1 (packed half) or
// 2 (fp32).  Returns KDW_ERR_TUNE without touching the error text when no tensor-core tile takes the shape (the
// caller then falls back to its CUDA-core kernels).
bool fprop_bnrelu_mma_fits(int64_t C, int64_t D) { return C >= 32 || C == 8 || (C == 16 && (D & 1) == 0); }

int launch_fprop_bnrelu_mma(const void* x, const float* scale, const float* shift, const void* w, void* y, int64_t N,
                            int64_t C, int64_t H, int64_t W, int64_t D, int64_t xsN, int64_t xsH, int64_t xsW,
                            int64_t ysN, int64_t ysH, int64_t ysW, bool packed_half, cudaStream_t stream) {
    PgArgs a{x, w, y, scale, shift, nullptr, 0, 0, 0, nullptr, 0, nullptr, N, C, H, W, D, xsN, xsH, xsW, H, ysN, ysH, ysW,
             0, (int)H, 0, stream};
    if (packed_half) {
        if (C == 8) return launch_fprop_pg<PCfg<8, 4, 4, 2, 4, 1, 0, 1>>(a);
        if (C == 16) return launch_fprop_pg<PCfg<16, 4, 2, 2, 4, 2, 0, 1>>(a);
        if (C == 32) return launch_fprop_pg<PCfg<32, 2, 2, 2, 4, 0, 0, 1>>(a);
        return launch_fprop_pg<PCfg<64, 2, 1, 2, 4, 0, 1, 1>>(a);
    }
    if (C == 8) return launch_fprop_pg<PCfg<8, 4, 4, 2, 4, 1, 0, 2>>(a);
    if (C == 16) return launch_fprop_pg<PCfg<16, 4, 2, 2, 4, 2, 0, 2>>(a);
    if (C == 32) return launch_fprop_pg<PCfg<32, 2, 2, 2, 4, 0, 0, 2>>(a);
    return launch_fprop_pg<PCfg<64, 2, 1, 2, 4, 0, 1, 2>>(a);
}

}  // namespace kdw
