// Depthwise 3x3x3 weight gradient on the tensor cores (warp-level mma.sync.m16n8k16), fp32 accumulation.
//
// Pass 1 of the weight gradient, replacing kerops/kernels/dw_conv.py:147-287 (_DWConv_wgrad_cl3d_impl) like
// wgrad_tma_kernel (dwconv_wgrad.cu), whose column march, TMA ring, per-CTA workspace rows and fixed-order second
// pass it shares.  The arithmetic is the transpose of the forward kernel's patch form (dwconv_fprop_mma.cu): with
// the x patch words A[block, (slot, cc)] and the grad words G[block, (out, cc')] of a unit of 16 blocks,
//     dW[(slot, cc), (out, cc')] += sum_blocks A[block, (slot, cc)] * G[block, (out, cc')]
// is an m16n8k16 product whose contraction runs over the blocks.  The entries with cc == cc' are the weight
// gradient of tap (b, t) = slot - out of channel c_cc, summed over the block's voxels; the others (products of two
// different channels) are never read.  Both operands have to be transposed with respect to the way channels-last
// words arrive in registers (a thread loads words of ONE block; the fragments want two blocks of one column per
// register): one movmatrix per register, 40 per 24 mma.  27 of 96 multiply-adds are useful, as in the forward
// kernel; every product is an exact fp16 x fp16 product accumulated in fp32.
//
// A thread keeps 96 fp32 accumulators (2 patch-row pairs x 4 channel pairs x 3 planes a x 4) for the whole run
// of a channel slice and the transposed grad words of three planes (a rotating window).  When the slice changes and
// at the end, every warp reduces its accumulators over the lanes that hold the same (tap, channel) through its own
// scratch area in shared memory and adds them to ITS row of the workspace - rows are per (CTA, spatial warp group),
// so no two warps write the same element, there is no CTA-wide barrier and no atomic, and the sum is reproducible.
#include "../../include/kdw.h"
#include "kdw_common.cuh"
#include "mma_patch.cuh"

namespace kdw {

template <int CS_, int WW_, int WD_, int UPW_, int ST_, int MODE_ = 0>
struct WPCfg {
    static constexpr int CS = CS_, WW = WW_, WD = WD_, UPW = UPW_, ST = ST_;
    static constexpr int NG = CS / 8;               // channel groups of 8
    static constexpr int SU = (WW / UPW) * WD;      // spatial warp groups: workspace rows per CTA
    static constexpr int NCW = NG * SU;             // consumer warps
    static constexpr int NT = NCW * 32;
    // Warps 0-3 form the helper warpgroup (warp 0 loads, the others leave at once), the consumer warps follow.  The
    // kernel is compiled for 168 registers per thread (12 warps); the helper warpgroup then hands registers back
    // (setmaxnreg) and the two consumer warpgroups take them: 96 accumulators, 48 grad words and the transposed
    // patch words do not fit in 168.
    static constexpr int NHELP = 4;
    static constexpr int NTHREADS = NT + NHELP * 32;
    static constexpr int REGS_HELPER = 40, REGS_CONSUMER = 232;
    static constexpr int WT = 4 * WW, DT = 16 * WD;
    static constexpr int VOXB = CS * 2;
    using Geo = TileGeo<CS, WT, DT, MODE_>;  // staging of the x ("in") and grad ("out") tiles and their TMA boxes
    static constexpr int SWZ = Geo::SWZ;
    static constexpr int X_BYTES = Geo::IN_BYTES, X_STRIDE = Geo::IN_STRIDE;
    static constexpr int G_BYTES = Geo::OUT_BYTES, G_STRIDE = Geo::OUT_STRIDE;
    static constexpr int STAGE = X_STRIDE + G_STRIDE;
    static constexpr int SCRATCH = 32 * 16 * 4;     // per warp: 16 floats per lane (one plane a of the flush)
    static constexpr int SMEM = ST * STAGE + NCW * SCRATCH + 16 * ST + 4 * ST + 128 + 1024;
    static_assert(CS == 8 || CS == 16 || CS == 32 || CS == 64, "a voxel must be one swizzle span (or 16 bytes)");
    static_assert(WW % UPW == 0 && NCW == 8, "two consumer warpgroups");
    static_assert(DT + 4 <= 256 && WT + 2 <= 256, "TMA box limits");
};

// x plane q of one unit against the grad planes q+1 (a=0), q (a=1), q-1 (a=2).  R = (step count) % 3 names the
// slot of the rotating grad window that receives plane q+1.  X[r]: the thread's voxel of input row r (as in the
// forward kernel); G0 / G1: its grad voxel (output t of block row g / g+8), zero when plane q+1 is not owned.
// The A quad of patch-row pair ks and channel pair cp is the transpose of the words of rows 2ks .. 2ks+3.
template <int R>
__device__ __forceinline__ void wg_step(const uint4 (&X)[6], const uint4& G0, const uint4& G1, uint32_t (&Gf)[3][4][2],
                                        float (&acc)[2][4][3][4]) {
    constexpr int SLOT[3] = {(R + 2) % 3, (R + 1) % 3, R % 3};  // slot of the grad plane paired with tap a
    const uint32_t* g0 = reinterpret_cast<const uint32_t*>(&G0);
    const uint32_t* g1 = reinterpret_cast<const uint32_t*>(&G1);
#pragma unroll
    for (int cp = 0; cp < 4; ++cp) {
        Gf[SLOT[0]][cp][0] = movmatrix_trans(g0[cp]);
        Gf[SLOT[0]][cp][1] = movmatrix_trans(g1[cp]);
    }
    const uint32_t* Xw = reinterpret_cast<const uint32_t*>(&X[0]);  // Xw[r * 4 + cp]
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
        Quad AT[4];
#pragma unroll
        for (int cp = 0; cp < 4; ++cp)
#pragma unroll
            for (int k = 0; k < 4; ++k) AT[cp].r[k] = movmatrix_trans(Xw[(2 * ks + k) * 4 + cp]);
#pragma unroll
        for (int a = 0; a < 3; ++a)
#pragma unroll
            for (int cp = 0; cp < 4; ++cp) mma16816<false>(acc[ks][cp][a], AT[cp], Gf[SLOT[a]][cp][0], Gf[SLOT[a]][cp][1]);
    }
}

// Adds the warp's accumulators to its workspace row and clears them.  Lane (g, t) holds, for patch-row pair ks,
// half h (row g / g + 8), channel pair cp and plane a, the entry (slot (pw = 2ks + h, pd = g >> 1), cc = g & 1) x
// (out t, cc' = e) in acc[ks][cp][a][2h + e]; the useful one has e = g & 1 and belongs to tap
// (b, tt) = (pw - (t >> 1), (g >> 1) - (t & 1)) of channel 2cp + (g & 1).  Per plane a the lanes park their 16
// useful values in the warp's scratch area; then lane j adds up, in a fixed order, the (at most four) entries of
// every (tap, channel) it is responsible for.
__device__ __forceinline__ void wg_flush(float (&acc)[2][4][3][4], float* scratch, float* row, int C, int cbase, int lane) {
    const int g = lane >> 2, e = g & 1;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        __syncwarp();
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int cp = 0; cp < 4; ++cp)  // (a register array must not be indexed with a run-time value)
                    scratch[lane * 16 + (ks * 2 + h) * 4 + cp] = e ? acc[ks][cp][a][2 * h + 1] : acc[ks][cp][a][2 * h];
        __syncwarp();
        for (int j = lane; j < 72; j += 32) {  // 9 taps x 8 channels
            const int ch = j & 7, tap = j >> 3, b = tap / 3, tt = tap % 3;
            float sum = 0.f;
#pragma unroll
            for (int ow = 0; ow < 2; ++ow)
#pragma unroll
                for (int od = 0; od < 2; ++od) {
                    const int pw = b + ow, pd = tt + od;  // the patch voxel output (ow, od) reads through this tap
                    if (pd > 3) continue;
                    const int src = (2 * pd + (ch & 1)) * 4 + 2 * ow + od;  // lane (g = 2pd + cc, t = 2ow + od)
                    sum += scratch[src * 16 + pw * 4 + (ch >> 1)];
                }
            row[(size_t)((a * 3 + b) * 3 + tt) * C + cbase + ch] += sum;
        }
    }
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
#pragma unroll
        for (int cp = 0; cp < 4; ++cp)
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[ks][cp][a][k] = 0.f;
}

// Issues the copies of the next x plane and grad plane (or the end marker) into the next stage, waiting for the
// stage to be free.  The position in the schedule lives in shared memory (ProdState).
template <class Cfg>
__device__ __forceinline__ void wg_produce(ProdState* ps, const Sched& s, const CUtensorMap& tmx, const CUtensorMap& tmg,
                                           uint32_t stage0, uint32_t full0, uint32_t empty0, uint32_t desc0, int g_h0,
                                           int* status, const WaitTest& wt) {
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
    const uint32_t bar = full0 + 8 * st;
    StepIter it = ps->it;
    if (!it.active) {  // end marker: completes the stage's barrier without a copy
        st_shared_u32(desc0 + 4 * st, 0xffffffffu);
        mbar_arrive(bar);
        ps->done = 1;
        return;
    }
    const bool with_g = it.q + 1 < it.g.he;  // grad plane q+1 is owned by the segment
    st_shared_u32(desc0 + 4 * st, ((uint32_t)it.g.c0 << 8) | (it.q == it.g.hb - 1 ? 2u : 0u) | (with_g ? 1u : 0u));
    mbar_expect_tx(bar, Cfg::X_BYTES + (with_g ? Cfg::G_BYTES : 0));
    tile_load_in<typename Cfg::Geo>(status, stage0 + st * Cfg::STAGE, &tmx, bar, it.g.c0, it.g.d0, it.g.w0, it.q, it.g.n);
    if (with_g)
        tile_load_out<typename Cfg::Geo>(status, stage0 + st * Cfg::STAGE + Cfg::X_STRIDE, &tmg, bar, it.g.c0, it.g.d0,
                                         it.g.w0, it.q + 1 - g_h0, it.g.n);
    it.next(s);
    ps->it = it;
    ps->pi = pi + 1;
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NTHREADS, 1)
    wgrad_pg_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmg,
                    float* __restrict__ ws, const Sched s, const int C, const int g_h0, int* status, const WaitTest wt) {
    constexpr int ST = Cfg::ST, NCW = Cfg::NCW, UPW = Cfg::UPW;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t stage0 = base;
    float* scratch0 = reinterpret_cast<float*>(base_ptr + ST * Cfg::STAGE);
    const uint32_t full0 = base + ST * Cfg::STAGE + NCW * Cfg::SCRATCH;  // full[ST], empty[ST], desc[ST]
    const uint32_t empty0 = full0 + 8 * ST;
    // desc[ST], written by the load warp before the copies of a stage are issued: bit 0 = the stage carries grad
    // plane q+1, bit 1 = first plane of a segment (the grad window restarts), bits 8.. = first channel of the
    // slice; 0xffffffff = no more planes
    const uint32_t desc0 = empty0 + 8 * ST;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int KC = 27 * C;
    if (tid == 0) {
        prefetch_tmap(&tmx);
        prefetch_tmap(&tmg);
        for (int k = 0; k < ST; ++k) {
            mbar_init(full0 + 8 * k, 1);
            mbar_init(empty0 + 8 * k, NCW);
        }
        mbar_fence_init();
    }
    // this CTA's rows of the workspace, one per spatial warp group
    for (int k = tid; k < Cfg::SU * KC; k += Cfg::NTHREADS) ws[(size_t)blockIdx.x * Cfg::SU * KC + k] = 0.f;
    __syncthreads();  // the only CTA-wide barrier

    ProdState* ps = reinterpret_cast<ProdState*>(base_ptr + (desc0 + 4 * ST + 15 - base) / 16 * 16);
    if (tid == 0) {
        ps->it.init(s, (int)blockIdx.x, (int)gridDim.x);
        ps->pi = 0;
        ps->done = 0;
    }
    __syncwarp();
    if (warp < Cfg::NHELP) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Cfg::REGS_HELPER));
        // ---------------- load warp ----------------
        if (tid == 0)
            while (!ps->done) wg_produce<Cfg>(ps, s, tmx, tmg, stage0, full0, empty0, desc0, g_h0, status, wt);
        return;
    }
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Cfg::REGS_CONSUMER));

    // ---------------- consumer warps ----------------
    const int cw = warp - Cfg::NHELP;
    const int ng = cw % Cfg::NG;
    const int su = cw / Cfg::NG;                   // spatial warp group
    const int uwg = su % (Cfg::WW / UPW), ud = su / (Cfg::WW / UPW);
    const int g = lane >> 2, t = lane & 3;
    using Geo = typename Cfg::Geo;
    constexpr uint32_t IN_ROW4 = Geo::IN_ROW4, G_ROW2 = Geo::OUT_ROW2;
    uint32_t in_off[4], g_off;
#pragma unroll
    for (int r = 0; r < 4; ++r)
        in_off[r] = swz<Cfg::SWZ>(Geo::in_off(4 * uwg * UPW + r, Geo::DPAD - 1 + 16 * ud + 2 * g + t) + 16 * ng);
    g_off = Cfg::X_STRIDE + swz<Cfg::SWZ>(Geo::out_off(4 * uwg * UPW + (t >> 1), 16 * ud + 2 * g + (t & 1)) + 16 * ng);
    float* scratch = scratch0 + cw * (Cfg::SCRATCH / 4);
    float* row = ws + ((size_t)blockIdx.x * Cfg::SU + su) * KC;

    float acc[2][4][3][4];
    uint32_t Gf[UPW][3][4][2];
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
#pragma unroll
        for (int cp = 0; cp < 4; ++cp)
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[ks][cp][a][k] = 0.f;

    uint32_t ci = 0;
    int cur_c0 = -1;
    bool failed = false;
    while (true) {
        const uint32_t st = ci % ST;
        const bool ok = mbar_wait_bounded(full0 + 8 * st, (ci / ST) & 1u, wt.limit_ns);
        if (__any_sync(0xffffffffu, !ok)) {
            if (lane == 0) atomicExch(status, (int)KDW_STATUS_TMA_TIMEOUT);
            failed = true;  // this warp leaves without adding its sums; every other wait is bounded as well
            break;
        }
        const uint32_t dsc = ld_shared_u32(desc0 + 4 * st);
        if (dsc == 0xffffffffu) break;
        const int c0 = (int)(dsc >> 8);
        if (c0 != cur_c0) {  // the accumulators belong to a channel slice
            if (cur_c0 >= 0) wg_flush(acc, scratch, row, C, cur_c0 + 8 * ng, lane);
            cur_c0 = c0;
        }
        if (dsc & 2u) {  // new segment: grad planes of the previous one must not meet this segment's x
#pragma unroll
            for (int u = 0; u < UPW; ++u)
#pragma unroll
                for (int sl = 0; sl < 3; ++sl)
#pragma unroll
                    for (int cp = 0; cp < 4; ++cp) Gf[u][sl][cp][0] = Gf[u][sl][cp][1] = 0u;
        }
        const bool with_g = (dsc & 1u) != 0;
        const uint32_t stage = stage0 + st * Cfg::STAGE;
#pragma unroll
        for (int u = 0; u < UPW; ++u) {
            uint4 X[6], G0 = make_uint4(0, 0, 0, 0), G1 = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int r = 0; r < 6; ++r) X[r] = lds128(stage + in_off[r & 3] + (uint32_t)((r >> 2) + u) * IN_ROW4);
            if (with_g) {
                G0 = lds128(stage + g_off + (uint32_t)(2 * u) * G_ROW2);
                G1 = lds128(stage + g_off + (uint32_t)(2 * u + 1) * G_ROW2);
            }
            if (u == UPW - 1) {
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * st);
            }
            switch (ci % 3) {
                case 0: wg_step<0>(X, G0, G1, Gf[u], acc); break;
                case 1: wg_step<1>(X, G0, G1, Gf[u], acc); break;
                default: wg_step<2>(X, G0, G1, Gf[u], acc); break;
            }
        }
        ++ci;
    }
    if (!failed && cur_c0 >= 0) wg_flush(acc, scratch, row, C, cur_c0 + 8 * ng, lane);
}

// ------------------------------------------------------------------------------------------------
// Host side (called from the dispatcher in dwconv_wgrad.cu)
// ------------------------------------------------------------------------------------------------
struct WpgArgs {
    const void* x;
    const void* g;
    float* ws;
    int64_t ws_rows;
    int64_t N, C, Hx, W, D, xsN, xsH, xsW, Hg, gsN, gsH, gsW;
    int h_begin, h_end, g_h0;
    cudaStream_t stream;
};

template <class Cfg>
static int launch_wgrad_pg(const WpgArgs& a, int* rows_used) {
    CUtensorMap tmx, tmg;
    int rc = encode_tile_map<typename Cfg::Geo>(&tmx, a.x, a.N, a.C, a.Hx, a.W, a.D, a.xsN, a.xsH, a.xsW, true);
    if (rc) return rc;
    rc = encode_tile_map<typename Cfg::Geo>(&tmg, a.g, a.N, a.C, a.Hg, a.W, a.D, a.gsN, a.gsH, a.gsW, false);
    if (rc) return rc;
    static KernelSetup setup;  // one per kernel instantiation
    auto kern = wgrad_pg_kernel<Cfg>;
    int sms = 0, occ = 0;
    rc = setup.get((const void*)kern, Cfg::NTHREADS, Cfg::SMEM, &sms, &occ);
    if (rc) return rc;
    int* status = nullptr;
    rc = status_ptr(&status);
    if (rc) return rc;
    long long target = (long long)sms * occ;
    if (target * Cfg::SU > a.ws_rows) target = a.ws_rows / Cfg::SU;  // one workspace row per (CTA, spatial warp group)
    if (target < 1) {
        set_error("wgrad: workspace has %lld rows, this variant needs %d per CTA", (long long)a.ws_rows, Cfg::SU);
        return KDW_ERR_WORKSPACE;
    }
    Sched s;
    const int grid = make_sched(&s, a.N, a.C, a.W, a.D, a.h_begin, a.h_end, Cfg::WT, Cfg::DT, Cfg::CS, (int)target);
    kern<<<grid, Cfg::NTHREADS, Cfg::SMEM, a.stream>>>(tmx, tmg, a.ws, s, (int)a.C, a.g_h0, status, wait_test());
    KDW_CUDA(cudaGetLastError());
    *rows_used = grid * Cfg::SU;
    return 0;
}

typedef int (*WpgLaunch)(const WpgArgs&, int*);
struct WpgVariant {
    int cs, dt, wt, mode;
    WpgLaunch f;
};
// WPCfg<CS, WW, WD, UPW, ST, MODE>: tile 4*WW x 16*WD voxels (w, d), CS channels; 8 consumer warps, two units each;
// MODE: how the tiles are staged (TileGeo): 0 any C that is a multiple of CS, 1 C == 8, 2 C == 16 and D even
#define KDW_WPG(CS, WW, WD, UPW, ST, MODE) {CS, 16 * WD, 4 * WW, MODE, &launch_wgrad_pg<WPCfg<CS, WW, WD, UPW, ST, MODE>>}
static const WpgVariant g_wpg_variants[] = {
    KDW_WPG(64, 2, 1, 2, 3, 0),  // 0: tile 8 x 16
    KDW_WPG(32, 4, 1, 2, 4, 0),  // 1: tile 16 x 16
    KDW_WPG(16, 4, 2, 2, 4, 0),  // 2: tile 16 x 32
    KDW_WPG(8, 4, 4, 2, 4, 0),   // 3: tile 16 x 64
    KDW_WPG(64, 2, 1, 2, 4, 0),  // 4: as 0, four stages
    KDW_WPG(32, 2, 2, 2, 4, 0),  // 5: tile 8 x 32
    KDW_WPG(8, 4, 4, 2, 4, 1),   // 6: C == 8, tile 16 x 64, long box rows
    KDW_WPG(16, 4, 2, 2, 4, 2),  // 7: C == 16, D even, tile 16 x 32, 64-byte box rows
    KDW_WPG(16, 8, 1, 2, 4, 2),  // 8: C == 16, D even, tile 32 x 16
};
#undef KDW_WPG
static const int g_n_wpg_variants = (int)(sizeof(g_wpg_variants) / sizeof(g_wpg_variants[0]));

int wgrad_mma_variants() { return g_n_wpg_variants; }

int wgrad_mma_variant_channels(int which) {
    if (which < 0 || which >= g_n_wpg_variants) return KDW_ERR_TUNE;
    return g_wpg_variants[which].cs;
}

void wgrad_mma_variant_tile(int which, int* wt, int* dt) {
    *wt = g_wpg_variants[which].wt;
    *dt = g_wpg_variants[which].dt;
}

bool wgrad_mma_variant_fits(int which, int64_t C, int64_t D) {
    const WpgVariant& v = g_wpg_variants[which];
    return C % v.cs == 0 && (v.mode == 0 || C == v.cs) && (v.mode != 2 || (D & 1) == 0);
}

int launch_wgrad_mma_variant(int which, const void* x, const void* grad, float* ws, int64_t ws_rows, int64_t N, int64_t C,
                             int64_t Hx, int64_t W, int64_t D, int64_t xsN, int64_t xsH, int64_t xsW, int64_t Hg,
                             int64_t gsN, int64_t gsH, int64_t gsW, int h_begin, int h_end, int g_h0,
                             cudaStream_t stream, int* rows_used) {
    if (which < 0 || which >= g_n_wpg_variants) {
        set_error("wgrad: no such tensor-core variant");
        return KDW_ERR_TUNE;
    }
    const WpgVariant& v = g_wpg_variants[which];
    if (C % v.cs != 0 || (v.mode != 0 && C != v.cs) || (v.mode == 2 && (D & 1))) {
        set_error("wgrad: tensor-core variant %d needs C %s %d%s (C=%lld, D=%lld)", which, v.mode ? "==" : "a multiple of",
                  v.cs, v.mode == 2 ? " and an even D" : "", (long long)C, (long long)D);
        return KDW_ERR_TUNE;
    }
    WpgArgs a{x, grad, ws, ws_rows, N, C, Hx, W, D, xsN, xsH, xsW, Hg, gsN, gsH, gsW, h_begin, h_end, g_h0, stream};
    return v.f(a, rows_used);
}

}  // namespace kdw
