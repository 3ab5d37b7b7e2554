// Tile configuration and per-thread step of the forward TMA kernel (see dwconv_fprop.cu).
// Kept in a header so the test-suite can run the same step code on the CPU.
#pragma once
#include "kdw_common.cuh"

namespace kdw {

template <int CS_, int DT_, int WT_, int M_, int CP_, int ST_, int MINB_>
struct FCfg {
    static constexpr int CS = CS_;      // channels per CTA slice
    static constexpr int DT = DT_;      // d extent of the tile
    static constexpr int WT = WT_;      // w extent of the tile
    static constexpr int M = M_;        // consecutive w outputs per thread
    static constexpr int CP = CP_;      // channel pairs (half2) per thread
    static constexpr int ST = ST_;      // input pipeline stages
    static constexpr int MINB = MINB_;  // CTAs per SM the register budget is set for
    static constexpr int CPG = CS / (2 * CP);  // threads that share a voxel
    static constexpr int WG = WT / M;
    static constexpr int NT = CPG * DT * WG;   // consumer threads
    static constexpr int NCW = NT / 32;        // consumer warps; warp NCW is the TMA producer
    static constexpr int DPW = 32 / CPG;       // d positions covered by one warp
    static constexpr int IN_BYTES = (WT + 2) * (DT + 2) * CS * 2;
    static constexpr int IN_STRIDE = (IN_BYTES + 127) / 128 * 128;
    static constexpr int OUTW_BYTES = M * DPW * CS * 2;  // one warp's output tile [M][DPW][CS]
    static constexpr int SMEM = ST * IN_STRIDE + 2 * NCW * OUTW_BYTES + 16 * ST + 128;
    static_assert(CS % (2 * CP) == 0 && WT % M == 0, "tile/thread shape");
    static_assert(CPG <= 32 && 32 % CPG == 0 && DT % DPW == 0, "a warp must cover whole voxels of one w group");
    static_assert(NT % 32 == 0 && NT + 32 <= 1024, "thread count");
    static_assert(OUTW_BYTES % 128 == 0, "out tile alignment");
    static_assert(DT + 2 <= 256 && WT + 2 <= 256 && CS <= 256, "TMA box limits");
};

// Which part of the tile a thread works on: channel pairs [2*CP*cg, 2*CP*(cg+1)), depth d,
// w positions [wg*M, wg*M + M).  Offsets are half indices.
template <class Cfg>
struct FThread {
    int cg, d, wg;
    int in_off;    // into an input stage [(WT+2)][(DT+2)][CS]
    int out_off;   // into the warp's output tile [M][DPW][CS]
    int warp_d0;   // first d of the warp's tile (relative to the CTA tile)
    KDW_HD explicit FThread(int tid) {
        cg = tid % Cfg::CPG;
        d = (tid / Cfg::CPG) % Cfg::DT;
        wg = tid / (Cfg::CPG * Cfg::DT);
        in_off = ((wg * Cfg::M) * (Cfg::DT + 2) + d) * Cfg::CS + cg * 2 * Cfg::CP;
        warp_d0 = d - (tid % 32) / Cfg::CPG;
        out_off = ((tid % 32) / Cfg::CPG) * Cfg::CS + cg * 2 * Cfg::CP;
    }
};

// One input plane q applied to the three output planes that use it: plane q+1 gets the a=0 taps, plane q
// the a=1 taps, plane q-1 the a=2 taps.  The thread sweeps its M+2 input columns once; an input column j
// feeds output m = j - b through tap b.  Carried between steps, per output m:
//   MODE 0 (KDW_ACC_F32): P1 = fp32 sum of plane q's a=0 taps, P2 = fp32 sum of plane q-1's a=0,1 taps;
//          every tap is one mixed-precision FMA (fp16 operands, exact product, fp32 accumulator), so the
//          only rounding to fp16 is the final one.
//   MODE 1 (KDW_ACC_F16): the same sums as packed-half chains (H1, H2), two channels per HFMA2.
// When `store` is set the finished plane q-1 is written to the warp's output tile `ob`.
template <class Cfg, int MODE>
KDW_HD void fprop_step(const __half* __restrict__ in, __half* __restrict__ ob, bool store,
                       const __half2 (&wgt)[27][Cfg::CP], float2 (&P1)[Cfg::M][Cfg::CP], float2 (&P2)[Cfg::M][Cfg::CP],
                       __half2 (&H1)[Cfg::M][Cfg::CP], __half2 (&H2)[Cfg::M][Cfg::CP]) {
    constexpr int CS = Cfg::CS, DT = Cfg::DT, M = Cfg::M, CP = Cfg::CP, DPW = Cfg::DPW;
    float2 F[3][3][CP];   // MODE 0: running fp32 sums of [a][output slot m % 3]
    __half2 S[3][3][CP];  // MODE 1: running packed-half chains
#pragma unroll
    for (int j = 0; j < M + 2; ++j) {
        __half2 xv[3][CP];
#pragma unroll
        for (int t = 0; t < 3; ++t) lds_h2<CP>(xv[t], in + (j * (DT + 2) + t) * CS);
#pragma unroll
        for (int a = 0; a < 3; ++a) {
#pragma unroll
            for (int b = 0; b < 3; ++b) {
                const int m = j - b;  // output this input column feeds through tap b
                if (m < 0 || m >= M) continue;
#pragma unroll
                for (int i = 0; i < CP; ++i) {
                    const __half2 w0 = wgt[(a * 3 + b) * 3 + 0][i];
                    const __half2 w1 = wgt[(a * 3 + b) * 3 + 1][i];
                    const __half2 w2 = wgt[(a * 3 + b) * 3 + 2][i];
                    if (MODE == 0) {
                        float2 f;
                        if (b == 0)
                            f = (a == 0) ? make_float2(0.f, 0.f) : (a == 1 ? P1[m][i] : P2[m][i]);
                        else
                            f = F[a][m % 3][i];
                        f = fma_h2_f2(w0, xv[0][i], f);
                        f = fma_h2_f2(w1, xv[1][i], f);
                        F[a][m % 3][i] = fma_h2_f2(w2, xv[2][i], f);
                    } else {
                        __half2 T;
                        if (b == 0) {
                            if (a == 0)
                                T = h2_mul(w0, xv[0][i]);
                            else
                                T = h2_fma(w0, xv[0][i], a == 1 ? H1[m][i] : H2[m][i]);
                        } else {
                            T = h2_fma(w0, xv[0][i], S[a][m % 3][i]);
                        }
                        T = h2_fma(w1, xv[1][i], T);
                        S[a][m % 3][i] = h2_fma(w2, xv[2][i], T);
                    }
                }
            }
        }
        const int m = j - 2;  // output whose nine taps of this plane are now complete
        if (m >= 0) {
            if (store) {  // plane q-1 is finished
                __half2 o[CP];
#pragma unroll
                for (int i = 0; i < CP; ++i) o[i] = (MODE == 0) ? __float22half2_rn(F[2][m % 3][i]) : S[2][m % 3][i];
                sts_h2<CP>(ob + (m * DPW) * CS, o);
            }
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                if (MODE == 0) {
                    P2[m][i] = F[1][m % 3][i];
                    P1[m][i] = F[0][m % 3][i];
                } else {
                    H2[m][i] = S[1][m % 3][i];
                    H1[m][i] = S[0][m % 3][i];
                }
            }
        }
    }
}

}  // namespace kdw
