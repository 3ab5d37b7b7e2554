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
    static constexpr int CPG = CS / (2 * CP);
    static constexpr int WG = WT / M;
    static constexpr int NT = CPG * DT * WG;
    static constexpr int IN_BYTES = (WT + 2) * (DT + 2) * CS * 2;
    static constexpr int IN_STRIDE = (IN_BYTES + 127) / 128 * 128;
    static constexpr int OUT_BYTES = WT * DT * CS * 2;
    static constexpr int SMEM = ST * IN_STRIDE + 2 * OUT_BYTES + 8 * ST + 128;
    static_assert(CS % (2 * CP) == 0 && WT % M == 0, "tile/thread shape");
    static_assert(NT % 32 == 0 && NT <= 1024, "thread count");
    static_assert(OUT_BYTES % 128 == 0, "out tile alignment");
    static_assert(DT + 2 <= 256 && WT + 2 <= 256 && CS <= 256, "TMA box limits");
};

// Which part of the tile a thread works on: channel pairs [2*CP*cg, 2*CP*(cg+1)), depth d,
// w positions [wg*M, wg*M + M).  Offsets are half indices into an input stage / output tile.
template <class Cfg>
struct FThread {
    int cg, d, wg, in_off, out_off;
    KDW_HD explicit FThread(int tid) {
        cg = tid % Cfg::CPG;
        d = (tid / Cfg::CPG) % Cfg::DT;
        wg = tid / (Cfg::CPG * Cfg::DT);
        in_off = ((wg * Cfg::M) * (Cfg::DT + 2) + d) * Cfg::CS + cg * 2 * Cfg::CP;
        out_off = ((wg * Cfg::M) * Cfg::DT + d) * Cfg::CS + cg * 2 * Cfg::CP;
    }
};

// One input plane applied to the (up to) three output planes selected by AM (bit a = taps a).
//
// MODE 0 (KDW_ACC_F32): every (a, b) row of three d-taps is a packed-half chain (mul, fma, fma) that is
//   added to an fp32 accumulator - the arithmetic of the reference kernel (fp16 products, fp16 sum of
//   the three d-taps, fp32 sum of the nine partials; kerops/kernels/dw_conv.py:49-52,71-121) with fused
//   multiply-adds.  Carried state: P1 = fp32 partial of plane q (its a=0 taps), P2 = of plane q-1
//   (a=0 and a=1 taps).
// MODE 1 (KDW_ACC_F16): all 27 taps of an output in one packed-half chain (carried in H1 / H2).
// MODE 2 (KDW_ACC_F32_PLANE): the nine taps of a plane in one packed-half chain, the three plane partials
//   added in fp32 (carried: H1 = half partial of plane q, P2 = fp32 partial of plane q-1).
template <class Cfg, int MODE, int AM>
KDW_HD void fprop_step(const __half* __restrict__ in, __half* __restrict__ ob, const __half2 (&wgt)[27][Cfg::CP],
                       float2 (&P1)[Cfg::M][Cfg::CP], float2 (&P2)[Cfg::M][Cfg::CP], __half2 (&H1)[Cfg::M][Cfg::CP],
                       __half2 (&H2)[Cfg::M][Cfg::CP]) {
    constexpr int CS = Cfg::CS, DT = Cfg::DT, M = Cfg::M, CP = Cfg::CP;
    __half2 S[3][3][CP];  // MODE 1/2: running chain of [a][output slot m % 3]
    float2 F[3][3][CP];   // MODE 0: running fp32 sum of [a][output slot m % 3]
#pragma unroll
    for (int j = 0; j < M + 2; ++j) {
        __half2 xv[3][CP];
#pragma unroll
        for (int t = 0; t < 3; ++t) lds_h2<CP>(xv[t], in + (j * (DT + 2) + t) * CS);
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            if (!((AM >> a) & 1)) continue;
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
                        __half2 T = h2_mul(w0, xv[0][i]);
                        T = h2_fma(w1, xv[1][i], T);
                        T = h2_fma(w2, xv[2][i], T);
                        if (b == 0) {
                            if (a == 0)
                                F[a][m % 3][i] = __half22float2(T);
                            else if (a == 1)
                                F[a][m % 3][i] = add_h2_f2(T, P1[m][i]);
                            else
                                F[a][m % 3][i] = add_h2_f2(T, P2[m][i]);
                        } else {
                            F[a][m % 3][i] = add_h2_f2(T, F[a][m % 3][i]);
                        }
                    } else {
                        __half2 T;
                        if (b == 0) {
                            if (MODE == 2 || a == 0)
                                T = h2_mul(w0, xv[0][i]);
                            else if (a == 1)
                                T = h2_fma(w0, xv[0][i], H1[m][i]);
                            else
                                T = h2_fma(w0, xv[0][i], H2[m][i]);
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
            if (AM & 4) {  // plane q-1 is finished
                __half2 o[CP];
#pragma unroll
                for (int i = 0; i < CP; ++i) {
                    if (MODE == 0)
                        o[i] = __float22half2_rn(F[2][m % 3][i]);
                    else if (MODE == 1)
                        o[i] = S[2][m % 3][i];
                    else
                        o[i] = __float22half2_rn(add_h2_f2(S[2][m % 3][i], P2[m][i]));
                }
                sts_h2<CP>(ob + (m * DT) * CS, o);
            }
            if (AM & 2) {  // plane q: what earlier steps gave it + this step's a=1 taps
#pragma unroll
                for (int i = 0; i < CP; ++i) {
                    if (MODE == 0)
                        P2[m][i] = F[1][m % 3][i];
                    else if (MODE == 1)
                        H2[m][i] = S[1][m % 3][i];
                    else
                        P2[m][i] = add_h2_f2(S[1][m % 3][i], __half22float2(H1[m][i]));
                }
            }
            if (AM & 1) {  // plane q+1: its first partial
#pragma unroll
                for (int i = 0; i < CP; ++i) {
                    if (MODE == 0)
                        P1[m][i] = F[0][m % 3][i];
                    else
                        H1[m][i] = S[0][m % 3][i];
                }
            }
        }
    }
}

}  // namespace kdw
