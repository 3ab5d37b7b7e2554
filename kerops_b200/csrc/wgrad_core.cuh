// Tile configuration and per-thread step of the weight-gradient TMA kernel (see dwconv_wgrad.cu).
// Kept in a header so the test-suite can run the same step code on the CPU.
#pragma once
#include "kdw_common.cuh"

namespace kdw {

template <int CS_, int DT_, int WT_, int M_, int CP_, int ST_, int MINB_>
struct WCfg {
    static constexpr int CS = CS_, DT = DT_, WT = WT_, M = M_, CP = CP_, ST = ST_, MINB = MINB_;
    static constexpr int CPG = CS / (2 * CP);
    static constexpr int WG = WT / M;
    static constexpr int NT = CPG * DT * WG;
    static constexpr int NW = NT / 32;
    static constexpr int X_BYTES = (WT + 2) * (DT + 2) * CS * 2;
    static constexpr int X_STRIDE = (X_BYTES + 127) / 128 * 128;
    static constexpr int G_BYTES = WT * DT * CS * 2;
    static constexpr int STAGE = X_STRIDE + G_BYTES;
    static constexpr int RED_BYTES = 27 * CS * 4;
    static constexpr int SMEM = ST * STAGE + RED_BYTES + 8 * ST + 128;
    static_assert(CS % (2 * CP) == 0 && WT % M == 0, "tile/thread shape");
    static_assert(NT % 32 == 0 && NT <= 1024, "thread count");
    static_assert(CPG <= 32 && (CPG & (CPG - 1)) == 0, "channel groups must fit a warp");
    static_assert(G_BYTES % 128 == 0, "grad tile alignment");
    static_assert(DT + 2 <= 256 && WT + 2 <= 256 && CS <= 256, "TMA box limits");
};

// Thread -> (channel pairs, depth, w group); offsets are half indices into the x / grad tiles of a stage.
template <class Cfg>
struct WThread {
    int cg, d, wg, x_off, g_off;
    KDW_HD explicit WThread(int tid) {
        cg = tid % Cfg::CPG;
        d = (tid / Cfg::CPG) % Cfg::DT;
        wg = tid / (Cfg::CPG * Cfg::DT);
        x_off = ((wg * Cfg::M) * (Cfg::DT + 2) + d) * Cfg::CS + cg * 2 * Cfg::CP;
        g_off = ((wg * Cfg::M) * Cfg::DT + d) * Cfg::CS + cg * 2 * Cfg::CP;
    }
};

// x plane q against the grad planes q+1 (a=0), q (a=1), q-1 (a=2) selected by AM.
template <class Cfg, int AM>
KDW_HD void wgrad_step(const __half* __restrict__ xin, const __half* __restrict__ gin,
                                           __half2 (&G)[3][Cfg::M][Cfg::CP], float2 (&acc)[27][Cfg::CP]) {
    constexpr int CS = Cfg::CS, DT = Cfg::DT, M = Cfg::M, CP = Cfg::CP;
    // slide the grad window: G[2] = plane q+1, G[1] = plane q, G[0] = plane q-1
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int i = 0; i < CP; ++i) {
            G[0][m][i] = G[1][m][i];
            G[1][m][i] = G[2][m][i];
        }
    if (AM & 1) {
#pragma unroll
        for (int m = 0; m < M; ++m) lds_h2<CP>(G[2][m], gin + (m * DT) * CS);
    }
    __half2 p[27][CP];  // this step's packed-half chains
#pragma unroll
    for (int j = 0; j < M + 2; ++j) {
        __half2 xv[3][CP];
#pragma unroll
        for (int t = 0; t < 3; ++t) lds_h2<CP>(xv[t], xin + (j * (DT + 2) + t) * CS);
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            if (!((AM >> a) & 1)) continue;
#pragma unroll
            for (int b = 0; b < 3; ++b) {
                const int m = j - b;  // grad position whose tap-b neighbour this x column is
                if (m < 0 || m >= M) continue;
#pragma unroll
                for (int t = 0; t < 3; ++t) {
#pragma unroll
                    for (int i = 0; i < CP; ++i) {
                        const int k = (a * 3 + b) * 3 + t;
                        if (m == 0)
                            p[k][i] = h2_mul(G[2 - a][m][i], xv[t][i]);
                        else
                            p[k][i] = h2_fma(G[2 - a][m][i], xv[t][i], p[k][i]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        if (!((AM >> a) & 1)) continue;
#pragma unroll
        for (int bt = 0; bt < 9; ++bt)
#pragma unroll
            for (int i = 0; i < CP; ++i) acc[a * 9 + bt][i] = add_h2_f2(p[a * 9 + bt][i], acc[a * 9 + bt][i]);
    }
}

}  // namespace kdw
