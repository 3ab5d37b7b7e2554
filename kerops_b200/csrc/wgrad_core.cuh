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
    static constexpr int NT = CPG * DT * WG;  // consumer threads
    static constexpr int NCW = NT / 32;       // consumer warps; warp NCW is the TMA producer
    static constexpr int X_BYTES = (WT + 2) * (DT + 2) * CS * 2;
    static constexpr int X_STRIDE = (X_BYTES + 127) / 128 * 128;
    static constexpr int G_BYTES = WT * DT * CS * 2;
    static constexpr int STAGE = X_STRIDE + G_BYTES;
    static constexpr int RED_BYTES = 27 * CS * 4;
    static constexpr int SMEM = ST * STAGE + RED_BYTES + 16 * ST + 128;
    static_assert(CS % (2 * CP) == 0 && WT % M == 0, "tile/thread shape");
    static_assert(NT % 32 == 0 && NT + 32 <= 1024, "thread count");
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

// x plane q against the grad planes q+1 (tap a=0), q (a=1) and q-1 (a=2):
//     acc[a][b][t] += grad[q+1-a][m] * x[q][m+b][d+t]      for the thread's M positions m,
// every product one mixed-precision FMA (exact fp16 product, fp32 accumulate).  The three grad planes sit
// in registers G[.]; R = (step count) % 3 says which slot holds which plane, so the window slides without
// register moves: slot (R+2)%3 receives plane q+1 (zeros when that plane is not owned by the segment),
// slot (R+1)%3 holds plane q, slot R holds plane q-1.
template <class Cfg, int R>
KDW_HD void wgrad_step(const __half* __restrict__ xin, const __half* __restrict__ gin, bool load_g,
                       __half2 (&G)[3][Cfg::M][Cfg::CP], float2 (&acc)[27][Cfg::CP]) {
    constexpr int CS = Cfg::CS, DT = Cfg::DT, M = Cfg::M, CP = Cfg::CP;
    constexpr int SLOT[3] = {(R + 2) % 3, (R + 1) % 3, R % 3};  // slot of the grad plane paired with tap a
#pragma unroll
    for (int m = 0; m < M; ++m) {
        if (load_g) {
            lds_h2<CP>(G[SLOT[0]][m], gin + (m * DT) * CS);
        } else {
#pragma unroll
            for (int i = 0; i < CP; ++i) G[SLOT[0]][m][i] = __float2half2_rn(0.f);
        }
    }
#pragma unroll
    for (int j = 0; j < M + 2; ++j) {
        __half2 xv[3][CP];
#pragma unroll
        for (int t = 0; t < 3; ++t) lds_h2<CP>(xv[t], xin + (j * (DT + 2) + t) * CS);
#pragma unroll
        for (int a = 0; a < 3; ++a) {
#pragma unroll
            for (int b = 0; b < 3; ++b) {
                const int m = j - b;  // grad position whose tap-b neighbour this x column is
                if (m < 0 || m >= M) continue;
#pragma unroll
                for (int t = 0; t < 3; ++t) {
#pragma unroll
                    for (int i = 0; i < CP; ++i) {
                        const int k = (a * 3 + b) * 3 + t;
                        acc[k][i] = fma_h2_f2(G[SLOT[a]][m][i], xv[t][i], acc[k][i]);
                    }
                }
            }
        }
    }
}

}  // namespace kdw
