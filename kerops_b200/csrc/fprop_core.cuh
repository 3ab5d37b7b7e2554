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
// feeds output m = j - b through tap b.  Two step functions follow, one per accumulate type.
//
// KDW_ACC_F16: the sums are packed-half chains, two channels per HFMA2.  Carried between steps, per output m:
// H1 = plane q's a=0 sum, H2 = plane q-1's a=0,1 sum.  When `store` is set the finished plane q-1 is written to
// the warp's output tile `ob`.
template <class Cfg>
KDW_HD void fprop_step_f16(const __half* __restrict__ in, __half* __restrict__ ob, bool store,
                           const __half2 (&wgt)[27][Cfg::CP], __half2 (&H1)[Cfg::M][Cfg::CP],
                           __half2 (&H2)[Cfg::M][Cfg::CP]) {
    constexpr int CS = Cfg::CS, DT = Cfg::DT, M = Cfg::M, CP = Cfg::CP, DPW = Cfg::DPW;
    __half2 S[3][3][CP];  // running chains of [a][output slot m % 3]
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
        const int m = j - 2;  // output whose nine taps of this plane are now complete
        if (m >= 0) {
            if (store) {  // plane q-1 is finished
                __half2 o[CP];
#pragma unroll
                for (int i = 0; i < CP; ++i) o[i] = S[2][m % 3][i];
                sts_h2<CP>(ob + (m * DPW) * CS, o);
            }
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                H2[m][i] = S[1][m % 3][i];
                H1[m][i] = S[0][m % 3][i];
            }
        }
    }
}

// KDW_ACC_F32: every tap is one mixed-precision FMA (fp16 operands, exact product, fp32 accumulator), so the
// only rounding to fp16 is the final one.  The carried fp32 sums are updated IN PLACE: A holds, per output m, the
// sum of plane q's a=0 taps on entry and of plane q's a=0,1 taps on exit; B holds plane q-1's a=0,1 sums on
// entry, is completed with the a=2 taps (and stored when `store` is set), and then receives plane q+1's a=0 sum.
// So the two arrays swap roles from one step to the next - the caller passes (A, B), then (B, A), ... - and no
// register is ever copied.
template <class Cfg>
KDW_HD void fprop_step_f32(const __half* __restrict__ in, __half* __restrict__ ob, bool store,
                               const __half2 (&wgt)[27][Cfg::CP], float2 (&A)[Cfg::M][Cfg::CP],
                               float2 (&B)[Cfg::M][Cfg::CP]) {
    constexpr int CS = Cfg::CS, DT = Cfg::DT, M = Cfg::M, CP = Cfg::CP, DPW = Cfg::DPW;
    float2 T[3][CP];  // running a=0 sums of the (at most three) outputs in flight
#pragma unroll
    for (int j = 0; j < M + 2; ++j) {
        __half2 xv[3][CP];
#pragma unroll
        for (int t = 0; t < 3; ++t) lds_h2<CP>(xv[t], in + (j * (DT + 2) + t) * CS);
        // a = 2: completes plane q-1 in B
#pragma unroll
        for (int b = 0; b < 3; ++b) {
            const int m = j - b;
            if (m < 0 || m >= M) continue;
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                float2 f = B[m][i];
                f = fma_h2_f2(wgt[(6 + b) * 3 + 0][i], xv[0][i], f);
                f = fma_h2_f2(wgt[(6 + b) * 3 + 1][i], xv[1][i], f);
                B[m][i] = fma_h2_f2(wgt[(6 + b) * 3 + 2][i], xv[2][i], f);
            }
        }
        if (j >= 2 && store) {
            __half2 o[CP];
#pragma unroll
            for (int i = 0; i < CP; ++i) o[i] = __float22half2_rn(B[j - 2][i]);
            sts_h2<CP>(ob + ((j - 2) * DPW) * CS, o);
        }
        // a = 1: plane q's sum grows in A
#pragma unroll
        for (int b = 0; b < 3; ++b) {
            const int m = j - b;
            if (m < 0 || m >= M) continue;
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                float2 f = A[m][i];
                f = fma_h2_f2(wgt[(3 + b) * 3 + 0][i], xv[0][i], f);
                f = fma_h2_f2(wgt[(3 + b) * 3 + 1][i], xv[1][i], f);
                A[m][i] = fma_h2_f2(wgt[(3 + b) * 3 + 2][i], xv[2][i], f);
            }
        }
        // a = 0: plane q+1 starts in T; its last tap lands in B[m], which the a = 2 pass has just released
#pragma unroll
        for (int b = 0; b < 3; ++b) {
            const int m = j - b;
            if (m < 0 || m >= M) continue;
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                float2 f = (b == 0) ? make_float2(0.f, 0.f) : T[m % 3][i];
                f = fma_h2_f2(wgt[b * 3 + 0][i], xv[0][i], f);
                f = fma_h2_f2(wgt[b * 3 + 1][i], xv[1][i], f);
                f = fma_h2_f2(wgt[b * 3 + 2][i], xv[2][i], f);
                if (b == 2)
                    B[m][i] = f;
                else
                    T[m % 3][i] = f;
            }
        }
    }
}

// fprop_step_f32 with a fused epilogue: the finished plane gets a residual added in fp16 (as a separate
// elementwise add of two fp16 tensors would) and, for the thread's `mv` valid outputs, the stored fp16 values
// and their squares are accumulated in fp32 (S1, S2) for per-channel statistics.  `res` points at the thread's
// first residual value in a [WT][DT][CS] tile.  The reference runs this as a second operator over the
// convolution's output (kerops/kernels/addition.py:5-37).
template <class Cfg>
KDW_HD void fprop_step_f32_addstats(const __half* __restrict__ in, const __half* __restrict__ res,
                                    __half* __restrict__ ob, bool store, int mv, const __half2 (&wgt)[27][Cfg::CP],
                                    float2 (&A)[Cfg::M][Cfg::CP], float2 (&B)[Cfg::M][Cfg::CP],
                                    float2 (&S1)[Cfg::CP], float2 (&S2)[Cfg::CP]) {
    constexpr int CS = Cfg::CS, DT = Cfg::DT, M = Cfg::M, CP = Cfg::CP, DPW = Cfg::DPW;
    float2 T[3][CP];
#pragma unroll
    for (int j = 0; j < M + 2; ++j) {
        __half2 xv[3][CP];
#pragma unroll
        for (int t = 0; t < 3; ++t) lds_h2<CP>(xv[t], in + (j * (DT + 2) + t) * CS);
#pragma unroll
        for (int b = 0; b < 3; ++b) {
            const int m = j - b;
            if (m < 0 || m >= M) continue;
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                float2 f = B[m][i];
                f = fma_h2_f2(wgt[(6 + b) * 3 + 0][i], xv[0][i], f);
                f = fma_h2_f2(wgt[(6 + b) * 3 + 1][i], xv[1][i], f);
                B[m][i] = fma_h2_f2(wgt[(6 + b) * 3 + 2][i], xv[2][i], f);
            }
        }
        if (j >= 2 && store) {
            const int m = j - 2;
            __half2 o[CP], r[CP];
            lds_h2<CP>(r, res + (m * DT) * CS);
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                o[i] = h2_add(__float22half2_rn(B[m][i]), r[i]);
                if (m < mv) {
                    S1[i] = add_h2_f2(o[i], S1[i]);
                    S2[i] = fma_h2_f2(o[i], o[i], S2[i]);
                }
            }
            sts_h2<CP>(ob + (m * DPW) * CS, o);
        }
#pragma unroll
        for (int b = 0; b < 3; ++b) {
            const int m = j - b;
            if (m < 0 || m >= M) continue;
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                float2 f = A[m][i];
                f = fma_h2_f2(wgt[(3 + b) * 3 + 0][i], xv[0][i], f);
                f = fma_h2_f2(wgt[(3 + b) * 3 + 1][i], xv[1][i], f);
                A[m][i] = fma_h2_f2(wgt[(3 + b) * 3 + 2][i], xv[2][i], f);
            }
        }
#pragma unroll
        for (int b = 0; b < 3; ++b) {
            const int m = j - b;
            if (m < 0 || m >= M) continue;
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                float2 f = (b == 0) ? make_float2(0.f, 0.f) : T[m % 3][i];
                f = fma_h2_f2(wgt[b * 3 + 0][i], xv[0][i], f);
                f = fma_h2_f2(wgt[b * 3 + 1][i], xv[1][i], f);
                f = fma_h2_f2(wgt[b * 3 + 2][i], xv[2][i], f);
                if (b == 2)
                    B[m][i] = f;
                else
                    T[m % 3][i] = f;
            }
        }
    }
}

// fprop_step_f32 with the BN-affine + ReLU applied to every value as it is read from the staged tile:
// x' = fp16(max(x * sc + sh, 0)).  The convolution pads the ACTIVATED tensor with zeros, so the positions outside
// the volume must give 0, not relu(sh): the tile is loaded with NaN as the out-of-bounds fill, NaN survives the
// multiply-add, and the maximum with 0 returns the operand that is a number - no masks, no bounds tests.  Each
// thread needs only the scale / shift of its own CP channel pairs.  A value is activated once per thread that
// reads it (about twice per element), which costs less than a cooperative pass over the tile with a CTA-wide
// barrier per step.
//
// PRO = 0: the multiply-add is computed in fp32 from fp32 scale / shift and rounded to fp16, like the reference's
//          operator (kerops/kernels/bnrelu.py:25-31).
// PRO = 1: scale and shift are rounded to fp16 and the multiply-add is ONE packed-half FMA per channel pair
//          (a single rounding), followed by the packed-half maximum.
template <class Cfg, int PRO>
KDW_HD void fprop_step_f32_bnrelu(const __half* __restrict__ in, __half* __restrict__ ob, bool store,
                                  const __half2 (&wgt)[27][Cfg::CP], const float2 (&sc)[Cfg::CP],
                                  const float2 (&sh)[Cfg::CP], float2 (&A)[Cfg::M][Cfg::CP],
                                  float2 (&B)[Cfg::M][Cfg::CP]) {
    constexpr int CS = Cfg::CS, DT = Cfg::DT, M = Cfg::M, CP = Cfg::CP, DPW = Cfg::DPW;
    float2 T[3][CP];
    __half2 sc16[CP], sh16[CP];
    if (PRO == 1) {
#pragma unroll
        for (int i = 0; i < CP; ++i) {
            sc16[i] = __float22half2_rn(sc[i]);
            sh16[i] = __float22half2_rn(sh[i]);
        }
    }
#pragma unroll
    for (int j = 0; j < M + 2; ++j) {
        __half2 xv[3][CP];
#pragma unroll
        for (int t = 0; t < 3; ++t) {
            lds_h2<CP>(xv[t], in + (j * (DT + 2) + t) * CS);
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                if (PRO == 1) {
                    xv[t][i] = h2_relu_nan0(h2_fma(xv[t][i], sc16[i], sh16[i]));
                } else {
                    float2 f = __half22float2(xv[t][i]);
                    f.x = fmaxf(fmaf(f.x, sc[i].x, sh[i].x), 0.f);  // fmaxf(NaN, 0) = 0
                    f.y = fmaxf(fmaf(f.y, sc[i].y, sh[i].y), 0.f);
                    xv[t][i] = __float22half2_rn(f);
                }
            }
        }
#pragma unroll
        for (int b = 0; b < 3; ++b) {
            const int m = j - b;
            if (m < 0 || m >= M) continue;
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                float2 f = B[m][i];
                f = fma_h2_f2(wgt[(6 + b) * 3 + 0][i], xv[0][i], f);
                f = fma_h2_f2(wgt[(6 + b) * 3 + 1][i], xv[1][i], f);
                B[m][i] = fma_h2_f2(wgt[(6 + b) * 3 + 2][i], xv[2][i], f);
            }
        }
        if (j >= 2 && store) {
            __half2 o[CP];
#pragma unroll
            for (int i = 0; i < CP; ++i) o[i] = __float22half2_rn(B[j - 2][i]);
            sts_h2<CP>(ob + ((j - 2) * DPW) * CS, o);
        }
#pragma unroll
        for (int b = 0; b < 3; ++b) {
            const int m = j - b;
            if (m < 0 || m >= M) continue;
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                float2 f = A[m][i];
                f = fma_h2_f2(wgt[(3 + b) * 3 + 0][i], xv[0][i], f);
                f = fma_h2_f2(wgt[(3 + b) * 3 + 1][i], xv[1][i], f);
                A[m][i] = fma_h2_f2(wgt[(3 + b) * 3 + 2][i], xv[2][i], f);
            }
        }
#pragma unroll
        for (int b = 0; b < 3; ++b) {
            const int m = j - b;
            if (m < 0 || m >= M) continue;
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                float2 f = (b == 0) ? make_float2(0.f, 0.f) : T[m % 3][i];
                f = fma_h2_f2(wgt[b * 3 + 0][i], xv[0][i], f);
                f = fma_h2_f2(wgt[b * 3 + 1][i], xv[1][i], f);
                f = fma_h2_f2(wgt[b * 3 + 2][i], xv[2][i], f);
                if (b == 2)
                    B[m][i] = f;
                else
                    T[m % 3][i] = f;
            }
        }
    }
}

}  // namespace kdw
