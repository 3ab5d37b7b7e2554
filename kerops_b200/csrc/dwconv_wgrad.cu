// Depthwise 3x3x3 channels-last fp16 weight gradient for sm_100a.
//
// Replaces kerops/kernels/dw_conv.py:147-287 (_DWConv_wgrad_cl3d_impl), the zero-filled fp16 partial
// buffer and the torch sum over it (kerops/ops/conv/dwconv_wgrad.py:54-77).
//
// Pass 1 (TMA kernel, C multiple of 8).  Same column march as the forward kernel: a producer warp streams,
// per step, the halo'd x plane q and the grad plane q+1 into a ring of shared-memory stages by TMA; full /
// empty mbarriers connect it to the consumer warps.  A consumer thread - fixed (channel pairs, d), M
// consecutive w positions - keeps the grad values of planes q-1, q, q+1 in registers and multiplies every x
// value it reads with the (up to) nine grad values whose tap it is:
//     dw[a][b][t] += grad[q+1-a][m] * x[q][m+b][d+t],
// each product one sm_100 mixed-precision FMA (fp16 operands, exact product, fp32 accumulator).  At the end
// of a segment the consumer warps reduce over their threads (warp shuffles, then warps in fixed order
// through shared memory) and add the [27][CS] result to the CTA's own fp32 row of the workspace.
// Pass 2 adds the rows in a fixed order and writes the fp32 and fp16 [3][3][3][C] results.
// There are no atomics anywhere, so results are bitwise reproducible.
//
// Plain pass 1 (any C, used for C < 8): one thread per (tap, channel), fp32 FMAs.
#include <mutex>

#include "../../include/kdw.h"
#include "kdw_common.cuh"
#include "wgrad_core.cuh"

namespace kdw {

static constexpr int kMaxRowsFloor = 1184;  // workspace rows are max(8 * SMs, this)

// ------------------------------------------------------------------------------------------------
// Pass 2: fixed-order sum over the CTA rows
// ------------------------------------------------------------------------------------------------
// One warp per output element k: lane l adds rows l, l+32, ... in order, then the 32 lane sums are combined
// by a fixed shuffle tree - the same order on every run.  OVERLAP: launched with launch_overlapping_previous,
// so pass 1 may still be running when the CTAs are placed.
template <bool OVERLAP>
__global__ void __launch_bounds__(128) wgrad_reduce_kernel(const float* __restrict__ ws, int rows, int KC,
                                                          float* __restrict__ dw32, __half* __restrict__ dw16) {
    const int k = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (k >= KC) return;
    if (OVERLAP) grid_dependency_wait();
    float acc = 0.f;
    for (int r = lane; r < rows; r += 32) acc += ws[(size_t)r * KC + k];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) {
        if (dw32) dw32[k] = acc;
        if (dw16) dw16[k] = __float2half_rn(acc);
    }
}

// ------------------------------------------------------------------------------------------------
// Plain pass 1
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) wgrad_plain_kernel(const __half* __restrict__ x, const __half* __restrict__ g,
                                                         float* __restrict__ ws, long long voxels, int C, int Hx, int W,
                                                         int D, long long xsN, long long xsH, long long xsW,
                                                         long long gsN, long long gsH, long long gsW, int h_begin,
                                                         int Hr, int g_h0) {
    const int KC = 27 * C;
    const long long lo = (long long)blockIdx.x * voxels / gridDim.x;
    const long long hi = (long long)(blockIdx.x + 1) * voxels / gridDim.x;
    for (int k = threadIdx.x; k < KC; k += blockDim.x) {
        const int c = k % C;
        const int tap = k / C;
        const int a = tap / 9, b = (tap / 3) % 3, t = tap % 3;
        float acc = 0.f;
        for (long long v = lo; v < hi; ++v) {
            long long r = v;
            const int d = (int)(r % D);
            r /= D;
            const int wv = (int)(r % W);
            r /= W;
            const int h = h_begin + (int)(r % Hr);
            const long long n = r / Hr;
            const int hh = h + a - 1, ww = wv + b - 1, dd = d + t - 1;
            if (hh < 0 || hh >= Hx || ww < 0 || ww >= W || dd < 0 || dd >= D) continue;
            const float gv = __half2float(g[n * gsN + (long long)(h - g_h0) * gsH + wv * gsW + (long long)d * C + c]);
            const float xv = __half2float(x[n * xsN + hh * xsH + ww * xsW + (long long)dd * C + c]);
            acc = fmaf(gv, xv, acc);
        }
        ws[(size_t)blockIdx.x * KC + k] = acc;
    }
}

// ------------------------------------------------------------------------------------------------
// TMA pass 1
// ------------------------------------------------------------------------------------------------
// Adds the consumer threads' accumulators for channel slice c0 to the CTA's workspace row and clears them:
// shuffle reduction over the lanes that share channels, then the warps take turns in a fixed order through
// shared memory (no atomics, so the sum is reproducible).  Called by all consumer threads of the CTA - also by
// warps whose bounded wait ran out (`failed`): the first barrier ORs that flag over all consumer threads, so
// either every warp adds its sums or none does, and no warp is left waiting at a barrier the others never reach.
// Returns true when the flush was abandoned.
template <class Cfg>
__device__ __forceinline__ bool flush_acc(float2 (&acc)[27][Cfg::CP], float* red, float* row, int C, int c0, int tid,
                                          bool failed) {
    constexpr int CS = Cfg::CS, CP = Cfg::CP, CPG = Cfg::CPG, NCW = Cfg::NCW;
    const int lane = tid & 31, warp = tid >> 5, cg = tid % CPG;
    if (named_barrier_or(1, Cfg::NT, failed)) return true;
#pragma unroll
    for (int k = 0; k < 27; ++k)
#pragma unroll
        for (int i = 0; i < CP; ++i) {
            float2 v = acc[k][i];
#pragma unroll
            for (int off = CPG; off < 32; off <<= 1) {
                v.x += __shfl_xor_sync(0xffffffffu, v.x, off);
                v.y += __shfl_xor_sync(0xffffffffu, v.y, off);
            }
            acc[k][i] = v;
        }
    for (int wi = 0; wi < NCW; ++wi) {
        if (warp == wi && lane < CPG) {
#pragma unroll
            for (int k = 0; k < 27; ++k)
#pragma unroll
                for (int i = 0; i < CP; ++i) {
                    float* dst = red + k * CS + cg * 2 * CP + 2 * i;
                    if (wi == 0) {
                        dst[0] = acc[k][i].x;
                        dst[1] = acc[k][i].y;
                    } else {
                        dst[0] += acc[k][i].x;
                        dst[1] += acc[k][i].y;
                    }
                }
        }
        named_barrier_sync(1, Cfg::NT);
    }
    for (int e = tid; e < 27 * CS; e += Cfg::NT) {
        const int k = e / CS, c = e % CS;
        row[k * C + c0 + c] += red[e];
    }
    named_barrier_sync(1, Cfg::NT);
#pragma unroll
    for (int k = 0; k < 27; ++k)
#pragma unroll
        for (int i = 0; i < CP; ++i) acc[k][i] = make_float2(0.f, 0.f);
    return false;
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NT + 32, Cfg::MINB)
    wgrad_tma_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmg,
                     float* __restrict__ ws, const Sched s, const int C, const int g_h0, int* status,
                     const WaitTest wt) {
    constexpr int CS = Cfg::CS, M = Cfg::M, CP = Cfg::CP, ST = Cfg::ST, CPG = Cfg::CPG, NCW = Cfg::NCW;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    unsigned char* stage_base = smem;  // ST stages of [x tile | grad tile]
    float* red = reinterpret_cast<float*>(smem + ST * Cfg::STAGE);
    const uint32_t full0 = smem_u32(smem + ST * Cfg::STAGE + Cfg::RED_BYTES);  // full[ST], then empty[ST]
    const uint32_t empty0 = full0 + 8 * ST;

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int KC = 27 * C;
    float* row = ws + (size_t)blockIdx.x * KC;  // this CTA's fp32 [27][C] row of the workspace

    if (tid == 0) {
        prefetch_tmap(&tmx);
        prefetch_tmap(&tmg);
        for (int k = 0; k < ST; ++k) {
            mbar_init(full0 + 8 * k, 1);
            mbar_init(empty0 + 8 * k, NCW);
        }
        mbar_fence_init();
    }
    for (int k = tid; k < KC; k += Cfg::NT + 32) row[k] = 0.f;
    __syncthreads();  // the only CTA-wide barrier

    if (warp == NCW) {
        // ---------------- producer warp ----------------
        if (lane != 0) return;
        StepIter it;
        it.init(s, (int)blockIdx.x, (int)gridDim.x);
        uint32_t pi = 0;
        bool ok = true;
        while (it.active) {
            if (wt.stop_after >= 0 && (int)pi >= wt.stop_after) return;  // test hook: the consumers' wait runs out
            const uint32_t st = pi % ST;
            if (pi >= ST) ok = mbar_wait_bounded(empty0 + 8 * st, ((pi / ST) & 1u) ^ 1u, wt.limit_ns);
            if (!ok) break;
            const bool with_g = it.q + 1 < it.g.he;  // grad plane q+1 is owned by the segment
            const uint32_t bar = full0 + 8 * st;
            mbar_expect_tx(bar, Cfg::X_BYTES + (with_g ? Cfg::G_BYTES : 0));
            tma_load_5d(status, smem_u32(stage_base + st * Cfg::STAGE), &tmx, bar, it.g.c0, it.g.d0 - 1, it.g.w0 - 1,
                        it.q, it.g.n);
            if (with_g)
                tma_load_5d(status, smem_u32(stage_base + st * Cfg::STAGE + Cfg::X_STRIDE), &tmg, bar, it.g.c0, it.g.d0,
                            it.g.w0, it.q + 1 - g_h0, it.g.n);
            ++pi;
            it.next(s);
        }
        if (!ok) {
            atomicExch(status, (int)KDW_STATUS_TMA_TIMEOUT);
            const uint32_t first = pi > ST ? pi - ST : 0;
            for (uint32_t k = first; k < pi; ++k)
                (void)mbar_wait_bounded(full0 + 8 * (k % ST), (k / ST) & 1u, wt.limit_ns);
        }
        return;
    }

    // ---------------- consumer warps ----------------
    const WThread<Cfg> th(tid);
    const int cg = th.cg;
    StepIter it;
    it.init(s, (int)blockIdx.x, (int)gridDim.x);

    __half2 G[3][M][CP];
    float2 acc[27][CP];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int i = 0; i < CP; ++i) G[0][m][i] = G[1][m][i] = G[2][m][i] = __float2half2_rn(0.f);
#pragma unroll
    for (int k = 0; k < 27; ++k)
#pragma unroll
        for (int i = 0; i < CP; ++i) acc[k][i] = make_float2(0.f, 0.f);

    uint32_t ci = 0;
    // A warp whose wait ran out keeps walking the schedule without waiting or computing, so that it still meets
    // the other consumer warps at every flush; the flush then decides for all of them (see flush_acc).
    bool failed = false;
    int cur_c0 = -1;  // channel slice the accumulators belong to
    while (it.active) {
        const uint32_t st = ci % ST;
        if (!failed) {
            const bool ok = mbar_wait_bounded(full0 + 8 * st, (ci / ST) & 1u, wt.limit_ns);
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0) atomicExch(status, (int)KDW_STATUS_TMA_TIMEOUT);
                failed = true;
            }
        }
        const int q = it.q;
        if (q == it.g.hb - 1) {
            // new segment: grad planes of the previous segment must not be paired with this segment's x
#pragma unroll
            for (int m = 0; m < M; ++m)
#pragma unroll
                for (int i = 0; i < CP; ++i) G[0][m][i] = G[1][m][i] = G[2][m][i] = __float2half2_rn(0.f);
            // The accumulators belong to a channel slice, not to a column: they are carried from segment to
            // segment and flushed to the workspace row only when the slice changes (in the round phase a CTA
            // keeps its slice whenever the CTA count is a multiple of the slice count) and at the end.
            if (it.g.c0 != cur_c0) {
                if (cur_c0 >= 0 && flush_acc<Cfg>(acc, red, row, C, cur_c0, tid, failed)) failed = true;
                cur_c0 = it.g.c0;
            }
        }
        if (!failed) {
            const bool load_g = q + 1 < it.g.he;
            const __half* xin = reinterpret_cast<const __half*>(stage_base + st * Cfg::STAGE) + th.x_off;
            const __half* gin =
                reinterpret_cast<const __half*>(stage_base + st * Cfg::STAGE + Cfg::X_STRIDE) + th.g_off;
            switch (ci % 3) {
                case 0: wgrad_step<Cfg, 0>(xin, gin, load_g, G, acc); break;
                case 1: wgrad_step<Cfg, 1>(xin, gin, load_g, G, acc); break;
                default: wgrad_step<Cfg, 2>(xin, gin, load_g, G, acc); break;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * st);  // this warp is done with the stage
        }
        it.next(s);
        ++ci;
    }
    if (cur_c0 >= 0) (void)flush_acc<Cfg>(acc, red, row, C, cur_c0, tid, failed);
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
struct WgradArgs {
    const void* x;
    const void* g;
    float* ws;
    int64_t ws_rows;
    int64_t N, C, Hx, W, D, xsN, xsH, xsW, Hg, gsN, gsH, gsW;
    int h_begin, h_end, g_h0;
    cudaStream_t stream;
};

template <class Cfg>
static int launch_wgrad_tma(const WgradArgs& a, int* rows_used) {
    CUtensorMap tmx, tmg;
    int rc = encode_volume_map(&tmx, a.x, a.N, a.C, a.Hx, a.W, a.D, a.xsN, a.xsH, a.xsW, Cfg::CS, Cfg::DT + 2,
                               Cfg::WT + 2);
    if (rc) return rc;
    rc = encode_volume_map(&tmg, a.g, a.N, a.C, a.Hg, a.W, a.D, a.gsN, a.gsH, a.gsW, Cfg::CS, Cfg::DT, Cfg::WT);
    if (rc) return rc;
    auto kern = wgrad_tma_kernel<Cfg>;
    static KernelSetup setup;  // one per kernel instantiation
    int occ = 0, sms = 0;
    rc = setup.get((const void*)kern, Cfg::NT + 32, Cfg::SMEM, &sms, &occ);
    if (rc) return rc;
    int* status = nullptr;
    rc = status_ptr(&status);
    if (rc) return rc;
    long long target = (long long)sms * occ;
    if (target > a.ws_rows) target = a.ws_rows;
    Sched s;
    const int grid = make_sched(&s, a.N, a.C, a.W, a.D, a.h_begin, a.h_end, Cfg::WT, Cfg::DT, Cfg::CS, (int)target);
    kern<<<grid, Cfg::NT + 32, Cfg::SMEM, a.stream>>>(tmx, tmg, a.ws, s, (int)a.C, a.g_h0, status, wait_test());
    KDW_CUDA(cudaGetLastError());
    *rows_used = grid;
    return 0;
}

typedef int (*WgradLaunch)(const WgradArgs&, int*);
struct WgradVariant {
    int cs, dt, wt;
    WgradLaunch f;
};
#define KDW_VARIANT(ID, CS, DT, WT, M, CP, ST, MINB) \
    {CS, DT, WT, &launch_wgrad_tma<WCfg<CS, DT, WT, M, CP, ST, MINB>>},
// index = id - 1
static const WgradVariant g_wgrad_variants[] = {
#include "wgrad_variants.inc"
};
#undef KDW_VARIANT
static const int g_n_table_wgrad_variants = (int)(sizeof(g_wgrad_variants) / sizeof(g_wgrad_variants[0]));

// tensor-core variants (dwconv_wgrad_mma.cu) are numbered after the table
int wgrad_mma_variants();
int wgrad_mma_variant_channels(int which);
int launch_wgrad_mma_variant(int which, const void* x, const void* grad, float* ws, int64_t ws_rows, int64_t N, int64_t C,
                             int64_t Hx, int64_t W, int64_t D, int64_t xsN, int64_t xsH, int64_t xsW, int64_t Hg,
                             int64_t gsN, int64_t gsH, int64_t gsW, int h_begin, int h_end, int g_h0,
                             cudaStream_t stream, int* rows_used);
static int n_wgrad_variants() { return g_n_table_wgrad_variants + wgrad_mma_variants(); }

// Built-in choice: per channel count a short list of candidates with their time relative to the best one, measured
// on B200 at (1,C,350,350,128); each candidate's time is scaled by the padded / real area of its tiles on this
// W x D and the cheapest one wins.  The tensor-core kernels (ids after the table, dwconv_wgrad_mma.cu) lead for
// every C; the CUDA-core tiles remain as candidates for shapes their tiles fit better.
struct WgradCand {
    int id;
    float rel;
};
void wgrad_mma_variant_tile(int which, int* wt, int* dt);
bool wgrad_mma_variant_fits(int which, int64_t C, int64_t D);
static const int kTW = (int)(sizeof(g_wgrad_variants) / sizeof(g_wgrad_variants[0]));  // tensor-core variant i: kTW + 1 + i
static const WgradCand kWgradCand8[] = {{kTW + 7, 1.00f}, {kTW + 4, 1.48f}, {24, 1.70f}, {11, 1.80f}, {1, 1.85f}};
static const WgradCand kWgradCand16[] = {{kTW + 8, 1.00f}, {kTW + 9, 1.10f}, {kTW + 3, 1.18f}, {1, 2.00f}, {2, 2.30f}};
static const WgradCand kWgradCand32[] = {{kTW + 2, 1.00f}, {kTW + 3, 1.03f}, {kTW + 6, 1.04f}, {14, 1.70f}};
static const WgradCand kWgradCand64[] = {{kTW + 1, 1.00f}, {kTW + 5, 1.03f}, {kTW + 6, 1.10f}, {kTW + 2, 1.11f}, {22, 1.65f}};
static const WgradCand kWgradCand128[] = {{kTW + 1, 1.00f}, {kTW + 5, 1.02f}, {kTW + 2, 1.14f}, {22, 1.78f}};

static void wgrad_variant_tile(int id, int* wt, int* dt) {
    if (id > kTW) {
        wgrad_mma_variant_tile(id - kTW - 1, wt, dt);
    } else {
        *wt = g_wgrad_variants[id - 1].wt;
        *dt = g_wgrad_variants[id - 1].dt;
    }
}

#define KDW_CANDS(a) cand = a, n = (int)(sizeof(a) / sizeof(a[0]))
// table_only: consider the CUDA-core tiles only (one workspace row per CTA; the built-in workspace of
// kdw_wgrad_f16_static is sized for that).
static int auto_wgrad_variant(int64_t C, int64_t W, int64_t D, bool table_only = false) {
    const WgradCand* cand;
    int n;
    if (C == 8) KDW_CANDS(kWgradCand8);
    else if (C == 16) KDW_CANDS(kWgradCand16);
    else if (C == 32) KDW_CANDS(kWgradCand32);
    else if (C == 64) KDW_CANDS(kWgradCand64);
    else KDW_CANDS(kWgradCand128);
    int best = 0;
    double best_cost = 0.0;
    for (int i = 0; i < n; ++i) {
        if (table_only && cand[i].id > kTW) continue;
        if (cand[i].id > kTW && !wgrad_mma_variant_fits(cand[i].id - kTW - 1, C, D)) continue;
        int wt = 1, dt = 1;
        wgrad_variant_tile(cand[i].id, &wt, &dt);
        const double padded = (double)((W + wt - 1) / wt * wt) * (double)((D + dt - 1) / dt * dt);
        const double cost = cand[i].rel * padded / ((double)W * (double)D);
        if (best == 0 || cost < best_cost) {
            best = cand[i].id;
            best_cost = cost;
        }
    }
    return best;
}
#undef KDW_CANDS

static int64_t ws_rows_for_device(int* rc_out) {
    int sms = 0;
    *rc_out = device_sm_count(&sms);
    if (*rc_out) return 0;
    int64_t rows = (int64_t)sms * 8;
    if (rows < kMaxRowsFloor) rows = kMaxRowsFloor;
    return rows;
}

static int wgrad_dispatch(const void* x, const void* grad, void* workspace, int64_t workspace_bytes, float* dw_f32,
                          void* dw_f16, int64_t N, int64_t C, int64_t Hx, int64_t W, int64_t D, int64_t xsN, int64_t xsH,
                          int64_t xsW, int64_t Hg, int64_t gsN, int64_t gsH, int64_t gsW, int64_t h_begin,
                          int64_t h_end, int64_t g_h0, int tune, void* stream) {
    if (!x || !grad || !workspace || (!dw_f32 && !dw_f16)) {
        set_error("wgrad: null pointer (x, grad, workspace and at least one output are required)");
        return KDW_ERR_ARG;
    }
    if (N <= 0 || C <= 0 || Hx <= 0 || W <= 0 || D <= 0 || Hg <= 0 || (C & (C - 1)) != 0) {
        set_error("wgrad: sizes must be positive and C a power of two (N=%lld C=%lld H=%lld W=%lld D=%lld)",
                  (long long)N, (long long)C, (long long)Hx, (long long)W, (long long)D);
        return KDW_ERR_ARG;
    }
    if (Hx > 0x7fffffff || W > 0x7fffffff || D > 0x7fffffff || N > 0x7fffffff || C > (1 << 20)) {
        set_error("wgrad: extent does not fit in 32 bits");
        return KDW_ERR_ARG;
    }
    if (h_begin < 0 || h_end > Hx || h_begin > h_end || h_begin - g_h0 < 0 || h_end - g_h0 > Hg) {
        set_error("wgrad: plane range [%lld,%lld) / g_h0=%lld outside x (%lld planes) or grad (%lld planes)",
                  (long long)h_begin, (long long)h_end, (long long)g_h0, (long long)Hx, (long long)Hg);
        return KDW_ERR_RANGE;
    }
    if (((uintptr_t)workspace & 15) != 0) {
        set_error("wgrad: workspace must be 16-byte aligned");
        return KDW_ERR_ALIGN;
    }
    if (tune < 0 || tune > n_wgrad_variants()) {
        set_error("wgrad: tune=%d names no kernel variant (1..%d)", tune, n_wgrad_variants());
        return KDW_ERR_TUNE;
    }
    int rc = 0;
    const int64_t rows_cap = ws_rows_for_device(&rc);
    if (rc) return rc;
    const int KC = (int)(27 * C);
    if (workspace_bytes < rows_cap * KC * 4) {
        set_error("wgrad: workspace has %lld bytes, needs %lld", (long long)workspace_bytes,
                  (long long)(rows_cap * KC * 4));
        return KDW_ERR_WORKSPACE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    float* ws = (float*)workspace;
    int rows = 0;
    if (h_begin == h_end) {
        // empty range: the gradient is zero
        if (dw_f32) KDW_CUDA(cudaMemsetAsync(dw_f32, 0, (size_t)KC * 4, st));
        if (dw_f16) KDW_CUDA(cudaMemsetAsync(dw_f16, 0, (size_t)KC * 2, st));
        return 0;
    }
    if (C < 8) {
        if (tune != 0) {
            set_error("wgrad: C=%lld < 8 runs the plain kernel; tune must be 0", (long long)C);
            return KDW_ERR_TUNE;
        }
        const long long voxels = (long long)N * (h_end - h_begin) * W * D;
        long long blocks = voxels < rows_cap ? voxels : rows_cap;
        wgrad_plain_kernel<<<(unsigned)blocks, 128, 0, st>>>((const __half*)x, (const __half*)grad, ws, voxels, (int)C,
                                                             (int)Hx, (int)W, (int)D, xsN, xsH, xsW, gsN, gsH, gsW,
                                                             (int)h_begin, (int)(h_end - h_begin), (int)g_h0);
        KDW_CUDA(cudaGetLastError());
        rows = (int)blocks;
    } else {
        const int id = tune ? tune : auto_wgrad_variant(C, W, D);
        if (id > g_n_table_wgrad_variants) {
            rc = launch_wgrad_mma_variant(id - g_n_table_wgrad_variants - 1, x, grad, ws, rows_cap, N, C, Hx, W, D, xsN,
                                          xsH, xsW, Hg, gsN, gsH, gsW, (int)h_begin, (int)h_end, (int)g_h0, st, &rows);
        } else {
            const WgradVariant& v = g_wgrad_variants[id - 1];
            if (C % v.cs != 0) {
                set_error("wgrad: variant %d works on %d-channel slices, C=%lld is not a multiple", id, v.cs,
                          (long long)C);
                return KDW_ERR_TUNE;
            }
            WgradArgs a{x,   grad, ws,  rows_cap, N,   C,          Hx,         W,          D,  xsN, xsH,
                        xsW, Hg,   gsN, gsH,      gsW, (int)h_begin, (int)h_end, (int)g_h0, st};
            rc = v.f(a, &rows);
        }
        if (rc) return rc;
    }
    KDW_CUDA(launch_overlapping_previous(wgrad_reduce_kernel<true>, (unsigned)((KC + 3) / 4), 128u, st, (const float*)ws,
                                         rows, KC, dw_f32, (__half*)dw_f16));
    return 0;
}

// ------------------------------------------------------------------------------------------------
// Weight gradient with a built-in workspace (no caller-provided scratch)
// ------------------------------------------------------------------------------------------------
// One fp32 [27][C] row per CTA, for at most kStaticRows CTAs and C <= kStaticMaxC: 296 * 27 * 128 * 4 bytes
// (3.9 MiB), resident on every GPU that loads the library until the process exits.
static constexpr int kStaticRows = 296;
static constexpr int kStaticMaxC = 128;
static __device__ __align__(256) float g_static_ws[kStaticRows * 27 * kStaticMaxC];

// In host code `g_static_ws` is only a handle for the runtime, not a device address: the address is looked up
// once per device (with that device current) and cached.
static int static_ws_ptr(float** out) {
    static float* cache[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    KDW_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_error("wgrad_static: device index %d is outside the supported range 0..63", dev);
        return KDW_ERR_ARG;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!cache[dev]) {
        void* addr = nullptr;
        KDW_CUDA(cudaGetSymbolAddress(&addr, g_static_ws));
        cache[dev] = (float*)addr;
    }
    *out = cache[dev];
    return 0;
}

static int wgrad_static_dispatch(const void* x, const void* grad, float* dw_f32, void* dw_f16, int64_t N, int64_t C,
                                 int64_t H, int64_t W, int64_t D, int64_t xsN, int64_t xsH, int64_t xsW, int64_t gsN,
                                 int64_t gsH, int64_t gsW, void* stream) {
    if (!x || !grad || (!dw_f32 && !dw_f16)) {
        set_error("wgrad_static: null pointer (x, grad and at least one output are required)");
        return KDW_ERR_ARG;
    }
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || D <= 0 || (C & (C - 1)) != 0) {
        set_error("wgrad_static: sizes must be positive and C a power of two (N=%lld C=%lld H=%lld W=%lld D=%lld)",
                  (long long)N, (long long)C, (long long)H, (long long)W, (long long)D);
        return KDW_ERR_ARG;
    }
    if (C > kStaticMaxC) {
        set_error("wgrad_static: C=%lld exceeds the built-in workspace (C <= %d); use kdw_wgrad_f16 with a "
                  "caller-provided workspace", (long long)C, kStaticMaxC);
        return KDW_ERR_WORKSPACE;
    }
    if (H > 0x7fffffff || W > 0x7fffffff || D > 0x7fffffff || N > 0x7fffffff) {
        set_error("wgrad_static: extent does not fit in 32 bits");
        return KDW_ERR_ARG;
    }
    float* ws = nullptr;
    int rc = static_ws_ptr(&ws);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const int KC = (int)(27 * C);
    int rows = 0;
    if (C < 8) {
        const long long voxels = (long long)N * H * W * D;
        const long long blocks = voxels < kStaticRows ? voxels : kStaticRows;
        wgrad_plain_kernel<<<(unsigned)blocks, 128, 0, st>>>((const __half*)x, (const __half*)grad, ws, voxels, (int)C,
                                                             (int)H, (int)W, (int)D, xsN, xsH, xsW, gsN, gsH, gsW, 0,
                                                             (int)H, 0);
        KDW_CUDA(cudaGetLastError());
        rows = (int)blocks;
    } else {
        const WgradVariant& v = g_wgrad_variants[auto_wgrad_variant(C, W, D, true) - 1];
        WgradArgs a{x, grad, ws, kStaticRows, N, C, H, W, D, xsN, xsH, xsW, H, gsN, gsH, gsW, 0, (int)H, 0, st};
        rc = v.f(a, &rows);  // the launcher never uses more CTAs (= rows) than a.ws_rows
        if (rc) return rc;
    }
    wgrad_reduce_kernel<false><<<(KC + 3) / 4, 128, 0, st>>>(ws, rows, KC, dw_f32, (__half*)dw_f16);
    KDW_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace kdw

extern "C" {

int kdw_wgrad_variants(void) { return kdw::n_wgrad_variants(); }

int kdw_wgrad_auto_variant(int64_t C, int64_t W, int64_t D) {
    if (C < 8 || (C & (C - 1)) != 0 || W <= 0 || D <= 0) return 0;
    return kdw::auto_wgrad_variant(C, W, D);
}

int kdw_wgrad_variant_channels(int id) {
    if (id < 1 || id > kdw::n_wgrad_variants()) return KDW_ERR_TUNE;
    if (id > kdw::g_n_table_wgrad_variants) return kdw::wgrad_mma_variant_channels(id - kdw::g_n_table_wgrad_variants - 1);
    return kdw::g_wgrad_variants[id - 1].cs;
}

int64_t kdw_wgrad_workspace_bytes(int64_t N, int64_t C, int64_t H, int64_t W, int64_t D) {
    (void)N;
    (void)H;
    (void)W;
    (void)D;
    if (C <= 0) return KDW_ERR_ARG;
    int rc = 0;
    const int64_t rows = kdw::ws_rows_for_device(&rc);
    if (rc) return -(int64_t)rc;
    return rows * 27 * C * 4;
}

int kdw_wgrad_f16(const void* x, const void* grad, void* workspace, int64_t workspace_bytes, float* dw_f32,
                  void* dw_f16, int64_t N, int64_t C, int64_t H, int64_t W, int64_t D, int64_t x_strideN,
                  int64_t x_strideH, int64_t x_strideW, int64_t g_strideN, int64_t g_strideH, int64_t g_strideW,
                  int tune, void* stream) {
    return kdw::wgrad_dispatch(x, grad, workspace, workspace_bytes, dw_f32, dw_f16, N, C, H, W, D, x_strideN,
                               x_strideH, x_strideW, H, g_strideN, g_strideH, g_strideW, 0, H, 0, tune, stream);
}

int kdw_wgrad_f16_static(const void* x, const void* grad, float* dw_f32, void* dw_f16, int64_t N, int64_t C, int64_t H,
                         int64_t W, int64_t D, int64_t x_strideN, int64_t x_strideH, int64_t x_strideW,
                         int64_t g_strideN, int64_t g_strideH, int64_t g_strideW, void* stream) {
    return kdw::wgrad_static_dispatch(x, grad, dw_f32, dw_f16, N, C, H, W, D, x_strideN, x_strideH, x_strideW, g_strideN,
                                      g_strideH, g_strideW, stream);
}

int kdw_wgrad_f16_range(const void* x, const void* grad, void* workspace, int64_t workspace_bytes, float* dw_f32,
                        void* dw_f16, int64_t N, int64_t C, int64_t Hx, int64_t W, int64_t D, int64_t x_strideN,
                        int64_t x_strideH, int64_t x_strideW, int64_t Hg, int64_t g_strideN, int64_t g_strideH,
                        int64_t g_strideW, int64_t h_begin, int64_t h_end, int64_t g_h0, int tune, void* stream) {
    return kdw::wgrad_dispatch(x, grad, workspace, workspace_bytes, dw_f32, dw_f16, N, C, Hx, W, D, x_strideN,
                               x_strideH, x_strideW, Hg, g_strideN, g_strideH, g_strideW, h_begin, h_end, g_h0, tune,
                               stream);
}

}  // extern "C"
