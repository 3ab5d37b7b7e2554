// CPU emulation of the TMA kernels, used only by the CPU test-suite.
//
// It runs the SAME host scheduler (make_sched), segment decoding (decode_segment / StepIter), thread
// mapping (FThread / WThread) and per-thread step functions (fprop_step_f32 / fprop_step_f16 / wgrad_step) as the CUDA
// kernels, one emulated thread after the other, and replaces only the hardware plumbing: a tiled TMA
// load becomes a box copy with zero fill, a TMA store a clipped box copy, the block reduction of the
// weight-gradient kernel a plain loop.  It lets the index arithmetic of every kernel variant be
// checked against the oracle on a machine without a GPU.
#include <string.h>

#include <vector>

#include "../../kerops_b200/csrc/fprop_core.cuh"
#include "../../kerops_b200/csrc/kdw_common.cuh"
#include "../../kerops_b200/csrc/wgrad_core.cuh"

using namespace kdw;

struct Vol {
    int64_t N, C, H, W, D, sN, sH, sW;
};

// box (CS, BD, BW) at (c0, d0, w0) of plane h of sample n; zero outside the volume
static void emu_tma_load(__half* dst, const __half* src, const Vol& v, int CS, int BD, int BW, int c0, int d0, int w0,
                         int h, int n, bool nan_fill = false) {
    for (int wj = 0; wj < BW; ++wj)
        for (int dd = 0; dd < BD; ++dd)
            for (int c = 0; c < CS; ++c) {
                const int w = w0 + wj, d = d0 + dd, ch = c0 + c;
                const bool in = h >= 0 && h < v.H && w >= 0 && w < v.W && d >= 0 && d < v.D && ch < v.C && n < v.N;
                dst[(wj * BD + dd) * CS + c] =
                    in ? src[n * v.sN + (int64_t)h * v.sH + (int64_t)w * v.sW + (int64_t)d * v.C + ch]
                       : (nan_fill ? __float2half(nanf("")) : __float2half(0.f));
            }
}
static void emu_tma_store(__half* dst, const __half* tile, const Vol& v, int CS, int BD, int BW, int c0, int d0, int w0,
                          int h, int n) {
    for (int wj = 0; wj < BW; ++wj)
        for (int dd = 0; dd < BD; ++dd)
            for (int c = 0; c < CS; ++c) {
                const int w = w0 + wj, d = d0 + dd, ch = c0 + c;
                const bool in = h >= 0 && h < v.H && w >= 0 && w < v.W && d >= 0 && d < v.D && ch < v.C && n < v.N;
                if (in) dst[n * v.sN + (int64_t)h * v.sH + (int64_t)w * v.sW + (int64_t)d * v.C + ch] = tile[(wj * BD + dd) * CS + c];
            }
}

template <class Cfg, int MODE>
static int emu_fprop_cfg(const __half* x, const __half* w, __half* y, Vol vx, Vol vy, int h_begin, int h_end, int y_h0,
                         int grid_target) {
    constexpr int M = Cfg::M, CP = Cfg::CP;
    struct TState {
        __half2 wgt[27][CP];
        float2 P1[M][CP], P2[M][CP];
        __half2 H1[M][CP], H2[M][CP];
    };
    Sched s;
    const int grid = make_sched(&s, vx.N, vx.C, vx.W, vx.D, h_begin, h_end, Cfg::WT, Cfg::DT, Cfg::CS, grid_target);
    std::vector<__half> stage(Cfg::IN_BYTES / 2);
    std::vector<__half> out((size_t)Cfg::NCW * Cfg::OUTW_BYTES / 2);  // one tile per consumer warp
    std::vector<TState> ts(Cfg::NT);
    for (int blk = 0; blk < grid; ++blk) {
        memset(ts.data(), 0, sizeof(TState) * ts.size());
        StepIter cons;
        cons.init(s, blk, grid);
        unsigned ci = 0;
        while (cons.active) {
            const int q = cons.q;
            const Seg& g = cons.g;
            emu_tma_load(stage.data(), x, vx, Cfg::CS, Cfg::DT + 2, Cfg::WT + 2, g.c0, g.d0 - 1, g.w0 - 1, q, g.n);
            const bool store = q - 1 >= g.hb;
            for (int tid = 0; tid < Cfg::NT; ++tid) {
                TState& t = ts[tid];
                const FThread<Cfg> th(tid);
                if (q == g.hb - 1) {
                    const __half* wp = w + g.c0 + th.cg * 2 * CP;
                    for (int k = 0; k < 27; ++k)
                        for (int i = 0; i < CP; ++i) t.wgt[k][i] = *reinterpret_cast<const __half2*>(wp + (size_t)k * vx.C + 2 * i);
                }
                const __half* in = stage.data() + th.in_off;
                __half* ob = out.data() + (size_t)(tid / 32) * (Cfg::OUTW_BYTES / 2) + th.out_off;
                if (MODE == 0) {  // as in the kernel: in-place sums, roles swap every step
                    if (ci & 1u)
                        fprop_step_f32<Cfg>(in, ob, store, t.wgt, t.P2, t.P1);
                    else
                        fprop_step_f32<Cfg>(in, ob, store, t.wgt, t.P1, t.P2);
                } else {
                    fprop_step_f16<Cfg>(in, ob, store, t.wgt, t.H1, t.H2);
                }
            }
            if (store) {
                for (int wp = 0; wp < Cfg::NCW; ++wp) {  // every warp stores its own box
                    const FThread<Cfg> th(wp * 32);
                    emu_tma_store(y, out.data() + (size_t)wp * (Cfg::OUTW_BYTES / 2), vy, Cfg::CS, Cfg::DPW, Cfg::M, g.c0,
                                  g.d0 + th.warp_d0, g.w0 + th.wg * Cfg::M, q - 1 - y_h0, g.n);
                }
            }
            cons.next(s);
            ++ci;
        }
    }
    return grid;
}

template <class Cfg>
static int emu_wgrad_cfg(const __half* x, const __half* gr, float* dw, Vol vx, Vol vg, int h_begin, int h_end, int g_h0,
                         int grid_target) {
    constexpr int M = Cfg::M, CP = Cfg::CP, CS = Cfg::CS;
    struct TState {
        __half2 G[3][M][CP];
        float2 acc[27][CP];
    };
    Sched s;
    const int grid = make_sched(&s, vx.N, vx.C, vx.W, vx.D, h_begin, h_end, Cfg::WT, Cfg::DT, Cfg::CS, grid_target);
    const int KC = 27 * (int)vx.C;
    std::vector<float> rows((size_t)grid * KC, 0.f);
    std::vector<__half> xs(Cfg::X_BYTES / 2), gs(Cfg::G_BYTES / 2);
    std::vector<TState> ts(Cfg::NT);
    for (int blk = 0; blk < grid; ++blk) {
        memset(ts.data(), 0, sizeof(TState) * ts.size());
        float* row = rows.data() + (size_t)blk * KC;
        StepIter cons;
        cons.init(s, blk, grid);
        unsigned ci = 0;
        int cur_c0 = -1;
        // like the kernel: the accumulators belong to a channel slice and are flushed when it changes and at the end
        auto flush = [&](int c0) {
            for (int tid = 0; tid < Cfg::NT; ++tid) {
                const WThread<Cfg> th(tid);
                for (int k = 0; k < 27; ++k)
                    for (int i = 0; i < CP; ++i) {
                        row[k * vx.C + c0 + th.cg * 2 * CP + 2 * i] += ts[tid].acc[k][i].x;
                        row[k * vx.C + c0 + th.cg * 2 * CP + 2 * i + 1] += ts[tid].acc[k][i].y;
                        ts[tid].acc[k][i] = make_float2(0.f, 0.f);
                    }
            }
        };
        while (cons.active) {
            const int q = cons.q;
            const Seg& g = cons.g;
            if (q == g.hb - 1 && g.c0 != cur_c0) {
                if (cur_c0 >= 0) flush(cur_c0);
                cur_c0 = g.c0;
            }
            emu_tma_load(xs.data(), x, vx, CS, Cfg::DT + 2, Cfg::WT + 2, g.c0, g.d0 - 1, g.w0 - 1, q, g.n);
            const bool load_g = q + 1 < g.he;
            if (load_g)
                emu_tma_load(gs.data(), gr, vg, CS, Cfg::DT, Cfg::WT, g.c0, g.d0, g.w0, q + 1 - g_h0, g.n);
            else
                for (auto& e : gs) e = __float2half(12345.f);  // stale data must never be used
            for (int tid = 0; tid < Cfg::NT; ++tid) {
                TState& t = ts[tid];
                const WThread<Cfg> th(tid);
                if (q == g.hb - 1) memset(t.G, 0, sizeof(t.G));
                const __half* xin = xs.data() + th.x_off;
                const __half* gin = gs.data() + th.g_off;
                switch (ci % 3) {
                    case 0: wgrad_step<Cfg, 0>(xin, gin, load_g, t.G, t.acc); break;
                    case 1: wgrad_step<Cfg, 1>(xin, gin, load_g, t.G, t.acc); break;
                    default: wgrad_step<Cfg, 2>(xin, gin, load_g, t.G, t.acc); break;
                }
            }
            cons.next(s);
            ++ci;
        }
        if (cur_c0 >= 0) flush(cur_c0);
    }
    for (int k = 0; k < KC; ++k) {
        float a = 0.f;
        for (int r = 0; r < grid; ++r) a += rows[(size_t)r * KC + k];
        dw[k] = a;
    }
    return grid;
}

#define EMU_FV(ID, CS, DT, WT, M, CP, ST, MINB)                                                                     \
    case ID: {                                                                                                      \
        using Cfg = FCfg<CS, DT, WT, M, CP, ST, MINB>;                                                              \
        const __half *xh = (const __half*)x, *wh = (const __half*)w;                                                \
        if (mode == 0) return emu_fprop_cfg<Cfg, 0>(xh, wh, (__half*)y, vx, vy, h_begin, h_end, y_h0, grid);        \
        return emu_fprop_cfg<Cfg, 1>(xh, wh, (__half*)y, vx, vy, h_begin, h_end, y_h0, grid);                       \
    }
#define EMU_WV(ID, CS, DT, WT, M, CP, ST, MINB)                                                                  \
    case ID:                                                                                                     \
        return emu_wgrad_cfg<WCfg<CS, DT, WT, M, CP, ST, MINB>>((const __half*)x, (const __half*)g, dw, vx, vg,  \
                                                                h_begin, h_end, g_h0, grid);

// The fused forward + residual add + statistics kernel (dwconv_fprop_addstats.cu), same walk as emu_fprop_cfg.
// stats receives [2][C] sums (not yet divided by the voxel count).
template <class Cfg>
static int emu_addstats_cfg(const __half* x, const __half* w, const __half* r, __half* y, double* stats, Vol v,
                            int grid_target) {
    constexpr int M = Cfg::M, CP = Cfg::CP;
    struct TState {
        __half2 wgt[27][CP];
        float2 P1[M][CP], P2[M][CP], S1[CP], S2[CP];
        int mv;
    };
    Sched s;
    const int grid = make_sched(&s, v.N, v.C, v.W, v.D, 0, (int)v.H, Cfg::WT, Cfg::DT, Cfg::CS, grid_target);
    std::vector<__half> stage(Cfg::IN_BYTES / 2), rt((size_t)Cfg::WT * Cfg::DT * Cfg::CS);
    std::vector<__half> out((size_t)Cfg::NCW * Cfg::OUTW_BYTES / 2);
    std::vector<TState> ts(Cfg::NT);
    for (int k = 0; k < 2 * v.C; ++k) stats[k] = 0.0;
    for (int blk = 0; blk < grid; ++blk) {
        memset(ts.data(), 0, sizeof(TState) * ts.size());
        std::vector<float> row(2 * v.C, 0.f);
        StepIter cons;
        cons.init(s, blk, grid);
        unsigned ci = 0;
        int cur_c0 = -1;
        auto flush = [&](int c0) {
            for (int tid = 0; tid < Cfg::NT; ++tid) {
                const FThread<Cfg> th(tid);
                for (int i = 0; i < CP; ++i) {
                    row[c0 + th.cg * 2 * CP + 2 * i] += ts[tid].S1[i].x;
                    row[c0 + th.cg * 2 * CP + 2 * i + 1] += ts[tid].S1[i].y;
                    row[v.C + c0 + th.cg * 2 * CP + 2 * i] += ts[tid].S2[i].x;
                    row[v.C + c0 + th.cg * 2 * CP + 2 * i + 1] += ts[tid].S2[i].y;
                    ts[tid].S1[i] = ts[tid].S2[i] = make_float2(0.f, 0.f);
                }
            }
        };
        while (cons.active) {
            const int q = cons.q;
            const Seg& g = cons.g;
            if (q == g.hb - 1 && g.c0 != cur_c0) {
                if (cur_c0 >= 0) flush(cur_c0);
                cur_c0 = g.c0;
            }
            emu_tma_load(stage.data(), x, v, Cfg::CS, Cfg::DT + 2, Cfg::WT + 2, g.c0, g.d0 - 1, g.w0 - 1, q, g.n);
            const bool store = q - 1 >= g.hb;
            if (store)
                emu_tma_load(rt.data(), r, v, Cfg::CS, Cfg::DT, Cfg::WT, g.c0, g.d0, g.w0, q - 1, g.n);
            else
                for (auto& e : rt) e = __float2half(12345.f);  // stale data must never be used
            for (int tid = 0; tid < Cfg::NT; ++tid) {
                TState& t = ts[tid];
                const FThread<Cfg> th(tid);
                if (q == g.hb - 1) {
                    const __half* wp = w + g.c0 + th.cg * 2 * CP;
                    for (int k = 0; k < 27; ++k)
                        for (int i = 0; i < CP; ++i) t.wgt[k][i] = *reinterpret_cast<const __half2*>(wp + (size_t)k * v.C + 2 * i);
                    int mv = (int)v.W - (g.w0 + th.wg * M);
                    mv = mv < 0 ? 0 : (mv > M ? M : mv);
                    if (g.d0 + th.d >= v.D) mv = 0;
                    t.mv = mv;
                }
                const __half* in = stage.data() + th.in_off;
                const __half* res = rt.data() + ((th.wg * M) * Cfg::DT + th.d) * Cfg::CS + th.cg * 2 * CP;
                __half* ob = out.data() + (size_t)(tid / 32) * (Cfg::OUTW_BYTES / 2) + th.out_off;
                if (ci & 1u)
                    fprop_step_f32_addstats<Cfg>(in, res, ob, store, t.mv, t.wgt, t.P2, t.P1, t.S1, t.S2);
                else
                    fprop_step_f32_addstats<Cfg>(in, res, ob, store, t.mv, t.wgt, t.P1, t.P2, t.S1, t.S2);
            }
            if (store) {
                for (int wp = 0; wp < Cfg::NCW; ++wp) {
                    const FThread<Cfg> th(wp * 32);
                    emu_tma_store(y, out.data() + (size_t)wp * (Cfg::OUTW_BYTES / 2), v, Cfg::CS, Cfg::DPW, Cfg::M, g.c0,
                                  g.d0 + th.warp_d0, g.w0 + th.wg * Cfg::M, q - 1, g.n);
                }
            }
            cons.next(s);
            ++ci;
        }
        if (cur_c0 >= 0) flush(cur_c0);
        for (int k = 0; k < 2 * v.C; ++k) stats[k] += row[k];
    }
    return grid;
}

// The fused BN-affine + ReLU prologue kernel (dwconv_fprop_bnrelu.cu): every thread activates the values it reads
// (fprop_step_f32_bnrelu) with its own channels' scale / shift; the tile's out-of-bounds fill is NaN.
template <class Cfg>
static int emu_bnrelu_cfg(const __half* x, const float* scale, const float* shift, const __half* w, __half* y, Vol v,
                          int grid_target) {
    constexpr int M = Cfg::M, CP = Cfg::CP, CS = Cfg::CS;
    struct TState {
        __half2 wgt[27][CP];
        float2 P1[M][CP], P2[M][CP], sc[CP], sh[CP];
    };
    Sched s;
    const int grid = make_sched(&s, v.N, v.C, v.W, v.D, 0, (int)v.H, Cfg::WT, Cfg::DT, Cfg::CS, grid_target);
    std::vector<__half> stage(Cfg::IN_BYTES / 2);
    std::vector<__half> out((size_t)Cfg::NCW * Cfg::OUTW_BYTES / 2);
    std::vector<TState> ts(Cfg::NT);
    for (int blk = 0; blk < grid; ++blk) {
        memset(ts.data(), 0, sizeof(TState) * ts.size());
        StepIter cons;
        cons.init(s, blk, grid);
        unsigned ci = 0;
        while (cons.active) {
            const int q = cons.q;
            const Seg& g = cons.g;
            emu_tma_load(stage.data(), x, v, CS, Cfg::DT + 2, Cfg::WT + 2, g.c0, g.d0 - 1, g.w0 - 1, q, g.n, true);
            const bool store = q - 1 >= g.hb;
            for (int tid = 0; tid < Cfg::NT; ++tid) {
                TState& t = ts[tid];
                const FThread<Cfg> th(tid);
                if (q == g.hb - 1) {
                    const __half* wp = w + g.c0 + th.cg * 2 * CP;
                    for (int k = 0; k < 27; ++k)
                        for (int i = 0; i < CP; ++i) t.wgt[k][i] = *reinterpret_cast<const __half2*>(wp + (size_t)k * v.C + 2 * i);
                    const int cb = g.c0 + th.cg * 2 * CP;
                    for (int i = 0; i < CP; ++i) {
                        t.sc[i] = make_float2(scale[cb + 2 * i], scale[cb + 2 * i + 1]);
                        t.sh[i] = make_float2(shift[cb + 2 * i], shift[cb + 2 * i + 1]);
                    }
                }
                const __half* in = stage.data() + th.in_off;
                __half* ob = out.data() + (size_t)(tid / 32) * (Cfg::OUTW_BYTES / 2) + th.out_off;
                if (ci & 1u)
                    fprop_step_f32_bnrelu<Cfg, 0>(in, ob, store, t.wgt, t.sc, t.sh, t.P2, t.P1);
                else
                    fprop_step_f32_bnrelu<Cfg, 0>(in, ob, store, t.wgt, t.sc, t.sh, t.P1, t.P2);
            }
            if (store) {
                for (int wp = 0; wp < Cfg::NCW; ++wp) {
                    const FThread<Cfg> th(wp * 32);
                    emu_tma_store(y, out.data() + (size_t)wp * (Cfg::OUTW_BYTES / 2), v, CS, Cfg::DPW, Cfg::M, g.c0,
                                  g.d0 + th.warp_d0, g.w0 + th.wg * Cfg::M, q - 1, g.n);
                }
            }
            cons.next(s);
            ++ci;
        }
    }
    return grid;
}

extern "C" {

// Returns the emulated grid size (> 0) or a negative error.  Volumes are dense channels-last.
int emu_fprop(int variant, const void* x, const void* w, void* y, int64_t N, int64_t C, int64_t Hx, int64_t W,
              int64_t D, int64_t Hy, int h_begin, int h_end, int y_h0, int mode, int grid) {
    const Vol vx{N, C, Hx, W, D, Hx * W * D * C, W * D * C, D * C};
    const Vol vy{N, C, Hy, W, D, Hy * W * D * C, W * D * C, D * C};
    switch (variant) {
#define KDW_VARIANT EMU_FV
#include "../../kerops_b200/csrc/fprop_variants.inc"
#undef KDW_VARIANT
    }
    return -1;
}

int emu_wgrad(int variant, const void* x, const void* g, float* dw, int64_t N, int64_t C, int64_t Hx, int64_t W,
              int64_t D, int64_t Hg, int h_begin, int h_end, int g_h0, int grid) {
    const Vol vx{N, C, Hx, W, D, Hx * W * D * C, W * D * C, D * C};
    const Vol vg{N, C, Hg, W, D, Hg * W * D * C, W * D * C, D * C};
    switch (variant) {
#define KDW_VARIANT EMU_WV
#include "../../kerops_b200/csrc/wgrad_variants.inc"
#undef KDW_VARIANT
    }
    return -1;
}

// Walks the schedule of every CTA exactly as the kernels do (make_sched + StepIter) and counts, per output unit
// (sample, channel slice, d tile, w tile, plane), how many segments own it; also returns the smallest and largest
// number of steps a CTA takes.  counts has N * nCS * nDT * nWT * (h_end - h_begin) entries, zero-initialised.
int emu_schedule(int64_t N, int64_t C, int64_t W, int64_t D, int h_begin, int h_end, int WT, int DT, int CS,
                 int grid_target, int* counts, int64_t* min_steps, int64_t* max_steps) {
    Sched s;
    const int grid = make_sched(&s, N, C, W, D, h_begin, h_end, WT, DT, CS, grid_target);
    const int Hr = h_end - h_begin;
    int64_t lo = -1, hi = -1;
    for (int blk = 0; blk < grid; ++blk) {
        StepIter it;
        it.init(s, blk, grid);
        int64_t steps = 0;
        while (it.active) {
            const Seg& g = it.g;
            if (it.q == g.hb - 1) {  // a new segment: owns planes hb .. he-1 of its column
                if (g.hb < h_begin || g.he > h_end || g.hb >= g.he) return -2;
                const int64_t col = (((int64_t)g.n * s.nCS + g.c0 / CS) * s.nDT + g.d0 / DT) * s.nWT + g.w0 / WT;
                for (int p = g.hb; p < g.he; ++p) ++counts[col * Hr + (p - h_begin)];
            }
            ++steps;
            it.next(s);
        }
        if (lo < 0 || steps < lo) lo = steps;
        if (steps > hi) hi = steps;
    }
    *min_steps = lo;
    *max_steps = hi;
    return grid;
}

// which: 1..5, the tiles of dwconv_fprop_addstats.cu in its order.
int emu_fprop_addstats(int which, const void* x, const void* w, const void* r, void* y, double* stats, int64_t N,
                       int64_t C, int64_t H, int64_t W, int64_t D, int grid) {
    const Vol v{N, C, H, W, D, H * W * D * C, W * D * C, D * C};
    const __half *xh = (const __half*)x, *wh = (const __half*)w, *rh = (const __half*)r;
    switch (which) {
        case 1: return emu_addstats_cfg<FCfg<8, 64, 8, 8, 1, 4, 2>>(xh, wh, rh, (__half*)y, stats, v, grid);
        case 2: return emu_addstats_cfg<FCfg<16, 32, 8, 8, 1, 4, 2>>(xh, wh, rh, (__half*)y, stats, v, grid);
        case 3: return emu_addstats_cfg<FCfg<32, 16, 8, 8, 1, 4, 2>>(xh, wh, rh, (__half*)y, stats, v, grid);
        case 4: return emu_addstats_cfg<FCfg<32, 32, 8, 8, 1, 3, 1>>(xh, wh, rh, (__half*)y, stats, v, grid);
        case 5: return emu_addstats_cfg<FCfg<64, 8, 8, 8, 1, 4, 2>>(xh, wh, rh, (__half*)y, stats, v, grid);
    }
    return -1;
}

// which: 1..6, the tiles of dwconv_fprop_bnrelu.cu in its order.
int emu_fprop_bnrelu(int which, const void* x, const float* scale, const float* shift, const void* w, void* y,
                     int64_t N, int64_t C, int64_t H, int64_t W, int64_t D, int grid) {
    const Vol v{N, C, H, W, D, H * W * D * C, W * D * C, D * C};
    const __half *xh = (const __half*)x, *wh = (const __half*)w;
    switch (which) {
        case 1: return emu_bnrelu_cfg<FCfg<8, 64, 8, 8, 1, 4, 2>>(xh, scale, shift, wh, (__half*)y, v, grid);
        case 2: return emu_bnrelu_cfg<FCfg<16, 64, 8, 8, 1, 3, 1>>(xh, scale, shift, wh, (__half*)y, v, grid);
        case 3: return emu_bnrelu_cfg<FCfg<16, 32, 8, 8, 1, 4, 2>>(xh, scale, shift, wh, (__half*)y, v, grid);
        case 4: return emu_bnrelu_cfg<FCfg<32, 32, 8, 8, 1, 3, 1>>(xh, scale, shift, wh, (__half*)y, v, grid);
        case 5: return emu_bnrelu_cfg<FCfg<32, 16, 8, 8, 1, 4, 2>>(xh, scale, shift, wh, (__half*)y, v, grid);
        case 6: return emu_bnrelu_cfg<FCfg<64, 8, 8, 8, 1, 4, 2>>(xh, scale, shift, wh, (__half*)y, v, grid);
    }
    return -1;
}

}  // extern "C"
