// Depthwise 3x3x3 channels-last fp16 forward pass for sm_100a.
//
// Replaces kerops/kernels/dw_conv.py:5-142 (_DWConv_cl3d_impl) and its launch loop
// (kerops/ops/conv/dwconv.py:42-61).
//
// TMA kernel (C multiple of 8).  A CTA owns a column (w-tile x d-tile x channel-slice) and marches
// along h.  A producer warp streams ONE halo'd input plane [(WT+2) x (DT+2) x CS] per step into a ring of
// shared-memory stages by tiled TMA loads (zero fill outside the volume = the padding on all three
// axes); full/empty mbarriers are the only synchronisation between it and the consumer warps.  Every
// consumer thread - fixed (channel pairs, d), M consecutive w positions - applies the plane to the three
// output planes that use it (plane q+1 gets the a=0 taps, plane q the a=1 taps, plane q-1 the a=2 taps)
// and carries the unfinished sums in registers, so each input plane is read from shared memory exactly
// once and the 27 x (channel pairs) taps stay in registers.  KDW_ACC_F32 uses the sm_100 mixed-precision
// FMA (fp16 operands, fp32 accumulator: exact products, one rounding to fp16 at the end);
// KDW_ACC_F16 uses packed-half FMA chains.  Neither has index arithmetic in the inner loop.  A warp
// stages its part of a finished plane in shared memory and stores it with its own TMA store, which
// clips the w/d tails.
//
// Plain kernel (any C): one thread per output element, fp32 FMAs, bounds checks.  Used for C < 8.
#include "../../include/kdw.h"
#include "fprop_core.cuh"
#include "kdw_common.cuh"

namespace kdw {

// ------------------------------------------------------------------------------------------------
// Plain kernel
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) fprop_plain_kernel(const __half* __restrict__ x, const __half* __restrict__ w,
                                                         __half* __restrict__ y, long long total, int C, int Hx, int W,
                                                         int D, long long xsN, long long xsH, long long xsW,
                                                         long long ysN, long long ysH, long long ysW, int h_begin,
                                                         int Hr, int y_h0, int acc16) {
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        long long r = idx;
        const int c = (int)(r % C);
        r /= C;
        const int d = (int)(r % D);
        r /= D;
        const int wv = (int)(r % W);
        r /= W;
        const int h = h_begin + (int)(r % Hr);
        const long long n = r / Hr;
        float acc = 0.f;
        __half acch = __float2half(0.f);
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            const int hh = h + a - 1;
            if (hh < 0 || hh >= Hx) continue;
#pragma unroll
            for (int b = 0; b < 3; ++b) {
                const int ww = wv + b - 1;
                if (ww < 0 || ww >= W) continue;
#pragma unroll
                for (int t = 0; t < 3; ++t) {
                    const int dd = d + t - 1;
                    if (dd < 0 || dd >= D) continue;
                    const __half xv = x[n * xsN + hh * xsH + ww * xsW + (long long)dd * C + c];
                    const __half wt = w[((a * 3 + b) * 3 + t) * C + c];
                    if (acc16)
                        acch = __hfma(xv, wt, acch);
                    else
                        acc = fmaf(__half2float(xv), __half2float(wt), acc);
                }
            }
        }
        y[n * ysN + (long long)(h - y_h0) * ysH + wv * ysW + (long long)d * C + c] =
            acc16 ? acch : __float2half_rn(acc);
    }
}

// ------------------------------------------------------------------------------------------------
// TMA kernel
// ------------------------------------------------------------------------------------------------
template <class Cfg, int MODE>
__global__ void __launch_bounds__(Cfg::NT + 32, Cfg::MINB)
    fprop_tma_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmy,
                     const __half* __restrict__ weight, const Sched s, const int C, const int y_h0, int* status,
                     const WaitTest wt) {
    constexpr int M = Cfg::M, CP = Cfg::CP, ST = Cfg::ST, NCW = Cfg::NCW;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    unsigned char* in_base = smem;                         // ST input stages
    unsigned char* out_base = smem + ST * Cfg::IN_STRIDE;  // per consumer warp: two output tiles
    const uint32_t full0 = smem_u32(out_base + 2 * NCW * Cfg::OUTW_BYTES);  // full[ST], then empty[ST]
    const uint32_t empty0 = full0 + 8 * ST;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        prefetch_tmap(&tmx);
        prefetch_tmap(&tmy);
        for (int k = 0; k < ST; ++k) {
            mbar_init(full0 + 8 * k, 1);     // the producer's arrive.expect_tx
            mbar_init(empty0 + 8 * k, NCW);  // one arrive per consumer warp
        }
        mbar_fence_init();
    }
    __syncthreads();  // the only CTA-wide barrier: from here on the warps only meet through mbarriers

    if (warp == NCW) {
        // ---------------- producer warp: one lane streams the input planes of the CTA's range ----------------
        if (lane != 0) return;
        StepIter it;
        it.init(s, (int)blockIdx.x, (int)gridDim.x);
        uint32_t pi = 0;
        bool ok = true;
        while (it.active && ok) {
            if (wt.stop_after >= 0 && (int)pi >= wt.stop_after) return;  // test hook: the consumers' wait runs out
            const uint32_t st = pi % ST;
            if (pi >= ST) ok = mbar_wait_bounded(empty0 + 8 * st, ((pi / ST) & 1u) ^ 1u, wt.limit_ns);  // released
            if (!ok) break;
            mbar_expect_tx(full0 + 8 * st, Cfg::IN_BYTES);
            tma_load_5d(status, smem_u32(in_base + st * Cfg::IN_STRIDE), &tmx, full0 + 8 * st, it.g.c0, it.g.d0 - 1,
                        it.g.w0 - 1, it.q, it.g.n);
            ++pi;
            it.next(s);
        }
        if (!ok) {
            atomicExch(status, (int)KDW_STATUS_TMA_TIMEOUT);
            // loads already issued still target this CTA's shared memory: give them a bounded chance to land
            const uint32_t first = pi > ST ? pi - ST : 0;
            for (uint32_t k = first; k < pi; ++k)
                (void)mbar_wait_bounded(full0 + 8 * (k % ST), (k / ST) & 1u, wt.limit_ns);
        }
        return;
    }

    // ---------------- consumer warps ----------------
    const FThread<Cfg> th(tid);
    unsigned char* my_out = out_base + warp * 2 * Cfg::OUTW_BYTES;
    StepIter it;
    it.init(s, (int)blockIdx.x, (int)gridDim.x);

    __half2 wgt[27][CP];           // taps of this thread's channels
    float2 P1[M][CP], P2[M][CP];   // carried fp32 partial sums (see fprop_step_f32)
    __half2 H1[M][CP], H2[M][CP];  // carried packed-half partial sums
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int i = 0; i < CP; ++i) {
            P1[m][i] = P2[m][i] = make_float2(0.f, 0.f);
            H1[m][i] = H2[m][i] = __float2half2_rn(0.f);
        }

    uint32_t ci = 0;  // steps consumed
    uint32_t oc = 0;  // planes stored by this warp
    while (it.active) {
        const int q = it.q;
        if (q == it.g.hb - 1) {  // new segment: this thread's taps for the segment's channel slice
            const __half* wp = weight + it.g.c0 + th.cg * 2 * CP;
#pragma unroll
            for (int k = 0; k < 27; ++k)
#pragma unroll
                for (int i = 0; i < CP; ++i)
                    wgt[k][i] = *reinterpret_cast<const __half2*>(wp + (size_t)k * C + 2 * i);
        }
        const uint32_t st = ci % ST;
        const bool ok = mbar_wait_bounded(full0 + 8 * st, (ci / ST) & 1u, wt.limit_ns);
        if (__any_sync(0xffffffffu, !ok)) {  // this warp leaves; the other warps' waits are bounded too
            if (lane == 0) atomicExch(status, (int)KDW_STATUS_TMA_TIMEOUT);
            break;
        }
        const bool store = q - 1 >= it.g.hb;  // plane q-1 is owned by the segment (q-1 < he always holds)
        unsigned char* ob_bytes = my_out + (oc & 1u) * Cfg::OUTW_BYTES;
        if (store && lane == 0) tma_wait_read<1>();  // the store issued two planes ago has released this tile
        __syncwarp();
        const __half* in = reinterpret_cast<const __half*>(in_base + st * Cfg::IN_STRIDE) + th.in_off;
        __half* ob = reinterpret_cast<__half*>(ob_bytes) + th.out_off;
        if (MODE == 0) {  // the two arrays swap roles every step
            if (ci & 1u)
                fprop_step_f32<Cfg>(in, ob, store, wgt, P2, P1);
            else
                fprop_step_f32<Cfg>(in, ob, store, wgt, P1, P2);
        } else {
            fprop_step_f16<Cfg>(in, ob, store, wgt, H1, H2);
        }
        if (store) fence_proxy_async_smem();  // the tile must be visible to the TMA store
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(empty0 + 8 * st);  // this warp is done with the input stage
            if (store) {
                tma_store_5d(status, &tmy, smem_u32(ob_bytes), it.g.c0, it.g.d0 + th.warp_d0, it.g.w0 + th.wg * M,
                             q - 1 - y_h0, it.g.n);
                tma_commit();
            }
        }
        if (store) ++oc;
        it.next(s);
        ++ci;
    }
    if (lane == 0) tma_wait_all();
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
struct FpropArgs {
    const void* x;
    const void* w;
    void* y;
    int64_t N, C, Hx, W, D, xsN, xsH, xsW, Hy, ysN, ysH, ysW;
    int h_begin, h_end, y_h0;
    cudaStream_t stream;
};

template <class Cfg, int MODE>
static int launch_fprop_tma(const FpropArgs& a) {
    CUtensorMap tmx, tmy;
    int rc = encode_volume_map(&tmx, a.x, a.N, a.C, a.Hx, a.W, a.D, a.xsN, a.xsH, a.xsW, Cfg::CS, Cfg::DT + 2,
                               Cfg::WT + 2);
    if (rc) return rc;
    rc = encode_volume_map(&tmy, a.y, a.N, a.C, a.Hy, a.W, a.D, a.ysN, a.ysH, a.ysW, Cfg::CS, Cfg::DPW, Cfg::M);
    if (rc) return rc;
    if (((uintptr_t)a.w & 3) != 0) {
        set_error("weight pointer must be 4-byte aligned");
        return KDW_ERR_ALIGN;
    }
    auto kern = fprop_tma_kernel<Cfg, MODE>;
    static KernelSetup setup;  // one per kernel instantiation
    int occ = 0, sms = 0;
    rc = setup.get((const void*)kern, Cfg::NT + 32, Cfg::SMEM, &sms, &occ);
    if (rc) return rc;
    int* status = nullptr;
    rc = status_ptr(&status);
    if (rc) return rc;
    Sched s;
    const int grid = make_sched(&s, a.N, a.C, a.W, a.D, a.h_begin, a.h_end, Cfg::WT, Cfg::DT, Cfg::CS, sms * occ);
    kern<<<grid, Cfg::NT + 32, Cfg::SMEM, a.stream>>>(tmx, tmy, (const __half*)a.w, s, (int)a.C, a.y_h0, status,
                                                      wait_test());
    KDW_CUDA(cudaGetLastError());
    return 0;
}

typedef int (*FpropLaunch)(const FpropArgs&);
struct FpropVariant {
    int cs, dt, wt;
    FpropLaunch mode[2];  // indexed by KDW_ACC_*
};
#define KDW_VARIANT(ID, CS, DT, WT, M, CP, ST, MINB)                            \
    {CS, DT, WT,                                                                \
     {&launch_fprop_tma<FCfg<CS, DT, WT, M, CP, ST, MINB>, 0>,                  \
      &launch_fprop_tma<FCfg<CS, DT, WT, M, CP, ST, MINB>, 1>}},
// index = id - 1
static const FpropVariant g_fprop_variants[] = {
#include "fprop_variants.inc"
};
#undef KDW_VARIANT
static const int g_n_table_variants = (int)(sizeof(g_fprop_variants) / sizeof(g_fprop_variants[0]));

// tensor-core variants (dwconv_fprop_mma.cu) are numbered after the table; they implement KDW_ACC_F32 only
int fprop_mma_variants();
int fprop_mma_variant_channels(int which);
int launch_fprop_mma_variant(int which, const void* x, const void* w, void* y, int64_t N, int64_t C, int64_t Hx,
                             int64_t W, int64_t D, int64_t xsN, int64_t xsH, int64_t xsW, int64_t Hy, int64_t ysN,
                             int64_t ysH, int64_t ysW, int h_begin, int h_end, int y_h0, cudaStream_t stream);
static int n_fprop_variants() { return g_n_table_variants + fprop_mma_variants(); }

// Built-in choice.  Per channel count and accumulate type a short list of candidates with their time relative to
// the best one, measured at (1, C, 350, 350, 128) on B200.  A tile that does not divide W or D computes padding:
// the candidate's time is scaled by the padded / real area and the cheapest one wins, so e.g. D = 40 does not run
// on a 64-deep tile.  The tensor-core kernels (ids after the table, dwconv_fprop_mma.cu: exact fp16 products, fp32
// sums) serve both accumulate types: KDW_ACC_F16 asks for no MORE than fp16 sums, and the fp32-accumulating mma
// kernel is both more accurate and faster than the packed-half FMA chains of the CUDA-core tiles, which run in
// that arithmetic only when a table variant is named explicitly together with KDW_ACC_F16.
struct FpropCand {
    int id;
    float rel;
};
void fprop_mma_variant_tile(int which, int* wt, int* dt);
bool fprop_mma_variant_fits(int which, int64_t C, int64_t D);
static const int kT = g_n_table_variants;  // tensor-core variant i has id kT + 1 + i
static const FpropCand kFpropCand8[] = {{kT + 7, 1.00f}, {kT + 4, 1.70f}, {1, 1.80f}, {2, 2.00f}};
static const FpropCand kFpropCand16[] = {{kT + 8, 1.00f}, {kT + 3, 1.21f}, {kT + 9, 1.31f}, {10, 1.80f}, {4, 1.85f}};
static const FpropCand kFpropCand32[] = {{kT + 5, 1.00f}, {kT + 3, 1.03f}, {kT + 2, 1.06f}, {11, 1.75f}};
static const FpropCand kFpropCand64[] = {{kT + 1, 1.00f}, {kT + 6, 1.02f}, {kT + 5, 1.09f}, {11, 1.80f}};
static const FpropCand kFpropCand128[] = {{kT + 1, 1.00f}, {kT + 6, 1.07f}, {kT + 2, 1.12f}, {8, 1.80f}};
static void fprop_variant_tile(int id, int* wt, int* dt) {
    if (id > g_n_table_variants) {
        fprop_mma_variant_tile(id - g_n_table_variants - 1, wt, dt);
    } else {
        *wt = g_fprop_variants[id - 1].wt;
        *dt = g_fprop_variants[id - 1].dt;
    }
}

#define KDW_CANDS(a) cand = a, n = (int)(sizeof(a) / sizeof(a[0]))
static int auto_fprop_variant(int64_t C, int64_t W, int64_t D, int acc_type) {
    const FpropCand* cand;
    int n;
    (void)acc_type;  // both accumulate types share the choice: see the comment above
    if (C == 8) KDW_CANDS(kFpropCand8);
    else if (C == 16) KDW_CANDS(kFpropCand16);
    else if (C == 32) KDW_CANDS(kFpropCand32);
    else if (C == 64) KDW_CANDS(kFpropCand64);
    else KDW_CANDS(kFpropCand128);
    int best = 0;
    double best_cost = 0.0;
    for (int i = 0; i < n; ++i) {
        if (cand[i].id > kT && !fprop_mma_variant_fits(cand[i].id - kT - 1, C, D)) continue;
        int wt = 1, dt = 1;
        fprop_variant_tile(cand[i].id, &wt, &dt);
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

static int fprop_dispatch(const void* x, const void* weight, void* y, int64_t N, int64_t C, int64_t Hx, int64_t W,
                          int64_t D, int64_t xsN, int64_t xsH, int64_t xsW, int64_t Hy, int64_t ysN, int64_t ysH,
                          int64_t ysW, int64_t h_begin, int64_t h_end, int64_t y_h0, int acc_type, int tune,
                          void* stream) {
    if (!x || !weight || !y) {
        set_error("fprop: null pointer");
        return KDW_ERR_ARG;
    }
    if (N <= 0 || C <= 0 || Hx <= 0 || W <= 0 || D <= 0 || Hy <= 0 || (C & (C - 1)) != 0) {
        set_error("fprop: sizes must be positive and C a power of two (N=%lld C=%lld H=%lld W=%lld D=%lld)",
                  (long long)N, (long long)C, (long long)Hx, (long long)W, (long long)D);
        return KDW_ERR_ARG;
    }
    if (acc_type != KDW_ACC_F32 && acc_type != KDW_ACC_F16) {
        set_error("fprop: acc_type must be KDW_ACC_F32 or KDW_ACC_F16");
        return KDW_ERR_ARG;
    }
    if (Hx > 0x7fffffff || W > 0x7fffffff || D > 0x7fffffff || N > 0x7fffffff || C > 0x7fffffff) {
        set_error("fprop: extent does not fit in 32 bits");
        return KDW_ERR_ARG;
    }
    if (h_begin < 0 || h_end > Hx || h_begin > h_end || h_begin - y_h0 < 0 || h_end - y_h0 > Hy) {
        set_error("fprop: plane range [%lld,%lld) / y_h0=%lld outside x (%lld planes) or y (%lld planes)",
                  (long long)h_begin, (long long)h_end, (long long)y_h0, (long long)Hx, (long long)Hy);
        return KDW_ERR_RANGE;
    }
    if (h_begin == h_end) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (tune < 0 || tune > n_fprop_variants()) {
        set_error("fprop: tune=%d names no kernel variant (1..%d)", tune, n_fprop_variants());
        return KDW_ERR_TUNE;
    }
    if (C < 8) {
        if (tune != 0) {
            set_error("fprop: C=%lld < 8 runs the plain kernel; tune must be 0", (long long)C);
            return KDW_ERR_TUNE;
        }
        const long long total = (long long)N * (h_end - h_begin) * W * D * C;
        long long blocks = (total + 255) / 256;
        if (blocks > 148 * 32) blocks = 148 * 32;
        fprop_plain_kernel<<<(unsigned)blocks, 256, 0, st>>>((const __half*)x, (const __half*)weight, (__half*)y,
                                                             total, (int)C, (int)Hx, (int)W, (int)D, xsN, xsH, xsW,
                                                             ysN, ysH, ysW, (int)h_begin, (int)(h_end - h_begin),
                                                             (int)y_h0, acc_type == KDW_ACC_F16);  // the plain kernel has one fp32 mode
        KDW_CUDA(cudaGetLastError());
        return 0;
    }
    const int id = tune ? tune : auto_fprop_variant(C, W, D, acc_type);
    if (id > g_n_table_variants) {
        return launch_fprop_mma_variant(id - g_n_table_variants - 1, x, weight, y, N, C, Hx, W, D, xsN, xsH, xsW, Hy, ysN,
                                        ysH, ysW, (int)h_begin, (int)h_end, (int)y_h0, st);
    }
    const FpropVariant& v = g_fprop_variants[id - 1];
    if (C % v.cs != 0) {
        set_error("fprop: variant %d works on %d-channel slices, C=%lld is not a multiple", id, v.cs, (long long)C);
        return KDW_ERR_TUNE;
    }
    FpropArgs a{x, weight, y, N, C, Hx, W, D, xsN, xsH, xsW, Hy, ysN, ysH, ysW, (int)h_begin, (int)h_end, (int)y_h0, st};
    return v.mode[acc_type](a);
}

}  // namespace kdw

extern "C" {

int kdw_fprop_variants(void) { return kdw::n_fprop_variants(); }

int kdw_fprop_auto_variant(int64_t C, int64_t W, int64_t D) {
    if (C < 8 || (C & (C - 1)) != 0 || W <= 0 || D <= 0) return 0;
    return kdw::auto_fprop_variant(C, W, D, KDW_ACC_F32);
}

int kdw_fprop_variant_channels(int id) {
    if (id < 1 || id > kdw::n_fprop_variants()) return KDW_ERR_TUNE;
    if (id > kdw::g_n_table_variants) return kdw::fprop_mma_variant_channels(id - kdw::g_n_table_variants - 1);
    return kdw::g_fprop_variants[id - 1].cs;
}

int kdw_fprop_f16(const void* x, const void* weight, void* y, int64_t N, int64_t C, int64_t H, int64_t W, int64_t D,
                  int64_t x_strideN, int64_t x_strideH, int64_t x_strideW, int64_t y_strideN, int64_t y_strideH,
                  int64_t y_strideW, int acc_type, int tune, void* stream) {
    return kdw::fprop_dispatch(x, weight, y, N, C, H, W, D, x_strideN, x_strideH, x_strideW, H, y_strideN, y_strideH,
                               y_strideW, 0, H, 0, acc_type, tune, stream);
}

int kdw_fprop_f16_range(const void* x, const void* weight, void* y, int64_t N, int64_t C, int64_t Hx, int64_t W,
                        int64_t D, int64_t x_strideN, int64_t x_strideH, int64_t x_strideW, int64_t Hy,
                        int64_t y_strideN, int64_t y_strideH, int64_t y_strideW, int64_t h_begin, int64_t h_end,
                        int64_t y_h0, int acc_type, int tune, void* stream) {
    return kdw::fprop_dispatch(x, weight, y, N, C, Hx, W, D, x_strideN, x_strideH, x_strideW, Hy, y_strideN,
                               y_strideH, y_strideW, h_begin, h_end, y_h0, acc_type, tune, stream);
}

}  // extern "C"
