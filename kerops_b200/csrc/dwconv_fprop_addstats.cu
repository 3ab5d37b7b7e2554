// Forward pass with a fused epilogue: out = fp16(DWConv(x, weight)) + residual, together with the per-channel
// mean and mean of squares of `out` - what the reference computes with a second operator over the convolution's
// output (AddStats, kerops/ops/addition.py:11-49 and kerops/kernels/addition.py:5-37; a full extra read of two
// tensors and a write of one).  Same pipeline as fprop_tma_kernel (dwconv_fprop.cu): a stage additionally holds
// the residual tile of the plane that the step finishes, the step adds it before the store and accumulates the
// statistics in registers, and the sums leave the CTA the way the weight gradient's accumulators do (flush on a
// change of channel slice and at the end, fixed order, one fp32 row per CTA, second pass over the rows).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/kdw.h"
#include "fprop_core.cuh"
#include "kdw_common.cuh"

namespace kdw {

template <class Cfg>
struct ACfg {
    static constexpr int R_BYTES = Cfg::WT * Cfg::DT * Cfg::CS * 2;  // residual tile [WT][DT][CS]
    static constexpr int STAGE = Cfg::IN_STRIDE + R_BYTES;
    static constexpr int RED_BYTES = 2 * Cfg::CS * 4;
    static constexpr int SMEM = Cfg::ST * STAGE + 2 * Cfg::NCW * Cfg::OUTW_BYTES + RED_BYTES + 16 * Cfg::ST + 128;
    static_assert(R_BYTES % 128 == 0, "residual tile alignment");
};

// Adds the consumer threads' statistics for channel slice c0 to the CTA's workspace row [2][C] and clears them.
template <class Cfg>
__device__ __forceinline__ bool flush_stats(float2 (&S1)[Cfg::CP], float2 (&S2)[Cfg::CP], float* red, float* row, int C,
                                            int c0, int tid, bool failed) {
    constexpr int CS = Cfg::CS, CP = Cfg::CP, CPG = Cfg::CPG, NCW = Cfg::NCW;
    const int lane = tid & 31, warp = tid >> 5, cg = tid % CPG;
    // all consumer warps come here, also those whose bounded wait ran out: either all add their sums or none does
    if (named_barrier_or(1, Cfg::NT, failed)) return true;
#pragma unroll
    for (int i = 0; i < CP; ++i) {
#pragma unroll
        for (int off = CPG; off < 32; off <<= 1) {
            S1[i].x += __shfl_xor_sync(0xffffffffu, S1[i].x, off);
            S1[i].y += __shfl_xor_sync(0xffffffffu, S1[i].y, off);
            S2[i].x += __shfl_xor_sync(0xffffffffu, S2[i].x, off);
            S2[i].y += __shfl_xor_sync(0xffffffffu, S2[i].y, off);
        }
    }
    for (int wi = 0; wi < NCW; ++wi) {
        if (warp == wi && lane < CPG) {
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                float* d1 = red + cg * 2 * CP + 2 * i;
                float* d2 = d1 + CS;
                if (wi == 0) {
                    d1[0] = S1[i].x, d1[1] = S1[i].y, d2[0] = S2[i].x, d2[1] = S2[i].y;
                } else {
                    d1[0] += S1[i].x, d1[1] += S1[i].y, d2[0] += S2[i].x, d2[1] += S2[i].y;
                }
            }
        }
        named_barrier_sync(1, Cfg::NT);
    }
    for (int e = tid; e < 2 * CS; e += Cfg::NT) row[(e / CS) * C + c0 + e % CS] += red[e];
    named_barrier_sync(1, Cfg::NT);
#pragma unroll
    for (int i = 0; i < CP; ++i) S1[i] = S2[i] = make_float2(0.f, 0.f);
    return false;
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NT + 32, Cfg::MINB)
    fprop_addstats_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmr,
                          const __grid_constant__ CUtensorMap tmy, const __half* __restrict__ weight,
                          float* __restrict__ ws, const Sched s, const int C, const int W, const int D, int* status) {
    using A = ACfg<Cfg>;
    constexpr int M = Cfg::M, CP = Cfg::CP, ST = Cfg::ST, NCW = Cfg::NCW;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    unsigned char* in_base = smem;                    // ST stages of [input tile | residual tile]
    unsigned char* out_base = smem + ST * A::STAGE;   // per consumer warp: two output tiles
    float* red = reinterpret_cast<float*>(out_base + 2 * NCW * Cfg::OUTW_BYTES);
    const uint32_t full0 = smem_u32(out_base + 2 * NCW * Cfg::OUTW_BYTES + A::RED_BYTES);
    const uint32_t empty0 = full0 + 8 * ST;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    float* row = ws + (size_t)blockIdx.x * 2 * C;  // this CTA's [2][C] sums
    if (tid == 0) {
        prefetch_tmap(&tmx);
        prefetch_tmap(&tmr);
        prefetch_tmap(&tmy);
        for (int k = 0; k < ST; ++k) {
            mbar_init(full0 + 8 * k, 1);
            mbar_init(empty0 + 8 * k, NCW);
        }
        mbar_fence_init();
    }
    for (int k = tid; k < 2 * C; k += Cfg::NT + 32) row[k] = 0.f;
    __syncthreads();

    if (warp == NCW) {
        // ---------------- producer warp ----------------
        if (lane != 0) return;
        StepIter it;
        it.init(s, (int)blockIdx.x, (int)gridDim.x);
        uint32_t pi = 0;
        bool ok = true;
        while (it.active && ok) {
            const uint32_t st = pi % ST;
            if (pi >= ST) ok = mbar_wait_bounded(empty0 + 8 * st, ((pi / ST) & 1u) ^ 1u);
            if (!ok) break;
            const bool with_r = it.q - 1 >= it.g.hb;  // this step finishes plane q-1: bring its residual tile
            const uint32_t bar = full0 + 8 * st;
            mbar_expect_tx(bar, Cfg::IN_BYTES + (with_r ? A::R_BYTES : 0));
            tma_load_5d(status, smem_u32(in_base + st * A::STAGE), &tmx, bar, it.g.c0, it.g.d0 - 1, it.g.w0 - 1, it.q,
                        it.g.n);
            if (with_r)
                tma_load_5d(status, smem_u32(in_base + st * A::STAGE + Cfg::IN_STRIDE), &tmr, bar, it.g.c0, it.g.d0,
                            it.g.w0, it.q - 1, it.g.n);
            ++pi;
            it.next(s);
        }
        if (!ok) {
            atomicExch(status, (int)KDW_STATUS_TMA_TIMEOUT);
            const uint32_t first = pi > ST ? pi - ST : 0;
            for (uint32_t k = first; k < pi; ++k) (void)mbar_wait_bounded(full0 + 8 * (k % ST), (k / ST) & 1u);
        }
        return;
    }

    // ---------------- consumer warps ----------------
    const FThread<Cfg> th(tid);
    const int res_off = ((th.wg * M) * Cfg::DT + th.d) * Cfg::CS + th.cg * 2 * CP;
    unsigned char* my_out = out_base + warp * 2 * Cfg::OUTW_BYTES;
    StepIter it;
    it.init(s, (int)blockIdx.x, (int)gridDim.x);

    __half2 wgt[27][CP];
    float2 P1[M][CP], P2[M][CP], S1[CP], S2[CP];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int i = 0; i < CP; ++i) P1[m][i] = P2[m][i] = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < CP; ++i) S1[i] = S2[i] = make_float2(0.f, 0.f);

    uint32_t ci = 0, oc = 0;
    int cur_c0 = -1;  // channel slice the statistics belong to
    int mv = 0;       // outputs of this thread that lie inside the volume (the tile may overhang W and D)
    bool failed = false;
    while (it.active) {
        const int q = it.q;
        if (q == it.g.hb - 1) {  // new segment
            const __half* wp = weight + it.g.c0 + th.cg * 2 * CP;
#pragma unroll
            for (int k = 0; k < 27; ++k)
#pragma unroll
                for (int i = 0; i < CP; ++i)
                    wgt[k][i] = *reinterpret_cast<const __half2*>(wp + (size_t)k * C + 2 * i);
            if (it.g.c0 != cur_c0) {
                if (cur_c0 >= 0 && flush_stats<Cfg>(S1, S2, red, row, C, cur_c0, tid, failed)) failed = true;
                cur_c0 = it.g.c0;
            }
            mv = W - (it.g.w0 + th.wg * M);
            mv = mv < 0 ? 0 : (mv > M ? M : mv);
            if (it.g.d0 + th.d >= D) mv = 0;
        }
        const uint32_t st = ci % ST;
        if (!failed) {
            const bool ok = mbar_wait_bounded(full0 + 8 * st, (ci / ST) & 1u);
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0) atomicExch(status, (int)KDW_STATUS_TMA_TIMEOUT);
                failed = true;  // keeps walking the schedule (no waits, no work) to meet the others at the flushes
            }
        }
        if (!failed) {
            const bool store = q - 1 >= it.g.hb;
            unsigned char* ob_bytes = my_out + (oc & 1u) * Cfg::OUTW_BYTES;
            if (store && lane == 0) tma_wait_read<1>();
            __syncwarp();
            const __half* in = reinterpret_cast<const __half*>(in_base + st * A::STAGE) + th.in_off;
            const __half* res = reinterpret_cast<const __half*>(in_base + st * A::STAGE + Cfg::IN_STRIDE) + res_off;
            __half* ob = reinterpret_cast<__half*>(ob_bytes) + th.out_off;
            if (ci & 1u)
                fprop_step_f32_addstats<Cfg>(in, res, ob, store, mv, wgt, P2, P1, S1, S2);
            else
                fprop_step_f32_addstats<Cfg>(in, res, ob, store, mv, wgt, P1, P2, S1, S2);
            if (store) fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(empty0 + 8 * st);
                if (store) {
                    tma_store_5d(status, &tmy, smem_u32(ob_bytes), it.g.c0, it.g.d0 + th.warp_d0, it.g.w0 + th.wg * M,
                                 q - 1, it.g.n);
                    tma_commit();
                }
            }
            if (store) ++oc;
        }
        it.next(s);
        ++ci;
    }
    if (lane == 0) tma_wait_all();
    if (cur_c0 >= 0) (void)flush_stats<Cfg>(S1, S2, red, row, C, cur_c0, tid, failed);
}

// One warp per output k in [0, 2C): rows added in a fixed order, scaled by 1 / (voxels per channel).
__global__ void __launch_bounds__(128) stats_reduce_kernel(const float* __restrict__ ws, int rows, int C, float inv_count,
                                                          float* __restrict__ mean, float* __restrict__ sqmean) {
    const int k = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (k >= 2 * C) return;
    grid_dependency_wait();  // launched with launch_overlapping_previous: pass 1 may still be running
    float acc = 0.f;
    for (int r = lane; r < rows; r += 32) acc += ws[(size_t)r * 2 * C + k];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) {
        if (k < C)
            mean[k] = acc * inv_count;
        else
            sqmean[k - C] = acc * inv_count;
    }
}

struct AddStatsArgs {
    const void *x, *w, *r;
    void* y;
    float* ws;
    int64_t ws_rows;
    int64_t N, C, H, W, D, xsN, xsH, xsW, rsN, rsH, rsW, ysN, ysH, ysW;
    cudaStream_t stream;
};

template <class Cfg>
static int launch_addstats(const AddStatsArgs& a, int* rows_used) {
    using A = ACfg<Cfg>;
    CUtensorMap tmx, tmr, tmy;
    int rc = encode_volume_map(&tmx, a.x, a.N, a.C, a.H, a.W, a.D, a.xsN, a.xsH, a.xsW, Cfg::CS, Cfg::DT + 2,
                               Cfg::WT + 2);
    if (rc) return rc;
    rc = encode_volume_map(&tmr, a.r, a.N, a.C, a.H, a.W, a.D, a.rsN, a.rsH, a.rsW, Cfg::CS, Cfg::DT, Cfg::WT);
    if (rc) return rc;
    rc = encode_volume_map(&tmy, a.y, a.N, a.C, a.H, a.W, a.D, a.ysN, a.ysH, a.ysW, Cfg::CS, Cfg::DPW, Cfg::M);
    if (rc) return rc;
    if (((uintptr_t)a.w & 3) != 0) {
        set_error("weight pointer must be 4-byte aligned");
        return KDW_ERR_ALIGN;
    }
    auto kern = fprop_addstats_kernel<Cfg>;
    KDW_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, A::SMEM));
    int occ = 0, sms = 0;
    KDW_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, Cfg::NT + 32, A::SMEM));
    if (occ < 1) {
        set_error("fprop_addstats kernel variant does not fit on this device");
        return KDW_ERR_TUNE;
    }
    rc = device_sm_count(&sms);
    if (rc) return rc;
    int* status = nullptr;
    rc = status_ptr(&status);
    if (rc) return rc;
    long long target = (long long)sms * occ;
    if (target > a.ws_rows) target = a.ws_rows;
    Sched s;
    const int grid = make_sched(&s, a.N, a.C, a.W, a.D, 0, (int)a.H, Cfg::WT, Cfg::DT, Cfg::CS, (int)target);
    kern<<<grid, Cfg::NT + 32, A::SMEM, a.stream>>>(tmx, tmr, tmy, (const __half*)a.w, a.ws, s, (int)a.C, (int)a.W,
                                                    (int)a.D, status);
    KDW_CUDA(cudaGetLastError());
    *rows_used = grid;
    return 0;
}

typedef int (*AddStatsLaunch)(const AddStatsArgs&, int*);
struct AddStatsVariant {
    int cs, dt, wt;
    AddStatsLaunch f;
};
// The tiles of the forward kernel whose stage still fits with the residual tile added.
static const AddStatsVariant g_addstats_variants[] = {
    {8, 64, 8, &launch_addstats<FCfg<8, 64, 8, 8, 1, 4, 2>>},    // C = 8
    {16, 32, 8, &launch_addstats<FCfg<16, 32, 8, 8, 1, 4, 2>>},  // C = 16
    {32, 16, 8, &launch_addstats<FCfg<32, 16, 8, 8, 1, 4, 2>>},  // C >= 32
    {32, 32, 8, &launch_addstats<FCfg<32, 32, 8, 8, 1, 3, 1>>},
    {64, 8, 8, &launch_addstats<FCfg<64, 8, 8, 8, 1, 4, 2>>},
};
static const int g_n_addstats_variants = (int)(sizeof(g_addstats_variants) / sizeof(g_addstats_variants[0]));

static int auto_addstats_variant(int64_t C, int64_t D) {
    if (C == 8) return 1;
    if (C == 16) return 2;
    if (C == 32) return (D % 32 == 0 || D > 96) ? 4 : 3;
    return 5;
}

// dwconv_fprop_mma.cu
bool fprop_addstats_mma_fits(int64_t C, int64_t D);
int launch_fprop_addstats_mma(const void* x, const void* w, const void* res, void* y, float* stats_ws, int64_t stats_rows,
                              int64_t N, int64_t C, int64_t H, int64_t W, int64_t D, int64_t xsN, int64_t xsH, int64_t xsW,
                              int64_t rsN, int64_t rsH, int64_t rsW, int64_t ysN, int64_t ysH, int64_t ysW,
                              cudaStream_t stream, int* rows_used);

static int64_t addstats_rows(int* rc_out) {
    int sms = 0;
    *rc_out = device_sm_count(&sms);
    if (*rc_out) return 0;
    int64_t rows = (int64_t)sms * 8;
    return rows < 1184 ? 1184 : rows;
}

}  // namespace kdw

extern "C" {

int64_t kdw_fprop_addstats_workspace_bytes(int64_t N, int64_t C, int64_t H, int64_t W, int64_t D) {
    (void)N, (void)H, (void)W, (void)D;
    if (C <= 0) return 0;
    int rc = 0;
    const int64_t rows = kdw::addstats_rows(&rc);
    if (rc) return 0;
    return rows * 2 * C * 4;
}

int kdw_fprop_addstats_variants(void) { return kdw::g_n_addstats_variants; }

int kdw_fprop_addstats_f16(const void* x, const void* weight, const void* residual, void* y, void* workspace,
                           int64_t workspace_bytes, float* mean, float* sqmean, int64_t N, int64_t C, int64_t H,
                           int64_t W, int64_t D, int64_t x_strideN, int64_t x_strideH, int64_t x_strideW,
                           int64_t r_strideN, int64_t r_strideH, int64_t r_strideW, int64_t y_strideN,
                           int64_t y_strideH, int64_t y_strideW, int tune, void* stream) {
    using namespace kdw;
    if (!x || !weight || !residual || !y || !workspace || !mean || !sqmean) {
        set_error("fprop_addstats: null pointer");
        return KDW_ERR_ARG;
    }
    if (N <= 0 || C < 8 || H <= 0 || W <= 0 || D <= 0 || (C & (C - 1)) != 0) {
        set_error("fprop_addstats: sizes must be positive and C a power of two >= 8 (N=%lld C=%lld H=%lld W=%lld D=%lld)",
                  (long long)N, (long long)C, (long long)H, (long long)W, (long long)D);
        return KDW_ERR_ARG;
    }
    if (H > 0x7fffffff || W > 0x7fffffff || D > 0x7fffffff || N > 0x7fffffff || C > 0x7fffffff) {
        set_error("fprop_addstats: extent does not fit in 32 bits");
        return KDW_ERR_ARG;
    }
    if (tune < 0 || tune > g_n_addstats_variants) {
        set_error("fprop_addstats: tune=%d names no kernel variant (1..%d)", tune, g_n_addstats_variants);
        return KDW_ERR_TUNE;
    }
    int rc = 0;
    const int64_t rows_cap = addstats_rows(&rc);
    if (rc) return rc;
    if (workspace_bytes < rows_cap * 2 * C * 4) {
        set_error("fprop_addstats: workspace of %lld bytes, %lld needed", (long long)workspace_bytes,
                  (long long)(rows_cap * 2 * C * 4));
        return KDW_ERR_WORKSPACE;
    }
    int rows = 0;
    if (tune == 0 && fprop_addstats_mma_fits(C, D)) {
        // built-in choice: the tensor-core forward kernel with the residual add and the sums in its epilogue
        rc = launch_fprop_addstats_mma(x, weight, residual, y, (float*)workspace, rows_cap, N, C, H, W, D, x_strideN,
                                       x_strideH, x_strideW, r_strideN, r_strideH, r_strideW, y_strideN, y_strideH,
                                       y_strideW, (cudaStream_t)stream, &rows);
        if (rc) return rc;
    } else {
        const int id = tune ? tune : auto_addstats_variant(C, D);
        const AddStatsVariant& v = g_addstats_variants[id - 1];
        if (C % v.cs != 0) {
            set_error("fprop_addstats: variant %d works on %d-channel slices, C=%lld is not a multiple", id, v.cs,
                      (long long)C);
            return KDW_ERR_TUNE;
        }
        AddStatsArgs a{x, weight, residual, y, (float*)workspace, rows_cap, N, C, H, W, D, x_strideN, x_strideH, x_strideW,
                       r_strideN, r_strideH, r_strideW, y_strideN, y_strideH, y_strideW, (cudaStream_t)stream};
        rc = v.f(a, &rows);
        if (rc) return rc;
    }
    const float inv = (float)(1.0 / ((double)N * (double)H * (double)W * (double)D));
    KDW_CUDA(launch_overlapping_previous(stats_reduce_kernel, (unsigned)((2 * (int)C + 3) / 4), 128u, (cudaStream_t)stream,
                                         (const float*)workspace, rows, (int)C, inv, mean, sqmean));
    return 0;
}

}  // extern "C"
