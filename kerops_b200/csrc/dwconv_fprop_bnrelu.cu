// Forward pass with a fused prologue: y = DWConv(relu(x * scale[c] + shift[c]), weight) - the reference's
// ApplyBNReLU (kerops/ops/bnrelu.py:11-43, kerops/kernels/bnrelu.py:5-31) followed by DWConv, without writing
// and re-reading the activated tensor.  Same pipeline as fprop_tma_kernel (dwconv_fprop.cu); the step activates
// every value as it reads it from the staged tile (fprop_step_f32_bnrelu).  The convolution pads the ACTIVATED
// tensor with zeros: x is loaded with NaN as the out-of-bounds fill and max(NaN, 0) = 0 restores the padding
// without masks.  (A cooperative in-place pass over the tile with a barrier per step was measured 20-40 % slower.)
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/kdw.h"
#include "fprop_core.cuh"
#include "kdw_common.cuh"

namespace kdw {

template <class Cfg>
struct BCfg {
    static constexpr int SMEM = Cfg::ST * Cfg::IN_STRIDE + 2 * Cfg::NCW * Cfg::OUTW_BYTES + 16 * Cfg::ST + 128;
};

template <class Cfg, int PRO>
__global__ void __launch_bounds__(Cfg::NT + 32, Cfg::MINB)
    fprop_bnrelu_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmy,
                        const __half* __restrict__ weight, const float* __restrict__ scale,
                        const float* __restrict__ shift, const Sched s, const int C, int* status) {
    using B = BCfg<Cfg>;
    constexpr int M = Cfg::M, CP = Cfg::CP, ST = Cfg::ST, NCW = Cfg::NCW;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    unsigned char* in_base = smem;
    unsigned char* out_base = smem + ST * Cfg::IN_STRIDE;
    const uint32_t full0 = smem_u32(out_base + 2 * NCW * Cfg::OUTW_BYTES);
    const uint32_t empty0 = full0 + 8 * ST;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        prefetch_tmap(&tmx);
        prefetch_tmap(&tmy);
        for (int k = 0; k < ST; ++k) {
            mbar_init(full0 + 8 * k, 1);
            mbar_init(empty0 + 8 * k, NCW);
        }
        mbar_fence_init();
    }
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
            mbar_expect_tx(full0 + 8 * st, Cfg::IN_BYTES);
            tma_load_5d(status, smem_u32(in_base + st * Cfg::IN_STRIDE), &tmx, full0 + 8 * st, it.g.c0, it.g.d0 - 1,
                        it.g.w0 - 1, it.q, it.g.n);
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
    unsigned char* my_out = out_base + warp * 2 * Cfg::OUTW_BYTES;
    StepIter it;
    it.init(s, (int)blockIdx.x, (int)gridDim.x);

    __half2 wgt[27][CP];
    float2 P1[M][CP], P2[M][CP];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int i = 0; i < CP; ++i) P1[m][i] = P2[m][i] = make_float2(0.f, 0.f);

    uint32_t ci = 0, oc = 0;
    float2 sc[CP], sh[CP];  // scale / shift of this thread's channels
    while (it.active) {
        const int q = it.q;
        if (q == it.g.hb - 1) {  // new segment
            const __half* wp = weight + it.g.c0 + th.cg * 2 * CP;
#pragma unroll
            for (int k = 0; k < 27; ++k)
#pragma unroll
                for (int i = 0; i < CP; ++i)
                    wgt[k][i] = *reinterpret_cast<const __half2*>(wp + (size_t)k * C + 2 * i);
            const int cb = it.g.c0 + th.cg * 2 * CP;
#pragma unroll
            for (int i = 0; i < CP; ++i) {
                sc[i] = make_float2(scale[cb + 2 * i], scale[cb + 2 * i + 1]);
                sh[i] = make_float2(shift[cb + 2 * i], shift[cb + 2 * i + 1]);
            }
        }
        const uint32_t st = ci % ST;
        const bool ok = mbar_wait_bounded(full0 + 8 * st, (ci / ST) & 1u);
        if (__any_sync(0xffffffffu, !ok)) {
            if (lane == 0) atomicExch(status, (int)KDW_STATUS_TMA_TIMEOUT);
            break;
        }
        const __half* tile = reinterpret_cast<const __half*>(in_base + st * Cfg::IN_STRIDE);
        const bool store = q - 1 >= it.g.hb;
        unsigned char* ob_bytes = my_out + (oc & 1u) * Cfg::OUTW_BYTES;
        if (store && lane == 0) tma_wait_read<1>();
        __syncwarp();
        const __half* in = tile + th.in_off;
        __half* ob = reinterpret_cast<__half*>(ob_bytes) + th.out_off;
        if (ci & 1u)
            fprop_step_f32_bnrelu<Cfg, PRO>(in, ob, store, wgt, sc, sh, P2, P1);
        else
            fprop_step_f32_bnrelu<Cfg, PRO>(in, ob, store, wgt, sc, sh, P1, P2);
        if (store) fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(empty0 + 8 * st);
            if (store) {
                tma_store_5d(status, &tmy, smem_u32(ob_bytes), it.g.c0, it.g.d0 + th.warp_d0, it.g.w0 + th.wg * M, q - 1,
                             it.g.n);
                tma_commit();
            }
        }
        if (store) ++oc;
        it.next(s);
        ++ci;
    }
    if (lane == 0) tma_wait_all();
}

struct BnReluArgs {
    const void *x, *w;
    const float *scale, *shift;
    void* y;
    int64_t N, C, H, W, D, xsN, xsH, xsW, ysN, ysH, ysW;
    cudaStream_t stream;
};

template <class Cfg, int PRO>
static int launch_bnrelu(const BnReluArgs& a) {
    using B = BCfg<Cfg>;
    CUtensorMap tmx, tmy;
    // out-of-bounds elements of x read as NaN: the activation turns them into the padding's zeros
    int rc = encode_volume_map(&tmx, a.x, a.N, a.C, a.H, a.W, a.D, a.xsN, a.xsH, a.xsW, Cfg::CS, Cfg::DT + 2,
                               Cfg::WT + 2, /*nan_fill=*/true);
    if (rc) return rc;
    rc = encode_volume_map(&tmy, a.y, a.N, a.C, a.H, a.W, a.D, a.ysN, a.ysH, a.ysW, Cfg::CS, Cfg::DPW, Cfg::M);
    if (rc) return rc;
    if (((uintptr_t)a.w & 3) != 0) {
        set_error("weight pointer must be 4-byte aligned");
        return KDW_ERR_ALIGN;
    }
    auto kern = fprop_bnrelu_kernel<Cfg, PRO>;
    KDW_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, B::SMEM));
    int occ = 0, sms = 0;
    KDW_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, Cfg::NT + 32, B::SMEM));
    if (occ < 1) {
        set_error("fprop_bnrelu kernel variant does not fit on this device");
        return KDW_ERR_TUNE;
    }
    rc = device_sm_count(&sms);
    if (rc) return rc;
    int* status = nullptr;
    rc = status_ptr(&status);
    if (rc) return rc;
    Sched s;
    const int grid = make_sched(&s, a.N, a.C, a.W, a.D, 0, (int)a.H, Cfg::WT, Cfg::DT, Cfg::CS, sms * occ);
    kern<<<grid, Cfg::NT + 32, B::SMEM, a.stream>>>(tmx, tmy, (const __half*)a.w, a.scale, a.shift, s, (int)a.C, status);
    KDW_CUDA(cudaGetLastError());
    return 0;
}

typedef int (*BnReluLaunch)(const BnReluArgs&);
struct BnReluVariant {
    int cs, dt, wt;
    BnReluLaunch f[2];  // indexed by the prologue arithmetic: KDW_ACC_F32 / KDW_ACC_F16
};
#define KDW_BNRELU_TILE(CS, DT, WT, M, CP, ST, MINB)                          \
    {CS, DT, WT,                                                              \
     {&launch_bnrelu<FCfg<CS, DT, WT, M, CP, ST, MINB>, 0>, &launch_bnrelu<FCfg<CS, DT, WT, M, CP, ST, MINB>, 1>}}
static const BnReluVariant g_bnrelu_variants[] = {
    KDW_BNRELU_TILE(8, 64, 8, 8, 1, 4, 2),   // C = 8
    KDW_BNRELU_TILE(16, 64, 8, 8, 1, 3, 1),  // C = 16
    KDW_BNRELU_TILE(16, 32, 8, 8, 1, 4, 2),
    KDW_BNRELU_TILE(32, 32, 8, 8, 1, 3, 1),  // C = 32, 64
    KDW_BNRELU_TILE(32, 16, 8, 8, 1, 4, 2),
    KDW_BNRELU_TILE(64, 8, 8, 8, 1, 4, 2),   // C >= 128
};
#undef KDW_BNRELU_TILE
static const int g_n_bnrelu_variants = (int)(sizeof(g_bnrelu_variants) / sizeof(g_bnrelu_variants[0]));

// dwconv_fprop_mma.cu
bool fprop_bnrelu_mma_fits(int64_t C, int64_t D);
int launch_fprop_bnrelu_mma(const void* x, const float* scale, const float* shift, const void* w, void* y, int64_t N,
                            int64_t C, int64_t H, int64_t W, int64_t D, int64_t xsN, int64_t xsH, int64_t xsW,
                            int64_t ysN, int64_t ysH, int64_t ysW, bool packed_half, cudaStream_t stream);

static int auto_bnrelu_variant(int64_t C, int64_t D) {
    if (C == 8) return 1;
    if (C == 16) return (D % 64 == 0 || D > 192) ? 2 : 3;
    if (C <= 64) return (D % 32 == 0 || D > 96) ? 4 : 5;
    return 6;
}

}  // namespace kdw

extern "C" {

int kdw_fprop_bnrelu_variants(void) { return kdw::g_n_bnrelu_variants; }

int kdw_fprop_bnrelu_f16(const void* x, const float* scale, const float* shift, const void* weight, void* y, int64_t N,
                         int64_t C, int64_t H, int64_t W, int64_t D, int64_t x_strideN, int64_t x_strideH,
                         int64_t x_strideW, int64_t y_strideN, int64_t y_strideH, int64_t y_strideW,
                         int prologue_type, int tune, void* stream) {
    using namespace kdw;
    if (!x || !scale || !shift || !weight || !y) {
        set_error("fprop_bnrelu: null pointer");
        return KDW_ERR_ARG;
    }
    if (N <= 0 || C < 8 || H <= 0 || W <= 0 || D <= 0 || (C & (C - 1)) != 0) {
        set_error("fprop_bnrelu: sizes must be positive and C a power of two >= 8 (N=%lld C=%lld H=%lld W=%lld D=%lld)",
                  (long long)N, (long long)C, (long long)H, (long long)W, (long long)D);
        return KDW_ERR_ARG;
    }
    if (H > 0x7fffffff || W > 0x7fffffff || D > 0x7fffffff || N > 0x7fffffff || C > 0x7fffffff) {
        set_error("fprop_bnrelu: extent does not fit in 32 bits");
        return KDW_ERR_ARG;
    }
    if (prologue_type != KDW_ACC_F32 && prologue_type != KDW_ACC_F16) {
        set_error("fprop_bnrelu: prologue_type must be KDW_ACC_F32 or KDW_ACC_F16");
        return KDW_ERR_ARG;
    }
    if (tune < 0 || tune > g_n_bnrelu_variants) {
        set_error("fprop_bnrelu: tune=%d names no kernel variant (1..%d)", tune, g_n_bnrelu_variants);
        return KDW_ERR_TUNE;
    }
    if (tune == 0 && fprop_bnrelu_mma_fits(C, D)) {
        // built-in choice: the tensor-core forward kernel with the activation applied to its operand words
        return launch_fprop_bnrelu_mma(x, scale, shift, weight, y, N, C, H, W, D, x_strideN, x_strideH, x_strideW,
                                       y_strideN, y_strideH, y_strideW, prologue_type == KDW_ACC_F16,
                                       (cudaStream_t)stream);
    }
    const int id = tune ? tune : auto_bnrelu_variant(C, D);
    const BnReluVariant& v = g_bnrelu_variants[id - 1];
    if (C % v.cs != 0) {
        set_error("fprop_bnrelu: variant %d works on %d-channel slices, C=%lld is not a multiple", id, v.cs,
                  (long long)C);
        return KDW_ERR_TUNE;
    }
    BnReluArgs a{x, weight, scale, shift, y, N, C, H, W, D, x_strideN, x_strideH, x_strideW, y_strideN, y_strideH,
                 y_strideW, (cudaStream_t)stream};
    return v.f[prologue_type](a);
}

}  // extern "C"
