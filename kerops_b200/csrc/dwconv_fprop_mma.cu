// Depthwise 3x3x3 forward pass on the tensor cores (warp-level mma.sync), fp32 accumulation.
//
// Same column march, TMA pipeline and producer warp as fprop_tma_kernel (dwconv_fprop.cu); only the arithmetic
// differs.  Channels are processed in slices of 8, so a voxel is one 16-byte row of the shared-memory tile.
// For 16 consecutive voxels along d and the 8 channels of the slice, one input plane contributes
//     out_a[v, c] += sum_{taps j} x[v + j, c] * w[a, j, c]          (a = 0, 1, 2: the three output planes it feeds)
// which is written as  D[16 x 8] += A[16 x 16] * B[16 x 8]  with
//     A[v, (j, c')] = x[v + tap_j, c']        two taps j per k16 step: an ldmatrix.x4 whose four 8x8 matrices are
//                                             the voxel rows of the two shifted positions - no data rearrangement,
//     B[(j, c'), c] = w[a, tap_j, c] if c' == c else 0      (kept in registers, rebuilt once per segment).
// Only the channel diagonal of B is non-zero, so 1/8 of the tensor-core multiply-adds are useful; the tensor pipe
// (about 940 multiply-adds per clock per SM for mma.sync on B200) still delivers as many useful ones as the FMA
// pipe, so the work is split: the tap pairs (t=0, t=1) go to the tensor cores, the t=2 taps stay on the FMA pipe
// as mixed-precision FMAs on the same fp32 accumulators (see fprop_mma_step).  fp16 x fp16 products are exact
// and sums are kept in fp32, as in KDW_ACC_F32.
#include "../../include/kdw.h"
#include "kdw_common.cuh"

namespace kdw {

template <int DT_, int WT_, int BW_, int ST_, int MINB_, bool MG_ = false>
struct MCfg {
    static constexpr bool MG = MG_;     // C == 8 only: tensor maps with the D and C axes merged (long TMA rows)
    static constexpr int CS = 8;        // channels per slice: one 16-byte row per voxel
    static constexpr int DT = DT_;      // d extent of the CTA tile (multiple of 16)
    static constexpr int WT = WT_;      // w extent of the CTA tile
    static constexpr int BW = BW_;      // w positions per warp (each a 16-voxel block along d)
    static constexpr int ST = ST_;      // input pipeline stages
    static constexpr int MINB = MINB_;
    static constexpr int WD = DT / 16;  // warps along d
    static constexpr int WW = WT / BW;  // warps along w
    static constexpr int NCW = WD * WW;  // compute warps; warp NCW is the TMA producer
    static constexpr int NT = NCW * 32;
    static constexpr int ROW = (DT + 2) * 16;  // bytes between consecutive w lines of an input stage
    static constexpr int IN_BYTES = (WT + 2) * ROW;
    static constexpr int IN_STRIDE = (IN_BYTES + 127) / 128 * 128;
    static constexpr int OUTW_BYTES = BW * 16 * 16;  // one warp's output tile [BW][16][8] halfs
    static constexpr int SMEM = ST * IN_STRIDE + 2 * NCW * OUTW_BYTES + 16 * ST + 128;
    static_assert(DT % 16 == 0 && WT % BW == 0, "tile shape");
    static_assert(OUTW_BYTES % 128 == 0, "out tile alignment");
    static_assert(DT + 2 <= 256 && WT + 2 <= 256, "TMA box limits");
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t (&r)[2]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
// d = a * b + c (m16n8k16, fp16 operands, fp32 accumulate); ZERO: c = 0
template <bool ZERO>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (ZERO) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
            "{%10, %10, %10, %10};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
            "{%0, %1, %2, %3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}
__device__ __forceinline__ void mma1688(float (&d)[4], const uint32_t (&a)[2], uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(b0));
}

// One input plane against the three output planes; R = (step count) % 3 rotates the roles of the three
// accumulator sets: set (R+2)%3 starts plane q+1 (taps a=0), set (R+1)%3 continues plane q (a=1), set R%3
// finishes plane q-1 (a=2) and is written to the warp's output tile when `store` is set.
//
// The warp walks the BW+2 input lines (w positions) of its tile once.  For a line it fetches the A fragment of
// the tap pair (t=0, t=1) with one ldmatrix.x4 and the t=2 values with two 4-byte loads, and uses them for the
// (up to) three outputs blk = line - b that read this line through tap b: 3 planes x 3 outputs = 9 mma (k16)
// on nine different accumulators, plus the t=2 taps as mixed-precision FMAs on the same accumulators (the mma
// accumulator fragment of a thread is rows g, g+8 x channels 2q, 2q+1 - exactly a pair of channel pairs).
// Splitting the taps this way keeps the tensor pipe, the FMA pipe and shared-memory bandwidth all below their
// limits: 9 mma + 18 packed FMAs per 16x8 outputs per plane step, 9 B of shared-memory reads per output.
template <class Cfg, int R>
__device__ __forceinline__ void fprop_mma_step(uint32_t stage_lane_addr, const unsigned char* stage_x2, unsigned char* ob,
                                               bool store, const uint32_t (&wbp)[3][3][2], const __half2 (&w2)[3][3],
                                               float (&acc)[3][Cfg::BW][4], int lane) {
    constexpr int SET[3] = {(R + 2) % 3, (R + 1) % 3, R % 3};
    constexpr int BW = Cfg::BW;
    const int g = lane >> 2, q = lane & 3;
#pragma unroll
    for (int wl = 0; wl < BW + 2; ++wl) {
        uint32_t a[4];
        ldsm_x4(stage_lane_addr + wl * Cfg::ROW, a);
        const __half2 x2g = *reinterpret_cast<const __half2*>(stage_x2 + wl * Cfg::ROW);             // row g,   t = 2
        const __half2 x2h = *reinterpret_cast<const __half2*>(stage_x2 + wl * Cfg::ROW + 8 * 16);    // row g+8, t = 2
#pragma unroll
        for (int b = 0; b < 3; ++b) {
            const int blk = wl - b;  // output position that reads this line through tap b
            if (blk < 0 || blk >= BW) continue;
#pragma unroll
            for (int r = 0; r < 3; ++r) {
                float(&d)[4] = acc[SET[r]][blk];
                if (r == 0 && b == 0)
                    mma16816<true>(d, a, wbp[r][b][0], wbp[r][b][1]);  // first taps of a new plane
                else
                    mma16816<false>(d, a, wbp[r][b][0], wbp[r][b][1]);
                float2 lo = fma_h2_f2(w2[r][b], x2g, make_float2(d[0], d[1]));
                float2 hi = fma_h2_f2(w2[r][b], x2h, make_float2(d[2], d[3]));
                d[0] = lo.x;
                d[1] = lo.y;
                d[2] = hi.x;
                d[3] = hi.y;
            }
        }
        const int blk = wl - 2;  // all nine taps of this plane are in
        if (blk >= 0 && store) {  // plane q-1 is finished: rows g and g+8 of the 16-voxel block, channels 2q, 2q+1
            const float(&d)[4] = acc[SET[2]][blk];
            *reinterpret_cast<__half2*>(ob + ((blk * 16 + g) * 8 + 2 * q) * 2) = __floats2half2_rn(d[0], d[1]);
            *reinterpret_cast<__half2*>(ob + ((blk * 16 + g + 8) * 8 + 2 * q) * 2) = __floats2half2_rn(d[2], d[3]);
        }
    }
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NT + 32, Cfg::MINB)
    fprop_mma_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmy,
                     const __half* __restrict__ weight, const Sched s, const int C, const int y_h0, int* status) {
    constexpr int ST = Cfg::ST, NCW = Cfg::NCW, BW = Cfg::BW;
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
    __syncthreads();  // the only CTA-wide barrier

    if (warp == NCW) {
        // ---------------- producer warp: one lane streams the input planes of the CTA's range ----------------
        if (lane != 0) return;
        StepIter it;
        it.init(s, (int)blockIdx.x, (int)gridDim.x);
        uint32_t pi = 0;
        bool ok = true;
        while (it.active) {
            const uint32_t st = pi % ST;
            if (pi >= ST) ok = mbar_wait_bounded(empty0 + 8 * st, ((pi / ST) & 1u) ^ 1u);
            if (!ok) break;
            mbar_expect_tx(full0 + 8 * st, Cfg::IN_BYTES);
            if (Cfg::MG)
                tma_load_5d(status, smem_u32(in_base + st * Cfg::IN_STRIDE), &tmx, full0 + 8 * st, (it.g.d0 - 1) * 8,
                            it.g.w0 - 1, it.q, it.g.n, 0);
            else
                tma_load_5d(status, smem_u32(in_base + st * Cfg::IN_STRIDE), &tmx, full0 + 8 * st, it.g.c0,
                            it.g.d0 - 1, it.g.w0 - 1, it.q, it.g.n);
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

    // ---------------- compute warps ----------------
    const int wd = warp % Cfg::WD, ww = warp / Cfg::WD;  // this warp's 16-voxel d block and group of BW w positions
    const int g = lane >> 2, q = lane & 3;
    // ldmatrix: lane L addresses row (L % 8) of matrix (L / 8); matrices 0,1 = voxels 0-7, 8-15 at the first tap of
    // a pair, matrices 2,3 = the same voxels at the second tap.  Byte offset of the lane's voxel row at tap (0, 0):
    const int vox = (lane & 7) + ((lane >> 3) & 1) * 8;
    // input line 0 of the warp, this lane's voxel row, tap t = lane / 16 (0 or 1)
    const uint32_t lane_off = (uint32_t)(((ww * BW) * (Cfg::DT + 2) + wd * 16 + vox + (lane >> 4)) * 16);
    // the same line at t = 2: row g, channels 2q, 2q+1 (row g+8 is 128 bytes further)
    const uint32_t x2_off = (uint32_t)(((ww * BW) * (Cfg::DT + 2) + wd * 16 + g + 2) * 16 + q * 4);
    unsigned char* my_out = out_base + warp * 2 * Cfg::OUTW_BYTES;

    StepIter it;
    it.init(s, (int)blockIdx.x, (int)gridDim.x);
    // B fragments of the tap pair (t=0, t=1) for plane a and tap b: the taps of channel g on the diagonal, i.e.
    // (w if 2q == g, w if 2q+1 == g), zeros elsewhere; w2[a][b]: the t=2 taps of channels 2q, 2q+1 for the FMAs
    uint32_t wbp[3][3][2];
    __half2 w2[3][3];
    float acc[3][BW][4];
#pragma unroll
    for (int r = 0; r < 3; ++r)
#pragma unroll
        for (int b = 0; b < BW; ++b)
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[r][b][k] = 0.f;

    uint32_t ci = 0, oc = 0;
    while (it.active) {
        const int qpl = it.q;
        if (qpl == it.g.hb - 1) {  // new segment: the taps of this slice's channel g, placed on the diagonal
            const unsigned short* wp = reinterpret_cast<const unsigned short*>(weight) + it.g.c0;
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int b = 0; b < 3; ++b) {
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        const uint32_t v = wp[(size_t)((a * 3 + b) * 3 + t) * C + g];
                        wbp[a][b][t] = (g == 2 * q) ? v : ((g == 2 * q + 1) ? (v << 16) : 0u);
                    }
                    w2[a][b] = *reinterpret_cast<const __half2*>(wp + (size_t)((a * 3 + b) * 3 + 2) * C + 2 * q);
                }
        }
        const uint32_t st = ci % ST;
        const bool ok = mbar_wait_bounded(full0 + 8 * st, (ci / ST) & 1u);
        if (__any_sync(0xffffffffu, !ok)) {
            if (lane == 0) atomicExch(status, (int)KDW_STATUS_TMA_TIMEOUT);
            break;
        }
        const bool store = qpl - 1 >= it.g.hb;
        unsigned char* ob = my_out + (oc & 1u) * Cfg::OUTW_BYTES;
        if (store && lane == 0) tma_wait_read<1>();
        __syncwarp();
        const uint32_t stage_lane_addr = smem_u32(in_base + st * Cfg::IN_STRIDE) + lane_off;
        const unsigned char* stage_x2 = in_base + st * Cfg::IN_STRIDE + x2_off;
        switch (ci % 3) {
            case 0: fprop_mma_step<Cfg, 0>(stage_lane_addr, stage_x2, ob, store, wbp, w2, acc, lane); break;
            case 1: fprop_mma_step<Cfg, 1>(stage_lane_addr, stage_x2, ob, store, wbp, w2, acc, lane); break;
            default: fprop_mma_step<Cfg, 2>(stage_lane_addr, stage_x2, ob, store, wbp, w2, acc, lane); break;
        }
        if (store) fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(empty0 + 8 * st);
            if (store) {
                if (Cfg::MG)
                    tma_store_5d(status, &tmy, smem_u32(ob), (it.g.d0 + wd * 16) * 8, it.g.w0 + ww * BW, qpl - 1 - y_h0,
                                 it.g.n, 0);
                else
                    tma_store_5d(status, &tmy, smem_u32(ob), it.g.c0, it.g.d0 + wd * 16, it.g.w0 + ww * BW,
                                 qpl - 1 - y_h0, it.g.n);
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
template <class Cfg>
static int launch_fprop_mma(const void* x, const void* w, void* y, int64_t N, int64_t C, int64_t Hx, int64_t W, int64_t D,
                            int64_t xsN, int64_t xsH, int64_t xsW, int64_t Hy, int64_t ysN, int64_t ysH, int64_t ysW,
                            int h_begin, int h_end, int y_h0, cudaStream_t stream) {
    CUtensorMap tmx, tmy;
    int rc;
    if (Cfg::MG) {
        if (C != 8) {
            set_error("fprop: this tensor-core variant needs C == 8");
            return KDW_ERR_TUNE;
        }
        rc = encode_merged_map(&tmx, x, N, C, Hx, W, D, xsN, xsH, xsW, (Cfg::DT + 2) * 8, Cfg::WT + 2);
        if (rc) return rc;
        rc = encode_merged_map(&tmy, y, N, C, Hy, W, D, ysN, ysH, ysW, 16 * 8, Cfg::BW);
    } else {
        rc = encode_volume_map(&tmx, x, N, C, Hx, W, D, xsN, xsH, xsW, Cfg::CS, Cfg::DT + 2, Cfg::WT + 2);
        if (rc) return rc;
        rc = encode_volume_map(&tmy, y, N, C, Hy, W, D, ysN, ysH, ysW, Cfg::CS, 16, Cfg::BW);
    }
    if (rc) return rc;
    if (((uintptr_t)w & 1) != 0) {
        set_error("weight pointer must be 2-byte aligned");
        return KDW_ERR_ALIGN;
    }
    auto kern = fprop_mma_kernel<Cfg>;
    KDW_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
    int occ = 0, sms = 0;
    KDW_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, Cfg::NT + 32, Cfg::SMEM));
    if (occ < 1) {
        set_error("fprop mma kernel variant does not fit on this device");
        return KDW_ERR_TUNE;
    }
    rc = device_sm_count(&sms);
    if (rc) return rc;
    int* status = nullptr;
    rc = status_ptr(&status);
    if (rc) return rc;
    Sched s;
    const int grid = make_sched(&s, N, C, W, D, h_begin, h_end, Cfg::WT, Cfg::DT, Cfg::CS, sms * occ);
    kern<<<grid, Cfg::NT + 32, Cfg::SMEM, stream>>>(tmx, tmy, (const __half*)w, s, (int)C, y_h0, status);
    KDW_CUDA(cudaGetLastError());
    return 0;
}

// Tensor-core variants, numbered after the variants of fprop_variants.inc by the dispatcher in dwconv_fprop.cu.
#define KDW_MMA_CASE(IDX, ...)                                                                                  \
    case IDX:                                                                                                  \
        return launch_fprop_mma<MCfg<__VA_ARGS__>>(x, w, y, N, C, Hx, W, D, xsN, xsH, xsW, Hy, ysN, ysH, ysW, h_begin, \
                                                   h_end, y_h0, stream);

int fprop_mma_variants() { return 10; }

int launch_fprop_mma_variant(int which, const void* x, const void* w, void* y, int64_t N, int64_t C, int64_t Hx,
                             int64_t W, int64_t D, int64_t xsN, int64_t xsH, int64_t xsW, int64_t Hy, int64_t ysN,
                             int64_t ysH, int64_t ysW, int h_begin, int h_end, int y_h0, cudaStream_t stream) {
    switch (which) {  // MCfg<DT, WT, BW, ST, MINB, MG>
        KDW_MMA_CASE(0, 64, 8, 4, 6, 1)
        KDW_MMA_CASE(1, 64, 6, 3, 4, 2)
        KDW_MMA_CASE(2, 64, 8, 4, 4, 2)
        KDW_MMA_CASE(3, 128, 6, 3, 3, 1)
        KDW_MMA_CASE(4, 64, 4, 2, 4, 2)
        KDW_MMA_CASE(5, 16, 32, 4, 4, 1, true)
        KDW_MMA_CASE(6, 16, 24, 3, 4, 2, true)
        KDW_MMA_CASE(7, 64, 8, 4, 10, 1)
        KDW_MMA_CASE(8, 64, 4, 2, 8, 2)
        KDW_MMA_CASE(9, 16, 32, 4, 10, 1, true)
    }
    set_error("fprop: no such tensor-core variant");
    return KDW_ERR_TUNE;
}

}  // namespace kdw
