// Per-SM issue rates of the instructions the depthwise-convolution kernels are built from, on the GPU it runs on.
// Not part of the library: a stand-alone program whose output backs the choice between the CUDA-core and the
// tensor-core formulation (27 multiply-adds per voxel-channel on a pipe that retires 128 of them per clock and SM,
// against mma.sync.m16n8k16 with 27 of 96 products useful).
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o issue_rate issue_rate.cu && ./issue_rate
//
// Every kernel runs 8 independent dependency chains per thread, 4, 8, 16 and 32 warps per SM; rates are per clock
// of the nominal SM frequency the runtime reports.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

constexpr int kChains = 8;
constexpr int kIters = 4096;

enum Op {
    FFMA, FFMA2, HFMA2, MIXED_LO, MIXED_PAIR, LOP3, IMAD, PRMT, CVT_PACK, HFMA2_LOP3, FFMA_LOP3, MMA_F32, MMA_F16,
    MOVMATRIX, SHFL, MOVMATRIX_LOP3
};

template <int OP>
__global__ void chains(float* out, int n, const unsigned* src) {
    float a[kChains], b[kChains];
    float2 a2[kChains];
    unsigned h[kChains], u[kChains], w[kChains];
    float c[kChains][4];
    const float seed = threadIdx.x * 1e-3f + 1.0f;
#pragma unroll
    for (int i = 0; i < kChains; ++i) {
        a[i] = seed + i, b[i] = seed - i, a2[i] = make_float2(seed + i, seed - i);
        h[i] = 0x3c003c00u + i, u[i] = threadIdx.x * 2654435761u + i, w[i] = src[(threadIdx.x + i) & 63];
        for (int j = 0; j < 4; ++j) c[i][j] = 0.f;
    }
    const float m1 = 1.0001f, m2 = 0.9999f;
    const unsigned hm = 0x3c013bffu;
    unsigned long long m64;
    {
        float2 t = make_float2(m1, m2);
        m64 = *reinterpret_cast<unsigned long long*>(&t);
    }
    for (int it = 0; it < n; ++it) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int i = 0; i < kChains; ++i) {
                if (OP == FFMA || OP == FFMA_LOP3) asm volatile("fma.rn.f32 %0, %0, %1, %2;" : "+f"(a[i]) : "f"(m1), "f"(m2));
                if (OP == FFMA2) {
                    unsigned long long v = *reinterpret_cast<unsigned long long*>(&a2[i]);
                    asm volatile("fma.rn.f32x2 %0, %0, %1, %1;" : "+l"(v) : "l"(m64));
                    a2[i] = *reinterpret_cast<float2*>(&v);
                }
                if (OP == HFMA2 || OP == HFMA2_LOP3) asm volatile("fma.rn.f16x2 %0, %0, %1, %1;" : "+r"(h[i]) : "r"(hm));
                if (OP == MIXED_LO)  // fp16 x fp16 + fp32, both operands the low half of a packed pair
                    asm volatile("{.reg .b16 al,ah,bl,bh; mov.b32 {al,ah}, %1; mov.b32 {bl,bh}, %2; fma.rn.f32.f16 %0, al, bl, %0;}"
                                 : "+f"(a[i]) : "r"(w[i]), "r"(w[(i + r) & 7]));
                if (OP == MIXED_PAIR)  // the (lo,lo) + (hi,hi) pair a channels-last word needs
                    asm volatile("{.reg .b16 al,ah,bl,bh; mov.b32 {al,ah}, %2; mov.b32 {bl,bh}, %3; fma.rn.f32.f16 %0, al, bl, %0; "
                                 "fma.rn.f32.f16 %1, ah, bh, %1;}"
                                 : "+f"(a[i]), "+f"(b[i]) : "r"(w[i]), "r"(w[(i + r) & 7]));
                if (OP == LOP3 || OP == HFMA2_LOP3 || OP == FFMA_LOP3)
                    asm volatile("lop3.b32 %0, %0, %1, %2, 0x96;" : "+r"(u[i]) : "r"(0x12345u), "r"(0x0ff0u));
                if (OP == IMAD) asm volatile("mad.lo.u32 %0, %0, %1, %2;" : "+r"(u[i]) : "r"(0x12345u), "r"(0x0ff0u));
                if (OP == PRMT) asm volatile("prmt.b32 %0, %0, %1, 0x3210;" : "+r"(u[i]) : "r"(0x55u));
                if (OP == CVT_PACK) {
                    unsigned v;
                    asm volatile("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(v) : "f"(a[i]), "f"(m1));
                    a[i] = __uint_as_float(v | 0x3f000000u);
                }
                if (OP == MMA_F32)
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(c[i][0]), "+f"(c[i][1]), "+f"(c[i][2]), "+f"(c[i][3])
                                 : "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]), "r"(h[4]), "r"(h[5]));
                if (OP == MMA_F16)
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f16.f16.f16.f16 {%0,%1}, {%2,%3,%4,%5}, {%6,%7}, {%0,%1};"
                                 : "+r"(u[i]), "+r"(w[i]) : "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]), "r"(h[4]), "r"(h[5]));
                if (OP == MOVMATRIX || OP == MOVMATRIX_LOP3)
                    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %0;" : "+r"(u[i]));
                if (OP == MOVMATRIX_LOP3)
                    asm volatile("lop3.b32 %0, %0, %1, %2, 0x96;" : "+r"(w[(i + 4) & 7]) : "r"(0x12345u), "r"(0x0ff0u));
                if (OP == SHFL) u[i] = __shfl_xor_sync(0xffffffffu, u[i], 1);
            }
        }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kChains; ++i)
        s += a[i] + b[i] + a2[i].x + a2[i].y + (float)h[i] + (float)u[i] + (float)w[i] + c[i][0] + c[i][1] + c[i][2] + c[i][3];
    out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

// `per` = instructions per chain step; `warp_wide`: report warp-instructions (mma, movmatrix, shfl) instead of lanes.
template <int OP>
void run(const char* name, int per, bool warp_wide) {
    int sms, khz;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, 0);
    float* out;
    unsigned* src;
    cudaMalloc(&out, (size_t)sms * 4 * 1024 * sizeof(float));
    cudaMalloc(&src, 64 * 4);
    cudaMemset(src, 0x3c, 64 * 4);
    printf("%-34s", name);
    for (int warps : {4, 8, 16, 32}) {
        const int threads = warps * 32 < 256 ? warps * 32 : 256, blocks = sms * (warps * 32 / threads);
        chains<OP><<<blocks, threads>>>(out, 16, src);
        cudaEvent_t e0, e1;
        cudaEventCreate(&e0), cudaEventCreate(&e1);
        cudaEventRecord(e0);
        chains<OP><<<blocks, threads>>>(out, kIters, src);
        cudaEventRecord(e1);
        cudaEventSynchronize(e1);
        float ms;
        cudaEventElapsedTime(&ms, e0, e1);
        const double inst = (double)blocks * threads * kIters * 4 * kChains * per / (warp_wide ? 32 : 1);
        printf("  %2d warps: %7.2f", warps, inst / (ms * 1e-3) / sms / (khz * 1e3));
        cudaEventDestroy(e0), cudaEventDestroy(e1);
    }
    printf("  %s/clk/SM\n", warp_wide ? "warp-inst" : "lane-inst");
    cudaFree(out), cudaFree(src);
}

int main() {
    int khz;
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, 0);
    printf("nominal SM clock %d MHz\n", khz / 1000);
    run<FFMA>("fma.rn.f32", 1, false);
    run<FFMA2>("fma.rn.f32x2 (2 FMAs each)", 1, false);
    run<HFMA2>("fma.rn.f16x2 (2 FMAs each)", 1, false);
    run<MIXED_LO>("fma.rn.f32.f16 lo*lo", 1, false);
    run<MIXED_PAIR>("fma.rn.f32.f16 lo*lo + hi*hi", 2, false);
    run<LOP3>("lop3", 1, false);
    run<IMAD>("mad.lo.u32", 1, false);
    run<PRMT>("prmt", 1, false);
    run<CVT_PACK>("cvt.rn.f16x2.f32 (+lop3)", 2, false);
    run<HFMA2_LOP3>("fma.rn.f16x2 + lop3", 2, false);
    run<FFMA_LOP3>("fma.rn.f32 + lop3", 2, false);
    run<MMA_F32>("mma.sync.m16n8k16 f16->f32", 1, true);
    run<MMA_F16>("mma.sync.m16n8k16 f16->f16", 1, true);
    run<MOVMATRIX>("movmatrix.m8n8.trans.b16", 1, true);
    run<SHFL>("shfl.bfly", 1, true);
    run<MOVMATRIX_LOP3>("movmatrix + lop3", 2, true);
    printf("%s\n", cudaGetErrorString(cudaDeviceSynchronize()));
    return 0;
}
