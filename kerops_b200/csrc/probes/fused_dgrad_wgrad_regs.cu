// Register budget of a fused input-gradient + weight-gradient step (compile-only).  Not part of the library.
//
// A single pass over grad that produces both gradients would run, per consumer warp, the weight-gradient step of
// dwconv_wgrad_mma.cu (96 fp32 accumulators that live for the whole range, three planes of transposed grad
// fragments) AND the forward step of dwconv_fprop_mma.cu applied to grad with the flipped taps (48 weight-fragment
// registers, two sets of 16 accumulators), on the same staged grad tile.  A consumer thread can own at most 232
// registers (12 warps per SM with the register hand-over the kernels already use).  This file puts the two steps,
// for ONE unit per warp, into one loop and lets the compiler report what that costs:
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -std=c++17 -O3 -maxrregcount 232 -Xptxas -v \
//        -I.. -c fused_dgrad_wgrad_regs.cu -o /dev/null
//
// and read the "bytes spill stores / spill loads" of fused_step_probe (the kernel is never launched).
#include "../dwconv_fprop_mma.cu"
#include "../dwconv_wgrad_mma.cu"

namespace kdw {

using ProbeCfg = PCfg<64, 2, 1, 2, 4, 0>;

__global__ void fused_step_probe(uint32_t stage, uint32_t out, const uint32_t* w, float* res, int n,
                                                        uint32_t zero, const int* dsc) {
    uint32_t Bf[4][3][2][2];  // flipped taps of the input gradient
    for (int i = 0; i < 48; ++i) (&Bf[0][0][0][0])[i] = w[i * 32 + threadIdx.x];
    float S0[4][4], S1[4][4];     // input-gradient planes in flight
    uint32_t Gf[3][4][2];         // transposed grad fragments of planes q-1, q, q+1
    float acc[2][4][3][4];        // weight gradient
    for (int i = 0; i < 24; ++i) (&Gf[0][0][0])[i] = 0u;
    for (int i = 0; i < 96; ++i) (&acc[0][0][0][0])[i] = 0.f;
    const uint32_t a = stage + threadIdx.x * 16;
    auto step = [&](float(&FIN)[4][4], float(&MID)[4][4], int it, auto rot) {
        uint4 X[6], GX[6];
#pragma unroll
        for (int r = 0; r < 6; ++r) X[r] = lds128(a + r * 4608 + (it & 3) * 40960);            // x plane q, halo rows
#pragma unroll
        for (int r = 0; r < 6; ++r) GX[r] = lds128(a + 20480 + r * 4608 + (it & 3) * 40960);   // grad plane, halo rows
        const uint4 G0 = lds128(a + 20480 + 4608 + 256), G1 = lds128(a + 20480 + 3 * 4608 + 256);  // its own voxels
        wg_step<decltype(rot)::value>(X, G0, G1, Gf, acc);
        pg_step<ProbeCfg>(GX, Bf, FIN, MID, (dsc[it & 7] & 1) != 0, out + threadIdx.x * 16, out + 8192 + threadIdx.x * 16,
                          zero);
    };
#pragma unroll 1
    for (int it = 0; it < n; it += 6) {  // six steps: the grad-plane rotation has period 3, the accumulator swap 2
        step(S0, S1, it, std::integral_constant<int, 0>{});
        step(S1, S0, it + 1, std::integral_constant<int, 1>{});
        step(S0, S1, it + 2, std::integral_constant<int, 2>{});
        step(S1, S0, it + 3, std::integral_constant<int, 0>{});
        step(S0, S1, it + 4, std::integral_constant<int, 1>{});
        step(S1, S0, it + 5, std::integral_constant<int, 2>{});
    }
    float s = 0.f;
    for (int i = 0; i < 96; ++i) s += (&acc[0][0][0][0])[i];
    for (int i = 0; i < 16; ++i) s += (&S0[0][0])[i] + (&S1[0][0])[i];
    res[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

}  // namespace kdw
