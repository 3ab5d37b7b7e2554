// tcgen05 probe.  Not part of the library: a stand-alone program of one CTA (128 threads) that
//  (1) checks the operand layout of a TS-form tcgen05.mma (A [128 x 16] in tensor memory, written by tcgen05.st:
//      column j of a lane holds k = 2j in the low half and k = 2j+1 in the high half; B [16 x N] in shared memory,
//      K-major without swizzle; D read back with tcgen05.ld) against a host product, and
//  (2) times streams of 480 M=128, K=16 MMAs with N = 16 ... 256 columns, issued by one elected lane of a
//      converged warp (and, for comparison, by a single diverged thread).
// The depthwise stencil has 8 to 16 useful output columns per MMA, so what matters is whether small-N MMAs get
// cheaper in proportion: they do (N/2 clocks each), but an M=128 tile still needs 128 rows of voxels per channel
// group in shared and tensor memory, which is what rules the instruction out for this operator.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o tcgen05_small_n tcgen05_small_n.cu && ./tcgen05_small_n
//
// Every mbarrier wait is bounded (0.2 s); tensor memory is freed on every path.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool try_wait(uint32_t bar, uint32_t par) {
    uint32_t ok;
    asm volatile("{.reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0,1,0,p;}"
                 : "=r"(ok) : "r"(bar), "r"(par) : "memory");
    return ok;
}
__device__ __forceinline__ bool waitb(uint32_t bar, uint32_t par) {
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (int i = 0;; ++i) {
        if (try_wait(bar, par)) return true;
        if ((i & 15) == 15) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t - t0 > 200000000ull) return false;
        }
    }
}
// K-major, no swizzle: core matrix = 8 rows (N) x 16 bytes (8 K elements), rows 16 B apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo & 0x3FFFF) >> 4) << 16;
    d |= (uint64_t)((sbo & 0x3FFFF) >> 4) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version for sm_100
    return d;
}
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ uint32_t elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
    return pred;
}
// all lanes execute this; only the elected lane issues
__device__ __forceinline__ void mma_ts_u(uint32_t el, uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p, e;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 e, %5, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc), "r"(el) : "memory");
}
__device__ __forceinline__ void mma_commit_u(uint32_t el, uint32_t bar) {
    asm volatile("{\n\t.reg .pred e;\n\tsetp.ne.b32 e, %1, 0;\n\t@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar), "r"(el) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t idesc_f16(int M, int N) {
    return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

#define NPAT 8
struct Out {
    float D[128 * 16];      // layout test result
    long long clk[64];      // timing results
    int err;
};

// mode 0: layout test.  mode 1: timing.
__global__ void __launch_bounds__(128) probe(const __half* __restrict__ A,  // [128][16]
                                             const __half* __restrict__ B,  // [16 K][16 N]
                                             Out* out, int lbo, int sbo) {
    __shared__ __align__(128) unsigned char bsm[16384];
    __shared__ __align__(128) unsigned char asm_[8192];
    __shared__ __align__(8) unsigned long long bar[2];
    __shared__ uint32_t tbase;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bar[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bar[1])));
        asm volatile("fence.mbarrier_init.release.cluster;");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(s32(&tbase)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // B into smem: element (n,k) at (n/8)*sbo + (k/8)*lbo + (n%8)*16 + (k%8)*2
    for (int i = tid; i < 16384 / 4; i += 128) reinterpret_cast<uint32_t*>(bsm)[i] = 0;
    for (int i = tid; i < 8192 / 4; i += 128) reinterpret_cast<uint32_t*>(asm_)[i] = 0;
    __syncthreads();
    for (int i = tid; i < 256; i += 128) {
        const int k = i / 16, n = i % 16;
        *reinterpret_cast<__half*>(bsm + (n / 8) * sbo + (k / 8) * lbo + (n % 8) * 16 + (k % 8) * 2) = B[k * 16 + n];
    }
    // A also into smem (K-major, 128 rows): (m/8)*256 + (k/8)*128 + (m%8)*16 + (k%8)*2  [lbo=128, sbo=256]
    for (int k = 0; k < 16; ++k)
        *reinterpret_cast<__half*>(asm_ + (tid / 8) * 256 + (k / 8) * 128 + (tid % 8) * 16 + (k % 8) * 2) = A[tid * 16 + k];
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tb = tbase;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    // A row -> TMEM columns [256, 264): column j = (k=2j low half, k=2j+1 high half)
    {
        uint32_t r[8];
        for (int j = 0; j < 8; ++j) r[j] = reinterpret_cast<const uint32_t*>(A + tid * 16)[j];
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                     ::"r"(tb + lane_base + 256), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]),
                       "r"(r[6]), "r"(r[7]) : "memory");
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint64_t bdesc = make_desc(s32(bsm), lbo, sbo);
    const uint64_t adesc = make_desc(s32(asm_), 128, 256);
    bool ok = true;
    // ---- layout test: D[128x16] at columns [0,16) = A (TMEM) x B ----
    if (tid == 0) {
        mma_ts(tb + 0, tb + 256, bdesc, idesc_f16(128, 16), 0);
        mma_commit(s32(&bar[0]));
    }
    ok = waitb(s32(&bar[0]), 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
        uint32_t v[16];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
              "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(tb + lane_base + 0) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        for (int j = 0; j < 16; ++j) out->D[tid * 16 + j] = __uint_as_float(v[j]);
    } else if (tid == 0) {
        out->err = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");


    // ---- timing patterns: warp 0 runs the loop uniformly, one elected lane issues ----
    if (ok) {
        uint32_t par = 1;
        for (int pat = 0; pat < NPAT && ok; ++pat) {
            const int L = 480;
            long long t0 = 0, t1 = 0;
            if (warp == 0) {
                const uint32_t el = elect_one();
                t0 = clock64();
                switch (pat) {
                case 0:
                    for (int i = 0; i < L; i += 8) {
#pragma unroll
                        for (int u = 0; u < 8; ++u) mma_ts_u(el, tb + 48 * u, tb + 384 + 8 * u, bdesc, idesc_f16(128, 48), 1);
                    }
                    break;
                case 1:
                    for (int i = 0; i < L; i += 8) {
#pragma unroll
                        for (int u = 0; u < 8; ++u) mma_ts_u(el, tb + 16 * u, tb + 384 + 8 * u, bdesc, idesc_f16(128, 16), 1);
                    }
                    break;
                case 2:
                    for (int i = 0; i < L; i += 8) {
#pragma unroll
                        for (int u = 0; u < 8; ++u) mma_ts_u(el, tb + 128 * (u & 1), tb + 384 + 8 * u, bdesc, idesc_f16(128, 128), 1);
                    }
                    break;
                case 3:
                    for (int i = 0; i < L; i += 8) {
#pragma unroll
                        for (int u = 0; u < 8; ++u) mma_ts_u(el, tb + 48 * u, tb + 384 + 8 * u, bdesc + (uint64_t)(u * 48), idesc_f16(128, 48), 1);
                    }
                    break;
                case 4:  // divergent single-thread issue, unrolled
                    if (tid == 0)
                        for (int i = 0; i < L; i += 8) {
#pragma unroll
                            for (int u = 0; u < 8; ++u) mma_ts(tb + 48 * u, tb + 384 + 8 * u, bdesc, idesc_f16(128, 48), 1);
                        }
                    __syncwarp();
                    break;
                case 5:
                    for (int i = 0; i < L; i += 8) {
#pragma unroll
                        for (int u = 0; u < 8; ++u) mma_ts_u(el, tb + 256 * 0, tb + 384 + 8 * u, bdesc, idesc_f16(128, 256), 1);
                    }
                    break;
                case 6:
                    for (int i = 0; i < L; i += 8) {
#pragma unroll
                        for (int u = 0; u < 8; ++u) mma_ts_u(el, tb + 64 * (u & 3), tb + 384 + 8 * u, bdesc, idesc_f16(128, 64), 1);
                    }
                    break;
                case 7:
                    for (int i = 0; i < L; i += 8) {
#pragma unroll
                        for (int u = 0; u < 8; ++u) mma_ts_u(el, tb + 32 * (u & 7), tb + 384 + 8 * u, bdesc, idesc_f16(128, 32), 1);
                    }
                    break;
                default: break;
                }
                mma_commit_u(el, s32(&bar[1]));
            }
            ok = waitb(s32(&bar[1]), par ^ 1u);
            par ^= 1u;
            if (tid == 0) {
                t1 = clock64();
                out->clk[pat] = t1 - t0;
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        if (!ok && tid == 0) out->err = 2;
    }
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tb) : "memory");
}

int main() {
    std::vector<__half> A(128 * 16), B(256);
    for (int r = 0; r < 128; ++r)
        for (int k = 0; k < 16; ++k) A[r * 16 + k] = __float2half((float)(r * 16 + k));
    // B[k][n] = 1 if n == (k+1)%16  (cyclic shift) plus 2 at (k=3, n=9) to break symmetries
    for (int k = 0; k < 16; ++k)
        for (int n = 0; n < 16; ++n) B[k * 16 + n] = __float2half(n == (k + 1) % 16 ? 1.f : 0.f);
    B[3 * 16 + 9] = __float2half(2.f);
    __half *dA, *dB;
    Out* dO;
    cudaMalloc(&dA, A.size() * 2);
    cudaMalloc(&dB, B.size() * 2);
    cudaMalloc(&dO, sizeof(Out));
    cudaMemcpy(dA, A.data(), A.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(dB, B.data(), B.size() * 2, cudaMemcpyHostToDevice);
    {
        const int lbo = 128, sbo = 256;  // leading-dimension (K) and stride-dimension (N) byte offsets of B
        cudaMemset(dO, 0, sizeof(Out));
        probe<<<1, 128>>>(dA, dB, dO, lbo, sbo);
        cudaError_t e = cudaDeviceSynchronize();
        printf("B descriptor lbo=%d sbo=%d: %s\n", lbo, sbo, cudaGetErrorString(e));
        if (e != cudaSuccess) return 1;
        Out h;
        cudaMemcpy(&h, dO, sizeof(Out), cudaMemcpyDeviceToHost);
        printf("  err=%d\n", h.err);
        // expected: D[r][n] = sum_k A[r][k] B[k][n]
        double maxerr = 0;
        for (int r = 0; r < 128; ++r)
            for (int n = 0; n < 16; ++n) {
                double ref = 0;
                for (int k = 0; k < 16; ++k) ref += (double)__half2float(A[r * 16 + k]) * __half2float(B[k * 16 + n]);
                double d = fabs(ref - h.D[r * 16 + n]);
                if (d > maxerr) maxerr = d;
            }
        printf("  layout max err %.3f\n", maxerr);
        for (int r : {0, 1, 37, 127}) {
            printf("  D[%3d]:", r);
            for (int n = 0; n < 16; ++n) printf(" %6.0f", h.D[r * 16 + n]);
            printf("\n");
        }
        const char* names[NPAT] = {"N=48, 8 accumulators",        "N=16, 8 accumulators",
                                   "N=128, 2 accumulators",       "N=48, 8 accumulators, 8 B tiles",
                                   "N=48, one diverged thread",   "N=256, 1 accumulator",
                                   "N=64, 4 accumulators",        "N=32, 8 accumulators"};
        for (int p = 0; p < NPAT; ++p) printf("  %-34s %8.1f clk per MMA (480 issued)\n", names[p], h.clk[p] / 480.0);
    }
    return 0;
}
