// How fast the TMA pipeline of the convolution kernels can move data as a function of the LENGTH OF A BOX ROW.
// Not part of the library: a stand-alone program.  One producer lane streams boxes of (BX channels) x (BY voxels)
// through an ST-stage shared-memory ring (TMA load -> mbarrier); one consumer lane writes every box back with a TMA
// store ("copy") or only releases the stage ("load").  No arithmetic at all, so the rates are ceilings for any
// kernel that tiles the volume into channel slices of BX channels.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o tma_rows tma_rows.cu -lcuda && ./tma_rows
//
// The tensor is (X channels, Y voxels, Z planes) of fp16; a box row is 2*BX bytes.  With X = 128 and BX < 128 the
// rows of a box are 256 bytes apart (channel slices of a 128-channel volume); with X = BX they are contiguous.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{.reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0,1,0,p;}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}

__device__ int g_abort;

// Every wait gives up after 0.1 s (or as soon as another CTA gave up) so that a mistake cannot hang the GPU.
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity) {
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (int i = 0;; ++i) {
        if (try_wait(bar, parity)) return true;
        if ((i & 15) == 15) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t - t0 > 100000000ull || *(volatile int*)&g_abort) {
                g_abort = 1;
                return false;
            }
        }
    }
}

template <int BX, int BY, int ST, int NW, int STORE>
__global__ void __launch_bounds__(NW * 32 + 32) stream_kernel(const __grid_constant__ CUtensorMap tin,
                                                              const __grid_constant__ CUtensorMap tout, int nx, int ny,
                                                              int nz, int* err) {
    constexpr int BOX = BX * BY * 2;
    constexpr int STRIDE = (BOX + 127) / 128 * 128;
    extern __shared__ unsigned char raw[];
    unsigned char* sm = raw + ((128 - (s32(raw) & 127)) & 127);
    const uint32_t full0 = s32(sm + ST * STRIDE), empty0 = full0 + 8 * ST;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < ST; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full0 + 8 * i));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty0 + 8 * i), "r"(NW));
        }
        asm volatile("fence.mbarrier_init.release.cluster;");
    }
    __syncthreads();
    const long long total = (long long)nx * ny * nz;
    const long long lo = blockIdx.x * total / gridDim.x, hi = (blockIdx.x + 1) * total / gridDim.x;
    if (warp == NW) {  // producer
        if (lane) return;
        uint32_t pi = 0;
        for (long long p = lo; p < hi; ++p, ++pi) {
            const int t = p / nz, z = p % nz, tx = t % nx, ty = t / nx;
            const uint32_t st = pi % ST;
            if (pi >= ST && !wait_bounded(empty0 + 8 * st, ((pi / ST) & 1) ^ 1)) {
                *err = 1;
                return;
            }
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full0 + 8 * st), "r"(BOX));
            asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2,%3,%4}], [%5];"
                         ::"r"(s32(sm + st * STRIDE)), "l"(&tin), "r"(tx * BX), "r"(ty * BY), "r"(z), "r"(full0 + 8 * st)
                         : "memory");
        }
        return;
    }
    uint32_t ci = 0;
    for (long long p = lo; p < hi; ++p, ++ci) {
        const int t = p / nz, z = p % nz, tx = t % nx, ty = t / nx;
        const uint32_t st = ci % ST;
        if (!wait_bounded(full0 + 8 * st, (ci / ST) & 1)) {
            if (lane == 0) *err = 2;
            return;
        }
        if (STORE && warp == 0 && lane == 0) {  // the box goes back straight from its stage
            asm volatile("fence.proxy.async.shared::cta;");
            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1,%2,%3}], [%4];"
                         ::"l"(&tout), "r"(tx * BX), "r"(ty * BY), "r"(z), "r"(s32(sm + st * STRIDE)) : "memory");
            asm volatile("cp.async.bulk.commit_group;");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty0 + 8 * st) : "memory");
    }
    if (warp == 0 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeFn g_encode;

static CUtensorMap make_map(void* base, long X, long Y, long Z, int bx, int by) {
    CUtensorMap m;
    cuuint64_t dims[3] = {(cuuint64_t)X, (cuuint64_t)Y, (cuuint64_t)Z};
    cuuint64_t strides[2] = {(cuuint64_t)X * 2, (cuuint64_t)X * Y * 2};
    cuuint32_t box[3] = {(cuuint32_t)bx, (cuuint32_t)by, 1}, elem[3] = {1, 1, 1};
    CUresult r = g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, base, dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r) {
        printf("cuTensorMapEncodeTiled failed: %d (box %d x %d)\n", (int)r, bx, by);
        exit(1);
    }
    return m;
}

template <int BX, int BY, int ST, int STORE>
void run(const char* name, __half* in, __half* out, long X, long Y, long Z, int* err) {
    constexpr int NW = 8;
    CUtensorMap ti = make_map(in, X, Y, Z, BX, BY), to = make_map(out, X, Y, Z, BX, BY);
    auto kern = stream_kernel<BX, BY, ST, NW, STORE>;
    constexpr int BOX = BX * BY * 2;
    const int smem = ST * ((BOX + 127) / 128 * 128) + 16 * ST + 128;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    int occ, sms;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, NW * 32 + 32, smem);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
    if (occ > 2) occ = 2;
    const int nx = X / BX, ny = (Y + BY - 1) / BY, grid = sms * occ;
    for (int i = 0; i < 2; ++i) kern<<<grid, NW * 32 + 32, smem>>>(ti, to, nx, ny, (int)Z, err);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0), cudaEventCreate(&e1);
    cudaEventRecord(e0);
    for (int i = 0; i < 5; ++i) kern<<<grid, NW * 32 + 32, smem>>>(ti, to, nx, ny, (int)Z, err);
    cudaEventRecord(e1);
    cudaEventSynchronize(e1);
    float ms;
    cudaEventElapsedTime(&ms, e0, e1);
    ms /= 5;
    const double bytes = (double)X * Y * Z * 2 * (STORE ? 2 : 1);
    const double rows = (double)X / BX * Y * Z * (STORE ? 2 : 1);
    int h;
    cudaMemcpy(&h, err, 4, cudaMemcpyDeviceToHost);
    printf("%-36s rows of %4d B, box %5.1f KB, %d stages, %d CTA/SM: %7.4f ms %7.1f GB/s %6.1f G rows/s %s err=%d %s\n", name,
           BX * 2, BOX / 1024.0, ST, occ, ms, bytes / ms / 1e6, rows / ms / 1e6, STORE ? "(load+store)" : "(load)", h,
           cudaGetErrorString(cudaGetLastError()));
    fflush(stdout);
    if (h) exit(2);
}

int main() {
    void* p;
    cudaDriverEntryPointQueryResult q;
    cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    g_encode = (EncodeFn)p;
    int* err;
    cudaMalloc(&err, 4);
    cudaMemset(err, 0, 4);
    {  // channel slices of a 128-channel volume: 100 planes of 350 x 128 voxels (1.15 GB per tensor)
        const long X = 128, Y = 350L * 128, Z = 100;
        __half *in, *out;
        cudaMalloc(&in, X * Y * Z * 2), cudaMalloc(&out, X * Y * Z * 2);
        cudaMemset(in, 0, X * Y * Z * 2);
        run<8, 256, 8, 1>("C=128, slices of 8", in, out, X, Y, Z, err);
        run<8, 256, 8, 0>("C=128, slices of 8", in, out, X, Y, Z, err);
        run<16, 256, 8, 1>("C=128, slices of 16", in, out, X, Y, Z, err);
        run<16, 256, 8, 0>("C=128, slices of 16", in, out, X, Y, Z, err);
        run<32, 256, 6, 1>("C=128, slices of 32", in, out, X, Y, Z, err);
        run<32, 256, 6, 0>("C=128, slices of 32", in, out, X, Y, Z, err);
        run<64, 160, 4, 1>("C=128, slices of 64", in, out, X, Y, Z, err);
        run<64, 160, 4, 0>("C=128, slices of 64", in, out, X, Y, Z, err);
        run<128, 80, 4, 1>("C=128, whole voxels", in, out, X, Y, Z, err);
        run<128, 80, 4, 0>("C=128, whole voxels", in, out, X, Y, Z, err);
        cudaFree(in), cudaFree(out);
    }
    {  // whole voxels of narrow volumes: the rows of a box are contiguous in memory
        const long Y = 350L * 128, Z = 350;
        __half *in, *out;
        cudaMalloc(&in, 32 * Y * Z * 2), cudaMalloc(&out, 32 * Y * Z * 2);
        cudaMemset(in, 0, 32 * Y * Z * 2);
        run<8, 256, 8, 1>("C=8, whole voxels (contiguous)", in, out, 8, Y, Z, err);
        run<16, 256, 8, 1>("C=16, whole voxels (contiguous)", in, out, 16, Y, Z, err);
        run<16, 256, 8, 0>("C=16, whole voxels (contiguous)", in, out, 16, Y, Z, err);
        run<8, 256, 8, 1>("C=16, slices of 8", in, out, 16, Y, Z, err);
        run<32, 256, 6, 1>("C=32, whole voxels (contiguous)", in, out, 32, Y, Z, err);
        cudaFree(in), cudaFree(out);
    }
    printf("%s\n", cudaGetErrorString(cudaDeviceSynchronize()));
    return 0;
}
