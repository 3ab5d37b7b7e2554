// Host-side helpers of the library: error string, device status word, tensor-map encoding,
// schedule construction.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "../../include/kdw.h"
#include "kdw_common.cuh"

namespace kdw {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return (int)e;
}

// One status word per device that loads the library.
static __device__ int g_status_word;

int status_ptr(int** p) {
    void* addr = nullptr;
    KDW_CUDA(cudaGetSymbolAddress(&addr, g_status_word));
    *p = (int*)addr;
    return 0;
}

int device_sm_count(int* sms) {
    int dev = 0;
    KDW_CUDA(cudaGetDevice(&dev));
    KDW_CUDA(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
    return 0;
}

int KernelSetup::get(const void* kernel, int threads, int smem, int* sms_out, int* occ_out) {
    static std::mutex mu;
    int dev = 0;
    KDW_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) {
        set_error("device index %d is outside the supported range 0..%d", dev, kMaxDevices - 1);
        return KDW_ERR_ARG;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!done[dev]) {
        KDW_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        int o = 0;
        KDW_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o, kernel, threads, smem));
        if (o < 1) {
            set_error("kernel variant does not fit on this device (%d threads, %d bytes of shared memory)", threads,
                      smem);
            return KDW_ERR_TUNE;
        }
        int n = 0;
        KDW_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
        occ[dev] = o;
        sms[dev] = n;
        done[dev] = true;
    }
    *sms_out = sms[dev];
    *occ_out = occ[dev];
    return 0;
}

static WaitTest g_wait_test = {2000000000ull, -1, 0u};
WaitTest wait_test() { return g_wait_test; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int get_encode_fn(EncodeTiledFn* out) {
    static EncodeTiledFn fn = nullptr;  // immutable once set; a race only repeats the lookup
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        KDW_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || !p) {
            set_error("cuTensorMapEncodeTiled is not available from this driver");
            return (int)cudaErrorNotSupported;
        }
        fn = (EncodeTiledFn)p;
    }
    *out = fn;
    return 0;
}

int encode_volume_map(CUtensorMap* map, const void* base, int64_t N, int64_t C, int64_t H, int64_t W, int64_t D,
                      int64_t strideN, int64_t strideH, int64_t strideW, int boxC, int boxD, int boxW, bool nan_fill,
                      int swizzle) {
    EncodeTiledFn fn;
    int rc = get_encode_fn(&fn);
    if (rc) return rc;
    if (((uintptr_t)base & 15) != 0 || (C % 8) != 0 || (strideW % 8) != 0 || (strideH % 8) != 0 ||
        (strideN % 8) != 0) {
        set_error("TMA path needs 16-byte aligned base and strides (C, strideW, strideH, strideN multiples of 8)");
        return KDW_ERR_ALIGN;
    }
    if (boxC < 8 || boxC > 256 || boxD < 1 || boxD > 256 || boxW < 1 || boxW > 256) {
        set_error("tensor-map box out of range");
        return KDW_ERR_ARG;
    }
    // a swizzled tile is used only with box rows exactly one swizzle span long (rows are then packed densely)
    if (swizzle != 0 && ((swizzle != 32 && swizzle != 64 && swizzle != 128) || boxC * 2 != swizzle)) {
        set_error("tensor-map swizzle %d does not match the %d-byte box rows", swizzle, boxC * 2);
        return KDW_ERR_ARG;
    }
    const CUtensorMapSwizzle sw = swizzle == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : swizzle == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                  : swizzle == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                  : CU_TENSOR_MAP_SWIZZLE_NONE;
    const cuuint64_t dims[5] = {(cuuint64_t)C, (cuuint64_t)D, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
    // byte strides of dims 1..4; a dimension of extent 1 still needs a legal (multiple of 16) stride
    cuuint64_t strides[4] = {(cuuint64_t)C * 2, (cuuint64_t)strideW * 2, (cuuint64_t)strideH * 2,
                             (cuuint64_t)strideN * 2};
    for (int i = 0; i < 4; ++i)
        if (strides[i] == 0) strides[i] = 16;
    const cuuint32_t box[5] = {(cuuint32_t)boxC, (cuuint32_t)boxD, (cuuint32_t)boxW, 1, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    nan_fill ? CU_TENSOR_MAP_FLOAT_OOB_FILL_NAN_REQUEST_ZERO_FMA : CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (dims C=%lld D=%lld W=%lld H=%lld N=%lld)", (int)r,
                  (long long)C, (long long)D, (long long)W, (long long)H, (long long)N);
        return (int)r;
    }
    return 0;
}

// The same volume with the D and C axes merged into one contiguous axis of D*C elements: dims (D*C, W, H, N, 1),
// box (boxDC, boxW, 1, 1, 1).  Rows of a box are then boxDC*2 bytes long instead of C*2, which matters for small
// C (a 16-byte row per voxel makes poor use of the TMA unit).  Zero fill works as before because W stays an
// axis of its own; only usable when a CTA takes all channels of a voxel.
int encode_merged_map(CUtensorMap* map, const void* base, int64_t N, int64_t C, int64_t H, int64_t W, int64_t D,
                      int64_t strideN, int64_t strideH, int64_t strideW, int boxDC, int boxW, bool nan_fill) {
    EncodeTiledFn fn;
    int rc = get_encode_fn(&fn);
    if (rc) return rc;
    if (((uintptr_t)base & 15) != 0 || (C % 8) != 0 || (strideW % 8) != 0 || (strideH % 8) != 0 ||
        (strideN % 8) != 0) {
        set_error("TMA path needs 16-byte aligned base and strides (C, strideW, strideH, strideN multiples of 8)");
        return KDW_ERR_ALIGN;
    }
    if (boxDC < 8 || boxDC > 256 || (boxDC % 8) != 0 || boxW < 1 || boxW > 256) {
        set_error("tensor-map box out of range");
        return KDW_ERR_ARG;
    }
    const cuuint64_t dims[5] = {(cuuint64_t)(D * C), (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N, 1};
    cuuint64_t strides[4] = {(cuuint64_t)strideW * 2, (cuuint64_t)strideH * 2, (cuuint64_t)strideN * 2,
                             (cuuint64_t)strideN * 2 * (cuuint64_t)N};
    for (int i = 0; i < 4; ++i)
        if (strides[i] == 0) strides[i] = 16;
    const cuuint32_t box[5] = {(cuuint32_t)boxDC, (cuuint32_t)boxW, 1, 1, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    nan_fill ? CU_TENSOR_MAP_FLOAT_OOB_FILL_NAN_REQUEST_ZERO_FMA : CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (merged D*C axis) failed with CUresult %d", (int)r);
        return (int)r;
    }
    return 0;
}

int encode_paired_map(CUtensorMap* map, const void* base, int64_t N, int64_t C, int64_t H, int64_t W, int64_t D,
                      int64_t strideN, int64_t strideH, int64_t strideW, int boxP, int boxW, bool nan_fill) {
    EncodeTiledFn fn;
    int rc = get_encode_fn(&fn);
    if (rc) return rc;
    if (((uintptr_t)base & 15) != 0 || C != 16 || (D & 1) != 0 || (strideW % 8) != 0 || (strideH % 8) != 0 ||
        (strideN % 8) != 0) {
        set_error("paired tensor map needs C == 16, an even D, a 16-byte aligned base and strides that are multiples of 8");
        return KDW_ERR_ALIGN;
    }
    if (boxP < 1 || boxP > 256 || boxW < 1 || boxW > 256) {
        set_error("tensor-map box out of range");
        return KDW_ERR_ARG;
    }
    const cuuint64_t dims[5] = {(cuuint64_t)(2 * C), (cuuint64_t)(D / 2), (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
    cuuint64_t strides[4] = {(cuuint64_t)C * 4, (cuuint64_t)strideW * 2, (cuuint64_t)strideH * 2, (cuuint64_t)strideN * 2};
    for (int i = 0; i < 4; ++i)
        if (strides[i] == 0) strides[i] = 16;
    const cuuint32_t box[5] = {(cuuint32_t)(2 * C), (cuuint32_t)boxP, (cuuint32_t)boxW, 1, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    nan_fill ? CU_TENSOR_MAP_FLOAT_OOB_FILL_NAN_REQUEST_ZERO_FMA : CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (paired d axis) failed with CUresult %d", (int)r);
        return (int)r;
    }
    return 0;
}

int make_sched(Sched* s, int64_t N, int64_t C, int64_t W, int64_t D, int h_begin, int h_end, int WT, int DT, int CS,
               int grid_target) {
    s->WT = WT;
    s->DT = DT;
    s->CS = CS;
    s->nWT = (int)((W + WT - 1) / WT);
    s->nDT = (int)((D + DT - 1) / DT);
    s->nCS = (int)(C / CS);
    s->Kc = s->nWT * s->nDT * s->nCS;
    s->Hr = h_end - h_begin;
    s->h_begin = h_begin;
    const long long Kall = (long long)N * s->Kc;
    const long long total = Kall * s->Hr;
    long long grid = grid_target;
    if (grid > total) grid = total;
    if (grid < 1) grid = 1;
    s->R = (int)(Kall / grid);
    s->Krem = (int)(Kall - (long long)s->R * grid);
    s->rem_total = (long long)s->Krem * s->Hr;
    s->PH = s->Hr;
    s->nh = 1;
    if (s->Krem > 0) {
        // planes per CTA in the remainder; chunk the h range so that one chunk row of all remaining columns is
        // about a whole number of CTA shares
        const double ppc = (double)s->rem_total / (double)grid;
        long long nh = (long long)((double)s->Hr / ppc + 0.5);
        if (nh < 1) nh = 1;
        if (nh > s->Hr) nh = s->Hr;
        s->PH = (int)((s->Hr + nh - 1) / nh);
        s->nh = (s->Hr + s->PH - 1) / s->PH;
    }
    return (int)grid;
}

}  // namespace kdw

extern "C" {

int kdw_version(void) { return 100; }

const char* kdw_last_error(void) { return kdw::g_err; }

int kdw_test_wait_limits(int64_t limit_ns, int stop_after) {
    if (limit_ns <= 0) {
        kdw::set_error("kdw_test_wait_limits: limit_ns must be positive");
        return KDW_ERR_ARG;
    }
    kdw::g_wait_test.limit_ns = (unsigned long long)limit_ns;
    kdw::g_wait_test.stop_after = stop_after < 0 ? -1 : stop_after;
    return 0;
}

int kdw_device_status(int* status) {
    if (!status) {
        kdw::set_error("kdw_device_status: status is NULL");
        return KDW_ERR_ARG;
    }
    KDW_CUDA(cudaDeviceSynchronize());
    int v = 0;
    KDW_CUDA(cudaMemcpyFromSymbol(&v, kdw::g_status_word, sizeof(int)));
    if (v != 0) {
        const int zero = 0;
        KDW_CUDA(cudaMemcpyToSymbol(kdw::g_status_word, &zero, sizeof(int)));
    }
    *status = v;
    return 0;
}

}  // extern "C"
