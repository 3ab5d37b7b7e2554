// Shared device/host helpers for the depthwise 3x3x3 channels-last kernels (sm_100a).
//
//  * PTX wrappers: mbarrier, tiled TMA load/store (cp.async.bulk.tensor, no cluster
//    multicast anywhere), proxy fences, the sm_100 mixed-precision add (f32 += f16).
//  * Balanced plane scheduler: the (sample, h-chunk, w-tile, d-tile, channel-slice, plane)
//    space is linearised and cut into gridDim.x equal ranges, so every CTA marches the same
//    number of h-planes (+-1) while CTAs that run at the same time work on neighbouring
//    columns of the same h-chunk (their halos then hit in L2).
//  * Host helpers: error string, tensor-map encoding through the driver entry point.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kdw {

// ------------------------------------------------------------------------------------------
// Status codes written by kernels into the per-library device status word.
// ------------------------------------------------------------------------------------------
enum : int {
    KDW_STATUS_OK = 0,
    KDW_STATUS_TMA_TIMEOUT = 1,  // a bounded mbarrier wait ran out
    KDW_STATUS_TMA_ARGS = 2,     // a TMA copy with a misaligned shared address or channel coordinate was skipped
};

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);  // records the message, returns (int)e

#define KDW_CUDA(expr)                                            \
    do {                                                          \
        cudaError_t _e = (expr);                                  \
        if (_e != cudaSuccess) return ::kdw::cuda_fail(_e, #expr); \
    } while (0)

// Encodes a 5-D fp16 tensor map over a channels-last volume: dims (C, D, W, H, N), element
// strides (1, C, strideW, strideH, strideN), box (boxC, boxD, boxW, 1, 1), zero fill for
// out-of-bounds elements.  Returns 0 or a negative argument error / positive driver error.
int encode_volume_map(CUtensorMap* map, const void* base, int64_t N, int64_t C, int64_t H, int64_t W, int64_t D,
                      int64_t strideN, int64_t strideH, int64_t strideW, int boxC, int boxD, int boxW,
                      bool nan_fill = false,  // out-of-bounds elements read as NaN instead of zero
                      int swizzle = 0);       // 0, or 32 / 64 / 128: swizzled shared-memory tile, boxC * 2 == swizzle

// As encode_volume_map with the D and C axes merged (see kdw_host.cu).
int encode_merged_map(CUtensorMap* map, const void* base, int64_t N, int64_t C, int64_t H, int64_t W, int64_t D,
                      int64_t strideN, int64_t strideH, int64_t strideW, int boxDC, int boxW, bool nan_fill = false);

// The volume with PAIRS of voxels along d as the innermost axis: dims (2*C, D/2, W, H, N), box (2*C, boxP, boxW, 1,
// 1), 64-byte swizzle.  Needs C == 16 (64-byte rows) and an even D.
int encode_paired_map(CUtensorMap* map, const void* base, int64_t N, int64_t C, int64_t H, int64_t W, int64_t D,
                      int64_t strideN, int64_t strideH, int64_t strideW, int boxP, int boxW, bool nan_fill = false);

int device_sm_count(int* sms);

#ifdef __CUDACC__
// Launches a small follow-up kernel (the fixed-order sums over per-CTA rows, the gradient exchange) with
// programmatic stream serialisation: its CTAs may be placed while the kernel before it in the stream is still
// draining, so the launch latency between two dependent kernels is hidden.  Such a kernel must execute
// grid_dependency_wait() before it touches anything the previous kernel wrote - the wait returns when that kernel
// has completed and its writes are visible; under an ordinary launch the wait returns at once.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapping_previous(void (*kernel)(KArgs...), unsigned grid, unsigned block, cudaStream_t st,
                                               Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

// Per kernel and device: the opt-in to `smem` bytes of dynamic shared memory, the CTAs per SM the kernel reaches
// with `threads` threads and the SM count - looked up on the first launch on a device and remembered (one
// static instance per kernel instantiation).
struct KernelSetup {
    static constexpr int kMaxDevices = 64;
    int occ[kMaxDevices];
    int sms[kMaxDevices];
    bool done[kMaxDevices];
    KernelSetup() {
        for (int i = 0; i < kMaxDevices; ++i) done[i] = false;
    }
    int get(const void* kernel, int threads, int smem, int* sms_out, int* occ_out);
};

// Limits of the kernels' bounded waits.  limit_ns is the time after which a wait on an mbarrier gives up (2 s by
// default); stop_after >= 0 makes the load warp of a TMA kernel stop after that many plane loads, so that the
// consumers' next wait runs out - the way the test-suite exercises the time-out path without any fault.
struct WaitTest {
    unsigned long long limit_ns;
    int stop_after;
    unsigned zero;  // always 0: a value the compiler cannot fold (see reg_copy in mma_patch.cuh)
};
WaitTest wait_test();

// Device address (on the current device) of the library's status word.
int status_ptr(int** p);

// Work decomposition shared by fprop and wgrad.  A COLUMN is (sample, w-tile, d-tile, channel-slice); a CTA
// marches a column along h.  With G CTAs and K columns:
//   * the first R = K / G "rounds" give CTA g the whole column r*G + g, so at any time the G resident CTAs
//     work on G neighbouring columns at about the same h and their halos hit in L2;
//   * the remaining K - R*G columns are cut along h into chunks, the (chunk, column, plane) space is
//     linearised and split into G equal ranges (+-1 plane), so the tail is balanced too.
struct Sched {
    long long rem_total;  // plane units of the remainder phase = Krem * Hr
    int R;                // full rounds
    int Krem;             // columns of the remainder phase
    int Kc;               // columns per sample = nWT * nDT * nCS
    int Hr;               // planes in [h_begin, h_end)
    int PH;               // planes per h-chunk (remainder phase)
    int nh;               // h-chunks (remainder phase)
    int nWT, nDT, nCS;
    int h_begin;
    int WT, DT, CS;       // tile extents (w, d, channels)
};

// Fills the schedule for `grid_target` CTAs; returns the grid size to launch.
int make_sched(Sched* s, int64_t N, int64_t C, int64_t W, int64_t D, int h_begin, int h_end, int WT, int DT, int CS,
               int grid_target);

// ------------------------------------------------------------------------------------------
// Device side
// ------------------------------------------------------------------------------------------
#ifdef __CUDACC__

#define KDW_HD __host__ __device__ __forceinline__

struct Seg {
    int n, w0, d0, c0;  // sample and tile origin
    int hb, he;         // owned planes [hb, he)
};

// Column index over all samples -> sample and tile origin.  Order: channel-slice fastest, then d-tile, w-tile, sample.
KDW_HD void decode_column(const Sched& s, int col_all, Seg& g) {
    g.n = col_all / s.Kc;
    int col = col_all - g.n * s.Kc;
    const int ics = col % s.nCS;
    col /= s.nCS;
    const int idt = col % s.nDT;
    const int iwt = col / s.nDT;
    g.w0 = iwt * s.WT;
    g.d0 = idt * s.DT;
    g.c0 = ics * s.CS;
}

// Remainder phase: decodes the segment that starts at linear position `pos` (< end) of the (h-chunk, column,
// plane) space; returns the number of plane units it covers.
KDW_HD int decode_remainder(const Sched& s, int first_col, long long pos, long long end, Seg& g) {
    const long long chunk_units = (long long)s.Krem * s.PH;
    int j = (int)(pos / chunk_units);
    if (j > s.nh - 1) j = s.nh - 1;
    const int len = (j < s.nh - 1) ? s.PH : s.Hr - (s.nh - 1) * s.PH;
    const long long r2 = pos - (long long)j * chunk_units;
    const int col = (int)(r2 / len);
    const int p = (int)(r2 - (long long)col * len);
    long long take = len - p;
    if (take > end - pos) take = end - pos;
    decode_column(s, first_col + col, g);
    g.hb = s.h_begin + j * s.PH + p;
    g.he = g.hb + (int)take;
    return (int)take;
}

// Walks the input planes hb-1 .. he of every segment of CTA `cta` of `ncta`.
struct StepIter {
    long long pos, end;  // remainder-phase range still to decode
    int r, cta, ncta;    // next full round
    Seg g;
    int q;
    bool active;
    KDW_HD void next_segment(const Sched& s) {
        if (r < s.R) {
            decode_column(s, r * ncta + cta, g);
            g.hb = s.h_begin;
            g.he = s.h_begin + s.Hr;
            ++r;
            q = g.hb - 1;
            active = true;
        } else if (pos < end) {
            pos += decode_remainder(s, s.R * ncta, pos, end, g);
            q = g.hb - 1;
            active = true;
        } else {
            active = false;
        }
    }
    KDW_HD void init(const Sched& s, int cta_, int ncta_) {
        cta = cta_;
        ncta = ncta_;
        r = 0;
        pos = (long long)cta_ * s.rem_total / ncta_;
        end = (long long)(cta_ + 1) * s.rem_total / ncta_;
        next_segment(s);
    }
    KDW_HD void next(const Sched& s) {
        if (++q > g.he) next_segment(s);
    }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// See launch_overlapping_previous: blocks until the previous kernel of the stream has completed.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Barrier among `nthreads` threads of the CTA (a multiple of 32) that does not involve the other warps.
__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// The same barrier with an OR-reduction of a per-thread flag: every participant gets the OR over all of them, so
// a decision such as "stop" is taken by all or by none (a warp that left alone would leave the others waiting).
__device__ __forceinline__ bool named_barrier_or(int id, int nthreads, bool flag) {
    int r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.s32 q, %3, 0;\n\t"
        "bar.red.or.pred p, %1, %2, q;\n\t"
        "selp.s32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"(id), "r"(nthreads), "r"((int)flag)
        : "memory");
    return r != 0;
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking test of a barrier phase.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: gives up after limit_ns (2 s by default) of wall time and returns false (the caller then raises
// the status word and leaves the kernel instead of spinning for ever).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  unsigned long long limit_ns = 2000000000ull) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 63u && global_ns() - t0 > limit_ns) return false;
    }
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// A tiled TMA copy needs a 128-byte aligned shared address and an innermost coordinate that is a
// multiple of 16 bytes (8 halfs); a copy that breaks either rule raises an illegal-instruction fault.
__device__ __forceinline__ bool tma_args_ok(uint32_t smem_addr, int c0) { return (smem_addr & 127u) == 0 && (c0 & 7) == 0; }

// The copies below check those two rules first; an offending copy is skipped and reported in *status.
__device__ __forceinline__ void tma_load_5d(int* status, uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1,
                                            int c2, int c3, int c4) {
    if (!tma_args_ok(dst, c0)) {
        atomicExch(status, (int)KDW_STATUS_TMA_ARGS);
        return;
    }
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
        ::"r"(dst), "l"(tm), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_store_5d(int* status, const CUtensorMap* tm, uint32_t src, int c0, int c1, int c2,
                                             int c3, int c4) {
    if (!tma_args_ok(src, c0)) {
        atomicExch(status, (int)KDW_STATUS_TMA_ARGS);
        return;
    }
    asm volatile(
        "cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%1, %2, %3, %4, %5}], [%6];"
        ::"l"(tm), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(src)
        : "memory");
}
__device__ __forceinline__ void tma_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's committed bulk stores still read their shared-memory source.
template <int N>
__device__ __forceinline__ void tma_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* tm) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tm) : "memory");
}

// Raw view of CP packed half2 values (type punning through a union).
template <int CP>
union H2Pack {
    static_assert(CP == 1 || CP == 2 || CP == 4, "CP must be 1, 2 or 4");
    __half2 h[CP];
    uint32_t u1;
    uint2 u2;
    uint4 u4;
    KDW_HD H2Pack() {}
};
// Packed-half multiply / fused multiply-add.  The host branches exist so that the per-thread step
// functions can also be executed on the CPU by the test-suite's kernel emulation.
KDW_HD __half2 h2_mul(__half2 a, __half2 b) {
#ifdef __CUDA_ARCH__
    return __hmul2(a, b);
#else
    const float2 fa = __half22float2(a), fb = __half22float2(b);
    return __floats2half2_rn(fa.x * fb.x, fa.y * fb.y);  // an fp16 x fp16 product is exact in fp32
#endif
}
KDW_HD __half2 h2_add(__half2 a, __half2 b) {
#ifdef __CUDA_ARCH__
    return __hadd2(a, b);
#else
    const float2 fa = __half22float2(a), fb = __half22float2(b);
    return __floats2half2_rn(fa.x + fb.x, fa.y + fb.y);  // the fp32 sum of two fp16 values is exact
#endif
}
// max(a, 0) per lane; a NaN lane gives 0 (the maximum returns the operand that is a number).
KDW_HD __half2 h2_relu_nan0(__half2 a) {
#ifdef __CUDA_ARCH__
    return __hmax2(a, __float2half2_rn(0.f));
#else
    const float2 f = __half22float2(a);
    return __floats2half2_rn(f.x > 0.f ? f.x : 0.f, f.y > 0.f ? f.y : 0.f);  // NaN > 0 is false
#endif
}
KDW_HD __half2 h2_fma(__half2 a, __half2 b, __half2 c) {
#ifdef __CUDA_ARCH__
    return __hfma2(a, b, c);
#else
    const float2 fa = __half22float2(a), fb = __half22float2(b), fc = __half22float2(c);
    const double lo = (double)fa.x * (double)fb.x + (double)fc.x;
    const double hi = (double)fa.y * (double)fb.y + (double)fc.y;
    return __halves2half2(__double2half(lo), __double2half(hi));
#endif
}

// c + a * b per lane with fp16 a, b and fp32 c: the sm_100 mixed-precision FMA.  The fp16 x fp16 product is
// exact, the sum is rounded once to fp32 - fp32 accumulation without separate converts.
KDW_HD float2 fma_h2_f2(__half2 a, __half2 b, float2 c) {
#ifdef __CUDA_ARCH__
    H2Pack<1> ka, kb;
    ka.h[0] = a;
    kb.h[0] = b;
    asm("{\n\t.reg .b16 al, ah, bl, bh;\n\t"
        "mov.b32 {al, ah}, %2;\n\t"
        "mov.b32 {bl, bh}, %3;\n\t"
        "fma.rn.f32.f16 %0, al, bl, %0;\n\t"
        "fma.rn.f32.f16 %1, ah, bh, %1;\n\t}"
        : "+f"(c.x), "+f"(c.y)
        : "r"(ka.u1), "r"(kb.u1));
    return c;
#else
    const float2 fa = __half22float2(a), fb = __half22float2(b);
    return make_float2(fmaf(fa.x, fb.x, c.x), fmaf(fa.y, fb.y, c.y));
#endif
}

// c + float(h), element-wise; on the device one sm_100 mixed-precision add per lane (no separate convert).
KDW_HD float2 add_h2_f2(__half2 h, float2 c) {
#ifdef __CUDA_ARCH__
    float2 r;
    H2Pack<1> k;
    k.h[0] = h;
    const uint32_t hu = k.u1;
    asm("{\n\t.reg .b16 lo, hi;\n\t"
        "mov.b32 {lo, hi}, %2;\n\t"
        "add.rn.f32.f16 %0, lo, %3;\n\t"
        "add.rn.f32.f16 %1, hi, %4;\n\t}"
        : "=f"(r.x), "=f"(r.y)
        : "r"(hu), "f"(c.x), "f"(c.y));
    return r;
#else
    const float2 f = __half22float2(h);
    return make_float2(f.x + c.x, f.y + c.y);
#endif
}

// CP consecutive half2 (4*CP bytes) from / to shared memory in one access.
template <int CP>
KDW_HD void lds_h2(__half2 (&v)[CP], const __half* p) {
    H2Pack<CP> k;
    if constexpr (CP == 1)
        k.u1 = *reinterpret_cast<const uint32_t*>(p);
    else if constexpr (CP == 2)
        k.u2 = *reinterpret_cast<const uint2*>(p);
    else
        k.u4 = *reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < CP; ++i) v[i] = k.h[i];
}
template <int CP>
KDW_HD void sts_h2(__half* p, const __half2 (&v)[CP]) {
    H2Pack<CP> k;
#pragma unroll
    for (int i = 0; i < CP; ++i) k.h[i] = v[i];
    if constexpr (CP == 1)
        *reinterpret_cast<uint32_t*>(p) = k.u1;
    else if constexpr (CP == 2)
        *reinterpret_cast<uint2*>(p) = k.u2;
    else
        *reinterpret_cast<uint4*>(p) = k.u4;
}

#endif  // __CUDACC__

}  // namespace kdw
