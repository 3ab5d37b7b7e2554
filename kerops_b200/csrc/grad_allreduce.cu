// Sum of the fp32 [27][C] weight gradients of several GPUs without a library collective: every rank PUSHES
// its gradient into a slot of every peer's exchange buffer (plain peer stores over NVLink), raises a flag
// there, waits - with a time limit - for the flags of all peers in its own buffer, and adds the slots in rank
// order.  One kernel per rank does all four steps; the result is bitwise identical on every rank.
//
// Exchange buffer of one rank (kdw_allreduce_buffer_bytes(capacity, world)):
//   [parity 0 | parity 1] x [source rank 0 .. world-1] x { payload: round_up(capacity,32) floats, flag line: 32 words }
// The layout depends on the CAPACITY the buffers were made for, never on the n of a call, so calls with different
// n on one set of buffers use the same slots and flags (a layout derived from n would let a small call's region
// overlap the region a slower peer is still summing for the previous, larger call).
// A call with sequence number s uses parity s & 1 and writes s into the flag word.  Two parities are enough:
// a rank can only start call s+2 after every peer has raised flag s+1, and a peer raises s+1 only after its
// own call s (the reader of the parity about to be overwritten) has finished, because calls on one rank are
// ordered by the stream they are enqueued on.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/kdw.h"
#include "kdw_common.cuh"

namespace kdw {

static constexpr int kMaxPushRanks = 16;
static constexpr int kPushThreads = 512;

struct PushPeers {
    float* buf[kMaxPushRanks];
};

__host__ __device__ inline long long push_payload_floats(long long n) { return (n + 31) / 32 * 32; }
__host__ __device__ inline long long push_slot_floats(long long n) { return push_payload_floats(n) + 32; }

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(kPushThreads) grad_push_sum_kernel(const float* __restrict__ local,
                                                                     float* __restrict__ out32,
                                                                     __half* __restrict__ out16, PushPeers peers, int n,
                                                                     long long capacity, int rank, int world, unsigned seq,
                                                                     unsigned long long timeout_ns, int* status) {
    __shared__ int s_failed;
    const int tid = threadIdx.x;
    const long long slot = push_slot_floats(capacity);
    const long long flag_off = push_payload_floats(capacity);
    const long long mine = ((long long)(seq & 1u) * world + rank) * slot;  // where this rank's data goes, in every buffer
    if (tid == 0) s_failed = 0;
    grid_dependency_wait();  // launched with launch_overlapping_previous: `local` is complete after this
    // 1. push the payload to every rank (own buffer included)
    for (int p = 0; p < world; ++p) {
        float* dst = peers.buf[p] + mine;
        for (int i = tid; i < n; i += kPushThreads) dst[i] = local[i];
    }
    __threadfence_system();
    __syncthreads();
    // 2. raise the flags, 3. wait for everybody's flag in the own buffer
    if (tid < world) {
        st_release_sys(reinterpret_cast<unsigned*>(peers.buf[tid] + mine + flag_off), seq);
        const unsigned* flag = reinterpret_cast<const unsigned*>(
            peers.buf[rank] + ((long long)(seq & 1u) * world + tid) * slot + flag_off);
        const unsigned long long t0 = global_timer_ns();
        while (ld_acquire_sys(flag) != seq) {
            if (global_timer_ns() - t0 > timeout_ns) {
                atomicExch(status, 3);
                s_failed = 1;
                break;
            }
            __nanosleep(200);
        }
    }
    __syncthreads();
    if (s_failed) return;  // outputs are left untouched
    // 4. add the slots in rank order (L2 loads: the slots were written by other GPUs)
    const float* base = peers.buf[rank] + (long long)(seq & 1u) * world * slot;
    for (int i = tid; i < n; i += kPushThreads) {
        float acc = 0.f;
        for (int s = 0; s < world; ++s) acc += __ldcg(base + s * slot + i);
        if (out32) out32[i] = acc;
        if (out16) out16[i] = __float2half_rn(acc);
    }
}

}  // namespace kdw

extern "C" {

int64_t kdw_allreduce_buffer_bytes(int64_t n, int world) {
    if (n <= 0 || world <= 0 || world > kdw::kMaxPushRanks) return 0;
    return 2 * (int64_t)world * kdw::push_slot_floats(n) * 4;
}

int kdw_allreduce_push_f32(const float* local, float* out_f32, void* out_f16, void* const* buffers, int64_t n,
                           int64_t capacity, int rank, int world, uint32_t seq, int64_t timeout_ns, void* stream) {
    using namespace kdw;
    if (!local || !buffers || (!out_f32 && !out_f16)) {
        set_error("allreduce_push: null pointer (local, buffers and at least one output are required)");
        return KDW_ERR_ARG;
    }
    if (n <= 0 || capacity > (1 << 24) || n > capacity || world <= 0 || world > kMaxPushRanks || rank < 0 ||
        rank >= world || timeout_ns <= 0) {
        set_error("allreduce_push: n=%lld capacity=%lld rank=%d world=%d timeout_ns=%lld out of range "
                  "(1 <= n <= capacity, 1 <= world <= %d)",
                  (long long)n, (long long)capacity, rank, world, (long long)timeout_ns, kMaxPushRanks);
        return KDW_ERR_ARG;
    }
    if (seq == 0) {
        set_error("allreduce_push: sequence numbers start at 1 (0 is the cleared state of the flags)");
        return KDW_ERR_ARG;
    }
    PushPeers peers;
    for (int p = 0; p < kMaxPushRanks; ++p) peers.buf[p] = nullptr;
    for (int p = 0; p < world; ++p) {
        if (!buffers[p] || ((uintptr_t)buffers[p] & 127) != 0) {
            set_error("allreduce_push: buffer of rank %d is null or not 128-byte aligned", p);
            return KDW_ERR_ALIGN;
        }
        peers.buf[p] = (float*)buffers[p];
    }
    int* status = nullptr;
    int rc = status_ptr(&status);
    if (rc) return rc;
    KDW_CUDA(launch_overlapping_previous(grad_push_sum_kernel, 1u, (unsigned)kPushThreads, (cudaStream_t)stream, local,
                                         out_f32, (__half*)out_f16, peers, (int)n, (long long)capacity, rank, world,
                                         (unsigned)seq, (unsigned long long)timeout_ns, status));
    return 0;
}

}  // extern "C"
