/*
 * kdw.h - C ABI of the B200 (sm_100a) depthwise 3x3x3 channels-last fp16 convolution library.
 *
 * The library replaces the device side of two kerops operators:
 *   kerops.ops.conv.DWConv       (kerops/ops/conv/dwconv.py:25-63,  kernel kerops/kernels/dw_conv.py:5-142)
 *   kerops.ops.conv.DWConvWGRAD  (kerops/ops/conv/dwconv_wgrad.py:31-79, kernel kerops/kernels/dw_conv.py:147-287)
 *
 * Conventions
 *   - Activations are channels_last_3d fp16 volumes.  kerops names the axes (N, C, H, W, D); the element
 *     offset of (n, c, h, w, d) is n*strideN + h*strideH + w*strideW + d*C + c, i.e. the channel stride is 1
 *     and the stride of the innermost spatial axis D is C.  Strides are in ELEMENTS.
 *   - Weights / weight gradients are [3][3][3][C] contiguous (taps along h, w, d, then channel), the layout
 *     asserted at kerops/ops/conv/dwconv.py:32.
 *   - Cross-correlation, stride 1, zero padding 1, no bias:
 *       y[n,h,w,d,c]  = sum_{a,b,t} x[n,h+a-1,w+b-1,d+t-1,c] * weight[a,b,t,c]
 *       dw[a,b,t,c]   = sum_{n,h,w,d} grad[n,h,w,d,c] * x[n,h+a-1,w+b-1,d+t-1,c]
 *   - Every function only ENQUEUES work on `stream` (a cudaStream_t passed as void*); none synchronises,
 *     allocates or frees device memory, or keeps a pointer after it returns.  Outputs and workspaces are
 *     allocated by the caller (the Python layer uses torch's allocator, like the reference's
 *     torch.empty_like / torch.zeros at dwconv.py:40 and dwconv_wgrad.py:54).
 *   - Return value: 0 on success, negative for an argument error, positive = cudaError_t / CUresult of a
 *     failed runtime or driver call.  kdw_last_error() gives the message of the calling thread's last failure.
 */
#ifndef KDW_H_
#define KDW_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* accumulate types, mirror the ACCTYPE keyword of the reference ('float32' | 'float16', dwconv.py:35) */
#define KDW_ACC_F32 0
#define KDW_ACC_F16 1

/* argument errors */
#define KDW_ERR_ARG (-1)         /* null pointer, non-positive size, bad enum            */
#define KDW_ERR_ALIGN (-2)       /* pointer or stride not usable by the selected kernel  */
#define KDW_ERR_WORKSPACE (-3)   /* workspace smaller than kdw_wgrad_workspace_bytes()   */
#define KDW_ERR_TUNE (-4)        /* `tune` names no kernel variant valid for this C      */
#define KDW_ERR_RANGE (-5)       /* plane range outside the tensor                       */

/* Library version (major*10000 + minor*100 + patch). No reference counterpart. */
int kdw_version(void);

/* Message of the last failure on the calling thread ("" if none). No reference counterpart. */
const char* kdw_last_error(void);

/*
 * Reads and clears the device-side status word of the CURRENT device (synchronises the device):
 * 0 = ok, 1 = a bounded wait on a TMA barrier ran out inside a kernel (the kernel stopped early and its
 * output is invalid), 2 = a TMA copy with a misaligned shared address or channel coordinate was skipped,
 * 3 = kdw_allreduce_push_f32 gave up waiting for a peer's flag (its outputs were not written).  No reference
 * counterpart (the reference has no device-side waits).
 */
int kdw_device_status(int* status);

/*
 * Test hook for the kernels' bounded waits (no reference counterpart; process-wide, not thread-safe, meant for
 * test programs only).  limit_ns: time after which a wait on a TMA barrier inside a forward or weight-gradient
 * kernel gives up (default 2 s).  stop_after >= 0: the load warp of those kernels stops after that many plane loads, so the next wait of
 * the compute warps runs out, the kernel raises status 1 (kdw_device_status) and returns with its output
 * incomplete - nothing faults and the context stays usable.  stop_after < 0 (default) switches the hook off.
 */
int kdw_test_wait_limits(int64_t limit_ns, int stop_after);

/*
 * Forward pass.  Replaces the launch loop of kerops/ops/conv/dwconv.py:47-61 (one launch per sample of
 * _DWConv_cl3d_impl) by one launch over the whole batch.
 *   x, y      fp16 volumes (N, C, H, W, D), strides in elements; y may have different N/H/W strides
 *   weight    fp16 [3][3][3][C]
 *   acc_type  KDW_ACC_F32: exact fp16 x fp16 products accumulated in fp32 (tensor-core mma or mixed-precision FMA,
 *             depending on the variant), rounded once to fp16 - at least as accurate as the reference's 'float32' mode (fp16 products, fp16 sum of three,
 *             fp32 sum of nine; kerops/kernels/dw_conv.py:49-52);  KDW_ACC_F16: sums of no more than fp16 accuracy
 *             are asked for - the built-in choice and the tensor-core variants then still accumulate in fp32 (more
 *             accurate and faster), only the CUDA-core variants named by `tune` run packed-half FMA chains
 *   tune      0 = built-in choice for this C, W and D; >0 = explicit kernel variant (see kdw_fprop_variants());
 *             takes the place of the num_warps / D_block keywords (dwconv.py:10-17)
 * C must be a power of two.  C >= 8 uses the TMA kernel (x, y 16-byte aligned, strides multiples of 8);
 * smaller C uses a plain kernel.
 */
int kdw_fprop_f16(const void* x, const void* weight, void* y, int64_t N, int64_t C, int64_t H, int64_t W,
                  int64_t D, int64_t x_strideN, int64_t x_strideH, int64_t x_strideW, int64_t y_strideN,
                  int64_t y_strideH, int64_t y_strideW, int acc_type, int tune, void* stream);

/*
 * Forward pass over a range of h-planes, for volumes sharded along H with halo planes (no reference
 * counterpart: the reference is single-GPU).  Computes output planes h in [h_begin, h_end) in x's plane
 * numbering, reading x planes h_begin-1 .. h_end (planes outside [0, Hx) read as zero), and writes them to
 * y plane (h - y_h0); y has Hy planes and 0 <= h_begin - y_h0, h_end - y_h0 <= Hy.
 */
int kdw_fprop_f16_range(const void* x, const void* weight, void* y, int64_t N, int64_t C, int64_t Hx, int64_t W,
                        int64_t D, int64_t x_strideN, int64_t x_strideH, int64_t x_strideW, int64_t Hy,
                        int64_t y_strideN, int64_t y_strideH, int64_t y_strideW, int64_t h_begin, int64_t h_end,
                        int64_t y_h0, int acc_type, int tune, void* stream);

/* Number of fprop kernel variants; variant ids are 1..count.  kdw_fprop_variant_channels(id) gives the
 * channel-slice width of a variant (usable when C is a multiple of it).  No reference counterpart. */
int kdw_fprop_variants(void);
int kdw_fprop_variant_channels(int id);
/* The variant tune = 0 selects for a (C, W, D): the fastest measured tile for this C, corrected for the padding
 * its tile computes when it does not divide W or D.  0 if C is not a power of two >= 8 (plain kernel) or a size is
 * not positive.  Takes the place of the reference's per-C tables (dwconv.py:10-17).  */
int kdw_fprop_auto_variant(int64_t C, int64_t W, int64_t D);

/*
 * Bytes of device workspace kdw_wgrad_f16 needs on the current device (upper bound for any tune).  Takes
 * the place of the fp16 partial buffer [N, grid, 3,3,3,C] the reference allocates (dwconv_wgrad.py:54).
 * The workspace needs no initialisation.
 */
int64_t kdw_wgrad_workspace_bytes(int64_t N, int64_t C, int64_t H, int64_t W, int64_t D);

/*
 * Weight gradient.  Replaces dwconv_wgrad.py:54-77: the zero-filled partial buffer, the per-sample launches
 * of _DWConv_wgrad_cl3d_impl and the torch sum over partials.
 *   x, grad    fp16 volumes (N, C, H, W, D)
 *   workspace  >= kdw_wgrad_workspace_bytes() bytes, 16-byte aligned; holds one fp32 [27][C] row per CTA
 *   dw_f32     optional fp32 [3][3][3][C] result (NULL to skip) - the quantity to all-reduce across GPUs
 *   dw_f16     optional fp16 [3][3][3][C] result (NULL to skip) - what DWConvWGRAD returns (dwconv_wgrad.py:77)
 * Pass 1 accumulates fp32 rows per CTA (per warp group in the tensor-core kernels): every product is an exact
 * fp16 x fp16 product added to an fp32 sum; pass 2 adds the rows in a fixed order.  No atomics: the result is
 * bitwise reproducible for a given device and shape.
 */
int kdw_wgrad_f16(const void* x, const void* grad, void* workspace, int64_t workspace_bytes, float* dw_f32,
                  void* dw_f16, int64_t N, int64_t C, int64_t H, int64_t W, int64_t D, int64_t x_strideN,
                  int64_t x_strideH, int64_t x_strideW, int64_t g_strideN, int64_t g_strideH, int64_t g_strideW,
                  int tune, void* stream);

/*
 * Weight gradient over a range of h-planes (H-sharded volumes; no reference counterpart).  Sums over grad
 * planes h in [h_begin, h_end) in x's plane numbering; grad plane index is (h - g_h0), grad has Hg planes.
 * x planes h_begin-1 .. h_end are read (zero outside [0, Hx)).
 */
int kdw_wgrad_f16_range(const void* x, const void* grad, void* workspace, int64_t workspace_bytes, float* dw_f32,
                        void* dw_f16, int64_t N, int64_t C, int64_t Hx, int64_t W, int64_t D, int64_t x_strideN,
                        int64_t x_strideH, int64_t x_strideW, int64_t Hg, int64_t g_strideN, int64_t g_strideH,
                        int64_t g_strideW, int64_t h_begin, int64_t h_end, int64_t g_h0, int tune, void* stream);

/*
 * Weight gradient of a whole volume without a caller-provided workspace (no counterpart in the reference).
 * For callers that must not allocate device memory around the call: a latency-critical training or serving
 * loop where cudaMalloc (a call that synchronises the device) is off limits, a process running under a fixed
 * device-memory budget, and embedders without access to an allocator (a plain C host, a plugin that is handed
 * only input and output buffers).  The per-CTA fp32 rows that kdw_wgrad_f16 keeps in `workspace` live in an
 * array built into the library instead.
 *   - Limit: C <= 128 (KDW_ERR_WORKSPACE beyond); the array is 296 x 27 x 128 floats = 3.9 MiB and stays
 *     resident on every GPU that loads the library until the process exits.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress); make that
 *     first call before any stream capture.  No call allocates or frees device memory.
 *   - All calls on a device share the array: calls that may overlap on the GPU (different streams) race and
 *     must be serialised by the caller.  Rows are re-initialised by every launch, so no state carries over.
 * Arguments and results as kdw_wgrad_f16; same kernels, so the result matches it to fp32 rounding (bit for bit
 * when both use the same number of CTAs).
 */
int kdw_wgrad_f16_static(const void* x, const void* grad, float* dw_f32, void* dw_f16, int64_t N, int64_t C, int64_t H,
                         int64_t W, int64_t D, int64_t x_strideN, int64_t x_strideH, int64_t x_strideW,
                         int64_t g_strideN, int64_t g_strideH, int64_t g_strideW, void* stream);

int kdw_wgrad_variants(void);
int kdw_wgrad_variant_channels(int id);
/* Same as kdw_fprop_auto_variant, for the weight gradient (dwconv_wgrad.py:10-22). */
int kdw_wgrad_auto_variant(int64_t C, int64_t W, int64_t D);

/*
 * Multi-GPU sum of weight gradients by peer stores (no reference counterpart: the reference is single-GPU).
 *
 * Every rank owns one exchange buffer of kdw_allreduce_buffer_bytes(capacity, world) bytes, zero-filled once
 * before the first call, and can address the buffers of all ranks (`buffers[r]`, device pointers valid in the calling
 * process, mapped with access for the calling GPU, e.g. torch symmetric memory or cuMemMap +
 * cuMemSetAccess; buffers[rank] is the rank's own).  One kernel on each
 * rank writes `local` (n fp32 values, e.g. the [3][3][3][C] gradient from kdw_wgrad_f16) into its slot of
 * every buffer, raises a flag there, waits for the flags of all ranks in its own buffer and writes the sum,
 * added in rank order, to out_f32 and/or out_f16 - the same bits on every rank.
 *   n           values to sum in this call, 1 <= n <= capacity; calls on one set of buffers may use different n
 *               (the same n on every rank within a call)
 *   capacity    the value the buffers were sized with; it alone fixes where slots and flags lie in a buffer
 *   seq         call counter, the same on every rank: 1 for the first call on these buffers, then 2, 3, ...
 *   timeout_ns  limit of the wait for the peers' flags; when it runs out the kernel sets the device status
 *               word to 3 (kdw_device_status) and leaves the outputs unwritten
 * All calls that use one set of buffers must be enqueued on the same stream of their rank.  world <= 16.
 * The function itself only enqueues the kernel; it returns KDW_ERR_ARG / KDW_ERR_ALIGN for bad arguments
 * (buffers must be 128-byte aligned).
 */
int64_t kdw_allreduce_buffer_bytes(int64_t capacity, int world);
int kdw_allreduce_push_f32(const float* local, float* out_f32, void* out_f16, void* const* buffers, int64_t n,
                           int64_t capacity, int rank, int world, uint32_t seq, int64_t timeout_ns, void* stream);

/*
 * Forward pass with a fused residual add and per-channel statistics:
 *   out = fp16(DWConv(x, weight)) + residual   (the add in fp16, like an elementwise add of two fp16 tensors)
 *   mean[c] = sum(out[..., c]) / (N*H*W*D),  sqmean[c] = sum(out[..., c]^2) / (N*H*W*D)   (fp32 sums of the fp16 values)
 * i.e. what the reference computes with two operators, AddStats(DWConv(x, weight), residual)
 * (kerops/ops/addition.py:11-49 on top of kerops/ops/conv/dwconv.py:25-63), without writing and re-reading the
 * convolution's output.  KDW_ACC_F32 arithmetic.  C a power of two >= 8; x, residual, y are (N, C, H, W, D) fp16
 * volumes with the layout rules of kdw_fprop_f16; mean, sqmean fp32 [C]; workspace of
 * kdw_fprop_addstats_workspace_bytes() bytes (no initialisation needed).  The sums are reproducible (no atomics).
 *   tune  0 = built-in choice (the tensor-core forward kernel with the add and the sums in its epilogue, where one
 *         of its tiles takes the shape); 1..kdw_fprop_addstats_variants() = explicit CUDA-core tile
 */
int64_t kdw_fprop_addstats_workspace_bytes(int64_t N, int64_t C, int64_t H, int64_t W, int64_t D);
int kdw_fprop_addstats_variants(void);
int kdw_fprop_addstats_f16(const void* x, const void* weight, const void* residual, void* y, void* workspace,
                           int64_t workspace_bytes, float* mean, float* sqmean, int64_t N, int64_t C, int64_t H,
                           int64_t W, int64_t D, int64_t x_strideN, int64_t x_strideH, int64_t x_strideW,
                           int64_t r_strideN, int64_t r_strideH, int64_t r_strideW, int64_t y_strideN,
                           int64_t y_strideH, int64_t y_strideW, int tune, void* stream);

/*
 * Forward pass with a fused per-channel affine map and ReLU on the INPUT:
 *   y = DWConv(relu(x * scale[c] + shift[c]), weight)
 * i.e. the reference's ApplyBNReLU(x, scale, shift) (kerops/ops/bnrelu.py:11-43; fp32 x*w+b, max 0, stored as fp16)
 * followed by DWConv (kerops/ops/conv/dwconv.py:25-63), without writing and re-reading the activated tensor.  The
 * zero padding of the convolution applies to the activated tensor.  The convolution itself uses KDW_ACC_F32
 * arithmetic.  C a power of two >= 8; scale, shift fp32 [C]; x, y as for kdw_fprop_f16.
 *   prologue_type  KDW_ACC_F32: activation computed in fp32 from the fp32 scale / shift and rounded to fp16 - the
 *                  reference operator's arithmetic;  KDW_ACC_F16: scale and shift rounded to fp16, activation one
 *                  packed-half fused multiply-add with ReLU (single rounding) - faster, differs from the fp32 form
 *                  only through the rounding of scale and shift
 *                  With tune = 0 both run on the tensor-core forward kernel where one of its tiles takes the shape (the
 *                  activation is applied to the operand words on their way from shared memory).
 *   tune           0 = built-in choice, 1..kdw_fprop_bnrelu_variants() = explicit tile
 */
int kdw_fprop_bnrelu_variants(void);
int kdw_fprop_bnrelu_f16(const void* x, const float* scale, const float* shift, const void* weight, void* y, int64_t N,
                         int64_t C, int64_t H, int64_t W, int64_t D, int64_t x_strideN, int64_t x_strideH,
                         int64_t x_strideW, int64_t y_strideN, int64_t y_strideH, int64_t y_strideW,
                         int prologue_type, int tune, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KDW_H_ */
