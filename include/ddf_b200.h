/*
 * ddf_b200.h -- C ABI of libddf_b200.so: the Decoupled Dynamic Filter (DDF)
 * operator, forward and backward, 'mul' and 'add' combine modes, as hand-written
 * sm_100a CUDA kernels.
 *
 * The library replaces the native layer of the reference project
 * (theFoxofSky/ddfnet).  There the native entry points are four pybind11
 * modules taking at::Tensor; here they are plain C functions taking device
 * pointers and sizes, so any host (ctypes, cffi, a torch extension, C++) can
 * bind them.  Each declaration cites the reference interface it replaces.
 *
 * Semantics (contiguous NCHW, r = (k-1)/2, OH = H/s, OW = W/s, floor):
 *   w[b,c,t,y,x]  = cf[b,c,i,j] * sf[b,t,y,x]   (mul)   or   cf + sf   (add),  t = i*k + j
 *   out[b,c,y,x]  = sum_t x[b,c, y*s + (i-r)*d, x*s + (j-r)*d] * w[b,c,t,y,x]   (zero padding)
 * and the three gradients of that expression.
 *
 * Conventions shared by all calls
 *   - Every pointer is a DEVICE pointer on the current CUDA device; the caller
 *     owns all memory.  The library allocates nothing, never synchronises the
 *     host, never exits the process and never throws: it returns a status.
 *   - All tensors are contiguous, of the element type `dtype`, shapes as below.
 *   - Every element of every output is written; outputs need not be zeroed.
 *   - Work is enqueued on `stream` (a cudaStream_t passed as void*; NULL is the
 *     legacy default stream).  Calls are asynchronous and re-entrant.
 *   - Status: 0 = success; negative = the argument check that failed
 *     (DDF_B200_E_*); positive = a cudaError_t reported by the CUDA runtime.
 */
#ifndef DDF_B200_H_
#define DDF_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
#define DDF_B200_F32 0
#define DDF_B200_F16 1
#define DDF_B200_BF16 2
#define DDF_B200_F64 3

/* combine modes: ddf/ddf.py:64-65 ('mul' | 'add') */
#define DDF_B200_MUL 0
#define DDF_B200_ADD 1

/* Kernel choice.  The reference's `version` argument (ddf/ddf.py:77-84) picks
 * between its generic ('o') and tiled ('f') forward; the same letters map to
 * GENERIC and STREAM here, '' to AUTO. */
#define DDF_B200_VARIANT_AUTO 0    /* STREAM where the shape qualifies, else GENERIC */
#define DDF_B200_VARIANT_GENERIC 1 /* one thread per element; any k, d, s, any type   */
#define DDF_B200_VARIANT_STREAM 2  /* TMA-fed persistent plane-streaming kernels      */

/* argument-check failures */
#define DDF_B200_E_NULL (-1)        /* a required pointer is NULL                      */
#define DDF_B200_E_SHAPE (-2)       /* B, C, H, W < 1 or H/s, W/s < 1                  */
#define DDF_B200_E_KERNEL (-3)      /* k even or < 1, d < 1, or s < 1 (ddf/ddf.py:63)  */
#define DDF_B200_E_COMBINE (-4)     /* combine not MUL / ADD                           */
#define DDF_B200_E_DTYPE (-5)       /* unknown dtype                                   */
#define DDF_B200_E_VARIANT (-6)     /* unknown variant                                 */
#define DDF_B200_E_UNSUPPORTED (-7) /* VARIANT_STREAM forced on a shape it cannot do   */
#define DDF_B200_E_WORKSPACE (-8)   /* workspace NULL or smaller than required         */
#define DDF_B200_E_TOO_LARGE (-9)   /* an index would not fit the kernels' ranges      */
#define DDF_B200_E_DEVICE (-10)     /* no usable CUDA device / not an sm_100 device    */
#define DDF_B200_E_SCRATCH_LIMIT (-11) /* ddf_b200_backward_noalloc: problem needs more
                                          scratch than the built-in array holds          */

/* Library version: major*10000 + minor*100 + patch. */
int ddf_b200_version(void);

/* Human-readable text for a status returned by this library (static storage). */
const char* ddf_b200_strerror(int status);

/*
 * Forward.  Replaces ddf_mul_forward / ddf_add_forward
 * (ddf/src/ddf_mul_ext.cpp:21-34, ddf/src/ddf_add_ext.cpp:21-34) and the
 * forward of the "faster" modules (ddf/src/ddf_mul_faster_ext.cpp:13-26), i.e.
 * the launchers DDFMulForwardLauncher (ddf/src/cuda/ddf_mul_cuda_kernel.cu:167-196)
 * and DDFMulFasterForwardLauncher (ddf/src/cuda/ddf_mul_faster_cuda_kernel.cu:165-199).
 *
 *   x   (B,C,H,W)   cf (B,C,k,k)   sf (B,k*k,H/s,W/s)   ->   out (B,C,H/s,W/s)
 */
int ddf_b200_forward(const void* x, const void* cf, const void* sf, void* out,
                     int B, int C, int H, int W, int k, int d, int s,
                     int combine, int dtype, int variant, void* stream);

/*
 * Forward with the spatial FilterNorm fused in.  `sf_raw` is the raw output of
 * the spatial branch's 1x1 convolution, shape (B,k*k,H/s,W/s); the kernel
 * normalises each pixel's k*k values itself -- (v - mean) / (std + 1e-10) * sf_scale,
 * std unbiased (divisor k*k - 1), statistics in float -- and then proceeds as
 * ddf_b200_forward.  Replaces FilterNorm(filter_type='spatial').forward
 * (ddf/ddf.py:146-157, built by build_spatial_branch, ddf/ddf.py:176-180, which
 * uses neither a running std nor a running mean) followed by the forward above;
 * sf_scale is that module's `std` attribute, calculate_gain(nonlinearity) / k
 * (ddf/ddf.py:135).  With head > 1 the caller has already folded heads into B.
 * Requires k >= 3.  The backward takes the normalised filter: recompute it and
 * call ddf_b200_backward.
 */
int ddf_b200_forward_sfnorm(const void* x, const void* cf, const void* sf_raw, void* out,
                            int B, int C, int H, int W, int k, int d, int s,
                            int combine, int dtype, int variant, double sf_scale, void* stream);

/*
 * Self-test of the bounded waits.  Runs the plane-ring forward kernel (2-byte element
 * types at the row widths it is built for; DDF_B200_E_UNSUPPORTED otherwise) with every
 * mbarrier wait limited to `wait_cycles` SM clocks.  With `starve` != 0 each stage is
 * announced 16 bytes larger than what is copied, so its barrier never completes: the
 * compute warps' waits run out, the kernel records fault 1 (a compute warp gave up
 * waiting for a stage) and returns with `out` partly unwritten, and the device context
 * stays usable.  ddf_b200_take_fault() then returns 1.  With `starve` == 0 the call is an
 * ordinary forward with a custom limit.  Replaces the reference's error convention for
 * this path -- print and exit(-1) on a failed launch
 * (ddf/src/cuda/ddf_mul_cuda_kernel.cu:190-194) -- with a status the host can read.
 */
int ddf_b200_forward_waitlimit(const void* x, const void* cf, const void* sf, void* out,
                               int B, int C, int H, int W, int k, int d, int s,
                               int combine, int dtype, long long wait_cycles, int starve,
                               void* stream);

/*
 * The spatial FilterNorm on its own, for the backward of ddf_b200_forward_sfnorm.
 * ddf_b200_sfnorm writes the normalised filter (same shape and type as `raw`,
 * (B,k*k,H',W')) that ddf_b200_backward takes as `sf`; ddf_b200_sfnorm_backward turns the
 * gradient with respect to the normalised filter (ddf_b200_backward's gsf) into the
 * gradient with respect to the raw filter.  Replace FilterNorm(filter_type='spatial').forward
 * (ddf/ddf.py:146-157) and the autograd of those torch operations.  Statistics in float
 * (double for F64).  k in {3, 5, 7}.
 */
int ddf_b200_sfnorm(const void* raw, void* normed, int B, int k, int OH, int OW, int dtype,
                    double sf_scale, void* stream);
int ddf_b200_sfnorm_backward(const void* raw, const void* grad_normed, void* grad_raw,
                             int B, int k, int OH, int OW, int dtype, double sf_scale, void* stream);

/*
 * Channels-innermost (NHWC, torch channels_last) forward.  The reference's op accepts
 * contiguous NCHW only (CHECK_CONTIGUOUS, ddf/src/cuda/ddf_mul_cuda.cpp:28-32), so a
 * network run with its --channels-last flag (train.py:369-370, 631-632) cannot reach it
 * without layout copies; this entry point takes the tensors as such a network holds them.
 *
 *   x   (B,H,W,C)     cf (B,C,k,k)     out (B,H/s,W/s,C)
 *   sf  k*k values per output pixel; the value of tap t at pixel (b,y,x) is read at element
 *       b*sf_batch_stride + (y*(W/s) + x)*sf_pixel_stride + t*sf_tap_stride, which covers a
 *       channels_last (B,G,H/s,W/s) tensor with G >= k*k maps (strides G*H'*W', G, 1) as well
 *       as the reference's planar (B,k*k,H/s,W/s) layout (strides k*k*H'*W', 1, H'*W').
 *   sf_bias (k*k floats or NULL) is added to the values read; with norm != 0 the spatial
 *       FilterNorm of ddf_b200_forward_sfnorm is then applied in float (sf_scale as there).
 *   out_scale / out_shift (C floats each, or both NULL) and relu: out = [relu](acc*scale+shift),
 *       i.e. the eval-mode BatchNorm and activation that follow the DDFPack in the model.
 * Built for k = 3, d = 1, s in {1, 2}, F16 / BF16, C a multiple of 8 that divides 2048;
 * anything else returns DDF_B200_E_UNSUPPORTED and the caller converts to NCHW.  In add mode
 * with norm != 0 the normalised filter is rounded to the element type before use, as the
 * reference's module sequence does when it stores it.
 *
 * ddf_b200_pool_nhwc leaves the float partial sums of x over tiles of 196 pixels,
 * partials (B, ddf_b200_pool_nhwc_tiles(H,W), C): the global average pool at the head of the
 * channel branch (ddf/ddf.py:186), in the form ddf_b200_channel_filter takes.
 */
int ddf_b200_forward_nhwc(const void* x, const void* cf, const void* sf, const float* sf_bias,
                          void* out, const float* out_scale, const float* out_shift, int relu,
                          int B, int C, int H, int W, int k, int d, int s, int combine, int dtype,
                          long long sf_batch_stride, long long sf_pixel_stride,
                          long long sf_tap_stride, int norm, double sf_scale, void* stream);
int ddf_b200_pool_nhwc_tiles(int H, int W);
int ddf_b200_pool_nhwc(const void* x, float* partials, int B, int C, int H, int W, int dtype,
                       void* stream);

/*
 * Measurement aids (no counterpart in the reference, which measures with wall-clock loops,
 * test_time.py:11-51).  ddf_b200_noop enqueues an empty kernel: replayed from a CUDA graph
 * it gives the launch floor the small shapes are compared with.  ddf_b200_rate_probe
 * measures how many warp instructions of one kind an SM issues per nanosecond
 * (mode 0 float FMA with repeated multiplicands, 1 float FMA with three distinct register
 * operands, 2 / 3 the mixed-precision FMA with bf16 / f16 multiplicands, 4 packed
 * fma.f32x2, 5 lop3); it needs ddf_b200_rate_probe_bytes() of scratch and, unlike every
 * other call, waits for its own kernels before it returns.
 */
int ddf_b200_noop(void* stream);
size_t ddf_b200_rate_probe_bytes(void);
int ddf_b200_rate_probe(int mode, void* scratch, size_t scratch_bytes, int iters,
                        double* warp_instr_per_ns_per_sm, void* stream);

/* Which variant (GENERIC or STREAM) AUTO resolves to for this problem; pointers
 * are assumed 16-byte aligned.  `backward` = 0 for the forward, 1 for the backward.
 * Returns a DDF_B200_VARIANT_* value, or a negative status. */
int ddf_b200_plan(int B, int C, int H, int W, int k, int d, int s,
                  int combine, int dtype, int backward);

/*
 * Bytes of scratch the backward needs for this problem (0 is possible).
 * The reference makes its caller allocate three zero-filled scratch tensors
 * (ddf/ddf.py:106-108, resized in ddf/src/cuda/ddf_mul_cuda.cpp:85-87); here the
 * caller provides one untyped block, 256-byte aligned, which need not be zeroed.
 */
size_t ddf_b200_backward_workspace(int B, int C, int H, int W, int k, int d, int s,
                                   int combine, int dtype, int variant);

/*
 * Backward.  Replaces ddf_mul_backward / ddf_add_backward
 * (ddf/src/ddf_mul_ext.cpp:36-55, ddf/src/ddf_add_ext.cpp:36-55), i.e.
 * DDFMulBackwardLauncher (ddf/src/cuda/ddf_mul_cuda_kernel.cu:423-527) and its
 * six launches (three transposes + DDFBackward_Feature / _Spatial_Filter /
 * _Channel_Filter).
 *
 *   go (B,C,H/s,W/s) , x , cf , sf   ->   gx like x, gcf like cf, gsf like sf
 *
 * Any of gx / gcf / gsf may be NULL: that gradient is then not computed
 * (the reference always computes all three).
 */
int ddf_b200_backward(const void* go, const void* x, const void* cf, const void* sf,
                      void* gx, void* gcf, void* gsf,
                      void* workspace, size_t workspace_bytes,
                      int B, int C, int H, int W, int k, int d, int s,
                      int combine, int dtype, int variant, void* stream);

/*
 * Backward for callers that cannot allocate device memory: same inputs, outputs
 * and results as ddf_b200_backward, but no workspace argument.  It has no
 * counterpart in the reference (whose Python wrapper allocates six tensors per
 * call, ddf/ddf.py:106-111).
 *
 * Who needs it: hosts that must not call cudaMalloc on this path -- a serving
 * runtime whose device arena was sized at start-up, a plugin invoked where an
 * allocation would synchronise the device or disturb a packed memory pool, a
 * caller with no allocator at hand at all.  The scratch the filter-gradient
 * kernel needs is a fixed array inside the library image instead:
 * ddf_b200_backward_noalloc_limit() bytes (16 MiB), held by every GPU that
 * loads the library until the process exits.
 *
 *   - Problems whose scratch need (what ddf_b200_backward_workspace reports)
 *     exceeds that limit are refused with DDF_B200_E_SCRATCH_LIMIT before
 *     anything is launched.
 *   - The call itself performs no cudaMalloc / cudaFree and uses no allocating
 *     library routine.
 *   - The first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress, with that device current).  Make that first call
 *     before starting any stream capture on the device.
 *   - All calls on a device share the one array and it keeps whatever the last
 *     call left in it.  The kernels write every scratch slot they later read, so
 *     nothing needs clearing between calls; but two calls whose kernels overlap
 *     on the GPU (different streams, no dependency) race on it -- serialise them.
 */
int ddf_b200_backward_noalloc(const void* go, const void* x, const void* cf, const void* sf,
                              void* gx, void* gcf, void* gsf,
                              int B, int C, int H, int W, int k, int d, int s,
                              int combine, int dtype, void* stream);

/* Size in bytes of the built-in scratch array used by ddf_b200_backward_noalloc. */
size_t ddf_b200_backward_noalloc_limit(void);

/*
 * Layout adapters for a channels-last (NHWC) network around the NCHW op: tiled
 * transposes of (B,H,W,C) <-> (B,C,H,W).  The reference has no counterpart: its
 * op rejects non-contiguous input (ddf/src/cuda/ddf_mul_cuda.cpp:28-32), so a
 * channels_last model (train.py --channels-last) pays generic strided copies
 * around every DDF layer.
 *
 * ddf_b200_nchw_to_nhwc can apply, on the way, dst = src * ch_scale[c] + ch_shift[c]
 * (both float arrays of C values, both NULL for none) and then max(., 0) when
 * `relu` is non-zero -- an eval-mode BatchNorm and ReLU following the op.
 * dtype: F32, F16 or BF16.  src and dst must not overlap and must be 16-byte
 * aligned (DDF_B200_E_UNSUPPORTED otherwise).
 */
int ddf_b200_nhwc_to_nchw(const void* src, void* dst, int B, int C, int H, int W, int dtype,
                          void* stream);
int ddf_b200_nchw_to_nhwc(const void* src, void* dst, int B, int C, int H, int W, int dtype,
                          const float* ch_scale, const float* ch_shift, int relu, void* stream);
/* NHWC -> NCHW taking only the first C of src_channels >= C channels per pixel, with the same
 * optional affine map and ReLU.  For the spatial branch: the library's 1x1 convolution is
 * several times faster with its k*k = 9 output maps padded to 16, and its bias can ride here. */
int ddf_b200_nhwc_to_nchw_affine(const void* src, void* dst, int B, int C, int H, int W,
                                 int src_channels, int dtype, const float* ch_scale,
                                 const float* ch_shift, int relu, void* stream);

/*
 * Front end of a DDF layer in a channels-last network: ONE pass over x (B,H,W,C)
 * produces the op's NCHW input and the channel branch's pooled sums.
 *   x_nchw (B,C,H,W)        x transposed (as ddf_b200_nhwc_to_nchw)
 *   pooled (B,NT,C) float   per-channel sums of x over each of the
 *                           NT = ddf_b200_frontend_tiles(H,W) 64-pixel tiles -- the
 *                           AdaptiveAvgPool2d of build_channel_branch (ddf/ddf.py:187)
 *                           as partial sums; feed them to ddf_b200_channel_filter with
 *                           n_partials = NT, pool_scale = 1/(H*W)
 * The reference reads x once for each of these.  Inference path (no gradients);
 * dtype F32 / F16 / BF16; C <= 2048; x_nhwc and x_nchw 16-byte aligned
 * (DDF_B200_E_UNSUPPORTED otherwise).
 */
int ddf_b200_frontend_tiles(int H, int W);
int ddf_b200_pack_frontend(const void* x_nhwc, void* x_nchw, float* pooled, int B, int C, int H,
                           int W, int dtype, void* stream);

/*
 * The channel branch of a DDF layer after its global average pool, as one launch:
 * 1x1 convolution C -> mid (w1 (mid,C), b1), ReLU, 1x1 convolution mid -> C*k*k
 * (w2s, b2), then FilterNorm(filter_type='channel', running_std=True):
 * per sample and channel the k*k values are centred, divided by their unbiased
 * std + 1e-10 and multiplied by gain[c*k*k + t] (the module's learnable `std`).
 * Replaces build_channel_branch minus its AdaptiveAvgPool2d (ddf/ddf.py:183-192,
 * FilterNorm at ddf/ddf.py:158-170), which the reference runs as about ten small
 * launches.  Weights, biases, gain and the output cf (B,C,k,k) have element type
 * `dtype` (F32, F16, BF16); arithmetic is float.
 *
 * w2s is the second convolution's weight (C*k*k, mid) RE-LAID-OUT as
 * (C / CW, mid, k*k, CW) with CW = ddf_b200_channel_filter_slice(C) channels per
 * slice -- w2.reshape(C/CW, CW, k*k, mid).permute(0, 3, 2, 1) -- so that each CTA's
 * share is one contiguous run for the bulk copies that feed it; do it once and keep
 * it (inference weights do not change).  w1 and w2s must be 16-byte aligned.
 *
 * pooled: float sums of x over pixels, laid out (B, n_partials, C); the kernel
 * adds the n_partials rows in order and multiplies by pool_scale (pass the mean
 * itself with n_partials = 1, pool_scale = 1).  k = 3 or 5, C <= 2048 and a multiple
 * of 8 (of 256 above 256), mid <= 512 (DDF_B200_E_UNSUPPORTED otherwise).  Inference
 * path: no gradients.
 */
int ddf_b200_channel_filter_slice(int C);
int ddf_b200_channel_filter(const float* pooled, int n_partials, float pool_scale,
                            const void* w1, const void* b1, const void* w2s, const void* b2,
                            const void* gain, void* cf, int B, int C, int mid, int k,
                            int dtype, void* stream);

/*
 * Reads and clears the per-device fault word that the streaming kernels set
 * when one of their bounded waits runs out (they then stop instead of spinning).
 * Synchronises the device.  0 = no fault recorded; otherwise a positive code
 * naming the wait that gave up.  Returns a negative status on a CUDA error.
 * No counterpart in the reference (its kernels have no waits).
 */
int ddf_b200_take_fault(void);

/* Number of kernel launches this library has enqueued since it was loaded
 * (all devices, all threads).  Used by the benchmark to report its launch count. */
unsigned long long ddf_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* DDF_B200_H_ */
