/*
 * wtconv_b200 -- C ABI of the B200 (sm_100a) WTConv forward kernels.
 *
 * Plain C, no torch types: raw device pointers, sizes, element strides and a
 * CUDA stream handle passed as void*.  The library never allocates or frees
 * device memory in the entry points below, never synchronises the stream
 * (wtconv_device_status excepted: it exists to do so) and never throws: every
 * call returns a status (0 = ok, <0 = rejected argument or un-built variant,
 * >0 = a cudaError_t from the launch).  All kernels run on the CURRENT device
 * of the calling thread, on the given stream.  The only state the library
 * keeps between calls is host-side and guarded by a mutex or read and written
 * atomically (a cache of launch plans keyed by the problem description,
 * per-device "kernel attribute set" flags) plus, on each device, the scratch
 * array of wtconv2d_forward_noalloc and the status word of
 * wtconv_device_status; the entry points may therefore be called concurrently
 * from several host threads (the reference's validate.py:263 nn.DataParallel
 * path does that).
 *
 * What each entry point replaces in the reference project (paths inside the
 * reference repository) is given beside its declaration.
 */
#ifndef WTCONV_B200_H_
#define WTCONV_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* activation / parameter element types */
#define WTCONV_F32 0
#define WTCONV_BF16 1
#define WTCONV_F16 2

/* status codes (negative = argument errors, positive = cudaError_t) */
#define WTCONV_OK 0
#define WTCONV_ERR_BAD_ARG (-1)        /* null pointer, non-positive size, bad dtype code  */
#define WTCONV_ERR_BAD_KERNEL_SIZE (-2)/* K is even or larger than 29 (gradients: 1,3,5,7)    */
#define WTCONV_ERR_BAD_LEVELS (-3)     /* wt_levels < 0 or beyond WTCONV_QUERY_MAX_LEVELS   */
#define WTCONV_ERR_WORKSPACE (-4)      /* workspace missing or smaller than *_workspace_bytes */
#define WTCONV_ERR_MISALIGNED (-5)     /* a pointer is not aligned to its element type      */
#define WTCONV_ERR_TOO_LARGE (-6)      /* a dimension overflows the 32-bit index plan       */
#define WTCONV_ERR_NO_DEVICE (-7)      /* no usable CUDA device / not an sm_100 device      */
#define WTCONV_ERR_SCRATCH_LIMIT (-8)  /* problem needs more than WTCONV_STATIC_SCRATCH_BYTES */
#define WTCONV_ERR_DEVICE_WAIT (-9)    /* a kernel gave up a bounded wait (wtconv_device_status) */

/* size of the scratch array built into the library for wtconv2d_forward_noalloc */
#define WTCONV_STATIC_SCRATCH_BYTES (16u << 20)

/* wtconv_query() selectors */
#define WTCONV_QUERY_VERSION 0         /* ABI version, currently 1                          */
#define WTCONV_QUERY_MAX_KERNEL_SIZE 1 /* largest K accepted: every odd K <= this works (29)   */
#define WTCONV_QUERY_MAX_LEVELS 2      /* largest wt_levels accepted                        */
#define WTCONV_QUERY_SM_ARCH 3         /* 100: built for sm_100a only                       */

/* Build facts.  Mirrors the build-ceiling check of the reference's CUDA backend
 * (fast_wtconv/cuda_haar/haar_cuda.py:65-105: MAX_KERNEL_SIZE / check_kernel_size). */
int wtconv_query(int what);

/* Human-readable text for a status returned by any entry point (static string).
 * Counterpart of the TORCH_CHECK messages of fast_wtconv/cuda_haar/fused_haar_conv.cu:399-417. */
const char* wtconv_status_string(int status);

/* Health check of the kernels that are fed by asynchronous bulk copies (TMA).  They poll the
 * completion barrier of a copy a bounded number of times; should a copy never complete, the
 * kernel sets a status word on the device and runs to its end instead of spinning for ever.
 * This call waits for `stream` (cudaStreamSynchronize), reads the word of the current device
 * and clears it.  Returns WTCONV_OK, or WTCONV_ERR_DEVICE_WAIT when some launch since the last
 * check gave up a wait (its output is then invalid), or a cudaError_t.  No counterpart in the
 * reference, whose kernels use no asynchronous copies. */
int wtconv_device_status(void* stream);

/* Number of floats of the packed parameter block for one layer.
 * ndim is 2 (WTConv2d) or 1 (WTConv1d). */
size_t wtconv_packed_param_floats(int ndim, int C, int K, int L);

/*
 * Fold a layer's parameters into the fp32 block the forward kernels read.
 * Replaces, per call of the reference forward, the _ScaleModule multiplications
 * (wtconv/wtconv2d.py:58,81,89-97) and the filter-bank tensors built by
 * wtconv/util/wavelet.py:23-43: the block holds, per channel, the base taps and
 * bias pre-multiplied by base_scale, and per level the four (two in 1-D)
 * sub-band tap sets pre-multiplied by wavelet_scale and by the product of the
 * analysis and synthesis taps of that depth, so the kernels run un-normalised
 * Haar butterflies (adds only).
 *
 *   param_dtype      element type of every parameter pointer below
 *   ana_tap, syn_tap magnitude of one analysis / synthesis filter tap as the
 *                    reference module holds it (wt_filter / iwt_filter, kept in
 *                    the module dtype: fp32 2-D taps are 0.49999997, 1-D taps
 *                    0.70710677; a bf16 module holds 0.5 / 0.70703125)
 *   base_w           (C,1,K,K) or (C,1,K) contiguous           base_conv.weight
 *   base_b           (C) or NULL                               base_conv.bias
 *   base_scale       (C)                                       base_scale.weight
 *   wavelet_w[i]     (S*C,1,K[,K]) contiguous, S=4 (2-D) / 2   wavelet_convs[i].weight
 *   wavelet_scale[i] (S*C)                                     wavelet_scale[i].weight
 *   wavelet_w / wavelet_scale are HOST arrays of L device pointers.
 *   packed           device buffer of wtconv_packed_param_floats() floats
 * One small kernel launch on `stream`.
 */
int wtconv_pack_params(int ndim, int C, int K, int L, int param_dtype,
                       double ana_tap, double syn_tap,
                       const void* base_w, const void* base_b, const void* base_scale,
                       const void* const* wavelet_w, const void* const* wavelet_scale,
                       float* packed, void* stream);

/*
 * Same block as wtconv_pack_params, for the ADJOINT of the layer: every tap set
 * is reversed (the K x K kernels flipped in both directions) and the bias slot
 * is zero.  The Haar transform is orthogonal and the reference pads / crops odd
 * sizes symmetrically (wtconv/wtconv2d.py:49-51,76), so running
 * wtconv2d_forward / wtconv1d_forward (stride 1) with this block on the
 * gradient of the output gives the gradient of the input -- what autograd
 * computes for wtconv/wtconv2d.py:38-87 and what the reference CUDA backend
 * computes in fused_haar_conv_scale_bwd (fast_wtconv/cuda_haar/
 * fused_haar_conv.cu:148-234).  Parameter gradients: wtconv2d_weight_grad_stats and
 * wtconv_param_grads below.
 */
int wtconv_pack_params_adjoint(int ndim, int C, int K, int L, int param_dtype,
                       double ana_tap, double syn_tap,
                       const void* base_w, const void* base_b, const void* base_scale,
                       const void* const* wavelet_w, const void* const* wavelet_scale,
                       float* packed, void* stream);

/*
 * Parameter gradients of WTConv2d (the weight-gradient half of the backward
 * pass; the input gradient is wtconv2d_forward on wtconv_pack_params_adjoint's
 * block).  The reference gets them from autograd through
 * wtconv/wtconv2d.py:46-85; its CUDA backend from
 * fused_haar_grad_weight_kernel and depthwise_grad_weight_kernel
 * (fast_wtconv/cuda_haar/fused_haar_conv.cu:257-342, depthwise_grad.cu:32-101).
 *
 * wtconv2d_pyramid writes the un-normalised Haar sub-bands of every level of a
 * tensor (x, or the gradient of the output at full resolution): level l as
 * fp32 (B, H_l, W_l, 4, C), levels concatenated, wtconv2d_pyramid_floats()
 * floats in all.  wtconv2d_weight_grad_stats then fills
 * stats[(1+4L)][K*K+1][C] (wtconv2d_weight_grad_stat_floats() floats; zeroed by
 * the call): for set 0 (base) and sets 1+4l+s (level l, sub-band s) the K x K
 * correlation sums between the two pyramids and, in slot K*K, the plain sum of
 * the gradient plane.  Per channel,
 *   d base_conv.weight = base_scale * stats[0],  d base_conv.bias = base_scale * stats[0][K*K],
 *   d base_scale = <base_conv.weight, stats[0]> + bias * stats[0][K*K],
 *   d wavelet_convs[l].weight[4c+s] = wavelet_scale[l][4c+s] * g_l * stats[1+4l+s],
 *   d wavelet_scale[l][4c+s] = g_l * <wavelet_convs[l].weight[4c+s], stats[1+4l+s]>,
 * with g_l = (ana_tap * syn_tap)^(l+1).  Sums are accumulated with floating-point
 * atomics (order not fixed, like the reference's kernels).  A 1-D layer
 * (wtconv/wtconv1d.py:46-85) passes its signal as a one-row image (H = 1, row
 * stride 0): its low / high band are sub-bands 0 and 2, its K taps the middle row
 * of the K x K sums.
 */
size_t wtconv2d_pyramid_floats(int B, int C, int H, int W, int L);
/*
 * wtconv_param_grads applies those factors: one small launch writes the gradient
 * of every parameter (contiguous buffers of the parameter dtype and shape;
 * pointer arguments as for wtconv_pack_params, g_* the gradients) from `stats`.
 * ndim = 1 reads the one-row-image sums as described below.
 */
int wtconv_param_grads(int ndim, int C, int K, int L, int param_dtype, double ana_tap, double syn_tap,
                       const float* stats, const void* base_w, const void* base_b, const void* base_scale,
                       const void* const* wavelet_w, const void* const* wavelet_scale, void* g_base_w,
                       void* g_base_b, void* g_base_scale, void* const* g_wavelet_w, void* const* g_wavelet_scale,
                       void* stream);
int wtconv2d_pyramid(const void* t, float* pyramid, int B, int C, int H, int W, int L, int dtype,
                     const long long* strides, void* stream);
size_t wtconv2d_weight_grad_stat_floats(int C, int K, int L);
int wtconv2d_weight_grad_stats(const void* x, const void* gy, const float* x_pyramid, const float* g_pyramid,
                               float* stats, int B, int C, int H, int W, int K, int L, int dtype,
                               const long long* x_strides, const long long* g_strides, void* stream);

/*
 * Scratch bytes wtconv2d_forward needs for this problem and memory layout (0
 * when the whole cascade of a plane is fused on chip, which is the case for
 * small planes; larger planes hand the reconstruction of their deep levels --
 * a quarter-resolution fp32 plane set or smaller -- from one launch to the next
 * through scratch).  x_strides / y_strides as for wtconv2d_forward (NULL =
 * NCHW-contiguous).  The launch chain also depends on whether the tensors start
 * on 16-byte boundaries (the tensor maps of the TMA-fed kernels need that); the
 * size reported covers both cases, so it is enough for any pointers with these
 * strides.
 * The reference has no counterpart: its intermediates are torch allocations
 * inside wtconv/wtconv2d.py:46-78.
 */
int wtconv2d_workspace_bytes(int B, int C, int H, int W, int K, int L, int dtype,
                             const long long* x_strides, const long long* y_strides, size_t* bytes);

/*
 * Number of kernel launches wtconv2d_forward enqueues for this problem and
 * layout (the stages of the launch chain plus the low-pass reductions feeding
 * them).  For accounting by benchmarks and profilers; the reference has no
 * counterpart (its forward issues about 8*L+3 ATen kernels,
 * wtconv/wtconv2d.py:46-85).
 */
int wtconv2d_launch_count(int B, int C, int H, int W, int K, int L, int stride, int dtype,
                          const long long* x_strides, const long long* y_strides, int* launches);

/*
 * WTConv2d forward: y = base_scale*(base_conv(x)) + inverse-wavelet cascade of
 * the scaled per-level sub-band depthwise convolutions, optionally subsampled
 * by `stride`.  Replaces the whole body of WTConv2d.forward
 * (wtconv/wtconv2d.py:38-87) including wavelet_2d_transform /
 * inverse_2d_wavelet_transform (wtconv/util/wavelet.py:62-75); it is also the
 * counterpart of the reference CUDA backend's fused_haar_conv_forward +
 * ihaar_cascade + cuDNN base conv (fast_wtconv/cuda_haar/haar.cpp:5-19).
 *
 *   x, y        device pointers, element type `dtype`; any H,W >= 1 (odd sizes
 *               are zero-extended in-kernel exactly like wtconv2d.py:49-51)
 *   x_strides   4 element strides (n,c,h,w) of x; y_strides likewise for y.
 *               NCHW-contiguous and channels-last are both native.
 *   y shape     (B,C,ceil(H/stride),ceil(W/stride))  (wtconv2d.py:33-34,84-85)
 *   packed      block written by wtconv_pack_params
 *   workspace   wtconv2d_workspace_bytes() bytes of device scratch or NULL if 0
 */
int wtconv2d_forward(const void* x, void* y, const float* packed,
                     void* workspace, size_t workspace_bytes,
                     int B, int C, int H, int W, int K, int L, int stride, int dtype,
                     const long long* x_strides, const long long* y_strides, void* stream);

/*
 * WTConv2d forward for callers that must not allocate device memory.
 *
 * Same arguments and result as wtconv2d_forward, minus the workspace: the
 * scratch planes that large inputs need (see wtconv2d_workspace_bytes) live in
 * an array of WTCONV_STATIC_SCRATCH_BYTES that is part of the library image, so
 * neither this call nor its caller runs cudaMalloc / cudaFree or any allocating
 * library routine.  It is meant for hosts that cannot allocate at call time:
 * code running inside a CUDA-graph capture or a real-time serving loop where an
 * allocation would synchronise the device, plug-ins that are handed fixed
 * buffers by an inference runtime and own no allocator, and embedders whose
 * memory budget is frozen after start-up.
 *
 *   - Problems whose scratch need exceeds WTCONV_STATIC_SCRATCH_BYTES are
 *     rejected with WTCONV_ERR_SCRATCH_LIMIT before anything is launched; the
 *     check plans with the pointers and strides of this very call (for example
 *     bf16 channels-last 56x56 planes with 5 levels need B*C*4704 bytes: up to
 *     B*C = 3566 planes fit).  Problems that need no scratch always pass.
 *   - Every GPU whose context loads the library holds the array until the
 *     process exits.
 *   - Every call looks up the array's address on the current device (one
 *     cudaGetSymbolAddress, a host-side table lookup once the kernels are
 *     loaded).  Make one call per device before starting any stream capture,
 *     so that loading the kernels does not fall into the capture.
 *   - All calls on a device share the one array, which keeps whatever the last
 *     call left in it.  The kernels overwrite every scratch plane they later
 *     read, so nothing has to be cleared between calls; but two calls that can
 *     overlap on the GPU (different streams, no ordering) race on it -- order
 *     them on one stream or with events.
 * This entry point has no counterpart in the reference, whose intermediates are
 * ordinary torch allocations.
 */
int wtconv2d_forward_noalloc(const void* x, void* y, const float* packed,
                             int B, int C, int H, int W, int K, int L, int stride, int dtype,
                             const long long* x_strides, const long long* y_strides, void* stream);

/*
 * WTConv1d forward, replaces WTConv1d.forward (wtconv/wtconv1d.py:38-87) and
 * wavelet_1d_transform / inverse_1d_wavelet_transform (wtconv/util/wavelet.py:46-59).
 *   x (B,C,N) with 3 element strides (n,c,t); y (B,C,floor(N/stride)) --
 *   stride>1 is a true average pool of `stride` samples (wtconv1d.py:34).
 * The 1-D cascade is always fused on chip; no scratch memory is used.
 * Limits of this build, narrower than the 2-D ones: wt_levels <= 8
 * (WTCONV_ERR_BAD_LEVELS beyond); B <= 65535, C*N < 2^31 and at most 65535
 * channel groups (WTCONV_ERR_TOO_LARGE); a signal tile must hold a multiple of
 * 2^wt_levels * 8 * stride samples, so deep cascades combined with a large
 * pooling stride on long signals (for example wt_levels 8, stride >= 6,
 * N > 12000) exceed the shared memory of an SM and are rejected with
 * WTCONV_ERR_TOO_LARGE as well.
 */
int wtconv1d_forward(const void* x, void* y, const float* packed,
                     int B, int C, int N, int K, int L, int stride, int dtype,
                     const long long* x_strides, const long long* y_strides, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* WTCONV_B200_H_ */
