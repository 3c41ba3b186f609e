/*
 * converse_b200 -- C ABI of the B200 (sm_100a) Converse2D library.
 *
 * Every entry point takes plain pointers and sizes, returns an int status
 * (0 = success, negative = error, see cvb_strerror), never throws, never exits
 * and never traps the device.  Device pointers are owned by the caller; work is
 * enqueued on the stream passed in (a cudaStream_t passed as void*).
 *
 * The functions replace, for the Converse2D forward path, what the reference
 * binds through its extension:
 *   - torch.ops.converse2d.forward   (Converse2D/torch_converse2d/converse2d.cpp:165-209,218-227)
 *   - torch.ops.converse2d.clear_cache (converse2d.cpp:211-216): the kernel-spectrum
 *     cache becomes an explicit, caller-owned "transfer table" (cvb_build_transfer).
 *   - the module-side pad / nearest-upsample / crop around the op
 *     (models/util_converse.py:144-145,166,189-190), which are fused into the kernel.
 */
#ifndef CONVERSE_B200_H_
#define CONVERSE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
enum {
  CVB_OK = 0,
  CVB_ERR_BAD_ARGUMENT = -1,     /* null pointer, non-positive size, bad enum */
  CVB_ERR_BAD_PADDING = -2,      /* circular needs p <= H,W; reflect needs p < H,W */
  CVB_ERR_UNSUPPORTED_SIZE = -3, /* padded length has a prime factor the FFT engine lacks */
  CVB_ERR_WORKSPACE = -4,        /* workspace missing or too small */
  CVB_ERR_CUDA = -5,             /* a CUDA runtime call failed; see cvb_last_cuda_error */
  CVB_ERR_KERNEL_TOO_LARGE = -6, /* k larger than the padded, upsampled plane */
  CVB_ERR_TOO_LARGE = -7         /* size beyond a stated fixed maximum */
};

/* boundary modes of F.pad (models/util_converse.py:144-145) */
enum { CVB_PAD_CIRCULAR = 0, CVB_PAD_REPLICATE = 1, CVB_PAD_REFLECT = 2, CVB_PAD_CONSTANT = 3 };

/* element type of x and out; spectra and arithmetic are always fp32 */
enum { CVB_F32 = 0, CVB_BF16 = 1 };

/* Library / ABI version (major*100 + minor). */
int cvb_version(void);

/* Human-readable text for a status code. */
const char* cvb_strerror(int status);

/* The cudaError_t (as int) of the last failing runtime call on this thread, 0 if none. */
int cvb_last_cuda_error(void);

/*
 * Process-wide routing options.  The defaults are what a caller wants; the options exist so that
 * every kernel family can be reached on any size (the tests compare the routes with one another).
 * They take the place of the reference's CONVERSE2D_BACKEND switch (models/util_converse.py:150),
 * which chooses between its two implementations per call.  Not thread-safe against calls in flight.
 */
enum {
  CVB_OPT_RUNTIME_PLAN = 0,   /* 1: planes that fit shared memory take the run-time-plan kernel     */
  CVB_OPT_MULTIPASS = 1,      /* 1: every plane takes the multi-pass path through the workspace     */
  CVB_OPT_PERSISTENT = 2,     /* 1: compile-time-plan kernels run as persistent blocks with prefetch */
  CVB_OPT_BLOCK_KERNELS = 3,  /* ConverseBlock 1x1 kernels: 0 CUDA cores, 1 tcgen05 single-buffered,
                                 2 tcgen05 warp-specialised, operand tiles in shared memory,
                                 3 tcgen05 warp-specialised, cp.async ring + operand in TMEM (default) */
  CVB_OPT_COUNT_ = 4
};
int cvb_set_option(int which, int value);   /* CVB_OK or CVB_ERR_BAD_ARGUMENT */
int cvb_get_option(int which);              /* the value, or CVB_ERR_BAD_ARGUMENT */

/*
 * Device-side status of the current device: 0, or non-zero after a kernel gave up a
 * bounded wait (its output is then incomplete).  Synchronises the device; clears the
 * word when `clear` is non-zero.  Negative on a runtime error.  (The reference has no
 * counterpart: its op only raises host-side c10::Error, converse2d.cpp:167-172.)
 */
int cvb_last_device_status(int clear);

/*
 * Size in bytes of the transfer table for C channels (or B*C planes when the
 * kernels differ per sample) at padded size h x w = (H+2p) x (W+2p).
 * Replaces the FB/FBC/F2B triple the reference caches per weight tensor
 * (converse2d.cpp:22-102).  Returns 0 on bad arguments or an unsupported size.
 */
size_t cvb_transfer_bytes(int C, int h, int w);

/*
 * Build the transfer table: psf2otf of the k x k taps (models/util_converse.py:218-235),
 * lambda = sigmoid(bias-9)+eps (:147), and the whole spectral algebra of :176-186
 * collapsed to one weights-only multiplier per frequency, evaluated in fp64 and
 * stored as fp32 in the layout the forward kernel reads.
 *   weight : device, (C, k, k) fp32      bias : device, (C) fp32
 *   h, w   : padded plane size           s    : scale
 *   table  : device, cvb_transfer_bytes(C, h, w) bytes, 16-byte aligned
 */
int cvb_build_transfer(const float* weight, const float* bias, int C, int k, int s, int h, int w,
                       float eps, void* table, void* stream);

/*
 * Table of the x0 term, same arguments and layout: the real multiplier
 * 1 / (mean over the s x s aliases of |FK|^2 + lambda), i.e. 1 / (invW + lambda) of
 * models/util_converse.py:183-184 (converse2d.cpp:199-201).  The raw operator
 * (converse2d.cpp:165,193) accepts an x0 that is not the nearest-upsampled input; its
 * extra term  d - corr(K, zero_insert(IFFT2(table . FFT2(decimate(K * d))))),
 * d = x0 - nearest(x), runs through cvb_converse2d_fwd at scale 1 with this table
 * (conversenet_b200/torch_converse2d.py).
 */
int cvb_build_x0_table(const float* weight, const float* bias, int C, int k, int s, int h, int w,
                       float eps, void* table, void* stream);

/*
 * Bytes of scratch the forward needs for this shape (0 when the plane fits in
 * shared memory and everything stays on chip).
 */
size_t cvb_converse2d_workspace_bytes(int B, int C, int H, int W, int s, int p, int io_dtype);

/*
 * Converse2D forward: out = crop(solve(pad(x))), the full body of
 * Converse2D.forward (models/util_converse.py:142-192) for x0 = nearest-upsample
 * of the padded input, which is what the module always passes (:166,172-173).
 *   x      : device, (B, C, H, W) contiguous, io_dtype
 *   out    : device, (B, C, s*H, s*W) contiguous, io_dtype
 *   table  : from cvb_build_transfer for (C, k, s, H+2p, W+2p)
 *   weight : device, (C, k, k) fp32 (read only when s > 1)
 *   fuse_gelu : 1 applies the exact (erf) GELU to the result before the store
 *               (the activation that follows the operator in ConverseBlock,
 *               models/util_converse.py:282)
 *   workspace / workspace_bytes : >= cvb_converse2d_workspace_bytes(...), may be
 *               NULL / 0 when that is 0
 */
int cvb_converse2d_fwd(const void* x, void* out, const void* table, const float* weight, int B,
                       int C, int H, int W, int k, int s, int p, int pad_mode, int io_dtype,
                       int fuse_gelu, void* workspace, size_t workspace_bytes, void* stream);

/*
 * ConverseBlock, first fused kernel: out = GELU( W . LayerNorm(x) + b ), C -> 2C channels,
 * i.e. conv1[0..2] of the block: channels_first LayerNorm (models/util_converse.py:60-68),
 * 1x1 Conv2d (:279), GELU (:280).  x (B,C,HW), out (B,2C,HW) contiguous, io_dtype;
 * ln_w, ln_b (C); w (2C,C); b (2C), all fp32 device pointers.  C must be 64
 * (CVB_ERR_UNSUPPORTED_SIZE otherwise).
 */
int cvb_ln_pw_gelu_fwd(const void* x, void* out, const float* ln_w, const float* ln_b, float ln_eps,
                       const float* w, const float* b, int B, int C, int HW, int io_dtype, void* stream);

/*
 * ConverseBlock, second fused kernel (models/util_converse.py:283, 285-288, 291-292; alphas :321-322):
 *   x1  = x + alpha1 * (W2 . t + b2)                              t (B,2C,HW): Converse2D output after GELU
 *   out = x1 + alpha2 * (W4 . GELU(W3 . LayerNorm(x1) + b3) + b4)
 * w2, w4 (C,2C); w3 (2C,C); b2, b4 (C); b3 (2C); alpha1, alpha2 (C) or NULL for 1.  C must be 64.
 */
int cvb_pw_res_mlp_fwd(const void* t, const void* x, void* out, const float* w2, const float* b2,
                       const float* alpha1, const float* ln_w, const float* ln_b, float ln_eps,
                       const float* w3, const float* b3, const float* w4, const float* b4,
                       const float* alpha2, int B, int C, int HW, int io_dtype, void* stream);

/*
 * One 1x1 convolution of ConverseBlock with its residual on the tensor cores (tcgen05):
 *   out = res + alpha * (W . t + b),  t (B,2C,HW) -> out (B,C,HW); w (C,2C), b (C), alpha (C) or NULL.
 * conv1[5] + first residual (models/util_converse.py:283,291) and conv2[3] + second residual
 * (:288,292).  fp32 or bf16 tensors, C = 64, HW a multiple of 128, t 16-byte aligned; otherwise
 * CVB_ERR_UNSUPPORTED_SIZE and the caller uses cvb_pw_res_mlp_fwd.
 */
int cvb_pw_res_fwd(const void* t, const void* res, void* out, const float* w, const float* b,
                   const float* alpha, int B, int C, int HW, int io_dtype, void* stream);

/*
 * Converse2D forward for callers that cannot allocate device memory.
 *
 * Same arguments, result and error codes as cvb_converse2d_fwd, minus the workspace:
 * the multi-pass kernels run with their scratch in a fixed array inside the library
 * (CVB_STATIC_SCRATCH_BYTES, held by every GPU that loads the library until the process
 * ends).  Meant for code that runs where an allocator call is impossible or unwelcome:
 * a plug-in that owns nothing but its input and output buffers, a region whose memory
 * pool must not change, a real-time loop that may not take the allocator lock.  The
 * function calls no cudaMalloc / cudaFree and no allocating library routine, and its
 * host side works in fixed-size stack storage (no heap allocation either).
 *   - Limit: one padded plane pair, 8*(H+2p)*(W+2p) bytes, must fit the array
 *     (about 1440 x 1440); larger planes return CVB_ERR_TOO_LARGE.
 *   - Set-up on first use: the first call on each device looks up the device addresses
 *     of the array and of the status word (runtime queries, no allocation), and the
 *     first call per device that meets a padded length with a large prime factor (268,
 *     for instance) also runs one small kernel that fills a constant table inside the
 *     library and waits for it on `stream` (cudaStreamSynchronize).  Make those first
 *     calls outside any stream capture.
 *   - A bounded wait that gives up inside a kernel is reported through
 *     cvb_last_device_status, as for cvb_converse2d_fwd.
 *   - All calls share the one array and it keeps the previous call's contents.  Nothing
 *     in it has to start at zero (every element is written before it is read), but two
 *     calls that overlap on the GPU -- different streams, or different host threads --
 *     race on it: serialise them.
 * No counterpart in the reference (its op lets ATen allocate every temporary).
 */
#define CVB_STATIC_SCRATCH_BYTES (16u << 20)
int cvb_converse2d_fwd_static_scratch(const void* x, void* out, const void* table, const float* weight,
                                      int B, int C, int H, int W, int k, int s, int p, int pad_mode,
                                      int io_dtype, int fuse_gelu, void* stream);

/*
 * Batch-summed cross spectrum for the parameter gradients.  The reference obtains dL/dweight and
 * dL/dbias from autograd through torch.fft (CompositeImplicitAutograd registration,
 * Converse2D/torch_converse2d/csrc/converse2d.cpp:223); here the batch reduction they need runs in
 * one kernel:
 *     out[seg][c][ky][kx] = sum over b = seg, seg + nseg, ... < B of
 *                           FFT2(pad(x[b,c]))[ky][kx] * conj(FFT2(q[b,c])[ky][kx])
 * x (B,C,H,W) and q (B,C,h,w) fp32, h = H + 2p, w = W + 2p, unnormalised forward transforms,
 * frequencies in natural order; out = nseg * C * h * w complex (float2) values, summed over seg
 * by the caller.  With q = dL/dout zero-extended to the padded plane (scale 1), or the adjoint of
 * the upsampling epilogue applied to it (scale >= 2), the loss depends on the operator's
 * multiplier M only through (1 / (h w)) Re sum M * out.  `table`: a transfer table built for
 * (C, h, w) (its twiddle tables are read).  1 <= nseg <= B.  cvb_cross_spectrum_supported: 1 when
 * two padded planes fit shared memory (radices with a butterfly); 2 when only one does: the nseg
 * blocks of a channel then add into ONE slab with atomics, out = C * h * w values, zero-filled by
 * this call (summation order, hence the last bits, vary from run to run); else 0.
 */
int cvb_cross_spectrum(const float* x, const float* q, const void* table, void* out, int nseg, int B, int C,
                       int H, int W, int p, int pad_mode, void* stream);
int cvb_cross_spectrum_supported(int h, int w);

/*
 * Direct tap term of dL/dweight at scale >= 2 (the reference: autograd through the correlation of
 * models/util_converse.py:171-173):
 *     out[seg][c][a][b] = sum over n = seg, seg + nseg, ... < B and cells (my, mx) of
 *         g_full[n,c,(s my - a + k/2) mod s h, (s mx - b + k/2) mod s w] * r[n,c,my,mx]
 * g_full (B,C,s h,s w) = dL/dout zero-extended to the padded grid, r (B,C,h,w) = IFFT2(P . FFT2(pad(x)))
 * (the forward at scale 1 on the padded planes), all fp32; out = nseg * C * k * k floats, summed over
 * seg by the caller.
 */
int cvb_tap_gradient(const float* g_full, const float* r, float* out, int nseg, int B, int C, int h, int w, int k,
                     int s, void* stream);

/*
 * Describe the FFT plan chosen for a padded length n: writes up to max_stages
 * radices, returns the stage count, 0 if n is unsupported.  Host-only, no GPU.
 */
int cvb_plan_radices(int n, int* radices, int max_stages);

/* 1 if the forward for this padded size runs in the single-kernel shared-memory
 * path, 0 if it takes the multi-pass path through the workspace, negative on error. */
int cvb_fits_shared(int h, int w);

#ifdef __cplusplus
}
#endif
#endif /* CONVERSE_B200_H_ */
