// Internal glue between the translation units of libconverse_b200.so.
#pragma once
#include "cvb_kernels.cuh"

namespace cvb {

// Records a failing CUDA runtime call for cvb_last_cuda_error and returns CVB_ERR_CUDA.
int cuda_fail(cudaError_t e);

#define CVB_CUDA(call)                                   \
  do {                                                   \
    cudaError_t e__ = (call);                            \
    if (e__ != cudaSuccess) return ::cvb::cuda_fail(e__); \
  } while (0)

// Tuning aids read the environment only in tuning builds (-DCVB_TUNING); a shipped library ignores them.
#ifdef CVB_TUNING
int env_int(const char* name, int dflt);
#define CVB_TUNE(name, dflt) ::cvb::env_int(name, dflt)
#else
#define CVB_TUNE(name, dflt) (dflt)
#endif

// Process-wide routing options (cvb_set_option / cvb_get_option in the C ABI).
int option(int which);
int sm_count();  // multiprocessors of the current device

// Number of (channel, batch-pair) work items = blocks of the shared-memory kernels.
inline int num_pairs(const FwdParams& P) { return P.C * ((P.B + 1) / 2); }

// Runtime-plan kernel (k_dynamic.cu).
int launch_dynamic(const FwdParams& P, int io_dtype, size_t smem, cudaStream_t st);
int launch_xspec(const XspecParams& Q, cudaStream_t st);
int launch_tap_gradient(const float* g, const float* r, float* out, int nseg, int B, int C, int h, int w, int k,
                        int s, cudaStream_t st);

// Multi-pass path through a workspace (k_strip.cu).
int launch_strip(const FwdParams& P, int io_dtype, void* workspace, size_t ws_bytes, cudaStream_t st);
// Same kernels, workspace = the library's own fixed device array (no allocation anywhere).
int launch_strip_static_scratch(const FwdParams& P, int io_dtype, cudaStream_t st);

// Fused channel-mixing kernels of ConverseBlock (k_block.cu).
struct BlockParams;
int launch_ln_pw_gelu(const BlockParams& P, int io_dtype, cudaStream_t st);
int launch_pw_res_mlp(const BlockParams& P, int io_dtype, int sms, cudaStream_t st);
// tcgen05 variant of the first kernel (k_block_tc.cu): fp32, HW a multiple of 128
int launch_ln_pw_gelu_tc(const BlockParams& P, int sms, int* status, cudaStream_t st);
// tcgen05: out = res + alpha * (W . t + b), 128 -> 64 channels (P.t, P.x = res, P.w_a, P.b_a, P.alpha1)
int launch_pw_res_tc(const BlockParams& P, int sms, int* status, cudaStream_t st);
// warp-specialised, double-buffered versions of the two (k_block_tc2.cu)
int launch_ln_pw_gelu_tc2(const BlockParams& P, int io_dtype, int sms, int* status, cudaStream_t st);
int launch_pw_res_tc2(const BlockParams& P, int io_dtype, int sms, int* status, cudaStream_t st);
int launch_ln_pw_gelu_tc3(const BlockParams& P, int io_dtype, int sms, int* status, cudaStream_t st);
int launch_pw_res_tc3(const BlockParams& P, int io_dtype, int sms, int* status, cudaStream_t st);

// Multi-pass kernels with a compile-time axis plan (k_strip2.cu, one object per registry line).
struct StripParams;
typedef int (*Strip2Launcher)(const StripParams& SP, int io_dtype, cudaStream_t st);
typedef int (*Strip2Resident)(int io_dtype, int k, int* blocks_per_sm);  // [3]: kernels A, B, C
struct Strip2Entry {
  int r0, r1, s0, s1;  // axis length r0 * r1; Rader sub-plan s0 * s1 of r0 - 1 (0, 0 if r0 is a register radix)
  Strip2Launcher A, B, C;
  Strip2Resident Q;
};

// Tensor-core multi-pass kernels (k_gemmdft.cu, one object per registry line).
namespace gd { struct Params; }
typedef int (*GdLauncher)(const gd::Params& P, int io_dtype, cudaStream_t st);
struct GdEntry {
  int r0;
  GdLauncher A, B1, B2, C;
};

// Compile-time-plan kernels (k_static.cu, one object per registry line).
typedef int (*StaticLauncher)(const FwdParams& P, int io_dtype, size_t smem, int blocks, cudaStream_t st);
struct StaticEntry {
  int ry0, ry1, rx0, rx1, nt, mb;
  StaticLauncher fn;          // one block per plane pair
  StaticLauncher fn_persist;  // persistent blocks with prefetch
};

}  // namespace cvb
