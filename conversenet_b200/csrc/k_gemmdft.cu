// Multi-pass kernels for padded lengths N = 4 * R0 with the R0-point transforms on the tensor
// cores (cvb_gemmdft.cuh).  Built once per line of the registry with -DCVB_G0=R0; kernels A and C
// use the plan of the column axis, B1 and B2 that of the row axis.
#include "../../include/converse_b200.h"
#include "cvb_internal.h"
#include "cvb_gemmdft.cuh"

#define CVB_GCAT_(n, a) launch_gd##n##_##a
#define CVB_GCAT(n, a) CVB_GCAT_(n, a)

namespace cvb {
namespace gd {

// Two blocks share an SM while the constant operand is small (R0 <= 96: 96 registers per thread);
// above that one block fills the SM's shared memory and may use the registers of two.
#if CVB_G0 <= 96
#define CVB_GD_MIN_BLOCKS 2
#else
#define CVB_GD_MIN_BLOCKS 1
#endif
template <int R0, int MODE, typename IO>
__global__ void __launch_bounds__(kThreads, CVB_GD_MIN_BLOCKS) gd_kernel(const Params P) {
  extern __shared__ unsigned char gd_smem[];
  body<R0, MODE, IO>(P, gd_smem);
}

namespace {
typedef Geo<CVB_G0> G;
// Constant operand (hi and lo halves of the cos / sin matrix in operand layout): a fixed array in
// the library image, filled by one small kernel the first time a device runs this plan.
static __device__ __align__(128) float g_bmat[2 * G::B_FLOATS];

static int bmat_ready(const float** out, cudaStream_t st) {
  static bool done[64] = {false};
  static float* addr[64] = {nullptr};
  int dev = 0;
  CVB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return CVB_ERR_BAD_ARGUMENT;
  if (!done[dev]) {
    void* p = nullptr;
    CVB_CUDA(cudaGetSymbolAddress(&p, g_bmat));
    addr[dev] = (float*)p;
    dft_matrix_kernel<CVB_G0><<<32, 256, 0, st>>>(addr[dev]);
    CVB_CUDA(cudaGetLastError());
    // Other streams may use the array from the next call on: finish the fill now.  Inside a stream
    // capture nothing can be waited for, so the fill stays part of every captured call.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    CVB_CUDA(cudaStreamIsCapturing(st, &cap));
    if (cap == cudaStreamCaptureStatusNone) {
      CVB_CUDA(cudaStreamSynchronize(st));
      done[dev] = true;
    }
  }
  *out = addr[dev];
  return CVB_OK;
}

template <typename K>
static int launch_k(K kernel, const Params& P0, int mode, cudaStream_t st) {
  Params P = P0;
  const int rc = bmat_ready(&P.bmat, st);
  if (rc != CVB_OK) return rc;
  const size_t smem = smem_bytes<CVB_G0>(mode);
  static int resident[4] = {0, 0, 0, 0};   // blocks per SM, asked once per kernel family
  CVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  if (!resident[mode]) {
    // ask for the largest shared-memory carve-out: with the default one the SM is configured for one
    // block's worth and a second block does not fit
    CVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kThreads, smem) != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      n = 1;
    }
    // Blocks per SM: TMEM (512 columns per SM) and shared memory decide.  The occupancy query answers
    // one block for the two-block configuration (R0 <= 96: 256 columns and ~112 KB each), but a grid of
    // two blocks per SM measured 1.4x faster than one, so the grid is sized from the resources directly.
    const int by_tmem = 512 / G::TMEM_COLS;
    const int by_smem = (int)((size_t)233472 / (smem + 1024));
    (void)n;
    resident[mode] = by_tmem < by_smem ? by_tmem : by_smem;
    if (resident[mode] < 1) resident[mode] = 1;
  }
  const int other = (mode == MODE_A || mode == MODE_C) ? P.f.w : P.f.h;
  const long long nlines = (long long)P.npair * other;
  const long long ntiles = (nlines + kLines - 1) / kLines;
  const long long cap = (long long)resident[mode] * sm_count();
  const int grid = (int)(ntiles < cap ? ntiles : cap);
  if (grid < 1) return CVB_OK;
  kernel<<<grid, kThreads, smem, st>>>(P);
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}
}  // namespace
}  // namespace gd

int CVB_GCAT(A, CVB_G0)(const gd::Params& P, int io_dtype, cudaStream_t st) {
  return io_dtype == CVB_F32 ? gd::launch_k(gd::gd_kernel<CVB_G0, gd::MODE_A, float>, P, gd::MODE_A, st)
                             : gd::launch_k(gd::gd_kernel<CVB_G0, gd::MODE_A, __nv_bfloat16>, P, gd::MODE_A, st);
}
int CVB_GCAT(B1, CVB_G0)(const gd::Params& P, int, cudaStream_t st) {
  return gd::launch_k(gd::gd_kernel<CVB_G0, gd::MODE_B1, float>, P, gd::MODE_B1, st);
}
int CVB_GCAT(B2, CVB_G0)(const gd::Params& P, int, cudaStream_t st) {
  return gd::launch_k(gd::gd_kernel<CVB_G0, gd::MODE_B2, float>, P, gd::MODE_B2, st);
}
int CVB_GCAT(C, CVB_G0)(const gd::Params& P, int io_dtype, cudaStream_t st) {
  return io_dtype == CVB_F32 ? gd::launch_k(gd::gd_kernel<CVB_G0, gd::MODE_C, float>, P, gd::MODE_C, st)
                             : gd::launch_k(gd::gd_kernel<CVB_G0, gd::MODE_C, __nv_bfloat16>, P, gd::MODE_C, st);
}

}  // namespace cvb
