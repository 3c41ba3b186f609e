// Multi-pass kernels with a compile-time axis plan N = R0 * R1 (Rader sub-plan S0 * S1 when
// R0 is a large prime).  Built once per line of the axis-plan registry with
// -DCVB_R0=.. -DCVB_R1=.. -DCVB_S0=.. -DCVB_S1=.. ; kernels A and C use the plan for the
// column axis, kernel B for the row axis.
#include "../../include/converse_b200.h"
#include "cvb_internal.h"
#include "cvb_strip2.cuh"

#define CVB_CAT_(n, a, b) launch_strip2##n##_##a##_##b
#define CVB_CAT(n, a, b) CVB_CAT_(n, a, b)

namespace cvb {

constexpr int kLines = strip2_lines(CVB_R0 * CVB_R1, CVB_R0);
constexpr int kThreads = strip2_threads(CVB_R0);
constexpr int kMinBlocks = 2;

template <typename IO, int R0, int R1, int S0, int S1>
__global__ void __launch_bounds__(kThreads, kMinBlocks) strip2_A_kernel(const StripParams SP) {
  extern __shared__ float2 smem[];
  strip2_A_body<IO, R0, R1, S0, S1>(SP, blockIdx.y, blockIdx.x, smem, 0);
}
template <int R0, int R1, int S0, int S1>
__global__ void __launch_bounds__(kThreads, kMinBlocks) strip2_B_kernel(const StripParams SP) {
  extern __shared__ float2 smem[];
  strip2_B_body<R0, R1, S0, S1>(SP, blockIdx.y, blockIdx.x, smem, 0);
}
template <typename IO, int R0, int R1, int S0, int S1>
__global__ void __launch_bounds__(kThreads, kMinBlocks) strip2_C_kernel(const StripParams SP) {
  extern __shared__ float2 smem[];
  strip2_C_body<IO, R0, R1, S0, S1>(SP, blockIdx.y, blockIdx.x, smem, 0);
}

namespace {
template <typename K>
int launch_k(K kernel, const StripParams& SP0, int nstrips, size_t smem, cudaStream_t st) {
  const StripParams& SP = SP0;
  CVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kernel<<<dim3(nstrips, SP.npair), kThreads, smem, st>>>(SP);
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}
template <typename K>
int resident_blocks(K kernel, size_t smem) {
  int n = 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kThreads, smem) != cudaSuccess || n < 1) {
    (void)cudaGetLastError();
    n = 2;
  }
  return n;
}
}  // namespace

// blocks of kernels A, B, C that one SM holds at a time (asked once per element type and tap count)
int CVB_CAT(Q, CVB_R0, CVB_R1)(int io_dtype, int k, int* bpsm) {
  static int key = -1, cached[3] = {2, 2, 2};
  const int want = io_dtype * 64 + k;
  if (key != want) {
    const size_t smem = strip2_smem(CVB_R0 * CVB_R1, kLines, CVB_R0, k);
    if (io_dtype == CVB_F32) {
      cached[0] = resident_blocks(strip2_A_kernel<float, CVB_R0, CVB_R1, CVB_S0, CVB_S1>, smem);
      cached[2] = resident_blocks(strip2_C_kernel<float, CVB_R0, CVB_R1, CVB_S0, CVB_S1>, smem);
    } else {
      cached[0] = resident_blocks(strip2_A_kernel<__nv_bfloat16, CVB_R0, CVB_R1, CVB_S0, CVB_S1>, smem);
      cached[2] = resident_blocks(strip2_C_kernel<__nv_bfloat16, CVB_R0, CVB_R1, CVB_S0, CVB_S1>, smem);
    }
    cached[1] = resident_blocks(strip2_B_kernel<CVB_R0, CVB_R1, CVB_S0, CVB_S1>, smem);
    key = want;
  }
  bpsm[0] = cached[0]; bpsm[1] = cached[1]; bpsm[2] = cached[2];
  return CVB_OK;
}

int CVB_CAT(A, CVB_R0, CVB_R1)(const StripParams& SP, int io_dtype, cudaStream_t st) {
  const size_t smem = strip2_smem(CVB_R0 * CVB_R1, kLines, CVB_R0, SP.f.k);
  const int n = (SP.f.w + kLines - 1) / kLines;
  return io_dtype == CVB_F32
             ? launch_k(strip2_A_kernel<float, CVB_R0, CVB_R1, CVB_S0, CVB_S1>, SP, n, smem, st)
             : launch_k(strip2_A_kernel<__nv_bfloat16, CVB_R0, CVB_R1, CVB_S0, CVB_S1>, SP, n, smem, st);
}
int CVB_CAT(B, CVB_R0, CVB_R1)(const StripParams& SP, int, cudaStream_t st) {
  const size_t smem = strip2_smem(CVB_R0 * CVB_R1, kLines, CVB_R0, SP.f.k);
  const int n = (SP.f.h + kLines - 1) / kLines;
  return launch_k(strip2_B_kernel<CVB_R0, CVB_R1, CVB_S0, CVB_S1>, SP, n, smem, st);
}
int CVB_CAT(C, CVB_R0, CVB_R1)(const StripParams& SP, int io_dtype, cudaStream_t st) {
  const size_t smem = strip2_smem(CVB_R0 * CVB_R1, kLines, CVB_R0, SP.f.k);
  const int cw = kLines - SP.halo_l - SP.halo_r;
  const int n = (SP.f.w + cw - 1) / cw;
  return io_dtype == CVB_F32
             ? launch_k(strip2_C_kernel<float, CVB_R0, CVB_R1, CVB_S0, CVB_S1>, SP, n, smem, st)
             : launch_k(strip2_C_kernel<__nv_bfloat16, CVB_R0, CVB_R1, CVB_S0, CVB_S1>, SP, n, smem, st);
}

}  // namespace cvb
