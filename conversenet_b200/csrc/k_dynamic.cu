// Runtime-plan shared-memory kernel: any padded size whose prime factors have a
// butterfly, one block per (channel, batch pair).
#include "../../include/converse_b200.h"
#include "cvb_internal.h"

namespace cvb {

template <typename IO>
__global__ void __launch_bounds__(512, 1) smem_dynamic_kernel(const FwdParams P) {
  extern __shared__ float2 smem[];
  smem_block_dynamic<IO>(P, blockIdx.x, smem, 0);
}

namespace {
template <typename IO>
int launch_t(const FwdParams& P, size_t smem, cudaStream_t st) {
  CVB_CUDA(cudaFuncSetAttribute(smem_dynamic_kernel<IO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int nthr = CVB_TUNE("CVB_THREADS", 0);
  if (nthr <= 0) {
    // enough threads for the stage with the fewest butterflies, at most 512
    const int by = P.w * (P.h / P.py.radix[0]), bx = P.h * (P.w / P.px.radix[0]);
    const int items = by > bx ? by : bx;
    nthr = (items + 31) / 32 * 32;
    if (nthr < 64) nthr = 64;
    if (nthr > 512) nthr = 512;
  }
  if (nthr > 512) nthr = 512;
  smem_dynamic_kernel<IO><<<num_pairs(P), nthr, smem, st>>>(P);
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}
}  // namespace

int launch_dynamic(const FwdParams& P, int io_dtype, size_t smem, cudaStream_t st) {
  return io_dtype == CVB_F32 ? launch_t<float>(P, smem, st) : launch_t<__nv_bfloat16>(P, smem, st);
}

}  // namespace cvb
