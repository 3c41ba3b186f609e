// Compile-time-plan shared-memory kernel.  Built once per line of the static
// registry with -DCVB_RY0=.. -DCVB_RY1=.. -DCVB_RX0=.. -DCVB_RX1=.. -DCVB_NT=.. -DCVB_MB=..
// (padded plane (RY0*RY1) x (RX0*RX1), NT threads, at least MB blocks per SM).
#include "../../include/converse_b200.h"
#include "cvb_internal.h"

#define CVB_CAT_(a, b, c, d) launch_static_##a##_##b##_##c##_##d
#define CVB_CAT(a, b, c, d) CVB_CAT_(a, b, c, d)

namespace cvb {

// The radices are template parameters so that every registry line gets its own
// kernel symbol: this file is compiled several times into one library.
template <typename IO, int RY0, int RY1, int RX0, int RX1>
__global__ void __launch_bounds__(CVB_NT, CVB_MB) smem_static_kernel(const FwdParams P) {
  extern __shared__ float2 smem[];
  smem_block_static<IO, RY0, RY1, RX0, RX1>(P, blockIdx.x, smem, 0);
}

namespace {
template <typename IO>
int launch_t(const FwdParams& P, size_t smem, cudaStream_t st) {
  auto kernel = smem_static_kernel<IO, CVB_RY0, CVB_RY1, CVB_RX0, CVB_RX1>;
  CVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int nthr = env_int("CVB_THREADS", CVB_NT);
  if (nthr < 32 || nthr > CVB_NT) nthr = CVB_NT;
  kernel<<<num_pairs(P), nthr, smem, st>>>(P);
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}
}  // namespace

int CVB_CAT(CVB_RY0, CVB_RY1, CVB_RX0, CVB_RX1)(const FwdParams& P, int io_dtype, size_t smem, cudaStream_t st) {
  return io_dtype == CVB_F32 ? launch_t<float>(P, smem, st) : launch_t<__nv_bfloat16>(P, smem, st);
}

}  // namespace cvb
