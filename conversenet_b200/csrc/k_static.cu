// Compile-time-plan shared-memory kernel.  Built once per line of the static
// registry with -DCVB_RY0=.. -DCVB_RY1=.. -DCVB_RX0=.. -DCVB_RX1=.. -DCVB_NT=.. -DCVB_MB=..
// (padded plane (RY0*RY1) x (RX0*RX1), NT threads, at least MB blocks per SM).
#include "../../include/converse_b200.h"
#include "cvb_internal.h"

#define CVB_CAT_(a, b, c, d, nt, mb, u) launch_static_##a##_##b##_##c##_##d##_##nt##_##mb##_##u
#define CVB_CAT(a, b, c, d, nt, mb, u) CVB_CAT_(a, b, c, d, nt, mb, u)

namespace cvb {

// The radices are template parameters so that every registry line gets its own
// kernel symbol: this file is compiled several times into one library.
#ifndef CVB_UNI
#define CVB_UNI 0
#endif
template <typename IO, int RY0, int RY1, int RX0, int RX1, int NT, int MB, int UNI>
__global__ void __launch_bounds__(NT, MB) smem_static_kernel(const FwdParams P) {
  extern __shared__ float2 smem[];
  smem_block_static<IO, RY0, RY1, RX0, RX1, NT, UNI != 0>(P, blockIdx.x, smem);
}

namespace {
template <typename IO>
int launch_t(const FwdParams& P, size_t smem, cudaStream_t st) {
  auto kernel = smem_static_kernel<IO, CVB_RY0, CVB_RY1, CVB_RX0, CVB_RX1, CVB_NT, CVB_MB, CVB_UNI>;
  CVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kernel<<<num_pairs(P), CVB_NT, smem, st>>>(P);  // the block size is baked into the index arithmetic
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}
}  // namespace

int CVB_CAT(CVB_RY0, CVB_RY1, CVB_RX0, CVB_RX1, CVB_NT, CVB_MB, CVB_UNI)(const FwdParams& P, int io_dtype, size_t smem, cudaStream_t st) {
  return io_dtype == CVB_F32 ? launch_t<float>(P, smem, st) : launch_t<__nv_bfloat16>(P, smem, st);
}

}  // namespace cvb
