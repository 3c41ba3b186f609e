// Compile-time-plan shared-memory kernels.  Built once per line of the static
// registry with -DCVB_RY0=.. -DCVB_RY1=.. -DCVB_RX0=.. -DCVB_RX1=.. -DCVB_NT=.. -DCVB_MB=..
// (padded plane (RY0*RY1) x (RX0*RX1), NT threads, at least MB blocks per SM).
//   launch_static_*  : one block per plane pair, x read straight from global memory.
//   launch_persist_* : MB blocks per SM loop over the pairs; the next pair's planes are
//                      prefetched by bulk asynchronous copies into shared memory.
#include "../../include/converse_b200.h"
#include "cvb_internal.h"

#define CVB_CAT_(n, a, b, c, d, nt, mb) launch_##n##_##a##_##b##_##c##_##d##_##nt##_##mb
#define CVB_CAT(n, a, b, c, d, nt, mb) CVB_CAT_(n, a, b, c, d, nt, mb)

namespace cvb {

// The radices are template parameters so that every registry line gets its own
// kernel symbol: this file is compiled several times into one library.
template <typename IO, int RY0, int RY1, int RX0, int RX1, int NT, int MB>
__global__ void __launch_bounds__(NT, MB) smem_static_kernel(const FwdParams P) {
  extern __shared__ float2 smem[];
  smem_block_static<IO, RY0, RY1, RX0, RX1, NT>(P, blockIdx.x, smem);
}

template <typename IO, int RY0, int RY1, int RX0, int RX1, int NT, int MB>
__global__ void __launch_bounds__(NT, MB) smem_persistent_kernel(const FwdParams P) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  smem_persistent_static<IO, RY0, RY1, RX0, RX1, NT>(P, smem_raw, blockIdx.x, gridDim.x);
}

namespace {
template <typename IO>
int launch_t(const FwdParams& P, size_t smem, cudaStream_t st) {
  auto kernel = smem_static_kernel<IO, CVB_RY0, CVB_RY1, CVB_RX0, CVB_RX1, CVB_NT, CVB_MB>;
  CVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kernel<<<num_pairs(P), CVB_NT, smem, st>>>(P);  // the block size is baked into the index arithmetic
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}

template <typename IO>
int launch_p(const FwdParams& P, size_t smem, int blocks, cudaStream_t st) {
  auto kernel = smem_persistent_kernel<IO, CVB_RY0, CVB_RY1, CVB_RX0, CVB_RX1, CVB_NT, CVB_MB>;
  CVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kernel<<<blocks, CVB_NT, smem, st>>>(P);
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}
}  // namespace

int CVB_CAT(static, CVB_RY0, CVB_RY1, CVB_RX0, CVB_RX1, CVB_NT, CVB_MB)(const FwdParams& P, int io_dtype,
                                                                       size_t smem, int, cudaStream_t st) {
  return io_dtype == CVB_F32 ? launch_t<float>(P, smem, st) : launch_t<__nv_bfloat16>(P, smem, st);
}

int CVB_CAT(persist, CVB_RY0, CVB_RY1, CVB_RX0, CVB_RX1, CVB_NT, CVB_MB)(const FwdParams& P, int io_dtype,
                                                                        size_t smem, int blocks,
                                                                        cudaStream_t st) {
  return io_dtype == CVB_F32 ? launch_p<float>(P, smem, blocks, st) : launch_p<__nv_bfloat16>(P, smem, blocks, st);
}

}  // namespace cvb
