// Kernels of the fused channel-mixing parts of ConverseBlock (see cvb_block.cuh).
#include "../../include/converse_b200.h"
#include "cvb_internal.h"
#include "cvb_block.cuh"

namespace cvb {

constexpr int kBlkThreads = 128;
constexpr int kK1Px = 2;  // pixels per thread in K1

template <typename IO>
__global__ void __launch_bounds__(kBlkThreads, 2) ln_pw_gelu_kernel(const BlockParams P) {
  extern __shared__ float bsm[];
  float* wt = bsm;                    // [C][2C]
  float* bf = bsm + kBlkC * kBlkM;    // [2C]
  k1_stage(threadIdx.x, kBlkThreads, P, wt, bf);
  __syncthreads();
  const long long total = (long long)P.B * P.HW;
  const long long pix0 = (long long)blockIdx.x * (kBlkThreads * kK1Px) + threadIdx.x;
  if (pix0 < total) k1_pixels<IO, kK1Px>(P, wt, bf, pix0, kBlkThreads, total);
}

template <typename IO>
__global__ void __launch_bounds__(kBlkThreads, 2) pw_res_mlp_kernel(const BlockParams P) {
  extern __shared__ float bsm[];
  const K3Smem m = k3_carve(bsm);
  k3_stage(threadIdx.x, kBlkThreads, P, m);
  __syncthreads();
  const long long total = (long long)P.B * P.HW;
  // a block walks several pixel groups so that the 96 KB of staged weights are reused
  for (long long pix = (long long)blockIdx.x * kBlkThreads + threadIdx.x; pix < total;
       pix += (long long)gridDim.x * kBlkThreads)
    k3_pixel<IO>(P, m, pix);
}

int launch_ln_pw_gelu(const BlockParams& P, int io_dtype, cudaStream_t st) {
  const size_t smem = (size_t)(kBlkC * kBlkM + kBlkM) * sizeof(float);
  const long long total = (long long)P.B * P.HW;
  const int grid = (int)((total + kBlkThreads * kK1Px - 1) / (kBlkThreads * kK1Px));
  if (io_dtype == CVB_F32) {
    CVB_CUDA(cudaFuncSetAttribute(ln_pw_gelu_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    ln_pw_gelu_kernel<float><<<grid, kBlkThreads, smem, st>>>(P);
  } else {
    CVB_CUDA(cudaFuncSetAttribute(ln_pw_gelu_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    ln_pw_gelu_kernel<__nv_bfloat16><<<grid, kBlkThreads, smem, st>>>(P);
  }
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}

int launch_pw_res_mlp(const BlockParams& P, int io_dtype, int sms, cudaStream_t st) {
  const size_t smem = k3_smem_floats() * sizeof(float);
  const long long total = (long long)P.B * P.HW;
  long long want = (total + kBlkThreads - 1) / kBlkThreads;
  const long long cap = (long long)sms * 2 * 4;  // a few waves of 2 blocks per SM
  const int grid = (int)(want < cap ? want : cap);
  if (io_dtype == CVB_F32) {
    CVB_CUDA(cudaFuncSetAttribute(pw_res_mlp_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    pw_res_mlp_kernel<float><<<grid, kBlkThreads, smem, st>>>(P);
  } else {
    CVB_CUDA(cudaFuncSetAttribute(pw_res_mlp_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    pw_res_mlp_kernel<__nv_bfloat16><<<grid, kBlkThreads, smem, st>>>(P);
  }
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}

}  // namespace cvb
