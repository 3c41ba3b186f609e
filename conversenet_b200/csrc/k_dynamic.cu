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

// batch-summed cross spectrum of (pad(x), q): one block per (channel, batch segment)
__global__ void __launch_bounds__(512, 1) smem_xspec_kernel(const XspecParams Q) {
  extern __shared__ float2 smem[];
  smem_block_xspec(Q, blockIdx.x, blockIdx.y, smem, 0);
}

int launch_xspec(const XspecParams& Q, cudaStream_t st) {
  const size_t smem = xspec_smem_bytes(Q.h, Q.w, Q.direct);
  if (Q.direct) CVB_CUDA(cudaMemsetAsync(Q.out, 0, (size_t)Q.C * Q.h * Q.w * sizeof(float2), st));
  CVB_CUDA(cudaFuncSetAttribute(smem_xspec_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int by = Q.w * (Q.h / Q.py.radix[0]), bx = Q.h * (Q.w / Q.px.radix[0]);
  int nthr = ((by > bx ? by : bx) + 31) / 32 * 32;
  if (nthr < 64) nthr = 64;
  if (nthr > 512) nthr = 512;
  smem_xspec_kernel<<<dim3(Q.C, Q.nseg), nthr, smem, st>>>(Q);
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}

// Direct tap term of the scale >= 2 parameter gradient:
//   out[seg][c][a][b] = sum over batch entries n = seg, seg + nseg, ... and cells m of
//                       g[n,c,(s my - a + cc) mod s h, (s mx - b + cc) mod s w] * r[n,c,my,mx],   cc = k / 2
// (the derivative of corr(K, zero_insert_s(r)) with respect to K, models/util_converse.py:171-173 collapsed).
// One block per (channel, segment); per tap a block-wide sum.
__global__ void __launch_bounds__(256) tap_gradient_kernel(const float* __restrict__ g, const float* __restrict__ r,
                                                           float* __restrict__ out, int nseg, int B, int C, int h,
                                                           int w, int k, int s) {
  __shared__ float red[8];
  const int c = blockIdx.x, seg = blockIdx.y, tid = threadIdx.x;
  const int sh = s * h, sw = s * w, cc = k / 2, cells = h * w;
  const float invw = 1.0f / (float)w;
  for (int t = 0; t < k * k; ++t) {
    const int a = t / k, b = t - a * k;
    float part = 0.f;
    for (int n = seg; n < B; n += nseg) {
      const float* gp = g + ((size_t)n * C + c) * sh * sw;
      const float* rp = r + ((size_t)n * C + c) * cells;
      for (int i = tid; i < cells; i += 256) {
        int my, mx;
        divmod_small(i, w, invw, my, mx);
        int gy = s * my - a + cc, gx = s * mx - b + cc;
        gy += gy < 0 ? sh : (gy >= sh ? -sh : 0);
        gx += gx < 0 ? sw : (gx >= sw ? -sw : 0);
        part = fmaf(gp[(size_t)gy * sw + gx], rp[i], part);
      }
    }
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if ((tid & 31) == 0) red[tid >> 5] = part;
    __syncthreads();
    if (tid == 0) {
      float v = 0.f;
      for (int i = 0; i < 8; ++i) v += red[i];
      out[((size_t)seg * C + c) * k * k + t] = v;
    }
    __syncthreads();
  }
}

// The same sums with the k x k taps of a cell kept in registers (compile-time K): a thread owns cells,
// reads the K x K window of g around (s my + cc, s mx + cc) and r once per cell; block-wide sums at the end.
template <int K>
__global__ void __launch_bounds__(256) tap_gradient_window_kernel(const float* __restrict__ g,
                                                                  const float* __restrict__ r,
                                                                  float* __restrict__ out, int nseg, int B, int C,
                                                                  int h, int w, int s) {
  __shared__ float red[8];
  const int c = blockIdx.x, seg = blockIdx.y, tid = threadIdx.x;
  const int sh = s * h, sw = s * w, cc = K / 2, cells = h * w;
  const float invw = 1.0f / (float)w;
  float acc[K * K];
#pragma unroll
  for (int t = 0; t < K * K; ++t) acc[t] = 0.f;
  for (int n = seg; n < B; n += nseg) {
    const float* gp = g + ((size_t)n * C + c) * sh * sw;
    const float* rp = r + ((size_t)n * C + c) * cells;
    for (int i = tid; i < cells; i += 256) {
      int my, mx;
      divmod_small(i, w, invw, my, mx);
      const float rv = rp[i];
      int gx[K];
#pragma unroll
      for (int b = 0; b < K; ++b) {
        int v = s * mx - b + cc;
        v += v < 0 ? sw : (v >= sw ? -sw : 0);
        gx[b] = v;
      }
#pragma unroll
      for (int a = 0; a < K; ++a) {
        int gy = s * my - a + cc;
        gy += gy < 0 ? sh : (gy >= sh ? -sh : 0);
        const float* row = gp + (size_t)gy * sw;
#pragma unroll
        for (int b = 0; b < K; ++b) acc[a * K + b] = fmaf(row[gx[b]], rv, acc[a * K + b]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < K * K; ++t) {
    float part = acc[t];
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if ((tid & 31) == 0) red[tid >> 5] = part;
    __syncthreads();
    if (tid == 0) {
      float v = 0.f;
      for (int i = 0; i < 8; ++i) v += red[i];
      out[((size_t)seg * C + c) * K * K + t] = v;
    }
    __syncthreads();
  }
}

int launch_tap_gradient(const float* g, const float* r, float* out, int nseg, int B, int C, int h, int w, int k,
                        int s, cudaStream_t st) {
  const dim3 grid(C, nseg);
  switch (k) {
    case 2: tap_gradient_window_kernel<2><<<grid, 256, 0, st>>>(g, r, out, nseg, B, C, h, w, s); break;
    case 3: tap_gradient_window_kernel<3><<<grid, 256, 0, st>>>(g, r, out, nseg, B, C, h, w, s); break;
    case 5: tap_gradient_window_kernel<5><<<grid, 256, 0, st>>>(g, r, out, nseg, B, C, h, w, s); break;
    case 7: tap_gradient_window_kernel<7><<<grid, 256, 0, st>>>(g, r, out, nseg, B, C, h, w, s); break;
    default: tap_gradient_kernel<<<grid, 256, 0, st>>>(g, r, out, nseg, B, C, h, w, k, s); break;
  }
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}

int launch_dynamic(const FwdParams& P, int io_dtype, size_t smem, cudaStream_t st) {
  return io_dtype == CVB_F32 ? launch_t<float>(P, smem, st) : launch_t<__nv_bfloat16>(P, smem, st);
}

}  // namespace cvb
