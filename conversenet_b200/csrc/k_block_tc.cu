// ConverseBlock first fused kernel on the 5th-generation tensor cores (tcgen05 + TMEM):
//   out = GELU( W1 . LN(x) + b1 ),  64 -> 128 channels, one 128-pixel tile per iteration.
// Per tile: (1) each warp loads 32 pixels x 64 channels, normalises them (LayerNorm across
// channels: 4 lanes share a pixel quad, two shuffles), splits every value into TF32 hi + lo and
// writes both in the K-major core-matrix layout; (2) one thread issues 8 K-steps x 3 MMAs
// (hi*hi + hi*lo + lo*hi, M = 128 pixels, N = 128 channels, K = 8) into a 128-column TMEM
// accumulator and commits to an mbarrier; (3) each warp reads its 32 TMEM lanes back, adds the
// bias, applies GELU and stores (coalesced: lane = pixel).  The folded weights (hi and lo, K-major
// core-matrix layout) are staged once per block; blocks loop over tiles.
// Every wait is bounded; on a time-out the block flags the status word, frees its TMEM and leaves.
#include "../../include/converse_b200.h"
#include "cvb_internal.h"
#include "cvb_block.cuh"
#include "cvb_tc.cuh"

namespace cvb {

constexpr int kTcThreads = 128;
constexpr int kTcTile = 128;                     // pixels per tile = MMA M
// Both operands are K-major (MN-major TF32 operands produced zeros on this part).  Bytes between
// 8-row groups / between the two 4-wide K halves of an MMA / between K steps.  A's strides are
// padded so that the staging stores of a quarter-warp fall into eight different 16-byte banks.
constexpr int kA_SBO = 128, kA_LBO = 2064, kA_KSTEP = 4128;
constexpr int kB_SBO = 128, kB_LBO = 2048, kB_KSTEP = 4096;
constexpr int kAFloats = (kBlkC / 8) * (kA_KSTEP / 4);  // one A operand (hi or lo)
constexpr int kBFloats = kBlkM * kBlkC;          // one B operand

__global__ void __launch_bounds__(kTcThreads, 1) ln_pw_gelu_tc_kernel(const BlockParams P, int* status) {
  extern __shared__ __align__(128) float tsm[];
  float* a_hi = tsm;
  float* a_lo = a_hi + kAFloats;
  float* b_hi = a_lo + kAFloats;
  float* b_lo = b_hi + kBFloats;
  float* bias = b_lo + kBFloats;                 // [128]
  uint64_t* mbar = (uint64_t*)(bias + kBlkM);
  uint32_t* tmem_holder = (uint32_t*)(mbar + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long ntiles = ((long long)P.B * P.HW) / kTcTile;

  // ---- once per block: weights (LayerNorm affine folded in), barrier, TMEM ----
  for (int i = tid; i < kBlkM * kBlkC; i += kTcThreads) {
    const int oc = i / kBlkC, ic = i - oc * kBlkC;
    float hi, lo;
    tc::split_tf32(P.w_a[i] * P.ln_w[ic], hi, lo);
    const int idx = (oc >> 3) * 32 + (oc & 7) * 4 + (ic & 3) + ((ic >> 2) & 1) * (kB_LBO / 4) + (ic >> 3) * (kB_KSTEP / 4);
    b_hi[idx] = hi;
    b_lo[idx] = lo;
  }
  for (int oc = tid; oc < kBlkM; oc += kTcThreads) {
    float s = P.b_a[oc];
    for (int ic = 0; ic < kBlkC; ++ic) s = fmaf(P.w_a[oc * kBlkC + ic], P.ln_b[ic], s);
    bias[oc] = s;
  }
  if (tid == 0) {
    mbar_init(mbar, 1);
    mbar_fence_init();
  }
  if (warp == 0) tc::tmem_alloc(tmem_holder, 128);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  constexpr uint32_t idesc = tc::idesc_tf32(kTcTile, kBlkM, /*a_mn_major=*/false, /*b_mn_major=*/false);

  const int q = lane >> 2, cg = lane & 3;        // pixel quad within the warp, channel group
  uint32_t parity = 0;
  bool failed = false;
  for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const long long pix0 = tile * kTcTile;
    const int b = (int)(pix0 / P.HW);
    const int p0 = (int)(pix0 - (long long)b * P.HW);
    // ---- (1) load, LayerNorm, split, stage A ----
    // lane = (pixel quad q, channel-group phase cg); the thread owns pixels 4q..4q+3 of its warp's 32
    // and the four channel groups g = cg + 4j (channels 4g..4g+3): a 4 x 4 block per group, read as four
    // float4 along pixels and written as four float4 along channels (the K-major 16-byte unit).
    const float* xb = (const float*)P.x + (size_t)b * kBlkC * P.HW + p0 + warp * 32 + q * 4;
    float4 v[16];  // v[4*j + e] = channel 4*(cg+4j)+e, pixels 4q..4q+3
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) v[4 * j + e] = *(const float4*)(xb + (size_t)(4 * (cg + 4 * j) + e) * P.HW);
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 16; ++j) { s.x += v[j].x; s.y += v[j].y; s.z += v[j].z; s.w += v[j].w; }
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      s.x += __shfl_xor_sync(0xffffffffu, s.x, o); s.y += __shfl_xor_sync(0xffffffffu, s.y, o);
      s.z += __shfl_xor_sync(0xffffffffu, s.z, o); s.w += __shfl_xor_sync(0xffffffffu, s.w, o);
    }
    const float4 mean = make_float4(s.x * (1.0f / kBlkC), s.y * (1.0f / kBlkC), s.z * (1.0f / kBlkC), s.w * (1.0f / kBlkC));
    float4 qv = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      v[j].x -= mean.x; v[j].y -= mean.y; v[j].z -= mean.z; v[j].w -= mean.w;
      qv.x = fmaf(v[j].x, v[j].x, qv.x); qv.y = fmaf(v[j].y, v[j].y, qv.y);
      qv.z = fmaf(v[j].z, v[j].z, qv.z); qv.w = fmaf(v[j].w, v[j].w, qv.w);
    }
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      qv.x += __shfl_xor_sync(0xffffffffu, qv.x, o); qv.y += __shfl_xor_sync(0xffffffffu, qv.y, o);
      qv.z += __shfl_xor_sync(0xffffffffu, qv.z, o); qv.w += __shfl_xor_sync(0xffffffffu, qv.w, o);
    }
    const float rstd[4] = {1.0f / sqrtf(qv.x * (1.0f / kBlkC) + P.ln_eps), 1.0f / sqrtf(qv.y * (1.0f / kBlkC) + P.ln_eps),
                           1.0f / sqrtf(qv.z * (1.0f / kBlkC) + P.ln_eps), 1.0f / sqrtf(qv.w * (1.0f / kBlkC) + P.ln_eps)};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int g = cg + 4 * j;                  // channel group: k = 4g .. 4g+3
      const int kof = (g & 1) * (kA_LBO / 4) + (g >> 1) * (kA_KSTEP / 4);
#pragma unroll
      for (int i = 0; i < 4; ++i) {              // pixel within the quad
        const int m = warp * 32 + q * 4 + i;
        const float px[4] = {i == 0 ? v[4 * j].x : i == 1 ? v[4 * j].y : i == 2 ? v[4 * j].z : v[4 * j].w,
                             i == 0 ? v[4 * j + 1].x : i == 1 ? v[4 * j + 1].y : i == 2 ? v[4 * j + 1].z : v[4 * j + 1].w,
                             i == 0 ? v[4 * j + 2].x : i == 1 ? v[4 * j + 2].y : i == 2 ? v[4 * j + 2].z : v[4 * j + 2].w,
                             i == 0 ? v[4 * j + 3].x : i == 1 ? v[4 * j + 3].y : i == 2 ? v[4 * j + 3].z : v[4 * j + 3].w};
        float4 hi, lo;
        tc::split_tf32(px[0] * rstd[i], hi.x, lo.x);
        tc::split_tf32(px[1] * rstd[i], hi.y, lo.y);
        tc::split_tf32(px[2] * rstd[i], hi.z, lo.z);
        tc::split_tf32(px[3] * rstd[i], hi.w, lo.w);
        const int idx = (m >> 3) * (kA_SBO / 4) + (m & 7) * 4 + kof;
        *(float4*)(a_hi + idx) = hi;
        *(float4*)(a_lo + idx) = lo;
      }
    }
    tc::fence_proxy_async();
    tc::fence_before_sync();
    __syncthreads();
    // ---- (2) MMAs ----
    if (tid == 0) {
      tc::fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < kBlkC / 8; ++ks) {
        const uint64_t ah = tc::smem_desc((const char*)a_hi + ks * kA_KSTEP, kA_LBO, kA_SBO);
        const uint64_t al = tc::smem_desc((const char*)a_lo + ks * kA_KSTEP, kA_LBO, kA_SBO);
        const uint64_t bh = tc::smem_desc((const char*)b_hi + ks * kB_KSTEP, kB_LBO, kB_SBO);
        const uint64_t bl = tc::smem_desc((const char*)b_lo + ks * kB_KSTEP, kB_LBO, kB_SBO);
        tc::mma_tf32(tmem, ah, bh, idesc, ks > 0 ? 1u : 0u);
        tc::mma_tf32(tmem, ah, bl, idesc, 1u);
        tc::mma_tf32(tmem, al, bh, idesc, 1u);
      }
      tc::mma_commit(mbar);
    }
    // ---- (3) wait, read TMEM, bias + GELU, store ----
    const bool ok = mbar_wait_bounded(mbar, parity, kWaitLimit);
    parity ^= 1u;
    if (__syncthreads_or(!ok)) { failed = true; break; }
    tc::fence_after_sync();
    float* ob = (float*)P.out + (size_t)b * kBlkM * P.HW + p0 + warp * 32 + lane;
#pragma unroll 1
    for (int c0 = 0; c0 < kBlkM; c0 += 32) {
      float acc[32];
      tc::tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, acc);
#pragma unroll
      for (int j = 0; j < 32; ++j) ob[(size_t)(c0 + j) * P.HW] = gelu_erf(acc[j] + bias[c0 + j]);
    }
    tc::fence_before_sync();
    __syncthreads();   // TMEM and the A buffers are free for the next tile
    tc::fence_after_sync();
  }
  if (failed && tid == 0 && status) atomicExch(status, 2);
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, 128);
}

// ---- second tensor-core kernel: out = res + alpha * (W . t + b), 128 -> 64 channels ----
// (conv1[5] with the first residual, models/util_converse.py:283,291, and conv2[3] with the second,
// :288,292).  No LayerNorm: the warp streams its 32 pixels x 128 channels in two halves straight into
// the K-major hi/lo tiles.  K = 128 -> 16 K-steps x 3 MMAs, N = 64 -> 64 TMEM columns.
constexpr int kR_K = kBlkM, kR_N = kBlkC;
constexpr int kRA_SBO = 128, kRA_LBO = 2064, kRA_KSTEP = 4128;
constexpr int kRB_SBO = 128, kRB_LBO = 1024, kRB_KSTEP = 2048;
constexpr int kRAFloats = (kR_K / 8) * (kRA_KSTEP / 4);
constexpr int kRBFloats = kR_N * kR_K;

__global__ void __launch_bounds__(kTcThreads, 1) pw_res_tc_kernel(const BlockParams P, int* status) {
  extern __shared__ __align__(128) float tsm[];
  float* a_hi = tsm;
  float* a_lo = a_hi + kRAFloats;
  float* b_hi = a_lo + kRAFloats;
  float* b_lo = b_hi + kRBFloats;
  float* bias = b_lo + kRBFloats;                // [64]
  float* alpha = bias + kR_N;                    // [64]
  uint64_t* mbar = (uint64_t*)(alpha + kR_N);
  uint32_t* tmem_holder = (uint32_t*)(mbar + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long ntiles = ((long long)P.B * P.HW) / kTcTile;
  for (int i = tid; i < kR_N * kR_K; i += kTcThreads) {
    const int oc = i / kR_K, ic = i - oc * kR_K;
    float hi, lo;
    tc::split_tf32(P.w_a[i], hi, lo);
    const int idx = (oc >> 3) * 32 + (oc & 7) * 4 + (ic & 3) + ((ic >> 2) & 1) * (kRB_LBO / 4) + (ic >> 3) * (kRB_KSTEP / 4);
    b_hi[idx] = hi;
    b_lo[idx] = lo;
  }
  for (int oc = tid; oc < kR_N; oc += kTcThreads) {
    bias[oc] = P.b_a[oc];
    alpha[oc] = P.alpha1 ? P.alpha1[oc] : 1.0f;
  }
  if (tid == 0) {
    mbar_init(mbar, 1);
    mbar_fence_init();
  }
  if (warp == 0) tc::tmem_alloc(tmem_holder, 64);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  constexpr uint32_t idesc = tc::idesc_tf32(kTcTile, kR_N, false, false);

  const int q = lane >> 2, cg = lane & 3;
  uint32_t parity = 0;
  bool failed = false;
  for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const long long pix0 = tile * kTcTile;
    const int b = (int)(pix0 / P.HW);
    const int p0 = (int)(pix0 - (long long)b * P.HW);
    const float* tb = (const float*)P.t + (size_t)b * kR_K * P.HW + p0 + warp * 32 + q * 4;
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      float4 v[16];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          v[4 * j + e] = *(const float4*)(tb + (size_t)(4 * (cg + 4 * (j + 4 * half)) + e) * P.HW);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int g = cg + 4 * (j + 4 * half);   // channel group: k = 4g .. 4g+3
        const int kof = (g & 1) * (kRA_LBO / 4) + (g >> 1) * (kRA_KSTEP / 4);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int m = warp * 32 + q * 4 + i;
          const float px[4] = {i == 0 ? v[4 * j].x : i == 1 ? v[4 * j].y : i == 2 ? v[4 * j].z : v[4 * j].w,
                               i == 0 ? v[4 * j + 1].x : i == 1 ? v[4 * j + 1].y : i == 2 ? v[4 * j + 1].z : v[4 * j + 1].w,
                               i == 0 ? v[4 * j + 2].x : i == 1 ? v[4 * j + 2].y : i == 2 ? v[4 * j + 2].z : v[4 * j + 2].w,
                               i == 0 ? v[4 * j + 3].x : i == 1 ? v[4 * j + 3].y : i == 2 ? v[4 * j + 3].z : v[4 * j + 3].w};
          float4 hi, lo;
          tc::split_tf32(px[0], hi.x, lo.x);
          tc::split_tf32(px[1], hi.y, lo.y);
          tc::split_tf32(px[2], hi.z, lo.z);
          tc::split_tf32(px[3], hi.w, lo.w);
          const int idx = (m >> 3) * (kRA_SBO / 4) + (m & 7) * 4 + kof;
          *(float4*)(a_hi + idx) = hi;
          *(float4*)(a_lo + idx) = lo;
        }
      }
    }
    tc::fence_proxy_async();
    tc::fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc::fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < kR_K / 8; ++ks) {
        const uint64_t ah = tc::smem_desc((const char*)a_hi + ks * kRA_KSTEP, kRA_LBO, kRA_SBO);
        const uint64_t al = tc::smem_desc((const char*)a_lo + ks * kRA_KSTEP, kRA_LBO, kRA_SBO);
        const uint64_t bh = tc::smem_desc((const char*)b_hi + ks * kRB_KSTEP, kRB_LBO, kRB_SBO);
        const uint64_t bl = tc::smem_desc((const char*)b_lo + ks * kRB_KSTEP, kRB_LBO, kRB_SBO);
        tc::mma_tf32(tmem, ah, bh, idesc, ks > 0 ? 1u : 0u);
        tc::mma_tf32(tmem, ah, bl, idesc, 1u);
        tc::mma_tf32(tmem, al, bh, idesc, 1u);
      }
      tc::mma_commit(mbar);
    }
    const bool ok = mbar_wait_bounded(mbar, parity, kWaitLimit);
    parity ^= 1u;
    if (__syncthreads_or(!ok)) { failed = true; break; }
    tc::fence_after_sync();
    const size_t off = (size_t)b * kR_N * P.HW + p0 + warp * 32 + lane;
    const float* rb = (const float*)P.x + off;
    float* ob = (float*)P.out + off;
#pragma unroll 1
    for (int c0 = 0; c0 < kR_N; c0 += 32) {
      float acc[32];
      tc::tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, acc);
      float r[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = rb[(size_t)(c0 + j) * P.HW];
#pragma unroll
      for (int j = 0; j < 32; ++j) ob[(size_t)(c0 + j) * P.HW] = fmaf(alpha[c0 + j], acc[j] + bias[c0 + j], r[j]);
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
  }
  if (failed && tid == 0 && status) atomicExch(status, 2);
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, 64);
}

int launch_pw_res_tc(const BlockParams& P, int sms, int* status, cudaStream_t st) {
  const size_t smem = (size_t)(2 * kRAFloats + 2 * kRBFloats + 2 * kR_N) * sizeof(float) + 64;
  CVB_CUDA(cudaFuncSetAttribute(pw_res_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const long long ntiles = ((long long)P.B * P.HW) / kTcTile;
  const int grid = (int)(ntiles < sms ? ntiles : sms);
  pw_res_tc_kernel<<<grid, kTcThreads, smem, st>>>(P, status);
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}

int launch_ln_pw_gelu_tc(const BlockParams& P, int sms, int* status, cudaStream_t st) {
  const size_t smem = (size_t)(2 * kAFloats + 2 * kBFloats + kBlkM) * sizeof(float) + 64;
  CVB_CUDA(cudaFuncSetAttribute(ln_pw_gelu_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const long long ntiles = ((long long)P.B * P.HW) / kTcTile;
  const int grid = (int)(ntiles < sms ? ntiles : sms);
  ln_pw_gelu_tc_kernel<<<grid, kTcThreads, smem, st>>>(P, status);
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}

}  // namespace cvb
