// Warp-specialised tcgen05 kernel for the 1x1 convolutions of ConverseBlock (128-pixel tiles):
//   MODE 0:  out = GELU( W . LN(x) + b )          K = 64  -> N = 128   (conv1[0..2] and conv2[0..2])
//   MODE 1:  out = res + alpha * ( W . t + b )    K = 128 -> N = 64    (conv1[5] / conv2[3] + residual)
// Tensors are fp32 or bf16 (IO); arithmetic, operands and accumulators are the same for both.
// Roles (288 threads): warps 0-3 produce -- load 32 pixels x 64 channels each, (LayerNorm), split into
// TF32 hi + lo, write the K-major core-matrix tiles of one 64-channel chunk; warp 8 issues the MMAs
// (8 K-steps x 3 per chunk) and commits; warps 4-7 consume -- read their 32 TMEM lanes, bias / GELU /
// alpha / residual, store.  Chunks flow through a ring of two shared-memory stages, tiles through two
// TMEM accumulators, so loading, tensor-core work and the epilogue of neighbouring tiles overlap.
//   full[s]       producers -> issuer   (128 arrivals)      chunk staged in stage s
//   empty[s]      issuer -> producers   (tcgen05.commit)    MMAs that read stage s are done
//   tfull[a]      issuer -> consumers   (tcgen05.commit)    accumulator a complete
//   tempty[a]     consumers -> issuer   (128 arrivals)      accumulator a has been read
// Every wait is bounded: on a time-out the waiting thread raises a block-wide abort flag, all roles
// leave their loops, the status word is set and TMEM is released after a last bounded wait.
#include "../../include/converse_b200.h"
#include "cvb_internal.h"
#include "cvb_block.cuh"
#include "cvb_tc.cuh"

namespace cvb {

constexpr int kT2Threads = 288;
constexpr int kT2Tile = 128;
constexpr int kT2Chunk = 64;                               // channels per staged chunk
constexpr int kT2A_SBO = 128, kT2A_LBO = 2064, kT2A_KSTEP = 4128;
constexpr int kT2AFloats = (kT2Chunk / 8) * (kT2A_KSTEP / 4);  // one of hi / lo of one stage

template <int MODE> struct T2Shape;
template <> struct T2Shape<0> { static constexpr int K = 64, N = 128; };
template <> struct T2Shape<1> { static constexpr int K = 128, N = 64; };

// bounded wait that also gives up when another thread raised the abort flag
__device__ __forceinline__ bool t2_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (int i = 0; i < kWaitLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255) == 255 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// four consecutive pixels of one channel: fp32 (16 bytes) or bf16 (8 bytes) tensors, fp32 in registers
template <typename IO> __device__ __forceinline__ float4 t2_load4(const IO* p);
template <> __device__ __forceinline__ float4 t2_load4<float>(const float* p) { return *(const float4*)p; }
template <> __device__ __forceinline__ float4 t2_load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 u = *(const uint2*)p;
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                     __uint_as_float(u.y & 0xffff0000u));
}

template <int MODE, typename IO>
__global__ void __launch_bounds__(kT2Threads, 1) tc_pw_kernel(const BlockParams P, int* status) {
  constexpr int K = T2Shape<MODE>::K, N = T2Shape<MODE>::N, CPT = K / kT2Chunk;
  constexpr int B_SBO = 128, B_LBO = (N / 8) * 128, B_KSTEP = 2 * B_LBO;
  constexpr int BFloats = N * K;
  extern __shared__ __align__(128) float tsm[];
  float* a_st = tsm;                              // [2 stages][hi, lo][kT2AFloats]
  float* b_hi = a_st + 4 * kT2AFloats;
  float* b_lo = b_hi + BFloats;
  float* bias = b_lo + BFloats;                   // [N]
  float* alpha = bias + N;                        // [N] (MODE 1)
  uint64_t* bars = (uint64_t*)(alpha + N);        // full[2], empty[2], tfull[2], tempty[2]
  uint32_t* tmem_holder = (uint32_t*)(bars + 8);
  volatile int* abort_flag = (volatile int*)(tmem_holder + 1);
  uint64_t* full = bars; uint64_t* empty = bars + 2; uint64_t* tfull = bars + 4; uint64_t* tempty = bars + 6;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long ntiles = ((long long)P.B * P.HW) / kT2Tile;

  // ---- set-up: weights (hi / lo, LayerNorm affine folded in for MODE 0), barriers, TMEM ----
  for (int i = tid; i < N * K; i += kT2Threads) {
    const int oc = i / K, ic = i - oc * K;
    float hi, lo;
    tc::split_tf32(MODE == 0 ? P.w_a[i] * P.ln_w[ic] : P.w_a[i], hi, lo);
    const int idx = (oc >> 3) * 32 + (oc & 7) * 4 + (ic & 3) + ((ic >> 2) & 1) * (B_LBO / 4) + (ic >> 3) * (B_KSTEP / 4);
    b_hi[idx] = hi;
    b_lo[idx] = lo;
  }
  for (int oc = tid; oc < N; oc += kT2Threads) {
    float s = P.b_a[oc];
    if (MODE == 0)
      for (int ic = 0; ic < K; ++ic) s = fmaf(P.w_a[oc * K + ic], P.ln_b[ic], s);
    bias[oc] = s;
    alpha[oc] = (MODE == 1 && P.alpha1) ? P.alpha1[oc] : 1.0f;
  }
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&full[i], 128);
      mbar_init(&empty[i], 1);
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 8) tc::tmem_alloc(tmem_holder, 2 * N);
  tc::fence_proxy_async();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  constexpr uint32_t idesc = tc::idesc_tf32(kT2Tile, N, false, false);

  if (warp < 4) {
    // ================= producers =================
    const int q = lane >> 2, cg = lane & 3;
    long long chunk = 0;
    // the loads of the NEXT chunk are issued before the current one is normalised and staged, so that
    // two chunks of global reads are in flight per producer thread
    auto load_chunk = [&](long long tile, int kc, float4 (&dst)[16]) {
      const long long pix0 = tile * kT2Tile;
      const int b = (int)(pix0 / P.HW);
      const int p0 = (int)(pix0 - (long long)b * P.HW);
      const IO* src = (const IO*)(MODE == 0 ? P.x : P.t) + (size_t)b * K * P.HW + p0 + warp * 32 + q * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          dst[4 * j + e] = t2_load4<IO>(src + (size_t)(kc * kT2Chunk + 4 * (cg + 4 * j) + e) * P.HW);
    };
    float4 vn[16];
    if ((long long)blockIdx.x < ntiles) load_chunk(blockIdx.x, 0, vn);
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
#pragma unroll 1
      for (int kc = 0; kc < CPT; ++kc, ++chunk) {
        const int st = (int)(chunk & 1);
        float4 v[16];  // v[4*j + e] = channel 64*kc + 4*(cg+4j)+e, pixels 4q..4q+3
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = vn[j];
        {
          const bool last_kc = (kc + 1 == CPT);
          const long long ntile = last_kc ? tile + gridDim.x : tile;
          if (ntile < ntiles) load_chunk(ntile, last_kc ? 0 : kc + 1, vn);
        }
        float rstd[4] = {1.f, 1.f, 1.f, 1.f};
        if (MODE == 0) {
          float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int j = 0; j < 16; ++j) { s.x += v[j].x; s.y += v[j].y; s.z += v[j].z; s.w += v[j].w; }
#pragma unroll
          for (int o = 1; o <= 2; o <<= 1) {
            s.x += __shfl_xor_sync(0xffffffffu, s.x, o); s.y += __shfl_xor_sync(0xffffffffu, s.y, o);
            s.z += __shfl_xor_sync(0xffffffffu, s.z, o); s.w += __shfl_xor_sync(0xffffffffu, s.w, o);
          }
          const float4 mean = make_float4(s.x * (1.0f / K), s.y * (1.0f / K), s.z * (1.0f / K), s.w * (1.0f / K));
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
          rstd[0] = 1.0f / sqrtf(qv.x * (1.0f / K) + P.ln_eps);
          rstd[1] = 1.0f / sqrtf(qv.y * (1.0f / K) + P.ln_eps);
          rstd[2] = 1.0f / sqrtf(qv.z * (1.0f / K) + P.ln_eps);
          rstd[3] = 1.0f / sqrtf(qv.w * (1.0f / K) + P.ln_eps);
        }
        // the stage must have been drained by the MMAs of two chunks ago
        if (!t2_wait(&empty[st], (uint32_t)(((chunk >> 1) & 1) ^ 1), abort_flag)) break;
        float* a_hi = a_st + st * 2 * kT2AFloats;
        float* a_lo = a_hi + kT2AFloats;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int g = cg + 4 * j;
          const int kof = (g & 1) * (kT2A_LBO / 4) + (g >> 1) * (kT2A_KSTEP / 4);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
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
            const int idx = (m >> 3) * (kT2A_SBO / 4) + (m & 7) * 4 + kof;
            *(float4*)(a_hi + idx) = hi;
            *(float4*)(a_lo + idx) = lo;
          }
        }
        tc::fence_proxy_async();
        mbar_arrive(&full[st]);
      }
      if (*abort_flag) break;
    }
  } else if (warp == 8) {
    // ================= MMA issuer (one lane) =================
    if (lane == 0) {
      long long chunk = 0, it = 0;
      for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
        const int acc = (int)(it & 1);
        // accumulator free again?  (first use of each passes at once)
        if (!t2_wait(&tempty[acc], (uint32_t)(((it >> 1) & 1) ^ 1), abort_flag)) break;
        tc::fence_after_sync();
        const uint32_t d = tmem + (uint32_t)(acc * N);
        bool ok = true;
#pragma unroll 1
        for (int kc = 0; kc < CPT; ++kc, ++chunk) {
          const int st = (int)(chunk & 1);
          if (!t2_wait(&full[st], (uint32_t)((chunk >> 1) & 1), abort_flag)) { ok = false; break; }
          tc::fence_after_sync();
          const char* a_hi = (const char*)(a_st + st * 2 * kT2AFloats);
          const char* a_lo = a_hi + kT2AFloats * 4;
#pragma unroll
          for (int ks = 0; ks < kT2Chunk / 8; ++ks) {
            const uint64_t ah = tc::smem_desc(a_hi + ks * kT2A_KSTEP, kT2A_LBO, kT2A_SBO);
            const uint64_t al = tc::smem_desc(a_lo + ks * kT2A_KSTEP, kT2A_LBO, kT2A_SBO);
            const int kb = kc * (kT2Chunk / 8) + ks;
            const uint64_t bh = tc::smem_desc((const char*)b_hi + kb * B_KSTEP, B_LBO, B_SBO);
            const uint64_t bl = tc::smem_desc((const char*)b_lo + kb * B_KSTEP, B_LBO, B_SBO);
            tc::mma_tf32(d, ah, bh, idesc, (kc > 0 || ks > 0) ? 1u : 0u);
            tc::mma_tf32(d, ah, bl, idesc, 1u);
            tc::mma_tf32(d, al, bh, idesc, 1u);
          }
          tc::mma_commit(&empty[st]);     // the stage may be refilled once these MMAs are done
        }
        if (!ok) break;
        tc::mma_commit(&tfull[acc]);      // accumulator complete
      }
    }
  } else {
    // ================= consumers (warps 4-7: TMEM lanes 32*(warp-4) ..) =================
    const int cw = warp - 4;
    long long it = 0;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
      const int acc = (int)(it & 1);
      const long long pix0 = tile * kT2Tile;
      const int b = (int)(pix0 / P.HW);
      const int p0 = (int)(pix0 - (long long)b * P.HW);
      const size_t off = (size_t)b * N * P.HW + p0 + cw * 32 + lane;
      IO* ob = (IO*)P.out + off;
      const IO* rb = (const IO*)P.x + off;   // residual (MODE 1)
      // MODE 1: the residual values of the first 32 channels are requested before the wait for the
      // accumulator, those of the next 32 before the first are used, so their latency is off the path
      float r[MODE == 1 ? 32 : 1];
      if (MODE == 1) {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = ld_io<IO>(rb, (size_t)j * P.HW);
      }
      if (!t2_wait(&tfull[acc], (uint32_t)((it >> 1) & 1), abort_flag)) break;
      tc::fence_after_sync();
#pragma unroll 1
      for (int c0 = 0; c0 < N; c0 += 32) {
        float a32[32];
        tc::tmem_ld32(tmem + ((uint32_t)(cw * 32) << 16) + (uint32_t)(acc * N + c0), a32);
        if (MODE == 0) {
#pragma unroll
          for (int j = 0; j < 32; ++j) st_io<IO>(ob, (size_t)(c0 + j) * P.HW, gelu_erf(a32[j] + bias[c0 + j]));
        } else {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaf(alpha[c0 + j], a32[j] + bias[c0 + j], r[j]);
          if (c0 + 32 < N) {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = ld_io<IO>(rb, (size_t)(c0 + 32 + j) * P.HW);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) st_io<IO>(ob, (size_t)(c0 + j) * P.HW, v[j]);
        }
      }
      tc::fence_before_sync();
      mbar_arrive(&tempty[acc]);
    }
  }
  // ---- common exit ----
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0 && status) atomicExch(status, 3);
    // let MMAs that may still be in flight finish before the accumulators are released
    if (warp == 8 && lane == 0) {
      mbar_wait_bounded(&tfull[0], 0, 4096);
      mbar_wait_bounded(&tfull[1], 0, 4096);
    }
    __syncthreads();
  }
  if (warp == 8) {
    __syncwarp();
    tc::tmem_dealloc(tmem, 2 * N);
  }
}

template <int MODE, typename IO>
static int launch_t2(const BlockParams& P, int sms, int* status, cudaStream_t st) {
  constexpr int K = T2Shape<MODE>::K, N = T2Shape<MODE>::N;
  const size_t smem = (size_t)(4 * kT2AFloats + 2 * N * K + 2 * N) * sizeof(float) + 8 * sizeof(uint64_t) + 64;
  CVB_CUDA(cudaFuncSetAttribute(tc_pw_kernel<MODE, IO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const long long ntiles = ((long long)P.B * P.HW) / kT2Tile;
  const int grid = (int)(ntiles < sms ? ntiles : sms);
  tc_pw_kernel<MODE, IO><<<grid, kT2Threads, smem, st>>>(P, status);
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}

int launch_ln_pw_gelu_tc2(const BlockParams& P, int io_dtype, int sms, int* status, cudaStream_t st) {
  return io_dtype == CVB_F32 ? launch_t2<0, float>(P, sms, status, st) : launch_t2<0, __nv_bfloat16>(P, sms, status, st);
}
int launch_pw_res_tc2(const BlockParams& P, int io_dtype, int sms, int* status, cudaStream_t st) {
  return io_dtype == CVB_F32 ? launch_t2<1, float>(P, sms, status, st) : launch_t2<1, __nv_bfloat16>(P, sms, status, st);
}

}  // namespace cvb
