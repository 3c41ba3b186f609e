// tcgen05 kernel for the 1x1 convolutions of ConverseBlock (128-pixel tiles) with the split operand A in
// tensor memory and the tensors streamed through a shared-memory ring of asynchronous copies:
//   MODE 0:  out = GELU( W . LN(x) + b )          K = 64  -> N = 128   (conv1[0..2] and conv2[0..2])
//   MODE 1:  out = res + alpha * ( W . t + b )    K = 128 -> N = 64    (conv1[5] / conv2[3] + residual)
// Tensors are fp32 or bf16 (IO); arithmetic, operands and accumulators are the same for both.
// Roles: warps 0-3 produce, warp 8 issues the MMAs, warps 4-7 consume; MODE 1 has a second set of consumers,
// warps 9-12, so that two warps share a TMEM quadrant and each takes half of the accumulator's columns
// (measured: 1x1 + residual on bf16 tensors 0.106 -> 0.089 ms; MODE 0 got slower with it, 0.104 -> 0.122 ms).
//   Producers copy chunks of 64 channels x 128 pixels (the tensor's own layout: one row of 128 pixels per
//   channel) into a ring of kRing raw slots with cp.async, kRing - 1 chunks ahead, holding nothing in
//   registers meanwhile.  When a chunk has landed, thread m takes pixel m: its 64 channel values sit in
//   one column of the slot, so LayerNorm's mean and variance are sums inside one thread; it splits the
//   values into TF32 hi + lo and writes them to its own lane of a 128-column operand stage in tensor
//   memory (tcgen05.st) -- no operand tiles in shared memory, no proxy fence.
//   The issuer runs 8 K-steps x 3 MMAs per chunk with A read from tensor memory and commits; consumers
//   read their 32 TMEM lanes, apply bias / GELU / alpha / residual and store.
//   full[s]       producers -> issuer   (128 arrivals)      chunk staged in operand stage s
//   empty[s]      issuer -> producers   (tcgen05.commit)    MMAs that read stage s are done
//   tfull[a]      issuer -> consumers   (tcgen05.commit)    accumulator a complete
//   tempty[a]     consumers -> issuer   (128 / 256 arrivals) accumulator a has been read
// TMEM columns: accumulators [0, 2N), operand stages at 2N + 128 s (hi [0,64), lo [64,128)).
// Every wait is bounded: on a time-out the waiting thread raises a block-wide abort flag, all roles
// leave their loops, the status word is set and TMEM is released after a last bounded wait.
#include "../../include/converse_b200.h"
#include "cvb_internal.h"
#include "cvb_block.cuh"
#include "cvb_tc.cuh"

namespace cvb {

template <int MODE> struct T3Threads { static constexpr int value = MODE == 1 ? 416 : 288; };
constexpr int kT3Tile = 128;
constexpr int kT3Chunk = 64;     // channels per chunk
constexpr int kT3Ring = 4;       // raw slots

template <int MODE> struct T3Shape;
template <> struct T3Shape<0> { static constexpr int K = 64, N = 128; };
template <> struct T3Shape<1> { static constexpr int K = 128, N = 64; };

__device__ __forceinline__ bool t3_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (int i = 0; i < kWaitLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255) == 255 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void t3_cp16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void t3_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void t3_wait_group() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void t3_bar_producers() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// sixteen consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void t3_st16(uint32_t taddr, const float (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
      "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
      "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
      : "memory");
}

template <int MODE, typename IO>
__global__ void __launch_bounds__(T3Threads<MODE>::value, 1) tc3_pw_kernel(const BlockParams P, int* status) {
  constexpr int kT3Threads = T3Threads<MODE>::value;
  constexpr int kConsumerSets = MODE == 1 ? 2 : 1;
  constexpr int K = T3Shape<MODE>::K, N = T3Shape<MODE>::N, CPT = K / kT3Chunk;
  constexpr int B_SBO = 128, B_LBO = (N / 8) * 128, B_KSTEP = 2 * B_LBO;
  constexpr int BFloats = N * K;
  constexpr int kSlotBytes = kT3Chunk * kT3Tile * (int)sizeof(IO);
  constexpr uint32_t A_BASE = 2 * N;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ __align__(128) unsigned char t3sm[];
  unsigned char* raw = t3sm;                                   // [kT3Ring][64 channels][128 pixels] IO
  float* b_hi = (float*)(raw + kT3Ring * kSlotBytes);
  float* b_lo = b_hi + BFloats;
  float* bias = b_lo + BFloats;                                // [N]
  float* alpha = bias + N;                                     // [N] (MODE 1)
  uint64_t* bars = (uint64_t*)(alpha + N);                     // full[2], empty[2], tfull[2], tempty[2]
  uint32_t* tmem_holder = (uint32_t*)(bars + 8);
  volatile int* abort_flag = (volatile int*)(tmem_holder + 1);
  uint64_t* full = bars; uint64_t* empty = bars + 2; uint64_t* tfull = bars + 4; uint64_t* tempty = bars + 6;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long ntiles = ((long long)P.B * P.HW) / kT3Tile;
  const long long my_tiles = ((long long)blockIdx.x < ntiles) ? (ntiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;

  // ---- set-up: weights (hi / lo, LayerNorm affine folded in for MODE 0), barriers, TMEM ----
  for (int i = tid; i < N * K; i += kT3Threads) {
    const int oc = i / K, ic = i - oc * K;
    float hi, lo;
    tc::split_tf32(MODE == 0 ? P.w_a[i] * P.ln_w[ic] : P.w_a[i], hi, lo);
    const int idx = (oc >> 3) * 32 + (oc & 7) * 4 + (ic & 3) + ((ic >> 2) & 1) * (B_LBO / 4) + (ic >> 3) * (B_KSTEP / 4);
    b_hi[idx] = hi;
    b_lo[idx] = lo;
  }
  for (int oc = tid; oc < N; oc += kT3Threads) {
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
      mbar_init(&tempty[i], 128 * kConsumerSets);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 8) tc::tmem_alloc(tmem_holder, TMEM_COLS);
  tc::fence_proxy_async();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  constexpr uint32_t idesc = tc::idesc_tf32(kT3Tile, N, false, false);

  if (warp < 4) {
    // ================= producers =================
    const long long nchunks = my_tiles * CPT;
    const IO* tensor = (const IO*)(MODE == 0 ? P.x : P.t);
    constexpr int kSegs = kT3Tile * (int)sizeof(IO) / 16;     // 16-byte segments per channel row
    constexpr int kRowsPerPass = 128 / kSegs;
    const int seg = tid % kSegs, r0 = tid / kSegs;
    auto issue_copy = [&](long long g) {
      const long long tile = blockIdx.x + (g / CPT) * gridDim.x;
      const int kc = (int)(g % CPT);
      const long long pix0 = tile * kT3Tile;
      const int b = (int)(pix0 / P.HW);
      const int p0 = (int)(pix0 - (long long)b * P.HW);
      const unsigned char* src = (const unsigned char*)(tensor + ((size_t)b * K + (size_t)kc * kT3Chunk) * P.HW + p0);
      unsigned char* dst = raw + (int)(g % kT3Ring) * kSlotBytes;
#pragma unroll
      for (int i = 0; i < kT3Chunk / kRowsPerPass; ++i) {
        const int row = r0 + i * kRowsPerPass;
        t3_cp16(dst + (size_t)row * kT3Tile * sizeof(IO) + seg * 16, src + (size_t)row * P.HW * sizeof(IO) + seg * 16);
      }
    };
    // kRing - 1 groups are always committed ahead (empty ones past the end keep the count uniform)
    for (int g = 0; g < kT3Ring - 1; ++g) {
      if (g < nchunks) issue_copy(g);
      t3_commit();
    }
    const uint32_t my_lane = tmem + ((uint32_t)(warp * 32) << 16);
    bool alive = true;   // false after a time-out: keep meeting the other producers on the barrier, do no work
    for (long long g = 0; g < nchunks; ++g) {
      t3_wait_group<kT3Ring - 2>();   // this thread's part of chunk g has landed
      t3_bar_producers();             // ... and everybody's; everybody has finished reading chunk g - 1
      if (alive && g + kT3Ring - 1 < nchunks) issue_copy(g + kT3Ring - 1);   // into the slot chunk g - 1 occupied
      t3_commit();
      if (*abort_flag) alive = false;
      if (!alive) continue;
      const int st = (int)(g & 1);
      const IO* col = (const IO*)(raw + (int)(g % kT3Ring) * kSlotBytes) + tid;   // pixel tid, channel c at col[c * 128]
      float v[kT3Chunk];
#pragma unroll
      for (int c = 0; c < kT3Chunk; ++c) v[c] = ld_io<IO>(col, (size_t)c * kT3Tile);
      if (MODE == 0) {
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < kT3Chunk; ++c) s += v[c];
        const float mean = s * (1.0f / K);
        float q = 0.f;
#pragma unroll
        for (int c = 0; c < kT3Chunk; ++c) { v[c] -= mean; q = fmaf(v[c], v[c], q); }
        const float rstd = 1.0f / sqrtf(q * (1.0f / K) + P.ln_eps);
#pragma unroll
        for (int c = 0; c < kT3Chunk; ++c) v[c] *= rstd;
      }
      // the operand stage must have been drained by the MMAs of two chunks ago
      if (!t3_wait(&empty[st], (uint32_t)(((g >> 1) & 1) ^ 1), abort_flag)) { alive = false; continue; }
      tc::fence_after_sync();
      const uint32_t a_st = my_lane + A_BASE + (uint32_t)st * 128u;
#pragma unroll
      for (int c0 = 0; c0 < kT3Chunk; c0 += 16) {
        float hi[16], lo[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) tc::split_tf32(v[c0 + e], hi[e], lo[e]);
        t3_st16(a_st + (uint32_t)c0, hi);
        t3_st16(a_st + 64u + (uint32_t)c0, lo);
      }
      tc::tmem_wait_st();
      tc::fence_before_sync();
      mbar_arrive(&full[st]);
    }
    t3_wait_group<0>();
  } else if (warp == 8) {
    // ================= MMA issuer (one lane) =================
    if (lane == 0) {
      long long chunk = 0, it = 0;
      for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
        const int acc = (int)(it & 1);
        // accumulator free again?  (first use of each passes at once)
        if (!t3_wait(&tempty[acc], (uint32_t)(((it >> 1) & 1) ^ 1), abort_flag)) break;
        tc::fence_after_sync();
        const uint32_t d = tmem + (uint32_t)(acc * N);
        bool ok = true;
#pragma unroll 1
        for (int kc = 0; kc < CPT; ++kc, ++chunk) {
          const int st = (int)(chunk & 1);
          if (!t3_wait(&full[st], (uint32_t)((chunk >> 1) & 1), abort_flag)) { ok = false; break; }
          tc::fence_after_sync();
          const uint32_t a_hi = tmem + A_BASE + (uint32_t)st * 128u, a_lo = a_hi + 64u;
#pragma unroll
          for (int ks = 0; ks < kT3Chunk / 8; ++ks) {
            const int kb = kc * (kT3Chunk / 8) + ks;
            const uint64_t bh = tc::smem_desc((const char*)b_hi + kb * B_KSTEP, B_LBO, B_SBO);
            const uint64_t bl = tc::smem_desc((const char*)b_lo + kb * B_KSTEP, B_LBO, B_SBO);
            tc::mma_tf32_ta(d, a_hi + (uint32_t)(ks * 8), bh, idesc, (kc > 0 || ks > 0) ? 1u : 0u);
            tc::mma_tf32_ta(d, a_hi + (uint32_t)(ks * 8), bl, idesc, 1u);
            tc::mma_tf32_ta(d, a_lo + (uint32_t)(ks * 8), bh, idesc, 1u);
          }
          tc::mma_commit(&empty[st]);     // the stage may be refilled once these MMAs are done
        }
        if (!ok) break;
        tc::mma_commit(&tfull[acc]);      // accumulator complete
      }
    }
  } else {
    // ================= consumers: warp w reads TMEM lanes 32 (w % 4) .., warps 4-7 the first half of the
    // accumulator's columns, warps 9-12 the second =================
    const int cw = warp & 3;
    constexpr int NH = N / kConsumerSets;
    const int cbase = warp >= 9 ? NH : 0;
    long long it = 0;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
      const int acc = (int)(it & 1);
      const long long pix0 = tile * kT3Tile;
      const int b = (int)(pix0 / P.HW);
      const int p0 = (int)(pix0 - (long long)b * P.HW);
      const size_t off = (size_t)b * N * P.HW + p0 + cw * 32 + lane;
      IO* ob = (IO*)P.out + off + (size_t)cbase * P.HW;
      const IO* rb = (const IO*)P.x + off + (size_t)cbase * P.HW;   // residual (MODE 1)
      // MODE 1: this warp's 32 residual values are requested before the wait for the accumulator
      float r[MODE == 1 ? 32 : 1];
      if (MODE == 1) {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = ld_io<IO>(rb, (size_t)j * P.HW);
      }
      if (!t3_wait(&tfull[acc], (uint32_t)((it >> 1) & 1), abort_flag)) break;
      tc::fence_after_sync();
#pragma unroll 1
      for (int c0 = 0; c0 < NH; c0 += 32) {
        float a32[32];
        tc::tmem_ld32(tmem + ((uint32_t)(cw * 32) << 16) + (uint32_t)(acc * N + cbase + c0), a32);
        if (MODE == 0) {
#ifdef __CUDA_ARCH__   // (the packed helpers exist in the device pass only)
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float2 bj = *(const float2*)(bias + cbase + c0 + j);
            const float2 g = gelu_erf2(a32[j] + bj.x, a32[j + 1] + bj.y);
            st_io<IO>(ob, (size_t)(c0 + j) * P.HW, g.x);
            st_io<IO>(ob, (size_t)(c0 + j + 1) * P.HW, g.y);
          }
#endif
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            st_io<IO>(ob, (size_t)(c0 + j) * P.HW, fmaf(alpha[cbase + c0 + j], a32[j] + bias[cbase + c0 + j], r[j]));
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
    tc::tmem_dealloc(tmem, TMEM_COLS);
  }
}

template <int MODE, typename IO>
static int launch_t3(const BlockParams& P, int sms, int* status, cudaStream_t st) {
  constexpr int K = T3Shape<MODE>::K, N = T3Shape<MODE>::N;
  const size_t smem = (size_t)kT3Ring * kT3Chunk * kT3Tile * sizeof(IO) + (size_t)(2 * N * K + 2 * N) * sizeof(float) +
                      8 * sizeof(uint64_t) + 64;
  CVB_CUDA(cudaFuncSetAttribute(tc3_pw_kernel<MODE, IO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const long long ntiles = ((long long)P.B * P.HW) / kT3Tile;
  const int grid = (int)(ntiles < sms ? ntiles : sms);
  tc3_pw_kernel<MODE, IO><<<grid, T3Threads<MODE>::value, smem, st>>>(P, status);
  CVB_CUDA(cudaGetLastError());
  return CVB_OK;
}

int launch_ln_pw_gelu_tc3(const BlockParams& P, int io_dtype, int sms, int* status, cudaStream_t st) {
  return io_dtype == CVB_F32 ? launch_t3<0, float>(P, sms, status, st) : launch_t3<0, __nv_bfloat16>(P, sms, status, st);
}
int launch_pw_res_tc3(const BlockParams& P, int io_dtype, int sms, int* status, cudaStream_t st) {
  return io_dtype == CVB_F32 ? launch_t3<1, float>(P, sms, status, st) : launch_t3<1, __nv_bfloat16>(P, sms, status, st);
}

}  // namespace cvb
