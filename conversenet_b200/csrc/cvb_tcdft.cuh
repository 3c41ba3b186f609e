// A prime-length DFT stage on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// The multi-pass kernels meet axis lengths N = R * R1 whose first radix R is a prime too large for
// a register butterfly (268 = 67 * 4 in ConverseDnCNN, 516 = 43 * 12 in ConverseUSRNet).  The R-point
// DFTs of such a stage are a dense contraction: for every "vector" (tile line c, inner index j)
//     X[k] = sum_q x[q] * exp(-2 pi i k q / R),   x[q] = tile[(q * R1 + j) * tp + c],
// so they run as one GEMM per 64 vectors.  With C[k][q] = cos(2 pi k q / R), S[k][q] = sin(..):
//     X[k]     = (C xr + S xi)[k] + i (C xi - S xr)[k]
//     X[R - k] = (C xr - S xi)[k] + i (C xi + S xr)[k],        k = 0 .. (R - 1) / 2,
// i.e. two real GEMMs D0 = Xr * B^T, D1 = Xi * B^T with the same constant operand B (rows 2k = C[k],
// 2k + 1 = S[k]) and the real / imaginary parts of the vectors as the M = 64 rows of operand A
// (M = 64 keeps the operands of a 16-line tile small enough for two blocks per SM, which is what
// hides one block's staging and waiting behind the other's; accumulator row r of an M = 64 MMA
// sits in TMEM lane 32 * (r / 16) + r % 16, checked on a B200 with index-valued operands).
// All operands are fp32 split into TF32 hi + lo, three MMAs per product (hi*hi + hi*lo + lo*hi),
// which keeps fp32 accuracy (error ~2^-21 per product).
//
// Pipeline per 64 vectors: K (= q) is staged eight values (one MMA K-step) at a time into a ring of
// three operand buffers.  Threads 0..127 stage the even chunk of a pair, threads 128..255 the odd
// one: each reads four consecutive q of its vector from the tile, applies the stage's input twiddle
// when the stage is an inverse one, splits and writes four 16-byte units in the K-major core-matrix
// layout, and arrives on a named barrier; a ninth warp waits there, issues the pair's 12 MMAs (two
// accumulators) and commits each chunk to its buffer's mbarrier, so that issuing overlaps the staging
// of the next pair.  Nobody waits for the tensor cores except to reuse a buffer three chunks later
// and once before the read-back: every warp then reads its TMEM quadrant (16
// vectors) 16 columns (= 8 values of k) at a time, forms X[k] and X[R - k], applies the output
// twiddle of a forward stage and writes them back into the tile in place.  The constant operand comes
// from a device-resident copy by one bulk copy (TMA) issued at block start.
// Every mbarrier wait is bounded; on a time-out the block flags the status word and carries on
// without the tensor cores' result (the caller reads the status after the launch).
//
// The host versions of the steps run the same index arithmetic on plain arrays (the operand layout
// is decoded by the "MMA"), so that the CPU emulation of the kernels covers it.
#pragma once
#include "cvb_kernels.cuh"
#ifdef __CUDA_ARCH__
#include "cvb_tc.cuh"
#endif

namespace cvb {
#if defined(CVB_PHASE_CLOCK) && defined(__CUDA_ARCH__)
extern __device__ unsigned long long g_phase_cycles[32];
#define CVB_TCTICK_INIT() long long tctick_prev_ = clock64()
#define CVB_TCTICK(i)                                                            \
  do {                                                                           \
    if (threadIdx.x == 0) {                                                      \
      const long long now_ = clock64();                                          \
      atomicAdd(&g_phase_cycles[i], (unsigned long long)(now_ - tctick_prev_));  \
      tctick_prev_ = now_;                                                       \
    }                                                                            \
  } while (0)
#else
#define CVB_TCTICK_INIT() do { } while (0)
#define CVB_TCTICK(i) do { } while (0)
#endif
namespace tcdft {

constexpr int kChunkK = 8;       // q values per chunk = one MMA K-step
constexpr int kTileM = 64;       // vectors per accumulator (MMA M)
constexpr int kNumBuf = 3;       // operand ring
constexpr int kItems = kTileM * (kChunkK / 4);   // 16-byte units of one chunk: 128

template <int R>
struct Geo {
  static constexpr int KH = (R - 1) / 2;                        // k = 0 .. KH are computed, R - k follow
  static constexpr int NB = ((2 * (KH + 1) + 7) / 8) * 8;       // rows of B = accumulator columns
  static constexpr int KP = ((R + kChunkK - 1) / kChunkK) * kChunkK;  // q padded to whole chunks
  static constexpr int NCHUNK = KP / kChunkK;
  // operand B: K-major, no swizzle: 8-row groups 128 B apart, the two 4-wide K halves LBO apart
  static constexpr int B_LBO = (NB / 8) * 128, B_KSTEP = 2 * B_LBO;   // bytes
  static constexpr int B_FLOATS = (KP / 8) * (B_KSTEP / 4);           // one array (hi or lo)
  // operand A, one chunk of one array: 8 row groups x two K halves
  static constexpr int A_LBO = (kTileM / 8) * 128;
  static constexpr int A_FLOATS = 2 * A_LBO / 4;                      // 512
  static constexpr size_t BYTES =
      (size_t)(2 * B_FLOATS + kNumBuf * 4 * A_FLOATS + 2 * R) * sizeof(float) + 64;
  static constexpr int TMEM_COLS = 2 * NB <= 32 ? 32 : 2 * NB <= 64 ? 64 : 2 * NB <= 128 ? 128 : 256;
};

// shared memory of the stage for a prime R (same figure as Geo<R>::BYTES)
CVB_HD constexpr size_t bytes(int R) {
  const int kh = (R - 1) / 2, nb = ((2 * (kh + 1) + 7) / 8) * 8;
  const int kp = ((R + kChunkK - 1) / kChunkK) * kChunkK;
  const int b_floats = (kp / 8) * (2 * (nb / 8) * 128 / 4);
  const int a_floats = 2 * ((kTileM / 8) * 128) / 4;
  return (size_t)(2 * b_floats + kNumBuf * 4 * a_floats + 2 * R) * sizeof(float) + 64;
}

// Views into the block's shared memory (base 128-byte aligned).
struct Ctx {
  float* b_hi; float* b_lo;        // constant operand
  float* a;                        // ring: [buffer][xr hi, xr lo, xi hi, xi lo][A_FLOATS]
  float* cs;                       // cos / sin (2 pi m / R), m < R (only when B is built in place)
  uint64_t* mbar;                  // [kNumBuf] buffer free again, then one for the arrival of B
  uint32_t* tmem_holder;
  uint32_t tmem;                   // accumulator base (device)
  uint32_t commits[kNumBuf];       // commits issued so far on each buffer's mbarrier
  uint32_t pairs;                  // pairs of chunks handed to the issuing warp so far
  int b_pending;                   // the bulk copy of B has not been waited for yet
  int failed;
  int* status;
};

template <int R>
CVB_HD Ctx carve(void* base, int* status) {
  typedef Geo<R> G;
  Ctx c;
  float* f = (float*)base;
  c.b_hi = f; f += G::B_FLOATS;
  c.b_lo = f; f += G::B_FLOATS;
  c.a = f; f += kNumBuf * 4 * G::A_FLOATS;
  c.cs = f; f += 2 * R;
  c.mbar = (uint64_t*)(((uintptr_t)f + 7) & ~(uintptr_t)7);
  c.tmem_holder = (uint32_t*)(c.mbar + kNumBuf + 1);
  c.tmem = 0; c.failed = 0; c.b_pending = 0; c.status = status;
  for (int i = 0; i < kNumBuf; ++i) c.commits[i] = 0;
  c.pairs = 0;
  return c;
}

// float index of element (row mn, column k) of a K-major operand
CVB_HD int operand_index(int mn, int k, int lbo_f, int kstep_f) {
  return (mn >> 3) * 32 + (mn & 7) * 4 + (k & 3) + ((k >> 2) & 1) * lbo_f + (k >> 3) * kstep_f;
}

CVB_HD void split_hi_lo(float a, float& hi, float& lo) {
#ifdef __CUDA_ARCH__
  tc::split_tf32(a, hi, lo);
#else
  // round to 10 mantissa bits (nearest, ties away): the host stand-in of cvt.rna.tf32
  uint32_t u;
  memcpy(&u, &a, 4);
  u = (u + 0x1000u) & 0xFFFFE000u;
  memcpy(&hi, &u, 4);
  lo = a - hi;
#endif
}

// cos / sin table, first step of building B in place (one thread per m)
template <int R>
CVB_HD void setup_table(int tid, int nthr, const Ctx& c) {
  for (int m = tid; m < R; m += nthr) {
    double sn, cs;
#ifdef __CUDA_ARCH__
    sincospi(2.0 * (double)m / (double)R, &sn, &cs);
#else
    sn = sin(2.0 * M_PI * (double)m / (double)R);
    cs = cos(2.0 * M_PI * (double)m / (double)R);
#endif
    c.cs[2 * m] = (float)cs;
    c.cs[2 * m + 1] = (float)sn;
  }
}
// constant operand B from the table (after a barrier)
template <int R>
CVB_HD void setup_matrix(int tid, int nthr, const Ctx& c) {
  typedef Geo<R> G;
  for (int i = tid; i < G::NB * G::KP; i += nthr) {
    const int n = i / G::KP, q = i - n * G::KP;
    const int k = n >> 1;
    float v = 0.f;
    if (k <= G::KH && q < R) v = c.cs[2 * ((k * q) % R) + (n & 1)];
    float hi, lo;
    split_hi_lo(v, hi, lo);
    const int idx = operand_index(n, q, G::B_LBO / 4, G::B_KSTEP / 4);
    c.b_hi[idx] = hi;
    c.b_lo[idx] = lo;
  }
}

// Staging of one 16-byte unit (vector m of the accumulator tile, q-quad qq of chunk ch):
// prepare_item() fills registers, commit_item() writes the ring buffer.
struct Staged {
  float rh[4], rl[4], ih[4], il[4];
};
template <int R, int R1, int LN>
CVB_HD void prepare_item(int item, const float2* cur, int tp, const float2* tw, int mt, int ch, bool pre,
                         Staged& s) {
  constexpr int NV = LN * R1;
  const int m = item & (kTileM - 1), qq = item / kTileM;
  const int v = mt * kTileM + m;
  const int j = v / LN, cc = v - j * LN;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int q = ch * kChunkK + qq * 4 + e;
    float2 x = make_float2(0.f, 0.f);
    if (v < NV && q < R) {
      x = cur[(q * R1 + j) * tp + cc];
      if (pre && j != 0) {
        const float2 wv = tw[j * q];
        x = make_float2(fmaf(x.y, wv.y, x.x * wv.x), fmaf(-x.x, wv.y, x.y * wv.x));
      }
    }
    split_hi_lo(x.x, s.rh[e], s.rl[e]);
    split_hi_lo(x.y, s.ih[e], s.il[e]);
  }
}
template <int R>
CVB_HD void commit_item(int item, float* buf, const Staged& s) {
  typedef Geo<R> G;
  const int m = item & (kTileM - 1), qq = item / kTileM;
  const int idx = operand_index(m, qq * 4, G::A_LBO / 4, 0);
  *(float4*)(buf + 0 * G::A_FLOATS + idx) = make_float4(s.rh[0], s.rh[1], s.rh[2], s.rh[3]);
  *(float4*)(buf + 1 * G::A_FLOATS + idx) = make_float4(s.rl[0], s.rl[1], s.rl[2], s.rl[3]);
  *(float4*)(buf + 2 * G::A_FLOATS + idx) = make_float4(s.ih[0], s.ih[1], s.ih[2], s.ih[3]);
  *(float4*)(buf + 3 * G::A_FLOATS + idx) = make_float4(s.il[0], s.il[1], s.il[2], s.il[3]);
}

// Outputs X[k0 .. k0 + NK) and their mirrors X[R - k] of vector v.  d0 / d1: 2 * NK accumulator
// columns (C xr, S xr interleaved; C xi, S xi interleaved).
template <int R, int R1, int LN, int NK>
CVB_HD void emit_group(float2* cur, int tp, const float2* tw, int v, int k0, const float (&d0)[2 * NK],
                       const float (&d1)[2 * NK], bool post, float osign) {
  typedef Geo<R> G;
  constexpr int NV = LN * R1;
  if (v >= NV) return;
  const int j = v / LN, cc = v - j * LN;
#pragma unroll
  for (int kk = 0; kk < NK; ++kk) {
    const int k = k0 + kk;
    if (k > G::KH) break;
    const float cxr = d0[2 * kk], sxr = d0[2 * kk + 1], cxi = d1[2 * kk], sxi = d1[2 * kk + 1];
    float ar = cxr + sxi, ai = cxi - sxr;     // X[k]
    float br = cxr - sxi, bi = cxi + sxr;     // X[R - k]
    if (post && j != 0) {
      const float2 wa = tw[j * k];
      const float tr = fmaf(ai, wa.y, ar * wa.x), ti = fmaf(-ar, wa.y, ai * wa.x);
      ar = tr; ai = ti;
      if (k > 0) {
        const float2 wb = tw[j * (R - k)];
        const float ur = fmaf(bi, wb.y, br * wb.x), ui = fmaf(-br, wb.y, bi * wb.x);
        br = ur; bi = ui;
      }
    }
    cur[(k * R1 + j) * tp + cc] = make_float2(ar, osign * ai);
    if (k > 0) cur[((R - k) * R1 + j) * tp + cc] = make_float2(br, osign * bi);
  }
}

#ifdef __CUDACC__
// The constant operand (hi then lo, operand layout) for a whole device, written once.
template <int R>
__global__ void dft_matrix_kernel(float* out) {
#ifdef __CUDA_ARCH__
  typedef Geo<R> G;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < G::NB * G::KP; i += gridDim.x * blockDim.x) {
    const int n = i / G::KP, q = i - n * G::KP;
    const int k = n >> 1;
    float v = 0.f;
    if (k <= G::KH && q < R) {
      double sn, cs;
      sincospi(2.0 * (double)((k * q) % R) / (double)R, &sn, &cs);
      v = (float)((n & 1) ? sn : cs);
    }
    float hi, lo;
    split_hi_lo(v, hi, lo);
    const int idx = operand_index(n, q, G::B_LBO / 4, G::B_KSTEP / 4);
    out[idx] = hi;
    out[G::B_FLOATS + idx] = lo;
  }
#else
  (void)out;
#endif
}
#endif

#ifdef __CUDA_ARCH__
// 32 lanes x 16 columns of fp32, twice (one wait for both loads)
__device__ __forceinline__ void tmem_ld16x2(uint32_t ta, uint32_t tb, float (&a)[16], float (&b)[16]) {
  uint32_t r[16], s[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(ta)
      : "memory");
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(s[0]), "=r"(s[1]), "=r"(s[2]), "=r"(s[3]), "=r"(s[4]), "=r"(s[5]), "=r"(s[6]), "=r"(s[7]),
        "=r"(s[8]), "=r"(s[9]), "=r"(s[10]), "=r"(s[11]), "=r"(s[12]), "=r"(s[13]), "=r"(s[14]), "=r"(s[15])
      : "r"(tb)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int j = 0; j < 16; ++j) { a[j] = __uint_as_float(r[j]); b[j] = __uint_as_float(s[j]); }
}

// Block set-up: constant operand (bulk copy from `matrix`, or built in place when it is null),
// mbarriers, TMEM.  All threads; ends with a barrier.
template <int R>
__device__ void setup(Ctx& c, const float* matrix) {
  typedef Geo<R> G;
  const int tid = threadIdx.x, nthr = blockDim.x;
  if (!matrix) setup_table<R>(tid, nthr, c);
  if (tid == 0) {
    for (int i = 0; i <= kNumBuf; ++i) mbar_init(&c.mbar[i], 1);
    mbar_fence_init();
    if (matrix) {   // b_hi and b_lo are adjacent in both places; lands while the tile is being loaded
      mbar_expect_tx(&c.mbar[kNumBuf], 2 * G::B_FLOATS * 4);
      bulk_g2s(c.b_hi, matrix, 2 * G::B_FLOATS * 4, &c.mbar[kNumBuf]);
    }
  }
  c.b_pending = matrix ? 1 : 0;
  if (tid < 32) tc::tmem_alloc(c.tmem_holder, G::TMEM_COLS);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  c.tmem = *c.tmem_holder;
  if (!matrix) {
    setup_matrix<R>(tid, nthr, c);
    tc::fence_proxy_async();
    __syncthreads();
  }
}
// Release the accumulators and report a time-out.  All threads, after the block's last stage.
template <int R>
__device__ __forceinline__ void finish(Ctx& c) {
  tc::fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) tc::tmem_dealloc(c.tmem, Geo<R>::TMEM_COLS);
  if (c.failed && threadIdx.x == 0 && c.status) atomicExch(c.status, 3);
}

// Named barrier between the 256 staging threads (arrive, never wait) and the issuing warp (sync).
constexpr int kProducers = 256, kStageThreads = kProducers + 32;
__device__ __forceinline__ void bar_arrive(int id) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(kStageThreads) : "memory");
}
__device__ __forceinline__ void bar_sync(int id) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(kStageThreads) : "memory");
}

// One stage over the whole tile, in place.  pre: twiddle the inputs (inverse stage); otherwise the
// outputs (forward stage); osign = -1 conjugates the result.  All 288 threads of the block: warps
// 0..7 stage and read back, warp 8 issues the MMAs.  The two named barriers alternate per pair of
// chunks; a staging thread can be at most one pair ahead of the issuing warp, because the buffer
// it fills next is released by a commit that the issuing warp makes after the pair before.
template <int R, int R1, int LN>
__device__ void stage(Ctx& c, float2* cur, int tp, const float2* tw, bool pre, float osign, int /*nthr_emu*/) {
  typedef Geo<R> G;
  static_assert(G::BYTES == bytes(R), "shared-memory figure out of step");
  constexpr int NV = LN * R1, MT = (NV + kTileM - 1) / kTileM;
  constexpr uint32_t idesc = tc::idesc_tf32(kTileM, G::NB, false, false);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, quad = warp & 3;
  const bool producer = tid < kProducers;
  const int half = (tid >> 7) & 1, item = tid & (kItems - 1);   // which chunk of a pair, which unit of it
  if (c.failed) return;
  CVB_TCTICK_INIT();
  bool ok = true;
  for (int mt = 0; mt < MT && ok; ++mt) {
    for (int ch0 = 0; ch0 < G::NCHUNK; ch0 += 2) {
      const int bar_id = 1 + (int)(c.pairs & 1u);
      if (producer) {
        const int ch = ch0 + half;
        if (ch < G::NCHUNK) {
          Staged s;
          prepare_item<R, R1, LN>(item, cur, tp, tw, mt, ch, pre, s);
          const int b = (mt * G::NCHUNK + ch) % kNumBuf;
          // the MMAs that read this buffer three chunks ago
          if (c.commits[b] > 0) ok = ok && mbar_wait_bounded(&c.mbar[b], (c.commits[b] - 1) & 1u, kWaitLimit);
          commit_item<R>(item, c.a + b * 4 * G::A_FLOATS, s);
        }
        tc::fence_proxy_async();
        tc::fence_before_sync();
        bar_arrive(bar_id);
      } else {
        bar_sync(bar_id);
        tc::fence_after_sync();
        if (lane == 0) {
          if (c.b_pending) ok = ok && mbar_wait_bounded(&c.mbar[kNumBuf], 0, kWaitLimit);
          if (ok) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int cc = ch0 + e;
              if (cc < G::NCHUNK) {
                const int b = (mt * G::NCHUNK + cc) % kNumBuf;
                const char* ab = (const char*)(c.a + b * 4 * G::A_FLOATS);
                const uint64_t bh = tc::smem_desc((const char*)c.b_hi + cc * G::B_KSTEP, G::B_LBO, 128);
                const uint64_t bl = tc::smem_desc((const char*)c.b_lo + cc * G::B_KSTEP, G::B_LBO, 128);
#pragma unroll
                for (int part = 0; part < 2; ++part) {
                  const uint64_t ah = tc::smem_desc(ab + (2 * part) * G::A_FLOATS * 4, G::A_LBO, 128);
                  const uint64_t al = tc::smem_desc(ab + (2 * part + 1) * G::A_FLOATS * 4, G::A_LBO, 128);
                  const uint32_t d = c.tmem + (uint32_t)(part * G::NB);
                  tc::mma_tf32(d, ah, bh, idesc, cc > 0 ? 1u : 0u);
                  tc::mma_tf32(d, ah, bl, idesc, 1u);
                  tc::mma_tf32(d, al, bh, idesc, 1u);
                }
                tc::mma_commit(&c.mbar[b]);
              }
            }
          }
        }
        __syncwarp();
      }
      c.b_pending = 0;
      c.pairs += 1;
      // every thread keeps the same count of commits per buffer as the issuing thread
#pragma unroll
      for (int e = 0; e < 2; ++e)
        if (ch0 + e < G::NCHUNK) c.commits[(mt * G::NCHUNK + ch0 + e) % kNumBuf] += 1;
    }
    CVB_TCTICK(16);
    // all MMAs of this accumulator tile are done when the last commit has arrived; the issuing
    // warp joins the block barrier only after it has made that commit
    {
      const int bl = (mt * G::NCHUNK + G::NCHUNK - 1) % kNumBuf;
      if (warp == 0) ok = ok && mbar_wait_bounded(&c.mbar[bl], (c.commits[bl] - 1) & 1u, kWaitLimit);
      if (__syncthreads_or(!ok)) {
        ok = false;
        break;
      }
    }
    CVB_TCTICK(17);
    tc::fence_after_sync();
    if (producer) {
      // accumulator row 16 * quad + lane lives in lane `lane` < 16 of the warp's quadrant
      const int v = mt * kTileM + quad * 16 + (lane & 15);
      for (int g = warp >> 2; 8 * g <= G::KH; g += 2) {
        float d0[16], d1[16];
        const uint32_t ta = c.tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(16 * g);
        tmem_ld16x2(ta, ta + (uint32_t)G::NB, d0, d1);
        // lanes 16..31 hold nothing of an M = 64 accumulator: they take the upper four k of the
        // vector of lane - 16
        float e0[8], e1[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float u0 = __shfl_sync(0xffffffffu, d0[8 + i], lane & 15);
          const float u1 = __shfl_sync(0xffffffffu, d1[8 + i], lane & 15);
          e0[i] = lane < 16 ? d0[i] : u0;
          e1[i] = lane < 16 ? d1[i] : u1;
        }
        emit_group<R, R1, LN, 4>(cur, tp, tw, v, 8 * g + (lane < 16 ? 0 : 4), e0, e1, !pre, osign);
      }
    }
    tc::fence_before_sync();
    __syncthreads();   // accumulators free, tile written
    tc::fence_after_sync();
    CVB_TCTICK(18);
  }
  if (!ok) c.failed = 1;   // uniform: decided by __syncthreads_or
}
#else
// ---- host stand-ins: same steps on plain arrays ----
template <int R>
inline void setup(Ctx& c, const float*) {
  setup_table<R>(0, 1, c);
  setup_matrix<R>(0, 1, c);
}
template <int R>
inline void finish(Ctx&) {}
template <int R, int R1, int LN>
inline void stage(Ctx& c, float2* cur, int tp, const float2* tw, bool pre, float osign, int /*nthr_emu*/) {
  typedef Geo<R> G;
  constexpr int NV = LN * R1, MT = (NV + kTileM - 1) / kTileM;
  static thread_local float D[2][kTileM][256];
  for (int mt = 0; mt < MT; ++mt) {
    for (int ch = 0; ch < G::NCHUNK; ++ch) {
      float* buf = c.a + ((mt * G::NCHUNK + ch) % kNumBuf) * 4 * G::A_FLOATS;
      for (int item = 0; item < kItems; ++item) {
        Staged s;
        prepare_item<R, R1, LN>(item, cur, tp, tw, mt, ch, pre, s);
        commit_item<R>(item, buf, s);
      }
      // the "MMA": decode the operand layouts
      for (int part = 0; part < 2; ++part)
        for (int m = 0; m < kTileM; ++m)
          for (int n = 0; n < G::NB; ++n) {
            float acc = (ch == 0) ? 0.f : D[part][m][n];
            for (int kk = 0; kk < kChunkK; ++kk) {
              const int ia = operand_index(m, kk, G::A_LBO / 4, 0);
              const int ib = operand_index(n, ch * kChunkK + kk, G::B_LBO / 4, G::B_KSTEP / 4);
              const float ah = buf[(2 * part) * G::A_FLOATS + ia], al = buf[(2 * part + 1) * G::A_FLOATS + ia];
              acc += ah * c.b_hi[ib] + ah * c.b_lo[ib] + al * c.b_hi[ib];
            }
            D[part][m][n] = acc;
          }
    }
    for (int row = 0; row < kTileM; ++row) {
      for (int g = 0; 8 * g <= G::KH; ++g) {
        float d0[16], d1[16];
        for (int i = 0; i < 16; ++i) {
          d0[i] = (16 * g + i < G::NB) ? D[0][row][16 * g + i] : 0.f;
          d1[i] = (16 * g + i < G::NB) ? D[1][row][16 * g + i] : 0.f;
        }
        emit_group<R, R1, LN, 8>(cur, tp, tw, mt * kTileM + row, 8 * g, d0, d1, !pre, osign);
      }
    }
  }
}
#endif

}  // namespace tcdft
}  // namespace cvb
