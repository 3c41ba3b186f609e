// A prime-length DFT stage on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// The multi-pass kernels meet axis lengths N = R * R1 whose first radix R is a prime too large for
// a register butterfly (268 = 67 * 4 in ConverseDnCNN, 516 = 43 * 12 in ConverseUSRNet).  The R-point
// DFTs of such a stage are a dense contraction: for every "vector" (tile line c, inner index j)
//     X[k] = sum_q x[q] * exp(-2 pi i k q / R),   x[q] = tile[(q * R1 + j) * tp + c],
// so they run as one GEMM per 128 vectors.  With C[k][q] = cos(2 pi k q / R), S[k][q] = sin(..):
//     X[k]     = (C xr + S xi)[k] + i (C xi - S xr)[k]
//     X[R - k] = (C xr - S xi)[k] + i (C xi + S xr)[k],        k = 0 .. (R - 1) / 2,
// i.e. two real GEMMs D0 = Xr * B^T, D1 = Xi * B^T with the same constant operand B (rows 2k = C[k],
// 2k + 1 = S[k]) and the real / imaginary parts of the vectors as the M = 128 rows of operand A.
// All operands are fp32 split into TF32 hi + lo, three MMAs per product (hi*hi + hi*lo + lo*hi),
// which keeps fp32 accuracy (error ~2^-21 per product).
//
// Per 128 vectors: K (= q) is staged in chunks of 24 (three K = 8 MMA steps): every thread reads four
// consecutive q of its vector from the tile, applies the stage's input twiddle when the stage is an
// inverse one, splits and writes four 16-byte units in the K-major core-matrix layout; one thread
// issues 18 MMAs (two accumulators) and commits to an mbarrier; after the last chunk every warp reads
// its 32 TMEM lanes (lane = vector) 16 columns (= 8 values of k) at a time, forms X[k] and X[R - k],
// applies the output twiddle of a forward stage and writes them back into the tile in place.
// Every mbarrier wait is bounded; on a time-out the block flags the status word and carries on
// without the tensor cores' result (the caller reads the status after the launch).
//
// The host versions of the three steps run the same index arithmetic on plain arrays (the operand
// layout is decoded by the "MMA"), so that the CPU emulation of the kernels covers it.
#pragma once
#include "cvb_kernels.cuh"
#ifdef __CUDA_ARCH__
#include "cvb_tc.cuh"
#endif

namespace cvb {
namespace tcdft {

constexpr int kChunkK = 24;      // q values staged per chunk (three MMA K-steps)
constexpr int kTileM = 128;      // vectors per accumulator (MMA M)
constexpr int kTmemCols = 256;   // two accumulators of up to 128 columns

template <int R>
struct Geo {
  static constexpr int KH = (R - 1) / 2;                        // k = 0 .. KH are computed, R - k follow
  static constexpr int NB = ((2 * (KH + 1) + 15) / 16) * 16;    // rows of B = accumulator columns
  static constexpr int KP = ((R + kChunkK - 1) / kChunkK) * kChunkK;  // q padded to whole chunks
  static constexpr int NCHUNK = KP / kChunkK;
  // operand B: K-major, no swizzle: 8-row groups 128 B apart, the two 4-wide K halves LBO apart
  static constexpr int B_LBO = (NB / 8) * 128, B_KSTEP = 2 * B_LBO;   // bytes
  static constexpr int B_FLOATS = (KP / 8) * (B_KSTEP / 4);           // one array (hi or lo)
  // operand A (one chunk): 16 row groups
  static constexpr int A_LBO = (kTileM / 8) * 128, A_KSTEP = 2 * A_LBO;
  static constexpr int A_FLOATS = (kChunkK / 8) * (A_KSTEP / 4);      // one of the four arrays
  static constexpr size_t BYTES = (size_t)(2 * B_FLOATS + 4 * A_FLOATS + 2 * R) * sizeof(float) + 64;
};

// shared memory of the stage for a prime R (same figure as Geo<R>::BYTES)
CVB_HD constexpr size_t bytes(int R) {
  const int kh = (R - 1) / 2, nb = ((2 * (kh + 1) + 15) / 16) * 16;
  const int kp = ((R + kChunkK - 1) / kChunkK) * kChunkK;
  const int b_floats = (kp / 8) * (2 * (nb / 8) * 128 / 4);
  const int a_floats = (kChunkK / 8) * (2 * (kTileM / 8) * 128 / 4);
  return (size_t)(2 * b_floats + 4 * a_floats + 2 * R) * sizeof(float) + 64;
}

// Views into the block's shared memory (base 128-byte aligned).
struct Ctx {
  float* b_hi; float* b_lo;        // constant operand
  float* a[4];                     // xr hi, xr lo, xi hi, xi lo of the current chunk
  float* cs;                       // cos / sin (2 pi m / R), m < R: [2m], [2m + 1]
  uint64_t* mbar;
  uint32_t* tmem_holder;
  uint32_t tmem;                   // accumulator base (device)
  uint32_t parity;
  int failed;
  int* status;
#ifndef __CUDA_ARCH__
  float* d_emu;                    // host: the two accumulators [2][128][NB]
#endif
};

template <int R>
CVB_HD Ctx carve(void* base, int* status) {
  typedef Geo<R> G;
  Ctx c;
  float* f = (float*)base;
  c.b_hi = f; f += G::B_FLOATS;
  c.b_lo = f; f += G::B_FLOATS;
  for (int i = 0; i < 4; ++i) { c.a[i] = f; f += G::A_FLOATS; }
  c.cs = f; f += 2 * R;
  c.mbar = (uint64_t*)(((uintptr_t)f + 7) & ~(uintptr_t)7);
  c.tmem_holder = (uint32_t*)(c.mbar + 1);
  c.tmem = 0; c.parity = 0; c.failed = 0; c.status = status;
#ifndef __CUDA_ARCH__
  c.d_emu = nullptr;
#endif
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

// cos / sin table, first step of the set-up (one thread per m)
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

// Stage chunk `ch` of the vectors mt * 128 .. + 127 (vector v = j * LN + c).
template <int R, int R1, int LN>
CVB_HD void stage_chunk(int tid, int nthr, const Ctx& c, const float2* cur, int tp, const float2* tw, int mt,
                        int ch, bool pre) {
  typedef Geo<R> G;
  constexpr int NV = LN * R1;
  for (int item = tid; item < kTileM * (kChunkK / 4); item += nthr) {
    const int m = item & (kTileM - 1), qq = item / kTileM;
    const int v = mt * kTileM + m;
    const int j = v / LN, cc = v - j * LN;
    float rh[4], rl[4], ih[4], il[4];
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
      split_hi_lo(x.x, rh[e], rl[e]);
      split_hi_lo(x.y, ih[e], il[e]);
    }
    const int idx = operand_index(m, qq * 4, G::A_LBO / 4, G::A_KSTEP / 4);
    *(float4*)(c.a[0] + idx) = make_float4(rh[0], rh[1], rh[2], rh[3]);
    *(float4*)(c.a[1] + idx) = make_float4(rl[0], rl[1], rl[2], rl[3]);
    *(float4*)(c.a[2] + idx) = make_float4(ih[0], ih[1], ih[2], ih[3]);
    *(float4*)(c.a[3] + idx) = make_float4(il[0], il[1], il[2], il[3]);
  }
}

// Outputs of the vectors of accumulator tile `mt`: thread (warp quadrant, lane) = vector, the warp's
// group index walks over the values of k eight at a time.  d0 / d1: 16 accumulator columns of the
// group (C xr, S xr interleaved; C xi, S xi interleaved).
template <int R, int R1, int LN>
CVB_HD void emit_group(float2* cur, int tp, const float2* tw, int v, int g, const float (&d0)[16],
                       const float (&d1)[16], bool post, float osign) {
  typedef Geo<R> G;
  constexpr int NV = LN * R1;
  if (v >= NV) return;
  const int j = v / LN, cc = v - j * LN;
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const int k = 8 * g + kk;
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

#ifdef __CUDA_ARCH__
// 32 lanes x 16 columns of fp32
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
}

// Block set-up: table, constant operand, mbarrier, TMEM.  All threads; ends with a barrier.
template <int R>
__device__ void setup(Ctx& c) {
  const int tid = threadIdx.x, nthr = blockDim.x;
  setup_table<R>(tid, nthr, c);
  if (tid == 0) {
    mbar_init(c.mbar, 1);
    mbar_fence_init();
  }
  if (tid < 32) tc::tmem_alloc(c.tmem_holder, kTmemCols);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  c.tmem = *c.tmem_holder;
  setup_matrix<R>(tid, nthr, c);
  tc::fence_proxy_async();
  __syncthreads();
}
// Release the accumulators and report a time-out.  All threads, after the block's last stage.
__device__ __forceinline__ void finish(Ctx& c) {
  tc::fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) tc::tmem_dealloc(c.tmem, kTmemCols);
  if (c.failed && threadIdx.x == 0 && c.status) atomicExch(c.status, 3);
}

// One stage over the whole tile, in place.  pre: twiddle the inputs (inverse stage); otherwise the
// outputs (forward stage); osign = -1 conjugates the result.  All threads of the block.
template <int R, int R1, int LN>
__device__ void stage(Ctx& c, float2* cur, int tp, const float2* tw, bool pre, float osign, int /*nthr_emu*/) {
  typedef Geo<R> G;
  static_assert(G::BYTES == bytes(R), "shared-memory figure out of step");
  constexpr int NV = LN * R1, MT = (NV + kTileM - 1) / kTileM;
  constexpr uint32_t idesc = tc::idesc_tf32(kTileM, G::NB, false, false);
  const int tid = threadIdx.x, nthr = blockDim.x, warp = tid >> 5, lane = tid & 31, quad = warp & 3;
  if (c.failed) return;
  for (int mt = 0; mt < MT; ++mt) {
    for (int ch = 0; ch < G::NCHUNK; ++ch) {
      stage_chunk<R, R1, LN>(tid, nthr, c, cur, tp, tw, mt, ch, pre);
      tc::fence_proxy_async();
      tc::fence_before_sync();
      __syncthreads();
      if (tid == 0) {
        tc::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < kChunkK / 8; ++ks) {
          const int kg = ch * (kChunkK / 8) + ks;
          const uint64_t bh = tc::smem_desc((const char*)c.b_hi + kg * G::B_KSTEP, G::B_LBO, 128);
          const uint64_t bl = tc::smem_desc((const char*)c.b_lo + kg * G::B_KSTEP, G::B_LBO, 128);
#pragma unroll
          for (int part = 0; part < 2; ++part) {
            const uint64_t ah = tc::smem_desc((const char*)c.a[2 * part] + ks * G::A_KSTEP, G::A_LBO, 128);
            const uint64_t al = tc::smem_desc((const char*)c.a[2 * part + 1] + ks * G::A_KSTEP, G::A_LBO, 128);
            const uint32_t d = c.tmem + (uint32_t)(part * G::NB);
            tc::mma_tf32(d, ah, bh, idesc, kg > 0 ? 1u : 0u);
            tc::mma_tf32(d, ah, bl, idesc, 1u);
            tc::mma_tf32(d, al, bh, idesc, 1u);
          }
        }
        tc::mma_commit(c.mbar);
      }
      const bool ok = mbar_wait_bounded(c.mbar, c.parity, kWaitLimit);
      c.parity ^= 1u;
      if (__syncthreads_or(!ok)) {   // the operand buffers are free again, or the wait ran out
        c.failed = 1;
        return;
      }
    }
    tc::fence_after_sync();
    const int v = mt * kTileM + quad * 32 + lane;
    for (int g = warp >> 2; 8 * g <= G::KH; g += nthr >> 7) {
      float d0[16], d1[16];
      const uint32_t ta = c.tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(16 * g);
      tmem_ld16(ta, d0);
      tmem_ld16(ta + (uint32_t)G::NB, d1);
      emit_group<R, R1, LN>(cur, tp, tw, v, g, d0, d1, !pre, osign);
    }
    tc::fence_before_sync();
    __syncthreads();   // accumulators free, tile written
    tc::fence_after_sync();
  }
}
#else
// ---- host stand-ins: same steps on plain arrays ----
template <int R>
inline void setup(Ctx& c) {
  setup_table<R>(0, 1, c);
  setup_matrix<R>(0, 1, c);
}
inline void finish(Ctx&) {}
template <int R, int R1, int LN>
inline void stage(Ctx& c, float2* cur, int tp, const float2* tw, bool pre, float osign, int nthr_emu) {
  typedef Geo<R> G;
  constexpr int NV = LN * R1, MT = (NV + kTileM - 1) / kTileM;
  static thread_local float D[2][kTileM][256];
  for (int mt = 0; mt < MT; ++mt) {
    for (int ch = 0; ch < G::NCHUNK; ++ch) {
      for (int tid = 0; tid < nthr_emu; ++tid) stage_chunk<R, R1, LN>(tid, nthr_emu, c, cur, tp, tw, mt, ch, pre);
      // the "MMA": decode the operand layouts
      for (int part = 0; part < 2; ++part)
        for (int m = 0; m < kTileM; ++m)
          for (int n = 0; n < G::NB; ++n) {
            float acc = (ch == 0) ? 0.f : D[part][m][n];
            for (int kk = 0; kk < kChunkK; ++kk) {
              const int ia = operand_index(m, kk, G::A_LBO / 4, G::A_KSTEP / 4);
              const int ib = operand_index(n, ch * kChunkK + kk, G::B_LBO / 4, G::B_KSTEP / 4);
              const float ah = c.a[2 * part][ia], al = c.a[2 * part + 1][ia];
              acc += ah * c.b_hi[ib] + ah * c.b_lo[ib] + al * c.b_hi[ib];
            }
            D[part][m][n] = acc;
          }
    }
    for (int tid = 0; tid < kTileM * 4; ++tid) {   // sixteen warps' worth of (quadrant, group) pairs
      const int warp = tid >> 5, lane = tid & 31, quad = warp & 3;
      const int v = mt * kTileM + quad * 32 + lane;
      for (int g = warp >> 2; 8 * g <= G::KH; g += 4) {
        float d0[16], d1[16];
        for (int i = 0; i < 16; ++i) {
          d0[i] = D[0][quad * 32 + lane][16 * g + i];
          d1[i] = D[1][quad * 32 + lane][16 * g + i];
        }
        emit_group<R, R1, LN>(cur, tp, tw, v, g, d0, d1, !pre, osign);
      }
    }
  }
}
#endif

}  // namespace tcdft
}  // namespace cvb
