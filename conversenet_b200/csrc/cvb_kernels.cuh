// Per-thread building blocks of the Converse2D forward kernels.
//
// Everything here is written as `__host__ __device__` functions of an explicit
// (tid, nthr) pair, and each kernel body is a sequence of CVB_PHASE(...) steps
// separated by block barriers.  Compiled for the device a phase runs once per
// thread followed by __syncthreads(); compiled for the host (test builds only)
// a phase is a loop over tid, so the index arithmetic of a whole block can be
// checked on a machine without a GPU.
//
// Math.  For one plane y = pad(x) of size h x w (models/util_converse.py:144-145)
// the reference's solve (:171-187) is linear in y and collapses to
//     s == 1 :  out = crop( IFFT2( G . FFT2(y) ) ),  G = (conj(FK)+lam) / (|FK|^2+lam)
//     s >= 2 :  r   = IFFT2( P . FFT2(y) ),          P = (1 - fold_s(FK.D)) / (fold_s(|FK|^2)+lam)
//               out = crop( nearest_s(y) + corr(K, zero_insert_s(r)) )
// with FK the kernel spectrum on the s*h x s*w grid (:218-235), D the spectrum of
// the s x s box that turns zero-insertion into nearest-upsampling, fold_s the
// mean over the s*s aliases (:182-183) and lam = sigmoid(bias-9)+eps (:147).
// Both FFTs are h x w whatever the scale.  Two planes that share a kernel (same
// channel, two batch entries) travel as the real and imaginary part of one
// complex plane: G and P are spectra of real filters, so the two never mix.
//
// FFT.  In-place mixed radix, decimation in frequency forward (natural order in,
// digit-reversed out) and decimation in time inverse (digit-reversed in, natural
// out); the transfer table is stored in digit-reversed order so nothing is ever
// permuted.  A stage with sub-length L, radix R, M = L/R handles butterfly
// t -> (blk = t / M, j = t % M) on elements blk*L + j + q*M.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>

#define CVB_HD __host__ __device__ __forceinline__
#include "fft_codelets.cuh"
#include "cvb_tma.cuh"

namespace cvb {

constexpr int kMaxStages = 8;
constexpr int kMaxTaps = 15;  // largest kernel_size the epilogue keeps in shared memory

struct Plan1D {
  int n;
  int nst;
  int radix[kMaxStages];
  int L[kMaxStages];  // sub-transform length entering stage i
  int M[kMaxStages];  // L / radix
  int gemm;           // 1: plan {n / 4, 4} of the tensor-core multi-pass kernels (cvb_gemmdft.cuh)
};

struct FwdParams {
  const void* x;
  void* out;
  const float2* table;  // [C][w][h] multiplier (transposed, digit-reversed), then twiddles
  const float* weight;  // (C,k,k), read when s > 1
  int B, C, H, W, k, s, p, pad_mode, fuse_gelu;
  int h, w, pitch;
  int skip_mask;  // tuning aid: bit i set = phase i is not executed (results are then wrong)
  int ystash;     // 1: shared memory also keeps the padded input (x0 of the s > 1 epilogue)
  int* status;    // device word set non-zero when a bounded wait gives up; may be null
  Plan1D py, px;
};

struct PassArgs {
  float2* sm;
  int es, ls, nlines;  // element stride, line stride (float2 units), number of lines
  int N, L, M, tws;    // transform length, stage sub-length, L/R, twiddle stride N/L
  const float2* tw;    // tw[n] = (cos, sin)(2 pi n / N)
  float inv_nlines, invM;
  int nl1, ls2;        // nl1 > 0: lines form a 2-level grid, line -> (line % nl1) * ls + (line / nl1) * ls2
  float inv_nl1;
  const float2* tab;   // PASS_MID multiplier when not the per-channel transfer table (else null)
  int tab_es, tab_ls;  //   its strides along the transform axis / across lines
};

struct IoArgs {
  const void* xa;
  const void* xb;  // second plane of the pair, may be null
  void* oa;
  void* ob;
  int H, W, p, pad_mode, gelu, h, w;
  const float2* tab;  // this channel's multiplier
  const int* rmap;    // padded row -> source row * W, or -1 (zero)
  const int* cmap;    // padded column -> source column, or -1 (zero)
  float2* ycopy;      // padded input of both planes, same layout as the FFT plane; null if not kept
  float2* ws;         // multi-pass workspace of this block's lines (PASS_SRC_WS / PASS_DST_WS)
  int wes, wls;       //   its element stride along the transform axis / stride between lines
  int xoff;           // plane column of line 0 (PASS_DST_GLOBAL of a column strip)
  int yoff;           // ycopy - plane, in float2 units
};

// ---------------------------------------------------------------- helpers
// Plain generic loads: the persistent kernel hands these functions its shared-memory prefetch buffers
// as well as global planes, so no global-only form (ld.global.nc / __ldg) may be used here.
template <typename IO> CVB_HD float ld_io(const void* p, size_t i);
template <> CVB_HD float ld_io<float>(const void* p, size_t i) {
  return ((const float*)p)[i];
}
template <> CVB_HD float ld_io<__nv_bfloat16>(const void* p, size_t i) {
  return __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
template <typename IO> CVB_HD void st_io(void* p, size_t i, float v);
template <> CVB_HD void st_io<float>(void* p, size_t i, float v) { ((float*)p)[i] = v; }
template <> CVB_HD void st_io<__nv_bfloat16>(void* p, size_t i, float v) {
  ((__nv_bfloat16*)p)[i] = __float2bfloat16(v);
}

CVB_HD float bf16_bits_to_float(unsigned short b) {
  const uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

// Exact (erf) GELU, branch-free: with t = |v| / sqrt(2), erfc(t) = 2^(-t * q(t)), q a degree-7 polynomial
// fitted to -log2(erfc(t)) / t on [0, 4.4] (absolute error of erfc below 6e-8, clamped beyond, where
// erfc < 5e-10);  Phi(v) = 1 - erfc(t) / 2 for v >= 0 and erfc(t) / 2 for v < 0.  Against the fp64 erf
// formula the result is within 3.9e-7 on [-6, 6], the rounding of the fp32 product itself, at about half
// the instructions of erff (no divergent branch).
CVB_HD float gelu_erf(float v) {
  const float t = fminf(fabsf(v) * 0.70710678118654752440f, 4.4f);
  float q = 3.7796224119226001e-05f;
  q = fmaf(q, t, -3.8324893763594527e-04f);
  q = fmaf(q, t, 1.2864194185710442e-03f);
  q = fmaf(q, t, 1.1106310484120274e-03f);
  q = fmaf(q, t, -2.8553848453755075e-02f);
  q = fmaf(q, t, 1.4862335641232380e-01f);
  q = fmaf(q, t, 9.1838461344425293e-01f);
  q = fmaf(q, t, 1.6279110826289691e+00f);
  const float half_erfc = 0.5f * exp2f(-q * t);
  return v * (v >= 0.f ? 1.0f - half_erfc : half_erfc);
}

#ifdef __CUDA_ARCH__
// Two GELUs at once: the polynomial, the product with t and the final product run on packed pairs
// (fma / mul .f32x2); |v|, the clamp, the two exp2 and the sign select stay per value.  Same polynomial
// and the same result as gelu_erf up to the rounding of the fused steps.
__device__ __forceinline__ float2 gelu_erf2(float vx, float vy) {
  const float tx = fminf(fabsf(vx) * 0.70710678118654752440f, 4.4f);
  const float ty = fminf(fabsf(vy) * 0.70710678118654752440f, 4.4f);
  const p2 t = p2_pack(tx, ty);
  p2 q = p2_pack(3.7796224119226001e-05f, 3.7796224119226001e-05f);
  q = p2_fma(q, t, p2_pack(-3.8324893763594527e-04f, -3.8324893763594527e-04f));
  q = p2_fma(q, t, p2_pack(1.2864194185710442e-03f, 1.2864194185710442e-03f));
  q = p2_fma(q, t, p2_pack(1.1106310484120274e-03f, 1.1106310484120274e-03f));
  q = p2_fma(q, t, p2_pack(-2.8553848453755075e-02f, -2.8553848453755075e-02f));
  q = p2_fma(q, t, p2_pack(1.4862335641232380e-01f, 1.4862335641232380e-01f));
  q = p2_fma(q, t, p2_pack(9.1838461344425293e-01f, 9.1838461344425293e-01f));
  q = p2_fma(q, t, p2_pack(1.6279110826289691e+00f, 1.6279110826289691e+00f));
  float ex, ey;
  p2_unpack(p2_mul(q, p2_mul(t, p2_pack(-1.0f, -1.0f))), ex, ey);   // -q t
  const float hx = 0.5f * exp2f(ex), hy = 0.5f * exp2f(ey);         // erfc / 2
  const p2 phi = p2_pack(vx >= 0.f ? 1.0f - hx : hx, vy >= 0.f ? 1.0f - hy : hy);
  float ox, oy;
  p2_unpack(p2_mul(p2_pack(vx, vy), phi), ox, oy);
  return make_float2(ox, oy);
}
#endif

// GELU of the two planes' values of one output position
CVB_HD void gelu_pair(float& a, float& b) {
#ifdef __CUDA_ARCH__
  const float2 g = gelu_erf2(a, b);
  a = g.x; b = g.y;
#else
  a = gelu_erf(a); b = gelu_erf(b);
#endif
}

// Index into the unpadded axis of length n for padded coordinate i (already
// shifted by -p), or -1 where constant padding supplies a zero.
CVB_HD int pad_index(int i, int n, int mode) {
  if (i >= 0 && i < n) return i;
  switch (mode) {
    case 0: return i < 0 ? i + n : i - n;           // circular
    case 1: return i < 0 ? 0 : n - 1;               // replicate
    case 2: return i < 0 ? -i : 2 * n - 2 - i;      // reflect
    default: return -1;                             // constant
  }
}

// wi -> (wi / d, wi % d) for small non-negative wi without an integer divide
CVB_HD void divmod_small(int wi, int d, float inv_d, int& q, int& r) {
  q = (int)((float)wi * inv_d);
  r = wi - q * d;
  if (r < 0) { r += d; --q; } else if (r >= d) { r -= d; ++q; }
}

// Position in the digit-reversed array -> frequency index.
CVB_HD int pos_to_freq(const Plan1D& pl, int pos) {
  int k = 0, mult = 1;
  for (int i = 0; i < pl.nst; ++i) {
    const int d = (pos / pl.M[i]) % pl.radix[i];
    k += d * mult;
    mult *= pl.radix[i];
  }
  return k;
}

// ---------------------------------------------------------------- one FFT stage
// One routine serves every stage of a kernel, selected by run-time flags, so that
// each butterfly is present once in the instruction stream (the kernels are
// instruction-cache bound otherwise).  All butterflies use the forward kernel:
//   forward stage (decimation in frequency): butterfly, then twiddle;
//   inverse stage (decimation in time)     : twiddle, then butterfly, applied to
//     the conjugated spectrum -- IDFT(W) = conj(DFT(conj(W))).  The conjugation
//     happens once in the PASS_MID stage and once at the final store (PASS_CONJ_OUT).
enum {
  PASS_PRE = 1,         // twiddle before the butterfly (inverse-type stage)
  PASS_SRC_GLOBAL = 2,  // first column stage: read x through the pad maps
  PASS_DST_GLOBAL = 4,  // last column stage at scale 1: crop and write out
  PASS_MID = 8,         // last row stage: butterfly, transfer multiply, conjugate, butterfly
  PASS_CONJ_OUT = 16,   // negate the imaginary part on the way out
  PASS_SRC_WS = 32,     // read the complex elements from a global workspace (io.ws, strides wes / wls)
  PASS_DST_WS = 64      // write them to the workspace instead of shared memory
};

// Transfer-table values of work item wi of a PASS_MID stage (same index arithmetic as fft_pass).
template <int R, int CN, int CL, int CM, int CNL>
CVB_HD void mid_table_load(const PassArgs& a, const IoArgs& io, int wi, float2 (&g)[R]) {
  int t, line;
  if constexpr (CNL != 0) {
    t = wi / CNL;
    line = wi - t * CNL;
  } else {
    divmod_small(wi, a.nlines, a.inv_nlines, t, line);
  }
  const int tes = a.tab ? a.tab_es : io.h;
  const float2* tp = a.tab ? a.tab + (t * R) * a.tab_es + line * a.tab_ls
                           : io.tab + (size_t)(t * R) * io.h + line;
#pragma unroll
  for (int p = 0; p < R; ++p) g[p] = tp[(size_t)p * tes];
}

// CN, CL, CM, CNL: compile-time transform length, stage sub-length, L/R and line
// count (0 = take the run-time value from PassArgs); strides stay run-time so that
// the row and the column stage of a square plane share one instantiation.
template <int R, typename IO, int CN = 0, int CL = 0, int CM = 0, int CNL = 0, int CFLAGS = -1>
CVB_HD void fft_pass(int tid, int nthr, const PassArgs& a, const IoArgs& io, int rt_flags) {
  const int flags = CFLAGS >= 0 ? CFLAGS : rt_flags;  // compile-time flags when given
  const int aN = CN ? CN : a.N, aL = CL ? CL : a.L, aM = CM ? CM : a.M, anl = CNL ? CNL : a.nlines;
  const int atws = CN ? CN / (CL ? CL : 1) : a.tws;
  const int nbf = aN / R;
  const int total = nbf * anl;
  const int nrep = (flags & PASS_MID) ? 2 : 1;
  const float osign = (flags & PASS_CONJ_OUT) ? -1.0f : 1.0f;
  const bool twiddle = aM > 1;
  constexpr bool kMidStatic = CFLAGS >= 0 && (CFLAGS & PASS_MID) != 0;
  float2 gtab[kMidStatic ? R : 1], gnext[kMidStatic ? R : 1];
  if constexpr (kMidStatic) {
    if (tid < total) mid_table_load<R, CN, CL, CM, CNL>(a, io, tid, gnext);
  }
  for (int wi = tid; wi < total; wi += nthr) {
    int t, line, blk, j;
    if constexpr (CNL != 0) {
      t = wi / CNL;
      line = wi - t * CNL;
      blk = t / CM;
      j = t - blk * CM;
    } else {
      divmod_small(wi, a.nlines, a.inv_nlines, t, line);
      divmod_small(t, a.M, a.invM, blk, j);
    }
    const int base = blk * aL + j;
    int loff = line * a.ls;
    if (a.nl1 > 0) {
      int l2, l1;
      divmod_small(line, a.nl1, a.inv_nl1, l2, l1);
      loff = l1 * a.ls + l2 * a.ls2;
    }
    float2* ptr = a.sm + loff + base * a.es;
    const int st = aM * a.es;
    const int tstep = j * atws;
    float re[R], im[R];
    // transfer-table values (global memory) are fetched one work item ahead, so that their
    // latency overlaps this item's shared-memory traffic and butterflies
    if constexpr (kMidStatic) {
#pragma unroll
      for (int p = 0; p < R; ++p) gtab[p] = gnext[p];
      const int wn = wi + nthr;
      if (wn < total) mid_table_load<R, CN, CL, CM, CNL>(a, io, wn, gnext);
    }

    if (flags & PASS_SRC_GLOBAL) {
      // rows base + q*M of padded column `line`, straight from x
      const int cx = io.cmap[line];
      if constexpr (sizeof(IO) == 2) {
        // bf16: all 16-bit loads first, the widening to fp32 afterwards, so that every load of the
        // item is in flight before the first use
        unsigned short ra[R], rb[R];
#pragma unroll
        for (int q = 0; q < R; ++q) {
          const int ro = io.rmap[base + q * aM];
          ra[q] = 0; rb[q] = 0;
          if ((cx | ro) >= 0) {
            const size_t off = (size_t)(ro + cx);
            ra[q] = ((const unsigned short*)io.xa)[off];
            if (io.xb) rb[q] = ((const unsigned short*)io.xb)[off];
          }
        }
#pragma unroll
        for (int q = 0; q < R; ++q) {
          re[q] = bf16_bits_to_float(ra[q]);
          im[q] = bf16_bits_to_float(rb[q]);
        }
      } else {
#pragma unroll
        for (int q = 0; q < R; ++q) {
          const int ro = io.rmap[base + q * aM];
          float va = 0.f, vb = 0.f;
          if ((cx | ro) >= 0) {
            const size_t off = (size_t)(ro + cx);
            va = ld_io<IO>(io.xa, off);
            if (io.xb) vb = ld_io<IO>(io.xb, off);
          }
          re[q] = va;
          im[q] = vb;
        }
      }
      if (io.ycopy) {  // after all loads are in flight
#pragma unroll
        for (int q = 0; q < R; ++q) ptr[io.yoff + q * st] = make_float2(re[q], im[q]);
      }
    } else if (flags & PASS_SRC_WS) {
      const float2* gp = io.ws + (size_t)line * io.wls + (size_t)base * io.wes;
#pragma unroll
      for (int q = 0; q < R; ++q) {
        const float2 v = gp[(size_t)(q * aM) * io.wes];
        re[q] = v.x;
        im[q] = v.y;
      }
    } else {
#pragma unroll
      for (int q = 0; q < R; ++q) {
        const float2 v = ptr[q * st];
        re[q] = v.x;
        im[q] = v.y;
      }
    }

    if ((flags & PASS_PRE) && twiddle) {
#pragma unroll
      for (int p = 1; p < R; ++p) {
        const float2 wv = a.tw[tstep * p];
        const float xr = re[p], xi = im[p];
        re[p] = fmaf(xi, wv.y, xr * wv.x);
        im[p] = fmaf(-xr, wv.y, xi * wv.x);
      }
    }

#pragma unroll 1
    for (int rep = 0; rep < nrep; ++rep) {
      Radix<R>::fwd(re, im);
      if ((flags & PASS_MID) && rep == 0) {
        // multiply by the transfer table and conjugate: the inverse runs on conj(spectrum)
        const int tes = a.tab ? a.tab_es : io.h;
        const float2* tp = a.tab ? a.tab + (t * R) * a.tab_es + line * a.tab_ls
                                 : io.tab + (size_t)(t * R) * io.h + line;
#pragma unroll
        for (int p = 0; p < R; ++p) {
          float2 g;
          if constexpr (kMidStatic) g = gtab[p];
          else g = tp[(size_t)p * tes];
          const float xr = re[p], xi = im[p];
          re[p] = fmaf(-xi, g.y, xr * g.x);
          im[p] = -fmaf(xr, g.y, xi * g.x);
        }
      }
    }

    if (!(flags & (PASS_PRE | PASS_MID)) && twiddle) {
#pragma unroll
      for (int p = 1; p < R; ++p) {
        const float2 wv = a.tw[tstep * p];
        const float xr = re[p], xi = im[p];
        re[p] = fmaf(xi, wv.y, xr * wv.x);
        im[p] = fmaf(-xr, wv.y, xi * wv.x);
      }
    }

    if (flags & PASS_DST_GLOBAL) {
      // crop and write both planes (column `line`, rows base + q*M)
      const int ox = line + io.xoff - io.p;
      if (ox >= 0 && ox < io.W) {
#pragma unroll
        for (int q = 0; q < R; ++q) {
          const int oy = base + q * aM - io.p;
          if (oy >= 0 && oy < io.H) {
            const size_t off = (size_t)oy * io.W + ox;
            float va = re[q], vb = osign * im[q];
            if (io.gelu) gelu_pair(va, vb);
            st_io<IO>(io.oa, off, va);
            if (io.ob) st_io<IO>(io.ob, off, vb);
          }
        }
      }
    } else if (flags & PASS_DST_WS) {
      float2* gp = io.ws + (size_t)line * io.wls + (size_t)base * io.wes;
#pragma unroll
      for (int q = 0; q < R; ++q) gp[(size_t)(q * aM) * io.wes] = make_float2(re[q], osign * im[q]);
    } else {
#pragma unroll
      for (int q = 0; q < R; ++q) ptr[q * st] = make_float2(re[q], osign * im[q]);
    }
  }
}

template <typename IO>
CVB_HD void run_pass(int R, int tid, int nthr, const PassArgs& a, const IoArgs& io, int flags) {
  switch (R) {
#define CVB_X(RR) \
  case RR: fft_pass<RR, IO>(tid, nthr, a, io, flags); break;
    CVB_FOR_EACH_RADIX(CVB_X)
#undef CVB_X
    default: break;
  }
}

CVB_HD PassArgs make_pass(float2* sm, bool along_y, int pitch, int h, int w, int N, int L, int M,
                          const float2* tw) {
  PassArgs a;
  a.sm = sm;
  a.es = along_y ? pitch : 1;
  a.ls = along_y ? 1 : pitch;
  a.nlines = along_y ? w : h;
  a.N = N;
  a.L = L;
  a.M = M;
  a.tws = N / L;
  a.tw = tw;
  a.inv_nlines = 1.0f / (float)a.nlines;
  a.invM = 1.0f / (float)M;
  a.nl1 = 0; a.ls2 = 0; a.inv_nl1 = 0.f;
  a.tab = nullptr; a.tab_es = 0; a.tab_ls = 0;
  return a;
}

// ---------------------------------------------------------------- s >= 2 epilogue
// out[i][j] = y[i/s][j/s] + sum_{a,b} K[a][b] * Z[i+a-c][j+b-c],  Z = zero-insert of r,
// c = k/2, on the s*h x s*w circular grid, cropped to [p*s, s*h - p*s).  `sm` holds r
// for both planes (x: plane a, y: plane b).  One thread per low-resolution cell.
CVB_HD int floordiv(int a, int b) { return (a >= 0) ? a / b : -((-a + b - 1) / b); }

template <typename IO>
CVB_HD void epilogue_generic(int tid, int nthr, const float2* sm, const float* wk, const FwdParams& P,
                             const IoArgs& io) {
  const int s = P.s, k = P.k, c = P.k / 2, p = P.p, h = P.h, w = P.w;
  const int cells = P.H * P.W;
  const int oW = P.W * s;
  const float invW = 1.0f / (float)P.W;
  for (int ci = tid; ci < cells; ci += nthr) {
    int my, mx;
    divmod_small(ci, P.W, invW, my, mx);
    const size_t xoff = (size_t)my * P.W + mx;
    float ya, yb;
    if (io.ycopy) {
      const float2 v = io.ycopy[(my + p) * P.pitch + mx + p];
      ya = v.x; yb = v.y;
    } else {
      ya = ld_io<IO>(io.xa, xoff);
      yb = io.xb ? ld_io<IO>(io.xb, xoff) : 0.f;
    }
    const int m = my + p, n = mx + p;
    for (int da = 0; da < s; ++da) {
      for (int db = 0; db < s; ++db) {
        float acca = ya, accb = yb;
        for (int a = 0; a < k; ++a) {
          const int ii = da + a - c;
          if (ii - floordiv(ii, s) * s != 0) continue;
          int rm = m + floordiv(ii, s);
          rm %= h; if (rm < 0) rm += h;
          for (int b = 0; b < k; ++b) {
            const int jj = db + b - c;
            if (jj - floordiv(jj, s) * s != 0) continue;
            int rn = n + floordiv(jj, s);
            rn %= w; if (rn < 0) rn += w;
            const float2 rv = sm[rm * P.pitch + rn];
            const float kv = wk[a * k + b];
            acca = fmaf(kv, rv.x, acca);
            accb = fmaf(kv, rv.y, accb);
          }
        }
        if (io.gelu) gelu_pair(acca, accb);
        const size_t off = (size_t)(my * s + da) * oW + (size_t)(mx * s + db);
        st_io<IO>(io.oa, off, acca);
        if (io.ob) st_io<IO>(io.ob, off, accb);
      }
    }
  }
}

// Store n consecutive outputs of one row; 16-byte vector stores when `vec`.
template <typename IO, int N>
CVB_HD void store_run(void* base, size_t off, const float (&v)[N], bool vec, int nvalid);
template <int N>
CVB_HD void store_run_f32(void* base, size_t off, const float (&v)[N], bool vec, int nvalid) {
  float* o = (float*)base + off;
  if constexpr (N % 4 == 0) {
    if (vec) {
#pragma unroll
      for (int i = 0; i < N; i += 4) {
#ifdef __CUDA_ARCH__
        __stcs((float4*)(o + i), make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]));   // written once, read by a later kernel
#else
        *(float4*)(o + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
#endif
      }
      return;
    }
  }
#pragma unroll
  for (int i = 0; i < N; ++i)
    if (i < nvalid) o[i] = v[i];
}
template <int N>
CVB_HD void store_run_bf16(void* base, size_t off, const float (&v)[N], bool vec, int nvalid) {
  __nv_bfloat16* o = (__nv_bfloat16*)base + off;
  if constexpr (N % 4 == 0 && N % 8 != 0) {
    if (vec) {   // 8-byte pieces: a warp still writes one contiguous run of an output row
#pragma unroll
      for (int i = 0; i < N; i += 4) {
        __nv_bfloat162 h0 = __floats2bfloat162_rn(v[i], v[i + 1]);
        __nv_bfloat162 h1 = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
        uint2 u;
        u.x = *(unsigned*)&h0; u.y = *(unsigned*)&h1;
        *(uint2*)(o + i) = u;
      }
      return;
    }
  }
  if constexpr (N % 8 == 0) {
    if (vec) {
#pragma unroll
      for (int i = 0; i < N; i += 8) {
        __nv_bfloat162 h0 = __floats2bfloat162_rn(v[i], v[i + 1]);
        __nv_bfloat162 h1 = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[i + 4], v[i + 5]);
        __nv_bfloat162 h3 = __floats2bfloat162_rn(v[i + 6], v[i + 7]);
        uint4 u;
        u.x = *(unsigned*)&h0; u.y = *(unsigned*)&h1; u.z = *(unsigned*)&h2; u.w = *(unsigned*)&h3;
        *(uint4*)(o + i) = u;
      }
      return;
    }
  }
#pragma unroll
  for (int i = 0; i < N; ++i)
    if (i < nvalid) o[i] = __float2bfloat16(v[i]);
}
template <> CVB_HD void store_run<float, 4>(void* b, size_t o, const float (&v)[4], bool vec, int n) { store_run_f32<4>(b, o, v, vec, n); }
template <> CVB_HD void store_run<float, 6>(void* b, size_t o, const float (&v)[6], bool vec, int n) { store_run_f32<6>(b, o, v, vec, n); }
template <> CVB_HD void store_run<float, 8>(void* b, size_t o, const float (&v)[8], bool vec, int n) { store_run_f32<8>(b, o, v, vec, n); }
template <> CVB_HD void store_run<float, 12>(void* b, size_t o, const float (&v)[12], bool vec, int n) { store_run_f32<12>(b, o, v, vec, n); }
template <> CVB_HD void store_run<float, 16>(void* b, size_t o, const float (&v)[16], bool vec, int n) { store_run_f32<16>(b, o, v, vec, n); }
template <> CVB_HD void store_run<__nv_bfloat16, 4>(void* b, size_t o, const float (&v)[4], bool vec, int n) { store_run_bf16<4>(b, o, v, vec, n); }
template <> CVB_HD void store_run<__nv_bfloat16, 6>(void* b, size_t o, const float (&v)[6], bool vec, int n) { store_run_bf16<6>(b, o, v, vec, n); }
template <> CVB_HD void store_run<__nv_bfloat16, 8>(void* b, size_t o, const float (&v)[8], bool vec, int n) { store_run_bf16<8>(b, o, v, vec, n); }
template <> CVB_HD void store_run<__nv_bfloat16, 12>(void* b, size_t o, const float (&v)[12], bool vec, int n) { store_run_bf16<12>(b, o, v, vec, n); }
template <> CVB_HD void store_run<__nv_bfloat16, 16>(void* b, size_t o, const float (&v)[16], bool vec, int n) { store_run_bf16<16>(b, o, v, vec, n); }

// Compile-time (S, K): the taps each output phase touches are resolved by the
// compiler.  A thread owns a strip of CW low-resolution columns and walks down a
// segment of rows with a sliding window of r (WIN rows x CW+WIN-1 columns): one new
// window row is read per step, and each of the S output rows of the step leaves as
// one run of CW*S values (16 bytes per lane, consecutive lanes = consecutive strips).
template <int S, int K, int CW, typename IO, bool GELU>
CVB_HD void epilogue_rows(int tid, int nthr, const float2* sm, const float* wk, const FwdParams& P,
                          const IoArgs& io) {
  constexpr int c = K / 2;
  constexpr int DMIN = (c == 0) ? 0 : -((c + S - 1) / S);
  constexpr int DMAX = (S - 1 + K - 1 - c) / S;
  constexpr int WIN = DMAX - DMIN + 1;
  constexpr int WC = CW + WIN - 1;
  constexpr int NO = CW * S;
  constexpr int VEC = (sizeof(IO) == 4 || NO % 8 != 0) ? 4 : 8;  // elements per vector store (16 bytes; 8 for short bf16 runs)
  const int p = P.p, h = P.h, w = P.w, pitch = P.pitch;
  const int spr = (P.W + CW - 1) / CW;  // strips per row
  int nseg = nthr / spr;                // row segments handled concurrently
  if (nseg < 1) nseg = 1;
  if (nseg > P.H) nseg = P.H;
  const int rps = (P.H + nseg - 1) / nseg;  // rows per segment
  const int nitems = nseg * spr;
  const int oW = P.W * S;
  const float inv_spr = 1.0f / (float)spr;
  const bool vec = (P.W % CW == 0) && (NO % VEC == 0) && (oW % VEC == 0) &&
                   (((size_t)io.oa) % 16 == 0) && (((size_t)io.ob) % 16 == 0);
  const bool nost = (P.skip_mask & 512) != 0;  // tuning aid: compute but do not store
  float kw[K * K];
#pragma unroll
  for (int i = 0; i < K * K; ++i) kw[i] = wk[i];
  for (int it = tid; it < nitems; it += nthr) {
    int seg, sx;
    divmod_small(it, spr, inv_spr, seg, sx);
    const int mx0 = sx * CW;
    const int ncell = (P.W - mx0) < CW ? (P.W - mx0) : CW;
    const int my_begin = seg * rps;
    const int my_end = (my_begin + rps) < P.H ? (my_begin + rps) : P.H;
    int cols[WC];
#pragma unroll
    for (int e = 0; e < WC; ++e) {
      int rn = mx0 + p + DMIN + e;
      if (rn < 0) rn += w;
      if (rn >= w) rn -= w;
      if (rn >= w) rn -= w;
      cols[e] = rn;
    }
    // window rows my + p + DMIN .. my + p + DMAX; preload all but the last
    float2 win[WIN][WC];
    int rm = my_begin + p + DMIN;
    if (rm < 0) rm += h;
    if (rm >= h) rm -= h;
#pragma unroll
    for (int d = 0; d + 1 < WIN; ++d) {
#pragma unroll
      for (int e = 0; e < WC; ++e) win[d][e] = sm[rm * pitch + cols[e]];
      rm = (rm + 1 == h) ? 0 : rm + 1;
    }
    for (int my = my_begin; my < my_end; ++my) {
#pragma unroll
      for (int e = 0; e < WC; ++e) win[WIN - 1][e] = sm[rm * pitch + cols[e]];
      rm = (rm + 1 == h) ? 0 : rm + 1;
      float ya[CW], yb[CW];
      if (io.ycopy) {
        const float2* yrow = io.ycopy + (my + p) * pitch + mx0 + p;
#pragma unroll
        for (int e = 0; e < CW; ++e) {
          const float2 v = yrow[e < ncell ? e : 0];
          ya[e] = v.x;
          yb[e] = v.y;
        }
      } else {
#pragma unroll
        for (int e = 0; e < CW; ++e) {
          const size_t xoff = (size_t)my * P.W + (mx0 + (e < ncell ? e : 0));
          ya[e] = ld_io<IO>(io.xa, xoff);
          yb[e] = io.xb ? ld_io<IO>(io.xb, xoff) : 0.f;
        }
      }
#pragma unroll
      for (int da = 0; da < S; ++da) {
        float oa[NO], ob[NO];
#pragma unroll
        for (int e = 0; e < CW; ++e) {
#pragma unroll
          for (int db = 0; db < S; ++db) {
            float acca = ya[e], accb = yb[e];
#pragma unroll
            for (int a = 0; a < K; ++a) {
              const int ii = da + a - c;
              const int fi = (ii >= 0) ? ii / S : -((-ii + S - 1) / S);
              if (ii - fi * S != 0) continue;
#pragma unroll
              for (int b = 0; b < K; ++b) {
                const int jj = db + b - c;
                const int fj = (jj >= 0) ? jj / S : -((-jj + S - 1) / S);
                if (jj - fj * S != 0) continue;
                const float2 rv = win[fi - DMIN][e + fj - DMIN];
                acca = fmaf(kw[a * K + b], rv.x, acca);
                accb = fmaf(kw[a * K + b], rv.y, accb);
              }
            }
            if (GELU) gelu_pair(acca, accb);
            oa[e * S + db] = acca;
            ob[e * S + db] = accb;
          }
        }
        const size_t off = (size_t)(my * S + da) * oW + (size_t)(mx0 * S);
        store_run<IO, NO>(io.oa, off, oa, vec && !nost, nost ? 0 : ncell * S);
        if (io.ob) store_run<IO, NO>(io.ob, off, ob, vec && !nost, nost ? 0 : ncell * S);
      }
      // slide the window down one row
#pragma unroll
      for (int d = 0; d + 1 < WIN; ++d) {
#pragma unroll
        for (int e = 0; e < WC; ++e) win[d][e] = win[d + 1][e];
      }
    }
  }
}

template <int S, int K, int CW, typename IO>
CVB_HD void epilogue_static(int tid, int nthr, const float2* sm, const float* wk, const FwdParams& P,
                            const IoArgs& io) {
  if (io.gelu) epilogue_rows<S, K, CW, IO, true>(tid, nthr, sm, wk, P, io);
  else epilogue_rows<S, K, CW, IO, false>(tid, nthr, sm, wk, P, io);
}

template <typename IO>
CVB_HD void run_epilogue(int tid, int nthr, const float2* sm, const float* wk, const FwdParams& P,
                         const IoArgs& io) {
  const int key = P.s * 100 + P.k;
  switch (key) {
    // CW cells per thread: CW * S outputs = 16 bytes of fp32 (8 of bf16: wider runs cost more
    // window registers than the kernel has), so that a warp's store covers consecutive pieces of
    // one output row
    case 202: epilogue_static<2, 2, 2, IO>(tid, nthr, sm, wk, P, io); break;
    case 203: epilogue_static<2, 3, 2, IO>(tid, nthr, sm, wk, P, io); break;
    case 205: epilogue_static<2, 5, 2, IO>(tid, nthr, sm, wk, P, io); break;
    case 303: epilogue_static<3, 3, 4, IO>(tid, nthr, sm, wk, P, io); break;
    case 305: epilogue_static<3, 5, 4, IO>(tid, nthr, sm, wk, P, io); break;
    case 407: epilogue_static<4, 7, 1, IO>(tid, nthr, sm, wk, P, io); break;
    default: epilogue_generic<IO>(tid, nthr, sm, wk, P, io); break;
  }
}

// ---------------------------------------------------------------- block bodies
#ifdef __CUDA_ARCH__
#define CVB_PHASE(call)                                  \
  do {                                                   \
    const int tid = threadIdx.x, nthr = blockDim.x;      \
    (void)tid; (void)nthr;                               \
    call;                                                \
    __syncthreads();                                     \
  } while (0)
#else
#define CVB_PHASE(call)                                  \
  do {                                                   \
    for (int tid = 0; tid < nthr_emu; ++tid) {           \
      const int nthr = nthr_emu;                         \
      (void)nthr;                                        \
      call;                                              \
    }                                                    \
  } while (0)
#endif

// Shared-memory layout of one block (float2 units unless noted).
struct SmemLayout {
  int plane;   // h * pitch
  int twy;     // h
  int twx;     // w
  int wk;      // k*k floats, rounded up to float2
  int maps;    // h + w ints (pad maps), rounded up to float2
  int ycopy;   // h * pitch when the padded input is kept, else 0
  __host__ __device__ size_t bytes() const {
    return (size_t)(plane + twy + twx + wk + maps + ycopy) * sizeof(float2);
  }
};
CVB_HD SmemLayout smem_layout(int h, int w, int pitch, int k, int ystash) {
  SmemLayout l;
  l.plane = h * pitch;
  l.twy = h;
  l.twx = w;
  l.wk = (k * k + 1) / 2;
  l.maps = (h + w + 1) / 2;
  l.ycopy = ystash ? h * pitch : 0;
  return l;
}

CVB_HD void load_tables(int tid, int nthr, const FwdParams& P, int c, float2* twy, float2* twx, float* wk,
                        int* maps) {
  const float2* gtw = P.table + (size_t)P.C * P.h * P.w;
  for (int i = tid; i < P.h; i += nthr) {
    twy[i] = gtw[i];
    const int ry = pad_index(i - P.p, P.H, P.pad_mode);
    maps[i] = ry < 0 ? -1 : ry * P.W;
  }
  for (int i = tid; i < P.w; i += nthr) {
    twx[i] = gtw[P.h + i];
    maps[P.h + i] = pad_index(i - P.p, P.W, P.pad_mode);
  }
  if (P.s > 1)
    for (int i = tid; i < P.k * P.k; i += nthr) wk[i] = P.weight[(size_t)c * P.k * P.k + i];
}

// pair index -> channel and the two planes
CVB_HD void pair_planes(const FwdParams& P, int pair, int& c, int& pa, int& pb) {
  c = pair % P.C;
  const int i = pair / P.C;
  pa = (2 * i) * P.C + c;
  pb = (2 * i + 1 < P.B) ? (2 * i + 1) * P.C + c : -1;
}

template <typename IO>
CVB_HD IoArgs make_io(const FwdParams& P, int c, int pa, int pb) {
  IoArgs io;
  const size_t in_plane = (size_t)P.H * P.W, out_plane = in_plane * P.s * P.s;
  io.xa = (const IO*)P.x + (size_t)pa * in_plane;
  io.xb = pb >= 0 ? (const void*)((const IO*)P.x + (size_t)pb * in_plane) : nullptr;
  io.oa = (IO*)P.out + (size_t)pa * out_plane;
  io.ob = pb >= 0 ? (void*)((IO*)P.out + (size_t)pb * out_plane) : nullptr;
  io.H = P.H; io.W = P.W; io.p = P.p; io.pad_mode = P.pad_mode; io.gelu = P.fuse_gelu;
  io.h = P.h; io.w = P.w;
  io.tab = P.table + (size_t)c * P.h * P.w;
  io.rmap = nullptr;
  io.cmap = nullptr;
  io.ycopy = nullptr;
  io.yoff = 0;
  io.ws = nullptr;
  io.wes = 0;
  io.wls = 0;
  io.xoff = 0;
  return io;
}

// Plain phases used by the runtime-plan kernel: padded load, table multiply, cropped store.
template <typename IO>
CVB_HD void phase_load_plane(int tid, int nthr, float2* plane, const FwdParams& P, const IoArgs& io) {
  const int total = P.h * P.w;
  const float invw = 1.0f / (float)P.w;
  for (int i = tid; i < total; i += nthr) {
    int row, col;
    divmod_small(i, P.w, invw, row, col);
    const int ry = pad_index(row - P.p, P.H, P.pad_mode);
    const int cx = pad_index(col - P.p, P.W, P.pad_mode);
    float va = 0.f, vb = 0.f;
    if (ry >= 0 && cx >= 0) {
      const size_t off = (size_t)ry * P.W + cx;
      va = ld_io<IO>(io.xa, off);
      if (io.xb) vb = ld_io<IO>(io.xb, off);
    }
    plane[row * P.pitch + col] = make_float2(va, vb);
    if (io.ycopy) io.ycopy[row * P.pitch + col] = make_float2(va, vb);
  }
}

CVB_HD void phase_multiply(int tid, int nthr, float2* plane, const FwdParams& P, const IoArgs& io) {
  const int total = P.h * P.w;
  const float invh = 1.0f / (float)P.h;
  for (int i = tid; i < total; i += nthr) {
    int posx, posy;
    divmod_small(i, P.h, invh, posx, posy);  // posy fastest: the table's order
    const float2 g = io.tab[i];
    float2* e = plane + posy * P.pitch + posx;
    const float2 v = *e;
    *e = make_float2(fmaf(-v.y, g.y, v.x * g.x), -fmaf(v.x, g.y, v.y * g.x));  // conj(v * g)
  }
}

template <typename IO>
CVB_HD void phase_store_plane(int tid, int nthr, const float2* plane, const FwdParams& P, const IoArgs& io) {
  const int total = P.H * P.W;
  const float invW = 1.0f / (float)P.W;
  for (int i = tid; i < total; i += nthr) {
    int oy, ox;
    divmod_small(i, P.W, invW, oy, ox);
    const float2 v = plane[(oy + P.p) * P.pitch + ox + P.p];
    float va = v.x, vb = v.y;
    if (io.gelu) gelu_pair(va, vb);
    st_io<IO>(io.oa, (size_t)i, va);
    if (io.ob) st_io<IO>(io.ob, (size_t)i, vb);
  }
}

// Runtime plan: any supported factorisation, radices picked by a switch; the
// load, multiply and store are separate sweeps (the compile-time kernels fuse them).
template <typename IO>
__host__ __device__ void smem_block_dynamic(const FwdParams& P, int pair, float2* smem, int nthr_emu) {
  (void)nthr_emu;
  const SmemLayout lay = smem_layout(P.h, P.w, P.pitch, P.k, P.ystash);
  float2* plane = smem;
  float2* twy = plane + lay.plane;
  float2* twx = twy + lay.twy;
  float* wk = (float*)(twx + lay.twx);
  int* maps = (int*)((float2*)wk + lay.wk);
  int c, pa, pb;
  pair_planes(P, pair, c, pa, pb);
  IoArgs io = make_io<IO>(P, c, pa, pb);
  io.rmap = maps;
  io.cmap = maps + P.h;
  if (P.ystash) { io.ycopy = (float2*)maps + lay.maps; io.yoff = (int)(io.ycopy - plane); }
  const Plan1D& py = P.py;
  const Plan1D& px = P.px;

  CVB_PHASE((load_tables(tid, nthr, P, c, twy, twx, wk, maps), phase_load_plane<IO>(tid, nthr, plane, P, io)));
  // One loop over all stages: forward columns, forward rows, (multiply), inverse rows, inverse columns.
  const int nf = py.nst + px.nst;
  for (int ph = 0; ph < 2 * nf; ++ph) {
    const bool inv = ph >= nf;
    const int q = inv ? 2 * nf - 1 - ph : ph;      // stage slot in forward order
    const bool along_y = q < py.nst;
    const Plan1D& pl = along_y ? py : px;
    const int i = along_y ? q : q - py.nst;
    int flags = inv ? PASS_PRE : 0;
    if (inv && q == 0) flags |= PASS_CONJ_OUT;
    if (ph == nf) CVB_PHASE(phase_multiply(tid, nthr, plane, P, io));
    CVB_PHASE((run_pass<float>(pl.radix[i], tid, nthr,
                               make_pass(plane, along_y, P.pitch, P.h, P.w, pl.n, pl.L[i], pl.M[i],
                                         along_y ? twy : twx), io, flags)));
  }
  if (P.s == 1) {
    CVB_PHASE(phase_store_plane<IO>(tid, nthr, plane, P, io));
  } else {
    CVB_PHASE(run_epilogue<IO>(tid, nthr, plane, wk, P, io));
  }
}

// ---- batch-summed cross spectrum (parameter gradients) ----
// The operator's multiplier M (G at scale 1, P at scale >= 2) enters the loss only through
//     L = (1 / (h w)) * Re sum_f M[f] * D[f],   D[f] = sum_b FFT2(pad(x_b))[f] * conj(FFT2(q_b)[f]),
// q = dL/dout zero-extended (scale 1) or the adjoint of the upsampling epilogue applied to it
// (scale >= 2), so dL/dweight and dL/dbias follow from D by the chain rule on one (C,h,w) tensor.
// D is what this kernel computes: a block owns channel c and the batch entries seg, seg + nseg, ...;
// per entry it loads z = pad(x) + i q into shared memory, runs the forward stages, and with
// P = Z[f], Q = Z[-f] adds  X conj(Qhat) = ( Im(P Q) / 2,  (|P|^2 - |Q|^2) / 4 )  to its accumulator
// plane (X = (P + conj Q) / 2 and Qhat = (P - conj Q) / 2i are the spectra of the two real planes).
// At the end the accumulator is written in natural frequency order: out[seg][c][ky][kx].
// Planes too large for two shared-memory planes (direct != 0) add every product straight into
// out[0][c][ky][kx] with atomics instead (the caller zero-fills it).
struct XspecParams {
  const float* x;     // (B,C,H,W)
  const float* q;     // (B,C,h,w)
  float2* out;        // [nseg][C][h][w]
  const float2* tw;   // (cos, sin)(2 pi n / h), n < h, then the same for w
  int B, C, H, W, p, pad_mode, h, w, pitch, nseg;
  int direct;         // 1: no accumulator plane, atomic adds into out[0]
  Plan1D py, px;
};

CVB_HD size_t xspec_smem_bytes(int h, int w, int direct) {
  const int pitch = w | 1;
  return (size_t)((direct ? 1 : 2) * h * pitch + h + w) * sizeof(float2) + (size_t)(3 * (h + w)) * sizeof(int);
}

CVB_HD void xspec_add(float* p, float v) {
#ifdef __CUDA_ARCH__
  atomicAdd(p, v);
#else
  *p += v;
#endif
}

__host__ __device__ inline void smem_block_xspec(const XspecParams& Q, int c, int seg, float2* smem, int nthr_emu) {
  (void)nthr_emu;
  const int h = Q.h, w = Q.w, pitch = Q.pitch;
  float2* plane = smem;
  float2* acc = plane + h * pitch;
  float2* twy = acc + (Q.direct ? 0 : h * pitch);
  float2* twx = twy + h;
  int* fy = (int*)(twx + w);   // position -> frequency
  int* fx = fy + h;
  int* ny = fx + w;            // position -> position of the negated frequency
  int* nx = ny + h;
  int* oy = nx + w;            // frequency -> position
  int* ox = oy + h;
  IoArgs io;
  io.xa = nullptr; io.xb = nullptr; io.oa = nullptr; io.ob = nullptr;
  io.H = Q.H; io.W = Q.W; io.p = Q.p; io.pad_mode = Q.pad_mode; io.gelu = 0; io.h = h; io.w = w;
  io.tab = nullptr; io.rmap = nullptr; io.cmap = nullptr; io.ycopy = nullptr; io.ws = nullptr;
  io.wes = 0; io.wls = 0; io.xoff = 0; io.yoff = 0;
  const float invw = 1.0f / (float)w;
  CVB_PHASE(([&] {
    for (int i = tid; i < h; i += nthr) {
      twy[i] = Q.tw[i];
      const int f = pos_to_freq(Q.py, i);
      fy[i] = f; oy[f] = i;
    }
    for (int i = tid; i < w; i += nthr) {
      twx[i] = Q.tw[h + i];
      const int f = pos_to_freq(Q.px, i);
      fx[i] = f; ox[f] = i;
    }
    if (!Q.direct)
      for (int i = tid; i < h * pitch; i += nthr) acc[i] = make_float2(0.f, 0.f);
  }()));
  CVB_PHASE(([&] {
    for (int i = tid; i < h; i += nthr) ny[i] = oy[(h - fy[i]) % h];
    for (int i = tid; i < w; i += nthr) nx[i] = ox[(w - fx[i]) % w];
  }()));
  const size_t in_plane = (size_t)Q.H * Q.W, q_plane = (size_t)h * w;
  const int nf = Q.py.nst + Q.px.nst;
  float2* op = Q.out + ((size_t)(Q.direct ? 0 : seg) * Q.C + c) * q_plane;
  for (int b = seg; b < Q.B; b += Q.nseg) {
    const float* xp = Q.x + ((size_t)b * Q.C + c) * in_plane;
    const float* qp = Q.q + ((size_t)b * Q.C + c) * q_plane;
    CVB_PHASE(([&] {
      for (int i = tid; i < h * w; i += nthr) {
        int row, col;
        divmod_small(i, w, invw, row, col);
        const int ry = pad_index(row - Q.p, Q.H, Q.pad_mode);
        const int cx = pad_index(col - Q.p, Q.W, Q.pad_mode);
        const float va = (ry >= 0 && cx >= 0) ? xp[(size_t)ry * Q.W + cx] : 0.f;
        plane[row * pitch + col] = make_float2(va, qp[i]);
      }
    }()));
    for (int ph = 0; ph < nf; ++ph) {
      const bool along_y = ph < Q.py.nst;
      const Plan1D& pl = along_y ? Q.py : Q.px;
      const int i = along_y ? ph : ph - Q.py.nst;
      CVB_PHASE((run_pass<float>(pl.radix[i], tid, nthr,
                                 make_pass(plane, along_y, pitch, h, w, pl.n, pl.L[i], pl.M[i],
                                           along_y ? twy : twx), io, 0)));
    }
    CVB_PHASE(([&] {
      for (int i = tid; i < h * w; i += nthr) {
        int row, col;
        divmod_small(i, w, invw, row, col);
        const float2 P = plane[row * pitch + col];
        const float2 N = plane[ny[row] * pitch + nx[col]];
        const float dre = 0.5f * fmaf(P.x, N.y, P.y * N.x);
        const float dim = 0.25f * (fmaf(P.x, P.x, P.y * P.y) - fmaf(N.x, N.x, N.y * N.y));
        if (Q.direct) {
          float* o = (float*)(op + (size_t)fy[row] * w + fx[col]);
          xspec_add(o, dre);
          xspec_add(o + 1, dim);
        } else {
          float2* a = acc + row * pitch + col;
          a->x += dre;
          a->y += dim;
        }
      }
    }()));
  }
  if (Q.direct) return;
  CVB_PHASE(([&] {
    for (int i = tid; i < h * w; i += nthr) {
      int row, col;
      divmod_small(i, w, invw, row, col);
      op[(size_t)fy[row] * w + fx[col]] = acc[row * pitch + col];
    }
  }()));
}

// Compile-time plan: h = RY0*RY1, w = RX0*RX1, two stages per axis, NT threads; all
// index arithmetic is folded by the compiler and only the four needed butterflies
// count against the kernel's register budget.
#ifdef __CUDA_ARCH__
#define CVB_PHASE_CT(call)                               \
  do {                                                   \
    const int tid = threadIdx.x;                         \
    constexpr int nthr = NT;                             \
    call;                                                \
    __syncthreads();                                     \
  } while (0)
#else
#define CVB_PHASE_CT(call)                               \
  do {                                                   \
    for (int tid = 0; tid < NT; ++tid) {                 \
      constexpr int nthr = NT;                           \
      call;                                              \
    }                                                    \
  } while (0)
#endif

// The seven FFT stages and the epilogue of one plane pair, every stage compiled with
// its own flags.  `io.xa/xb` may point to global memory or to a staged copy in shared
// memory; the stage code is the same.
template <typename IO, int RY0, int RY1, int RX0, int RX1, int NT>
CVB_HD void static_stages(const FwdParams& P, const IoArgs& io, float2* plane, const float2* twy,
                          const float2* twx, const float* wk) {
  constexpr int h = RY0 * RY1, w = RX0 * RX1;
  constexpr int pitch = w | 1;
  const PassArgs ay0 = make_pass(plane, true, pitch, h, w, h, h, RY1, twy);
  const PassArgs ay1 = make_pass(plane, true, pitch, h, w, h, RY1, 1, twy);
  const PassArgs ax0 = make_pass(plane, false, pitch, h, w, w, w, RX1, twx);
  const PassArgs ax1 = make_pass(plane, false, pitch, h, w, w, RX1, 1, twx);
  const int sk = P.skip_mask;
  if (!(sk & 2)) CVB_PHASE_CT((fft_pass<RY0, IO, h, h, RY1, w, PASS_SRC_GLOBAL>(tid, nthr, ay0, io, 0)));
  if (!(sk & 4)) CVB_PHASE_CT((fft_pass<RY1, IO, h, RY1, 1, w, 0>(tid, nthr, ay1, io, 0)));
  if (!(sk & 8)) CVB_PHASE_CT((fft_pass<RX0, IO, w, w, RX1, h, 0>(tid, nthr, ax0, io, 0)));
  if (!(sk & 16)) CVB_PHASE_CT((fft_pass<RX1, IO, w, RX1, 1, h, PASS_MID>(tid, nthr, ax1, io, 0)));
  if (!(sk & 32)) CVB_PHASE_CT((fft_pass<RX0, IO, w, w, RX1, h, PASS_PRE>(tid, nthr, ax0, io, 0)));
  if (!(sk & 64)) CVB_PHASE_CT((fft_pass<RY1, IO, h, RY1, 1, w, PASS_PRE>(tid, nthr, ay1, io, 0)));
  if (!(sk & 128)) {
    if (P.s == 1) {
      CVB_PHASE_CT((fft_pass<RY0, IO, h, h, RY1, w, PASS_PRE | PASS_CONJ_OUT | PASS_DST_GLOBAL>(tid, nthr, ay0, io, 0)));
    } else {
      CVB_PHASE_CT((fft_pass<RY0, IO, h, h, RY1, w, PASS_PRE | PASS_CONJ_OUT>(tid, nthr, ay0, io, 0)));
    }
  }
  if (P.s != 1 && !(sk & 256)) CVB_PHASE_CT(run_epilogue<IO>(tid, nthr, plane, wk, P, io));
}

// One block = one plane pair.
template <typename IO, int RY0, int RY1, int RX0, int RX1, int NT>
__host__ __device__ void smem_block_static(const FwdParams& P, int pair, float2* smem) {
  constexpr int h = RY0 * RY1, w = RX0 * RX1;
  constexpr int pitch = w | 1;
  const SmemLayout lay = smem_layout(h, w, pitch, P.k, P.ystash);
  float2* plane = smem;
  float2* twy = plane + lay.plane;
  float2* twx = twy + lay.twy;
  float* wk = (float*)(twx + lay.twx);
  int* maps = (int*)((float2*)wk + lay.wk);
  int c, pa, pb;
  pair_planes(P, pair, c, pa, pb);
  IoArgs io = make_io<IO>(P, c, pa, pb);
  io.h = h; io.w = w;
  io.rmap = maps;
  io.cmap = maps + h;
  if (P.ystash) { io.ycopy = (float2*)maps + lay.maps; io.yoff = (int)(io.ycopy - plane); }
  CVB_PHASE_CT(load_tables(tid, nthr, P, c, twy, twx, wk, maps));
  static_stages<IO, RY0, RY1, RX0, RX1, NT>(P, io, plane, twy, twx, wk);
}

// Persistent variant: a block loops over plane pairs (pair = block, block + nblocks, ...).
// The raw planes of the NEXT pair are fetched by bulk asynchronous copies (TMA) into one
// half of a double buffer while the current pair is transformed, so no thread ever
// waits on HBM latency, and the stores of one pair drain while the next is computed.
// The first column stage and the epilogue read x from the staged copy.
constexpr int kWaitLimit = 1 << 18;  // polls of mbarrier.try_wait before giving up

CVB_HD size_t persistent_xin_bytes(int H, int W, int esize) {
  return ((size_t)2 * H * W * esize + 127) / 128 * 128;
}
CVB_HD size_t persistent_smem_bytes(int h, int w, int H, int W, int k, int esize) {
  return 2 * persistent_xin_bytes(H, W, esize) + smem_layout(h, w, w | 1, k, 0).bytes() + 2 * sizeof(uint64_t);
}

template <typename IO>
CVB_HD void persistent_issue(const FwdParams& P, int pair, IO* dst, uint64_t* bar) {
  int c, pa, pb;
  pair_planes(P, pair, c, pa, pb);
  const size_t HW = (size_t)P.H * P.W;
  const uint32_t bytes = (uint32_t)(HW * sizeof(IO));
  mbar_expect_tx(bar, pb >= 0 ? 2 * bytes : bytes);
  bulk_g2s(dst, (const IO*)P.x + (size_t)pa * HW, bytes, bar);
  if (pb >= 0) bulk_g2s(dst + HW, (const IO*)P.x + (size_t)pb * HW, bytes, bar);
}

template <typename IO, int RY0, int RY1, int RX0, int RX1, int NT>
__host__ __device__ void smem_persistent_static(const FwdParams& P, unsigned char* smem, int block, int nblocks) {
  constexpr int h = RY0 * RY1, w = RX0 * RX1;
  constexpr int pitch = w | 1;
  const size_t HW = (size_t)P.H * P.W;
  const size_t xin_bytes = persistent_xin_bytes(P.H, P.W, (int)sizeof(IO));
  IO* xin0 = (IO*)smem;
  IO* xin1 = (IO*)(smem + xin_bytes);
  const SmemLayout lay = smem_layout(h, w, pitch, P.k, 0);
  float2* plane = (float2*)(smem + 2 * xin_bytes);
  float2* twy = plane + lay.plane;
  float2* twx = twy + lay.twy;
  float* wk = (float*)(twx + lay.twx);
  int* maps = (int*)((float2*)wk + lay.wk);
  uint64_t* mbar = (uint64_t*)((float2*)maps + lay.maps);
  const int npairs = P.C * ((P.B + 1) / 2);
  if (block >= npairs) return;

#ifdef __CUDA_ARCH__
  if (threadIdx.x == 0) {
    mbar_init(&mbar[0], 1);
    mbar_init(&mbar[1], 1);
    mbar_fence_init();
    persistent_issue<IO>(P, block, xin0, &mbar[0]);
  }
#else
  persistent_issue<IO>(P, block, xin0, &mbar[0]);
#endif
  CVB_PHASE_CT(load_tables(tid, nthr, P, 0, twy, twx, wk, maps));

  int it = 0;
  for (int pair = block; pair < npairs; pair += nblocks, ++it) {
    const int buf = it & 1;
    const uint32_t parity = (uint32_t)((it >> 1) & 1);
    IO* cur = buf ? xin1 : xin0;
    IO* nxt = buf ? xin0 : xin1;
    int c, pa, pb;
    pair_planes(P, pair, c, pa, pb);
    IoArgs io = make_io<IO>(P, c, pa, pb);
    io.h = h; io.w = w;
    io.rmap = maps;
    io.cmap = maps + h;
    io.xa = cur;
    io.xb = pb >= 0 ? (const void*)(cur + HW) : nullptr;
    const bool more = pair + nblocks < npairs;
#ifdef __CUDA_ARCH__
    {
      const int tid = threadIdx.x;
      // the other half was last read in the previous iteration, which ended with a barrier
      if (tid == 0 && more) persistent_issue<IO>(P, pair + nblocks, nxt, &mbar[buf ^ 1]);
      if (P.s > 1)
        for (int i = tid; i < P.k * P.k; i += NT) wk[i] = P.weight[(size_t)c * P.k * P.k + i];
      const bool ok = mbar_wait_bounded(&mbar[buf], parity, kWaitLimit);
      if (__syncthreads_or(!ok)) {
        // give up: flag it, let the copy in flight (if any) land, and leave
        if (tid == 0 && P.status) atomicExch(P.status, 1);
        if (more) mbar_wait_bounded(&mbar[buf ^ 1], (uint32_t)(((it + 1) >> 1) & 1), kWaitLimit);
        return;
      }
    }
#else
    if (more) persistent_issue<IO>(P, pair + nblocks, nxt, &mbar[buf ^ 1]);
    if (P.s > 1)
      for (int i = 0; i < P.k * P.k; ++i) wk[i] = P.weight[(size_t)c * P.k * P.k + i];
#endif
    static_stages<IO, RY0, RY1, RX0, RX1, NT>(P, io, plane, twy, twx, wk);
  }
}

// ---------------------------------------------------------------- transfer table
// Rader's algorithm for a large prime R that is the first stage of an axis plan (used by
// the multi-pass kernels): tables of one axis, stored in the transfer blob behind the twiddles
// as [bhat: R-1 float2][twiddles of R-1: R-1 float2][g^q mod R: R-1 int][g^-m mod R: R-1 int].
struct RaderInfo {
  int R;        // 0 = not used on this axis
  int g;        // primitive root of R
  Plan1D sub;   // plan of length R-1
  int off;      // float2 offset of this axis' tables from the end of the twiddles
};

struct TransferParams {
  const float* weight;  // (C,k,k)
  const float* bias;    // (C)
  float2* table;
  int C, k, s, h, w;
  float eps;
  int kind;  // 0: the operator's multiplier; 1: 1 / (alias mean of |FK|^2 + lambda), the x0 term's multiplier
  Plan1D py, px;
  RaderInfo ry, rx;
};

// One table entry, straightforward form (one sine / cosine pair per tap and alias); kept for
// scales above kFastMaxScale.  fp64 throughout.
__host__ __device__ inline void transfer_entry_slow(const TransferParams& T, int c, int posy, int posx) {
  const int s = T.s, k = T.k, h = T.h, w = T.w, cc = T.k / 2;
  const int u = pos_to_freq(T.py, posy), v = pos_to_freq(T.px, posx);
  const double lam = 1.0 / (1.0 + exp(-((double)T.bias[c] - 9.0))) + (double)T.eps;
  const int Nh = s * h, Nw = s * w;
  const float* K = T.weight + (size_t)c * k * k;
  double num_r = 0.0, num_i = 0.0, den = 0.0;  // sums over the s*s aliases
  for (int ia = 0; ia < s; ++ia) {
    const int U = u + ia * h;
    // D_h(U) = sum_{a<s} exp(-2 pi i a U / Nh)
    double dhr = 0.0, dhi = 0.0;
    for (int a = 0; a < s; ++a) {
      const long long m = ((long long)a * U) % Nh;
      dhr += cos(-2.0 * M_PI * (double)m / Nh);
      dhi += sin(-2.0 * M_PI * (double)m / Nh);
    }
    for (int ib = 0; ib < s; ++ib) {
      const int V = v + ib * w;
      double dwr = 0.0, dwi = 0.0;
      for (int b = 0; b < s; ++b) {
        const long long m = ((long long)b * V) % Nw;
        dwr += cos(-2.0 * M_PI * (double)m / Nw);
        dwi += sin(-2.0 * M_PI * (double)m / Nw);
      }
      // FK[U,V] = sum_{a,b} K[a][b] exp(-2 pi i ((a-c) U / Nh + (b-c) V / Nw))
      double fr = 0.0, fi = 0.0;
      for (int a = 0; a < k; ++a) {
        long long ma = ((long long)(a - cc) * U) % Nh; if (ma < 0) ma += Nh;
        const double ear = cos(-2.0 * M_PI * (double)ma / Nh), eai = sin(-2.0 * M_PI * (double)ma / Nh);
        double rr = 0.0, ri = 0.0;
        for (int b = 0; b < k; ++b) {
          long long mb = ((long long)(b - cc) * V) % Nw; if (mb < 0) mb += Nw;
          const double kv = (double)K[a * k + b];
          rr += kv * cos(-2.0 * M_PI * (double)mb / Nw);
          ri += kv * sin(-2.0 * M_PI * (double)mb / Nw);
        }
        fr += ear * rr - eai * ri;
        fi += ear * ri + eai * rr;
      }
      den += fr * fr + fi * fi;
      if (s == 1) {
        num_r = fr; num_i = -fi;  // conj(FK)
      } else {
        const double dr = dhr * dwr - dhi * dwi, di = dhr * dwi + dhi * dwr;
        num_r += fr * dr - fi * di;
        num_i += fr * di + fi * dr;
      }
    }
  }
  const double inv_alias = 1.0 / (double)(s * s);
  const double norm = 1.0 / ((double)h * (double)w);
  double tr, ti;
  if (T.kind == 1) {
    tr = 1.0 / (den * inv_alias + lam);
    ti = 0.0;
  } else if (s == 1) {
    const double d = den + lam;
    tr = (num_r + lam) / d;
    ti = num_i / d;
  } else {
    const double d = den * inv_alias + lam;
    tr = (1.0 - num_r * inv_alias) / d;
    ti = (-num_i * inv_alias) / d;
  }
  T.table[((size_t)c * w + posx) * h + posy] = make_float2((float)(tr * norm), (float)(ti * norm));
}

// exp(-2 pi i m / N) in fp64
__host__ __device__ inline void cis_neg(long long m, int N, double& cr, double& ci) {
#ifdef __CUDA_ARCH__
  double sn, cs;
  sincospi(-2.0 * (double)m / (double)N, &sn, &cs);
  cr = cs; ci = sn;
#else
  const double a = -2.0 * M_PI * (double)m / (double)N;
  cr = cos(a); ci = sin(a);
#endif
}

constexpr int kFastMaxScale = 4;

// One table entry: position (posx, posy) of channel c.  fp64 throughout.  The kernel spectrum is
// separable in its exponentials: with ey = exp(-2 pi i U / Nh), ex = exp(-2 pi i V / Nw),
//   FK[U,V] = sum_a ey^(a-c) * ( sum_b K[a][b] * ex^(b-c) ),
// so one sine / cosine pair per axis and alias and k*k real-by-complex multiply-adds per alias
// replace a sine / cosine pair per tap.  (The per-sample data step of USRNet rebuilds this table
// at every call, models/converse_usrnet.py:203-211, so its cost is on the hot path there.)
// CK, CS: compile-time kernel size and scale (0 = run-time values): with both known the small
// per-alias arrays live in registers.
template <int CK, int CS>
__host__ __device__ inline void transfer_entry_t(const TransferParams& T, int c, int posy, int posx) {
  const int s = CS ? CS : T.s, k = CK ? CK : T.k, h = T.h, w = T.w, cc = k / 2;
  if (s > kFastMaxScale) {
    transfer_entry_slow(T, c, posy, posx);
    return;
  }
  const int u = pos_to_freq(T.py, posy), v = pos_to_freq(T.px, posx);
  const double lam = 1.0 / (1.0 + exp(-((double)T.bias[c] - 9.0))) + (double)T.eps;
  const int Nh = s * h, Nw = s * w;
  const float* K = T.weight + (size_t)c * k * k;
  // per alias along x: tx[ib][a] = sum_b K[a][b] ex^(b-c), and the box factor D_w
  constexpr int AS = CS ? CS : kFastMaxScale, AK = CK ? CK : kMaxTaps;
  double txr[AS][AK], txi[AS][AK], dwr[AS], dwi[AS];
#pragma unroll
  for (int ib = 0; ib < (CS ? CS : s); ++ib) {
    const int V = v + ib * w;
    double er, ei, pr, pi;
    cis_neg(V, Nw, er, ei);
    // ex^(-c)
    cis_neg((long long)(-cc) * V % Nw + ((long long)(-cc) * V % Nw < 0 ? Nw : 0), Nw, pr, pi);
#pragma unroll
    for (int a = 0; a < (CK ? CK : k); ++a) { txr[ib][a] = 0.0; txi[ib][a] = 0.0; }
#pragma unroll
    for (int b = 0; b < (CK ? CK : k); ++b) {
#pragma unroll
      for (int a = 0; a < (CK ? CK : k); ++a) {
        const double kv = (double)K[a * k + b];
        txr[ib][a] += kv * pr;
        txi[ib][a] += kv * pi;
      }
      const double nr = pr * er - pi * ei, ni = pr * ei + pi * er;
      pr = nr; pi = ni;
    }
    double sr = 0.0, si = 0.0, qr = 1.0, qi = 0.0;  // D_w = sum_{b<s} ex^b
    for (int b = 0; b < s; ++b) {
      sr += qr; si += qi;
      const double nr = qr * er - qi * ei, ni = qr * ei + qi * er;
      qr = nr; qi = ni;
    }
    dwr[ib] = sr; dwi[ib] = si;
  }
  double num_r = 0.0, num_i = 0.0, den = 0.0;
#pragma unroll
  for (int ia = 0; ia < (CS ? CS : s); ++ia) {
    const int U = u + ia * h;
    double er, ei, p0r, p0i;
    cis_neg(U, Nh, er, ei);
    cis_neg((long long)(-cc) * U % Nh + ((long long)(-cc) * U % Nh < 0 ? Nh : 0), Nh, p0r, p0i);
    double dhr = 0.0, dhi = 0.0, qr = 1.0, qi = 0.0;  // D_h = sum_{a<s} ey^a
    for (int a = 0; a < s; ++a) {
      dhr += qr; dhi += qi;
      const double nr = qr * er - qi * ei, ni = qr * ei + qi * er;
      qr = nr; qi = ni;
    }
#pragma unroll
    for (int ib = 0; ib < (CS ? CS : s); ++ib) {
      double fr = 0.0, fi = 0.0, pr = p0r, pi = p0i;
#pragma unroll
      for (int a = 0; a < (CK ? CK : k); ++a) {
        fr += pr * txr[ib][a] - pi * txi[ib][a];
        fi += pr * txi[ib][a] + pi * txr[ib][a];
        const double nr = pr * er - pi * ei, ni = pr * ei + pi * er;
        pr = nr; pi = ni;
      }
      den += fr * fr + fi * fi;
      if (s == 1) {
        num_r = fr; num_i = -fi;  // conj(FK)
      } else {
        const double dr = dhr * dwr[ib] - dhi * dwi[ib], di = dhr * dwi[ib] + dhi * dwr[ib];
        num_r += fr * dr - fi * di;
        num_i += fr * di + fi * dr;
      }
    }
  }
  const double inv_alias = 1.0 / (double)(s * s);
  const double norm = 1.0 / ((double)h * (double)w);
  double tr, ti;
  if (T.kind == 1) {
    tr = 1.0 / (den * inv_alias + lam);
    ti = 0.0;
  } else if (s == 1) {
    const double d = den + lam;
    tr = (num_r + lam) / d;
    ti = num_i / d;
  } else {
    const double d = den * inv_alias + lam;
    tr = (1.0 - num_r * inv_alias) / d;
    ti = (-num_i * inv_alias) / d;
  }
  T.table[((size_t)c * w + posx) * h + posy] = make_float2((float)(tr * norm), (float)(ti * norm));
}

// per-entry form with run-time kernel size and scale (scales above kFastMaxScale take the slow form)
__host__ __device__ inline void transfer_entry(const TransferParams& T, int c, int posy, int posx) {
  transfer_entry_t<0, 0>(T, c, posy, posx);
}

// ---- tiled form of the table build: one block = one channel x kTransferTile table columns.
// The x half of the separable sum (tx[alias][column][a] and the box factor D_w) depends only on
// the column, so it is computed once per block into shared memory (transfer_tile_x, one work item
// per alias and column); each thread then owns table rows (posy), keeps its y phasors in
// registers and spends k complex multiply-adds per alias pair and entry (transfer_tile_y).
// Same arithmetic as transfer_entry_t, same fp64, same table layout.
constexpr int kTransferTile = 32;
struct TransferTileSmem {
  double txr[kFastMaxScale][kTransferTile][kMaxTaps];
  double txi[kFastMaxScale][kTransferTile][kMaxTaps];
  double dwr[kFastMaxScale][kTransferTile], dwi[kFastMaxScale][kTransferTile];
};

template <int CK, int CS>
__host__ __device__ inline void transfer_tile_x(const TransferParams& T, int c, int x0, int item,
                                                TransferTileSmem& S) {
  const int s = CS ? CS : T.s, k = CK ? CK : T.k, w = T.w, cc = k / 2;
  const int ib = item / kTransferTile, xi = item % kTransferTile;
  if (ib >= s || x0 + xi >= w) return;
  const int Nw = s * w;
  const int V = pos_to_freq(T.px, x0 + xi) + ib * w;
  const float* K = T.weight + (size_t)c * k * k;
  double er, ei, pr, pi;
  cis_neg(V, Nw, er, ei);
  const long long m0 = (long long)(-cc) * V % Nw;
  cis_neg(m0 < 0 ? m0 + Nw : m0, Nw, pr, pi);  // ex^(-c)
  constexpr int AK = CK ? CK : kMaxTaps;
  double ar[AK], ai[AK];
#pragma unroll
  for (int a = 0; a < (CK ? CK : k); ++a) { ar[a] = 0.0; ai[a] = 0.0; }
#pragma unroll
  for (int b = 0; b < (CK ? CK : k); ++b) {
#pragma unroll
    for (int a = 0; a < (CK ? CK : k); ++a) {
      const double kv = (double)K[a * k + b];
      ar[a] += kv * pr;
      ai[a] += kv * pi;
    }
    const double nr = pr * er - pi * ei, ni = pr * ei + pi * er;
    pr = nr; pi = ni;
  }
#pragma unroll
  for (int a = 0; a < (CK ? CK : k); ++a) { S.txr[ib][xi][a] = ar[a]; S.txi[ib][xi][a] = ai[a]; }
  double sr = 0.0, si = 0.0, qr = 1.0, qi = 0.0;  // D_w = sum_{b<s} ex^b
  for (int b = 0; b < s; ++b) {
    sr += qr; si += qi;
    const double nr = qr * er - qi * ei, ni = qr * ei + qi * er;
    qr = nr; qi = ni;
  }
  S.dwr[ib][xi] = sr; S.dwi[ib][xi] = si;
}

template <int CK, int CS>
__host__ __device__ inline void transfer_tile_y(const TransferParams& T, int c, int x0, int posy,
                                                const TransferTileSmem& S) {
  const int s = CS ? CS : T.s, k = CK ? CK : T.k, h = T.h, w = T.w, cc = k / 2;
  const int Nh = s * h;
  const int u = pos_to_freq(T.py, posy);
  const double lam = 1.0 / (1.0 + exp(-((double)T.bias[c] - 9.0))) + (double)T.eps;
  constexpr int AS = CS ? CS : kFastMaxScale, AK = CK ? CK : kMaxTaps;
  double pr[AS][AK], pi[AS][AK], dhr[AS], dhi[AS];  // ey^(a-c) per alias, and D_h
#pragma unroll
  for (int ia = 0; ia < (CS ? CS : s); ++ia) {
    const int U = u + ia * h;
    double er, ei, qr, qi;
    cis_neg(U, Nh, er, ei);
    const long long m0 = (long long)(-cc) * U % Nh;
    cis_neg(m0 < 0 ? m0 + Nh : m0, Nh, qr, qi);
#pragma unroll
    for (int a = 0; a < (CK ? CK : k); ++a) {
      pr[ia][a] = qr; pi[ia][a] = qi;
      const double nr = qr * er - qi * ei, ni = qr * ei + qi * er;
      qr = nr; qi = ni;
    }
    double sr = 0.0, si = 0.0;
    qr = 1.0; qi = 0.0;
    for (int a = 0; a < s; ++a) {
      sr += qr; si += qi;
      const double nr = qr * er - qi * ei, ni = qr * ei + qi * er;
      qr = nr; qi = ni;
    }
    dhr[ia] = sr; dhi[ia] = si;
  }
  const double inv_alias = 1.0 / (double)(s * s);
  const double norm = 1.0 / ((double)h * (double)w);
  const int nx = (w - x0 < kTransferTile) ? w - x0 : kTransferTile;
  for (int xi = 0; xi < nx; ++xi) {
    double num_r = 0.0, num_i = 0.0, den = 0.0;
#pragma unroll
    for (int ia = 0; ia < (CS ? CS : s); ++ia) {
#pragma unroll
      for (int ib = 0; ib < (CS ? CS : s); ++ib) {
        double fr = 0.0, fi = 0.0;
#pragma unroll
        for (int a = 0; a < (CK ? CK : k); ++a) {
          const double tr = S.txr[ib][xi][a], ti = S.txi[ib][xi][a];
          fr += pr[ia][a] * tr - pi[ia][a] * ti;
          fi += pr[ia][a] * ti + pi[ia][a] * tr;
        }
        den += fr * fr + fi * fi;
        if (s == 1) {
          num_r = fr; num_i = -fi;  // conj(FK)
        } else {
          const double dr = dhr[ia] * S.dwr[ib][xi] - dhi[ia] * S.dwi[ib][xi];
          const double di = dhr[ia] * S.dwi[ib][xi] + dhi[ia] * S.dwr[ib][xi];
          num_r += fr * dr - fi * di;
          num_i += fr * di + fi * dr;
        }
      }
    }
    double tr, ti;
    if (T.kind == 1) {
      tr = 1.0 / (den * inv_alias + lam);
      ti = 0.0;
    } else if (s == 1) {
      const double d = den + lam;
      tr = (num_r + lam) / d;
      ti = num_i / d;
    } else {
      const double d = den * inv_alias + lam;
      tr = (1.0 - num_r * inv_alias) / d;
      ti = (-num_i * inv_alias) / d;
    }
    T.table[((size_t)c * w + x0 + xi) * h + posy] = make_float2((float)(tr * norm), (float)(ti * norm));
  }
}


template <int CK, int CS>
__host__ __device__ inline void transfer_tile_items(const TransferParams& T, int c, int x0, int tid,
                                                    int nthreads, TransferTileSmem& S) {
  const int s = CS ? CS : T.s;
  for (int item = tid; item < s * kTransferTile; item += nthreads) transfer_tile_x<CK, CS>(T, c, x0, item, S);
}
template <int CK, int CS>
__host__ __device__ inline void transfer_tile_rows(const TransferParams& T, int c, int x0, int tid,
                                                   int nthreads, const TransferTileSmem& S) {
  for (int posy = tid; posy < T.h; posy += nthreads) transfer_tile_y<CK, CS>(T, c, x0, posy, S);
}

// One block of the tiled build (block index -> channel, column tile); the host emulation calls it
// with any thread count.
template <int CK, int CS>
__host__ __device__ inline void transfer_tile_block(const TransferParams& T, long long block, int nthr_emu,
                                                    TransferTileSmem& S) {
  (void)nthr_emu;
  const int xtiles = (T.w + kTransferTile - 1) / kTransferTile;
  const int c = (int)(block / xtiles), x0 = (int)(block % xtiles) * kTransferTile;
  CVB_PHASE((transfer_tile_items<CK, CS>(T, c, x0, tid, nthr, S)));
  CVB_PHASE((transfer_tile_rows<CK, CS>(T, c, x0, tid, nthr, S)));
}

// (kernel size, scale) pairs with a compile-time instance of the tiled build; X(k, s)
#define CVB_TRANSFER_CASES(X) X(7, 1) X(7, 2) X(7, 4) X(5, 1) X(5, 2) X(3, 1) X(3, 2) X(2, 2)

__host__ __device__ inline void twiddle_entry(const TransferParams& T, int i) {
  // tw[n] = (cos, sin)(2 pi n / N); first h entries for the column length, then w
  float2* tw = T.table + (size_t)T.C * T.h * T.w;
  const int N = i < T.h ? T.h : T.w;
  const int n = i < T.h ? i : i - T.h;
  const double th = 2.0 * M_PI * (double)n / (double)N;
  tw[i] = make_float2((float)cos(th), (float)sin(th));
}

__host__ __device__ inline void rader_entry(const TransferParams& T, const RaderInfo& rb, int i) {
  const int R = rb.R, n = R - 1;
  float2* base = T.table + (size_t)T.C * T.h * T.w + T.h + T.w + rb.off;
  int* perm_in = (int*)(base + 2 * n);
  int* perm_out = perm_in + n;
  long long gp = 1;
  for (int e = 0; e < i; ++e) gp = gp * rb.g % R;
  perm_in[i] = (int)gp;                       // g^i
  long long ginv = 1;
  for (int e = 0; e < n - 1; ++e) ginv = ginv * rb.g % R;  // g^(n-1) = g^-1
  long long gm = 1;
  for (int e = 0; e < i; ++e) gm = gm * ginv % R;
  perm_out[i] = (int)gm;                      // g^-i
  const double th = 2.0 * M_PI * (double)i / (double)n;
  base[n + i] = make_float2((float)cos(th), (float)sin(th));
  // bhat at digit-reversed position i: (1/n) sum_q b_q exp(-2 pi i q f / n), b_q = exp(-2 pi i g^-q / R)
  const int f = pos_to_freq(rb.sub, i);
  double sr = 0.0, si = 0.0;
  long long e = 1;
  for (int q = 0; q < n; ++q) {
    const double a1 = -2.0 * M_PI * (double)e / (double)R;
    const double a2 = -2.0 * M_PI * (double)(((long long)q * f) % n) / (double)n;
    const double br = cos(a1), bi = sin(a1), cr = cos(a2), ci = sin(a2);
    sr += br * cr - bi * ci;
    si += br * ci + bi * cr;
    e = e * ginv % R;
  }
  base[i] = make_float2((float)(sr / n), (float)(si / n));
}

}  // namespace cvb
