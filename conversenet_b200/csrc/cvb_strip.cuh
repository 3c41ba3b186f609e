// Multi-pass path for planes that do not fit in shared memory (or whose length has a
// prime factor above the largest register butterfly).
//
// The 2-D transform is split into three kernels that meet in a workspace S holding, per
// plane pair, the h x w complex plane (float2):
//   strip_colfwd : a strip of CW columns, full height, in shared memory: read x through
//                  the pad maps, all forward column stages, write S (rows digit-reversed);
//   strip_rowmid : a strip of RH rows, full width: forward row stages, transfer multiply,
//                  inverse row stages, back to S in place;
//   strip_colinv : column strips again (plus the halo columns the s > 1 epilogue needs):
//                  inverse column stages, then crop + store (s == 1) or the upsampling
//                  epilogue.
// Pairs are processed in chunks small enough for S to stay in the 126 MB L2, so the two
// round trips through S cost L2 bandwidth, not HBM bandwidth.
//
// Prime lengths above 23 (43, 67, ...) use a direct O(R^2) conjugate-pair butterfly that
// reads its R inputs from one shared-memory buffer and writes to a second one.
#pragma once
#include "cvb_kernels.cuh"

namespace cvb {

constexpr int kBigPairs = 8;          // output pairs (k, R-k) accumulated per work item
constexpr int kMaxRegisterRadix = 26; // radices above this take the direct butterfly

struct StripParams {
  FwdParams f;
  float2* ws;       // workspace: [pairs_in_chunk][h][w] float2
  int pair0;        // first global pair of this chunk
  int npair;        // pairs in this chunk
  int cw;           // columns per column strip
  int rh;           // rows per row strip
  int halo_l, halo_r;  // extra columns the epilogue reads left / right of a strip (s > 1)
  int big_y, big_x;    // the column / row plan has a large-prime stage (second tile buffer present)
  RaderInfo ry, rx;
};

// ---- direct butterfly for a large prime radix, out of place (src -> dst) ----
// item = (line, butterfly t, group g); group g produces X_0 (g == 0) and the pairs
// (k, R-k) for k = g*kBigPairs+1 .. ; lanes run along lines so the twiddle reads are
// broadcasts.  `post`: multiply output k by W_L^(j k) (forward stage); inverse-type
// stages pre-twiddle with twiddle_sweep() instead.
CVB_HD void bigprime_pass(int tid, int nthr, const float2* src, float2* dst, const PassArgs& a, int R,
                          bool post, float osign) {
  const int hn = (R - 1) / 2;
  const int G = (hn + kBigPairs - 1) / kBigPairs;
  const int nbf = a.N / R;
  const int total = a.nlines * nbf * G;
  const int rstep = a.N / R;  // tw index step for angle 2 pi / R
  const float inv_lg = 1.0f / (float)(a.nlines);
  for (int wi = tid; wi < total; wi += nthr) {
    int rest, line, g, t, blk, j;
    divmod_small(wi, a.nlines, inv_lg, rest, line);
    t = rest / G;
    g = rest - t * G;
    blk = t / a.M;
    j = t - blk * a.M;
    const int base = blk * a.L + j;
    const float2* ip = src + line * a.ls + base * a.es;
    float2* op = dst + line * a.ls + base * a.es;
    const int st = a.M * a.es;
    const int k0 = g * kBigPairs + 1;
    float ar[kBigPairs], ai[kBigPairs], br[kBigPairs], bi[kBigPairs];
    int idx[kBigPairs];
    const float2 x0 = ip[0];
#pragma unroll
    for (int u = 0; u < kBigPairs; ++u) { ar[u] = x0.x; ai[u] = x0.y; br[u] = 0.f; bi[u] = 0.f; idx[u] = 0; }
    float s0r = x0.x, s0i = x0.y;
    for (int q = 1; q <= hn; ++q) {
      const float2 xa = ip[q * st], xb = ip[(R - q) * st];
      const float sr = xa.x + xb.x, si = xa.y + xb.y, dr = xa.x - xb.x, di = xa.y - xb.y;
      s0r += sr; s0i += si;
#pragma unroll
      for (int u = 0; u < kBigPairs; ++u) {
        int m = idx[u] + (k0 + u);
        if (m >= R) m -= R;
        idx[u] = m;  // (q * k) mod R
        const float2 cs = a.tw[m * rstep];
        ar[u] = fmaf(cs.x, sr, ar[u]);
        ai[u] = fmaf(cs.x, si, ai[u]);
        br[u] = fmaf(cs.y, dr, br[u]);
        bi[u] = fmaf(cs.y, di, bi[u]);
      }
    }
    if (g == 0) op[0] = make_float2(s0r, osign * s0i);
#pragma unroll
    for (int u = 0; u < kBigPairs; ++u) {
      const int k = k0 + u;
      if (k > hn) break;
      float x1r = ar[u] + bi[u], x1i = ai[u] - br[u];   // X_k
      float x2r = ar[u] - bi[u], x2i = ai[u] + br[u];   // X_{R-k}
      if (post && a.M > 1) {
        const float2 w1 = a.tw[j * a.tws * k], w2 = a.tw[j * a.tws * (R - k)];
        const float t1r = fmaf(x1i, w1.y, x1r * w1.x), t1i = fmaf(-x1r, w1.y, x1i * w1.x);
        const float t2r = fmaf(x2i, w2.y, x2r * w2.x), t2i = fmaf(-x2r, w2.y, x2i * w2.x);
        x1r = t1r; x1i = t1i; x2r = t2r; x2i = t2i;
      }
      op[k * st] = make_float2(x1r, osign * x1i);
      op[(R - k) * st] = make_float2(x2r, osign * x2i);
    }
  }
}

// In-place multiply of element p of every butterfly by W_L^(j p): the pre-twiddle of an
// inverse-type stage whose butterfly is the out-of-place one above.
CVB_HD void twiddle_sweep(int tid, int nthr, float2* buf, const PassArgs& a, int R) {
  if (a.M <= 1) return;
  const int total = a.nlines * a.N;
  const float inv_nl = 1.0f / (float)a.nlines;
  for (int wi = tid; wi < total; wi += nthr) {
    int e, line;
    divmod_small(wi, a.nlines, inv_nl, e, line);
    const int blk = e / a.L, r = e - blk * a.L;
    const int p = r / a.M, j = r - p * a.M;
    if (p == 0 || j == 0) continue;
    const float2 wv = a.tw[j * p * a.tws];
    float2* ptr = buf + line * a.ls + e * a.es;
    const float2 v = *ptr;
    *ptr = make_float2(fmaf(v.y, wv.y, v.x * wv.x), fmaf(-v.x, wv.y, v.y * wv.x));
  }
}


// ---- Rader stage: shared-memory tables of one axis ----
struct RaderSmem {
  const float2* bhat;   // FFT of the fixed sequence, digit-reversed, scaled by 1/(R-1)
  const float2* tw;     // twiddles of length R-1
  const int* perm_in;   // g^q mod R
  const int* perm_out;  // g^-m mod R
};
CVB_HD int rader_floats2(int R) { return 3 * (R - 1); }  // bhat, tw, two int tables (= one float2 table)
CVB_HD RaderSmem rader_views(const float2* base, int R) {
  RaderSmem r;
  r.bhat = base;
  r.tw = base + (R - 1);
  r.perm_in = (const int*)(base + 2 * (R - 1));
  r.perm_out = r.perm_in + (R - 1);
  return r;
}

// gather: oth[p = q+1] = x[g^q] (pre-twiddled by W_N^(j p) for an inverse-type stage), oth[0] = x[0]
template <int CM = 0>
CVB_HD void rader_gather(int tid, int nthr, const float2* cur, float2* oth, const PassArgs& a, int R,
                         const RaderSmem& rs, bool pre) {
  const int aM = CM ? CM : a.M;
  const int total = a.nlines * aM * R;
  const float inv_nl = 1.0f / (float)a.nlines;
  for (int wi = tid; wi < total; wi += nthr) {
    int rest, line;
    divmod_small(wi, a.nlines, inv_nl, rest, line);
    const int q = rest / aM, j = rest - q * aM;  // q = 0 .. R-1; q == R-1 stands for element 0
    const int src_p = (q == R - 1) ? 0 : rs.perm_in[q];
    const int dst_p = (q == R - 1) ? 0 : q + 1;
    float2 v = cur[line * a.ls + (j + src_p * aM) * a.es];
    if (pre && src_p != 0 && j != 0) {
      const float2 wv = a.tw[j * src_p * a.tws];
      v = make_float2(fmaf(v.y, wv.y, v.x * wv.x), fmaf(-v.x, wv.y, v.y * wv.x));
    }
    oth[line * a.ls + (j + dst_p * aM) * a.es] = v;
  }
}

// X_0 = sum of the (pre-twiddled) inputs, which `oth` now holds; written to its final place in cur
CVB_HD void rader_dc(int tid, int nthr, float2* cur, const float2* oth, const PassArgs& a, int R, float osign) {
  const int total = a.nlines * a.M;
  const float inv_nl = 1.0f / (float)a.nlines;
  for (int wi = tid; wi < total; wi += nthr) {
    int j, line;
    divmod_small(wi, a.nlines, inv_nl, j, line);
    const float2* ip = oth + line * a.ls + j * a.es;
    float sr = 0.f, si = 0.f;
    for (int p = 0; p < R; ++p) {
      const float2 v = ip[p * a.M * a.es];
      sr += v.x; si += v.y;
    }
    cur[line * a.ls + j * a.es] = make_float2(sr, osign * si);
  }
}

// scatter: X[g^-m] = x_0 + conj(c_m), post-twiddled by W_N^(j k) for a forward stage
template <int CM = 0>
CVB_HD void rader_scatter(int tid, int nthr, float2* cur, const float2* oth, const PassArgs& a, int R,
                          const RaderSmem& rs, bool post, float osign) {
  const int aM = CM ? CM : a.M;
  const int total = a.nlines * aM * (R - 1);
  const float inv_nl = 1.0f / (float)a.nlines;
  for (int wi = tid; wi < total; wi += nthr) {
    int rest, line;
    divmod_small(wi, a.nlines, inv_nl, rest, line);
    const int m = rest / aM, j = rest - m * aM;
    const float2* ip = oth + line * a.ls + j * a.es;
    const float2 x0 = ip[0];
    const float2 c = ip[(m + 1) * aM * a.es];
    float vr = x0.x + c.x, vi = x0.y - c.y;
    const int k = rs.perm_out[m];
    if (post && j != 0) {
      const float2 wv = a.tw[j * k * a.tws];
      const float tr = fmaf(vi, wv.y, vr * wv.x), ti = fmaf(-vr, wv.y, vi * wv.x);
      vr = tr; vi = ti;
    }
    cur[line * a.ls + (j + k * aM) * a.es] = make_float2(vr, osign * vi);
  }
}

// PassArgs of stage `i` of the length-(R-1) sub-transform living in `oth` behind element 0
CVB_HD PassArgs rader_sub_pass(float2* oth, const PassArgs& a, const RaderInfo& ri, int i, const RaderSmem& rs) {
  PassArgs s = a;
  s.sm = oth + a.M * a.es;          // element p = 1 of every sub-line
  s.es = a.M * a.es;
  s.nl1 = a.nlines;                 // sub-line (line, j): offset line * ls + j * (outer es)
  s.inv_nl1 = 1.0f / (float)a.nlines;
  s.ls2 = a.es;
  s.nlines = a.nlines * a.M;
  s.inv_nlines = 1.0f / (float)s.nlines;
  s.N = ri.sub.n; s.L = ri.sub.L[i]; s.M = ri.sub.M[i]; s.tws = ri.sub.n / ri.sub.L[i];
  s.invM = 1.0f / (float)s.M;
  s.tw = rs.tw;
  s.tab = rs.bhat; s.tab_es = 1; s.tab_ls = 0;
  return s;
}

// One FFT stage on a shared-memory tile.  Register radices work in place; a large
// prime goes src -> dst and the caller swaps the buffers.  Expands to whole phases.
#define CVB_TILE_STAGE(pl, i, along_y_, cur, oth, tpitch, nlines_, twp, flags_, rinfo, rsm)                \
  do {                                                                                                   \
    PassArgs a_ = make_pass(cur, along_y_, tpitch, 0, 0, (pl).n, (pl).L[i], (pl).M[i], twp);            \
    a_.nlines = (nlines_);                                                                               \
    a_.inv_nlines = 1.0f / (float)(nlines_);                                                             \
    const int R_ = (pl).radix[i];                                                                        \
    const bool pre_ = ((flags_) & PASS_PRE) != 0;                                                        \
    const float osg_ = ((flags_) & PASS_CONJ_OUT) ? -1.0f : 1.0f;                                        \
    if (R_ <= kMaxRegisterRadix) {                                                                       \
      CVB_PHASE((run_pass<float>(R_, tid, nthr, a_, io, (flags_))));                                     \
    } else if ((i) == 0 && (rinfo).R == R_) {                                                            \
      CVB_PHASE(rader_gather(tid, nthr, cur, oth, a_, R_, rsm, pre_));                                   \
      CVB_PHASE(rader_dc(tid, nthr, cur, oth, a_, R_, osg_));                                            \
      const int ns_ = (rinfo).sub.nst;                                                                   \
      for (int u_ = 0; u_ + 1 < ns_; ++u_) {                                                             \
        const PassArgs s_ = rader_sub_pass(oth, a_, rinfo, u_, rsm);                                     \
        CVB_PHASE((run_pass<float>((rinfo).sub.radix[u_], tid, nthr, s_, io, 0)));                       \
      }                                                                                                  \
      {                                                                                                  \
        const PassArgs s_ = rader_sub_pass(oth, a_, rinfo, ns_ - 1, rsm);                                \
        CVB_PHASE((run_pass<float>((rinfo).sub.radix[ns_ - 1], tid, nthr, s_, io, PASS_MID)));           \
      }                                                                                                  \
      for (int u_ = ns_ - 2; u_ >= 0; --u_) {                                                            \
        const PassArgs s_ = rader_sub_pass(oth, a_, rinfo, u_, rsm);                                     \
        CVB_PHASE((run_pass<float>((rinfo).sub.radix[u_], tid, nthr, s_, io, PASS_PRE)));                \
      }                                                                                                  \
      CVB_PHASE(rader_scatter(tid, nthr, cur, oth, a_, R_, rsm, !pre_, osg_));                           \
    } else {                                                                                             \
      if (pre_) CVB_PHASE(twiddle_sweep(tid, nthr, cur, a_, R_));                                        \
      CVB_PHASE(bigprime_pass(tid, nthr, cur, oth, a_, R_, !pre_, osg_));                                \
      float2* t_ = cur; cur = oth; oth = t_;                                                             \
    }                                                                                                    \
  } while (0)

template <typename IO>
CVB_HD IoArgs strip_io(const FwdParams& P, int pair, int& c) {
  int pa, pb;
  pair_planes(P, pair, c, pa, pb);
  return make_io<IO>(P, c, pa, pb);
}

CVB_HD void copy_floats(int tid, int nthr, float* dst, const float* src, int n) {
  for (int i = tid; i < n; i += nthr) dst[i] = src[i];
}
CVB_HD void copy_twiddles(int tid, int nthr, float2* dst, const float2* src, int n) {
  for (int i = tid; i < n; i += nthr) dst[i] = src[i];
}

constexpr int kTileUnroll = 8;  // independent global accesses in flight per thread in the tile copies

// tile[row][col] = padded x at (row, xfirst + col) for both planes; columns wrap modulo w
template <typename IO>
CVB_HD void tile_load_x(int tid, int nthr, float2* tile, int tp, int nc, int xfirst, const FwdParams& P,
                        const IoArgs& io) {
  const float inv_nc = 1.0f / (float)nc;
  const int total = P.h * nc;
  for (int i0 = tid; i0 < total; i0 += nthr * kTileUnroll) {
    float va[kTileUnroll], vb[kTileUnroll];
    int dst[kTileUnroll];
#pragma unroll
    for (int u = 0; u < kTileUnroll; ++u) {
      const int i = i0 + u * nthr;
      va[u] = 0.f; vb[u] = 0.f; dst[u] = -1;
      if (i < total) {
        int row, col;
        divmod_small(i, nc, inv_nc, row, col);
        dst[u] = row * tp + col;
        const int ry = pad_index(row - P.p, P.H, P.pad_mode);
        const int cx = pad_index(xfirst + col - P.p, P.W, P.pad_mode);
        if (ry >= 0 && cx >= 0) {
          const size_t off = (size_t)ry * P.W + cx;
          va[u] = ld_io<IO>(io.xa, off);
          if (io.xb) vb[u] = ld_io<IO>(io.xb, off);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kTileUnroll; ++u)
      if (dst[u] >= 0) tile[dst[u]] = make_float2(va[u], vb[u]);
  }
}

// tile (nr rows x nc cols, pitch tp) <-> S rows ys.. , columns (xfirst + col) mod w
CVB_HD void tile_from_ws(int tid, int nthr, float2* tile, int tp, int nr, int nc, const float2* S, int w,
                         int xfirst) {
  const float inv_nc = 1.0f / (float)nc;
  const int total = nr * nc;
  for (int i0 = tid; i0 < total; i0 += nthr * kTileUnroll) {
    float2 v[kTileUnroll];
    int dst[kTileUnroll];
#pragma unroll
    for (int u = 0; u < kTileUnroll; ++u) {
      const int i = i0 + u * nthr;
      dst[u] = -1;
      v[u] = make_float2(0.f, 0.f);
      if (i < total) {
        int row, col;
        divmod_small(i, nc, inv_nc, row, col);
        int x = xfirst + col;
        if (x < 0) x += w;
        if (x >= w) x -= w;
        dst[u] = row * tp + col;
        v[u] = S[(size_t)row * w + x];
      }
    }
#pragma unroll
    for (int u = 0; u < kTileUnroll; ++u)
      if (dst[u] >= 0) tile[dst[u]] = v[u];
  }
}
CVB_HD void tile_to_ws(int tid, int nthr, const float2* tile, int tp, int nr, int nc, float2* S, int w,
                       int xfirst) {
  const float inv_nc = 1.0f / (float)nc;
  for (int i = tid; i < nr * nc; i += nthr) {
    int row, col;
    divmod_small(i, nc, inv_nc, row, col);
    S[(size_t)row * w + xfirst + col] = tile[row * tp + col];
  }
}

// conj(v * table) on a row strip; table order is [posx][posy], posy fastest across threads
CVB_HD void tile_multiply(int tid, int nthr, float2* tile, int tp, int nr, int w, int h, int y0,
                          const float2* tab) {
  const float inv_nr = 1.0f / (float)nr;
  const int total = nr * w;
  for (int i0 = tid; i0 < total; i0 += nthr * kTileUnroll) {
    float2 g[kTileUnroll];
    int dst[kTileUnroll];
#pragma unroll
    for (int u = 0; u < kTileUnroll; ++u) {
      const int i = i0 + u * nthr;
      dst[u] = -1;
      g[u] = make_float2(0.f, 0.f);
      if (i < total) {
        int posx, r;
        divmod_small(i, nr, inv_nr, posx, r);
        g[u] = tab[(size_t)posx * h + y0 + r];
        dst[u] = r * tp + posx;
      }
    }
#pragma unroll
    for (int u = 0; u < kTileUnroll; ++u) {
      if (dst[u] < 0) continue;
      const float2 v = tile[dst[u]];
      tile[dst[u]] = make_float2(fmaf(-v.y, g[u].y, v.x * g[u].x), -fmaf(v.x, g[u].y, v.y * g[u].x));
    }
  }
}

// ---- kernel 1: column strip, forward column stages -> workspace ----
template <typename IO>
__host__ __device__ void strip_colfwd_body(const StripParams& SP, int lp, int strip, float2* smem, int nthr_emu) {
  (void)nthr_emu;
  const FwdParams& P = SP.f;
  const int h = P.h, w = P.w;
  const int x0 = strip * SP.cw;
  const int nc = (w - x0) < SP.cw ? (w - x0) : SP.cw;
  const int tp = SP.cw | 1;
  const bool big = SP.big_y != 0;
  float2* cur = smem;
  float2* oth = big ? smem + h * tp : smem;
  float2* twy = oth + h * tp;
  float2* rtab = twy + h;
  const int nrt = SP.ry.R ? rader_floats2(SP.ry.R) : 0;
  const RaderSmem rsm = rader_views(rtab, SP.ry.R ? SP.ry.R : 1);
  const float2* blob = P.table + (size_t)P.C * h * w;
  int c;
  const IoArgs io = strip_io<IO>(P, SP.pair0 + lp, c);
  CVB_PHASE((copy_twiddles(tid, nthr, twy, blob, h), copy_twiddles(tid, nthr, rtab, blob + h + w + SP.ry.off, nrt),
             tile_load_x<IO>(tid, nthr, cur, tp, nc, x0, P, io)));
  for (int i = 0; i < P.py.nst; ++i) CVB_TILE_STAGE(P.py, i, true, cur, oth, tp, nc, twy, 0, SP.ry, rsm);
  CVB_PHASE(tile_to_ws(tid, nthr, cur, tp, h, nc, SP.ws + (size_t)lp * h * w, w, x0));
}

// ---- kernel 2: row strip, forward row stages, transfer multiply, inverse row stages ----
__host__ __device__ inline void strip_rowmid_body(const StripParams& SP, int lp, int strip, float2* smem,
                                                 int nthr_emu) {
  (void)nthr_emu;
  const FwdParams& P = SP.f;
  const int h = P.h, w = P.w;
  const int y0 = strip * SP.rh;
  const int nr = (h - y0) < SP.rh ? (h - y0) : SP.rh;
  const int tp = w | 1;
  const bool big = SP.big_x != 0;
  float2* cur = smem;
  float2* oth = big ? smem + SP.rh * tp : smem;
  float2* twx = oth + SP.rh * tp;
  float2* rtab = twx + w;
  const int nrt = SP.rx.R ? rader_floats2(SP.rx.R) : 0;
  const RaderSmem rsm = rader_views(rtab, SP.rx.R ? SP.rx.R : 1);
  const float2* blob = P.table + (size_t)P.C * h * w;
  int c;
  const IoArgs io = strip_io<float>(P, SP.pair0 + lp, c);
  float2* S = SP.ws + (size_t)lp * h * w + (size_t)y0 * w;
  CVB_PHASE((copy_twiddles(tid, nthr, twx, blob + h, w), copy_twiddles(tid, nthr, rtab, blob + h + w + SP.rx.off, nrt),
             tile_from_ws(tid, nthr, cur, tp, nr, w, S, w, 0)));
  for (int i = 0; i < P.px.nst; ++i) CVB_TILE_STAGE(P.px, i, false, cur, oth, tp, nr, twx, 0, SP.rx, rsm);
  CVB_PHASE(tile_multiply(tid, nthr, cur, tp, nr, w, h, y0, io.tab));
  for (int i = P.px.nst - 1; i >= 0; --i) CVB_TILE_STAGE(P.px, i, false, cur, oth, tp, nr, twx, PASS_PRE, SP.rx, rsm);
  CVB_PHASE(tile_to_ws(tid, nthr, cur, tp, nr, w, S, w, 0));
}

// ---- kernel 3: column strip (+ halo), inverse column stages, crop / epilogue ----
// Tile column tc holds plane column (x0 - halo_l + tc) mod w.  At s == 1 the strip's own
// columns are cropped and stored; at s > 1 every output pixel whose low-resolution
// column lies in the strip is produced from the tile (taps reach into the halo).
template <typename IO>
CVB_HD void tile_store_crop(int tid, int nthr, const float2* tile, int tp, int nc, int x0, const FwdParams& P,
                            const IoArgs& io) {
  const float inv_nc = 1.0f / (float)nc;
  for (int i = tid; i < P.H * nc; i += nthr) {
    int oy, col;
    divmod_small(i, nc, inv_nc, oy, col);
    const int ox = x0 + col - P.p;
    if (ox < 0 || ox >= P.W) continue;
    const float2 v = tile[(oy + P.p) * tp + col];
    float va = v.x, vb = v.y;
    if (io.gelu) gelu_pair(va, vb);
    const size_t off = (size_t)oy * P.W + ox;
    st_io<IO>(io.oa, off, va);
    if (io.ob) st_io<IO>(io.ob, off, vb);
  }
}

template <typename IO>
CVB_HD void tile_epilogue(int tid, int nthr, const float2* tile, int tp, int nc, int x0, int halo_l,
                          const float* wk, const FwdParams& P, const IoArgs& io) {
  const int s = P.s, k = P.k, c = P.k / 2, p = P.p, h = P.h;
  const int oW = P.W * s;
  const float inv_nc = 1.0f / (float)nc;
  for (int i = tid; i < P.H * nc; i += nthr) {
    int my, col;
    divmod_small(i, nc, inv_nc, my, col);
    const int mx = x0 + col - p;  // unpadded low-resolution column
    if (mx < 0 || mx >= P.W) continue;
    const size_t xoff = (size_t)my * P.W + mx;
    const float ya = ld_io<IO>(io.xa, xoff);
    const float yb = io.xb ? ld_io<IO>(io.xb, xoff) : 0.f;
    const int m = my + p;
    for (int da = 0; da < s; ++da) {
      for (int db = 0; db < s; ++db) {
        float acca = ya, accb = yb;
        for (int a = 0; a < k; ++a) {
          const int ii = da + a - c;
          const int fi = floordiv(ii, s);
          if (ii - fi * s != 0) continue;
          int rm = m + fi;
          rm %= h; if (rm < 0) rm += h;
          for (int b = 0; b < k; ++b) {
            const int jj = db + b - c;
            const int fj = floordiv(jj, s);
            if (jj - fj * s != 0) continue;
            const float2 rv = tile[rm * tp + (col + halo_l + fj)];
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

template <typename IO>
__host__ __device__ void strip_colinv_body(const StripParams& SP, int lp, int strip, float2* smem, int nthr_emu) {
  (void)nthr_emu;
  const FwdParams& P = SP.f;
  const int h = P.h, w = P.w;
  const int x0 = strip * SP.cw;
  const int nc = (w - x0) < SP.cw ? (w - x0) : SP.cw;
  const int hl = P.s > 1 ? SP.halo_l : 0, hr = P.s > 1 ? SP.halo_r : 0;
  const int nt = nc + hl + hr;              // tile columns
  const int tp = (SP.cw + SP.halo_l + SP.halo_r) | 1;
  const bool big = SP.big_y != 0;
  float2* cur = smem;
  float2* oth = big ? smem + h * tp : smem;
  float2* twy = oth + h * tp;
  float2* rtab = twy + h;
  const int nrt = SP.ry.R ? rader_floats2(SP.ry.R) : 0;
  const RaderSmem rsm = rader_views(rtab, SP.ry.R ? SP.ry.R : 1);
  const float2* blob = P.table + (size_t)P.C * h * w;
  float* wk = (float*)(rtab + nrt);
  int c;
  const IoArgs io = strip_io<IO>(P, SP.pair0 + lp, c);
  const float2* S = SP.ws + (size_t)lp * h * w;
  CVB_PHASE((copy_twiddles(tid, nthr, twy, blob, h), copy_twiddles(tid, nthr, rtab, blob + h + w + SP.ry.off, nrt),
             tile_from_ws(tid, nthr, cur, tp, h, nt, S, w, x0 - hl)));
  if (P.s > 1) {
    const float* gw = P.weight + (size_t)c * P.k * P.k;
    CVB_PHASE(copy_floats(tid, nthr, wk, gw, P.k * P.k));
  }
  for (int i = P.py.nst - 1; i >= 0; --i)
    CVB_TILE_STAGE(P.py, i, true, cur, oth, tp, nt, twy, PASS_PRE | (i == 0 ? PASS_CONJ_OUT : 0), SP.ry, rsm);
  if (P.s == 1) {
    CVB_PHASE(tile_store_crop<IO>(tid, nthr, cur, tp, nc, x0, P, io));
  } else {
    CVB_PHASE(tile_epilogue<IO>(tid, nthr, cur, tp, nc, x0, hl, wk, P, io));
  }
}

}  // namespace cvb
