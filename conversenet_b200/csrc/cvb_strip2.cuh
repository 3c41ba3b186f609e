// Multi-pass path, compile-time axis plans.  Same three kernels as cvb_strip.cuh, but
//   * every axis plan is two stages N = R0 * R1 known at compile time (R0 may be a large
//     prime handled by Rader with a compile-time sub-plan R0 - 1 = S0 * S1);
//   * global traffic is fused into the FFT stages wherever the access is coalesced;
//   * the workspace is kept TRANSPOSED, S^T[pair][x][pos_y], so that the row transform (kernel
//     B) is again a transform along the slow axis: its loads and stores run along pos_y,
//     contiguous, exactly the order of the transfer table.
//
//   A (column strip): x --stage R0 (reads x through the pad maps)--> tile --stage R1--> tile
//                     --transposed copy--> S^T
//   B (pos_y strip):  S^T --stage R0 (reads S^T)--> tile --stage R1 . table . stage R1'--> tile
//                     --stage R0' (writes S^T in place)
//   C (column strip): S^T --transposed copy--> tile --stage R1'--> tile --stage R0'--> crop +
//                     store (s == 1), or tile + upsampling epilogue (s > 1)
#pragma once
#include "cvb_strip.cuh"

namespace cvb {

// A first radix R0 that is a prime beyond the register codelets runs as Rader's algorithm
// with a compile-time sub-plan (516 = 43 * 12).  (Sizes 4 * R0 with a large R0 do not come
// here: their first stage is a dense contraction on the tensor cores, cvb_gemmdft.cuh.)
CVB_HD constexpr bool strip2_rader(int R0) { return R0 > kMaxRegisterRadix; }
CVB_HD constexpr int strip2_threads(int) { return 256; }
// lines per strip (columns for A / C, pos_y values for B): the widest of 32 / 16 / 8 whose
// tile stays under ~76 KB, so that three blocks share an SM
CVB_HD constexpr int strip2_lines(int N, int R0) {
  if (strip2_rader(R0))   // two tile buffers
    return 2 * N * 33 * 8 <= 76 * 1024 ? 32 : 2 * N * 17 * 8 <= 76 * 1024 ? 16 : 8;
  return N * 33 * 8 <= 76 * 1024 ? 32 : N * 17 * 8 <= 76 * 1024 ? 16 : 8;
}

// shared memory (bytes) of one block: tile, twiddles, maps / taps
CVB_HD size_t strip2_smem(int N, int lines, int R0, int k) {
  const size_t f2 = (size_t)(strip2_rader(R0) ? 2 : 1) * N * (lines | 1) + N + (N + lines + 1) / 2 +
                    (k * k + 1) / 2 + (strip2_rader(R0) ? rader_floats2(R0) : 0);
  return f2 * sizeof(float2);
}

// ---- Rader stage with a compile-time sub-plan R - 1 = S0 * S1, gather and scatter fused ----
// Three phases: (1) X_0 by a direct sum + first sub-stage reading its inputs through the g^q
// permutation straight from the tile; (2) second sub-stage with the B-hat multiply and its inverse
// (fft_pass, PASS_MID); (3) inverse first sub-stage writing x_0 + conj(c_m) through the g^-m permutation
// back into the tile.  `oth` holds the length-(R-1) sequences (element p = e + 1) and x_0 at p = 0.
template <int CM>
CVB_HD void rader_dc_fused(int tid, int nthr, float2* cur, float2* oth, const PassArgs& a, int R, bool pre,
                           float osign) {
  const int total = a.nlines * CM;
  const float inv_nl = 1.0f / (float)a.nlines;
  for (int wi = tid; wi < total; wi += nthr) {
    int j, line;
    divmod_small(wi, a.nlines, inv_nl, j, line);
    float2* ip = cur + line * a.ls + j * a.es;
    const float2 x0 = ip[0];
    float sr = x0.x, si = x0.y;
    for (int p = 1; p < R; ++p) {
      float2 v = ip[p * CM * a.es];
      if (pre && j != 0) {
        const float2 wv = a.tw[j * p * a.tws];
        v = make_float2(fmaf(v.y, wv.y, v.x * wv.x), fmaf(-v.x, wv.y, v.y * wv.x));
      }
      sr += v.x; si += v.y;
    }
    oth[line * a.ls + j * a.es] = x0;
    ip[0] = make_float2(sr, osign * si);
  }
}

template <int S0, int S1, int CM>
CVB_HD void rader_first_pass(int tid, int nthr, const float2* cur, float2* oth, const PassArgs& a, int R,
                             const RaderSmem& rs, bool pre) {
  const int total = a.nlines * CM * S1;
  const float inv_nl = 1.0f / (float)a.nlines;
  for (int wi = tid; wi < total; wi += nthr) {
    int rest, line;
    divmod_small(wi, a.nlines, inv_nl, rest, line);
    const int jp = rest / CM, jj = rest - jp * CM;   // butterfly of the sub-transform, outer j
    const float2* bc = cur + line * a.ls + jj * a.es;
    float2* bo = oth + line * a.ls + (jj + CM) * a.es;
    float re[S0], im[S0];
#pragma unroll
    for (int q = 0; q < S0; ++q) {
      const int p = rs.perm_in[jp + S1 * q];
      float2 v = bc[p * CM * a.es];
      if (pre && jj != 0) {
        const float2 wv = a.tw[jj * p * a.tws];
        v = make_float2(fmaf(v.y, wv.y, v.x * wv.x), fmaf(-v.x, wv.y, v.y * wv.x));
      }
      re[q] = v.x; im[q] = v.y;
    }
    Radix<S0>::fwd(re, im);
#pragma unroll
    for (int q = 1; q < S0; ++q) {
      const float2 wv = rs.tw[jp * q];
      const float xr = re[q], xi = im[q];
      re[q] = fmaf(xi, wv.y, xr * wv.x);
      im[q] = fmaf(-xr, wv.y, xi * wv.x);
    }
#pragma unroll
    for (int q = 0; q < S0; ++q) bo[(jp + S1 * q) * CM * a.es] = make_float2(re[q], im[q]);
  }
}

template <int S0, int S1, int CM>
CVB_HD void rader_last_pass(int tid, int nthr, float2* cur, const float2* oth, const PassArgs& a, int R,
                            const RaderSmem& rs, bool post, float osign) {
  const int total = a.nlines * CM * S1;
  const float inv_nl = 1.0f / (float)a.nlines;
  for (int wi = tid; wi < total; wi += nthr) {
    int rest, line;
    divmod_small(wi, a.nlines, inv_nl, rest, line);
    const int jp = rest / CM, jj = rest - jp * CM;
    const float2* bo = oth + line * a.ls + (jj + CM) * a.es;
    float2* bc = cur + line * a.ls + jj * a.es;
    const float2 x0 = oth[line * a.ls + jj * a.es];
    float re[S0], im[S0];
#pragma unroll
    for (int q = 0; q < S0; ++q) {
      const float2 v = bo[(jp + S1 * q) * CM * a.es];
      re[q] = v.x; im[q] = v.y;
    }
#pragma unroll
    for (int q = 1; q < S0; ++q) {
      const float2 wv = rs.tw[jp * q];
      const float xr = re[q], xi = im[q];
      re[q] = fmaf(xi, wv.y, xr * wv.x);
      im[q] = fmaf(-xr, wv.y, xi * wv.x);
    }
    Radix<S0>::fwd(re, im);
#pragma unroll
    for (int q = 0; q < S0; ++q) {
      const int k = rs.perm_out[jp + S1 * q];
      float vr = x0.x + re[q], vi = x0.y - im[q];   // x_0 + conj(c_m)
      if (post && jj != 0) {
        const float2 wv = a.tw[jj * k * a.tws];
        const float tr = fmaf(vi, wv.y, vr * wv.x), ti = fmaf(-vr, wv.y, vi * wv.x);
        vr = tr; vi = ti;
      }
      bc[k * CM * a.es] = make_float2(vr, osign * vi);
    }
  }
}

#define CVB_RADER_STATIC(R, R1_, S0, S1, cur, oth, a_, rinfo, rsm, pre_, osg_)                              \
  do {                                                                                                    \
    CVB_PHASE((rader_dc_fused<R1_>(tid, nthr, cur, oth, a_, R, pre_, osg_),                               \
               rader_first_pass<S0, S1, R1_>(tid, nthr, cur, oth, a_, R, rsm, pre_)));                    \
    {                                                                                                     \
      const PassArgs s_ = rader_sub_pass(oth, a_, rinfo, 1, rsm);                                         \
      CVB_PHASE((fft_pass<S1, float, R - 1, S1, 1, 0, PASS_MID>(tid, nthr, s_, io, 0)));                  \
    }                                                                                                     \
    CVB_PHASE((rader_last_pass<S0, S1, R1_>(tid, nthr, cur, oth, a_, R, rsm, !(pre_), osg_)));            \
  } while (0)

CVB_HD PassArgs strip_pass(float2* tile, int tp, int nlines, int N, int L, int M, const float2* tw) {
  PassArgs a = make_pass(tile, true, tp, 0, 0, N, L, M, tw);
  a.nlines = nlines;
  a.inv_nlines = 1.0f / (float)nlines;
  return a;
}

// tile[r][c] <-> S^T[(xfirst + c) mod w][r].  A warp takes one column c at a time with its lanes
// along r (contiguous in S^T, odd stride tp in the tile), so no index is divided; all loads of a
// column are issued before the first store.
template <int H>
CVB_HD void tileT_from_ws(int tid, int nthr, float2* tile, int tp, int nc, const float2* ST, int w, int xfirst) {
  constexpr int U = (H + 31) / 32;
  const int nwarps = nthr >= 32 ? nthr / 32 : 1, lanes = nthr >= 32 ? 32 : nthr;
  const int warp = tid / lanes, lane = tid % lanes;
  if (warp >= nwarps) return;
  for (int c = warp; c < nc; c += nwarps) {
    int x = xfirst + c;
    if (x < 0) x += w;
    if (x >= w) x -= w;
    const float2* src = ST + (size_t)x * H;
    for (int r0 = lane; r0 < 32; r0 += lanes) {  // one trip on the GPU; covers short emulated warps
      float2 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int r = r0 + 32 * u;
        v[u] = (r < H) ? src[r] : make_float2(0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int r = r0 + 32 * u;
        if (r < H) tile[r * tp + c] = v[u];
      }
    }
  }
}
template <int H>
CVB_HD void tileT_to_ws(int tid, int nthr, const float2* tile, int tp, int nc, float2* ST, int xfirst) {
  constexpr int U = (H + 31) / 32;
  const int nwarps = nthr >= 32 ? nthr / 32 : 1, lanes = nthr >= 32 ? 32 : nthr;
  const int warp = tid / lanes, lane = tid % lanes;
  if (warp >= nwarps) return;
  for (int c = warp; c < nc; c += nwarps) {
    float2* dst = ST + (size_t)(xfirst + c) * H;
    for (int r0 = lane; r0 < 32; r0 += lanes) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int r = r0 + 32 * u;
        if (r < H) dst[r] = tile[r * tp + c];
      }
    }
  }
}
// tile[x][c] <-> S^T[x][y0 + c], lanes along c
CVB_HD void tile_rows_from_ws(int tid, int nthr, float2* tile, int tp, int w, int nc, const float2* ST, int h,
                              int y0) {
  const float inv_nc = 1.0f / (float)nc;
  const int total = w * nc;
  for (int i0 = tid; i0 < total; i0 += nthr * kTileUnroll) {
    float2 v[kTileUnroll];
    int dst[kTileUnroll];
#pragma unroll
    for (int u = 0; u < kTileUnroll; ++u) {
      const int i = i0 + u * nthr;
      dst[u] = -1;
      v[u] = make_float2(0.f, 0.f);
      if (i < total) {
        int x, c;
        divmod_small(i, nc, inv_nc, x, c);
        dst[u] = x * tp + c;
        v[u] = ST[(size_t)x * h + y0 + c];
      }
    }
#pragma unroll
    for (int u = 0; u < kTileUnroll; ++u)
      if (dst[u] >= 0) tile[dst[u]] = v[u];
  }
}
CVB_HD void tile_rows_to_ws(int tid, int nthr, const float2* tile, int tp, int w, int nc, float2* ST, int h,
                            int y0) {
  const float inv_nc = 1.0f / (float)nc;
  for (int i = tid; i < w * nc; i += nthr) {
    int x, c;
    divmod_small(i, nc, inv_nc, x, c);
    ST[(size_t)x * h + y0 + c] = tile[x * tp + c];
  }
}

// ---- tile <-> global copies of the large-prime plans: a warp covers 32 / LN_ tile rows at a time
// with LN_ lanes along the lines (contiguous in global memory), four row groups in flight, and no
// index is divided ----
template <int LN_>
struct LaneMap {
  static constexpr int RPW = 32 / LN_;   // tile rows per warp and step
  int lc, row0, step;                    // lane's line, first row, row stride
  CVB_HD LaneMap(int tid, int nthr) {
    const int lanes = nthr >= 32 ? 32 : nthr;   // short "warps" only in the host emulation
    const int nwarps = nthr / lanes, warp = tid / lanes, lane = tid % lanes;
    lc = lane % LN_;
    row0 = warp * RPW + lane / LN_;
    step = nwarps * RPW;
    if (warp >= nwarps || lane / LN_ >= RPW) row0 = 1 << 30;   // idle thread
  }
};

// x (through the pad maps) -> tile[r][c]
// U: row groups in flight per thread (a block of 256 threads covers the tile in one trip when
// U = ceil(rows / (8 * RPW)), so that the whole tile is one round of memory latency)
template <typename IO, int LN_, int U>
CVB_HD void tile_load_maps(int tid, int nthr, float2* tile, int tp, int nc, int h, const int* rmap,
                           const int* cmap, const IoArgs& io) {
  const LaneMap<LN_> lm(tid, nthr);
  if (lm.lc >= nc) return;
  const int cx = cmap[lm.lc];
  for (int r0 = lm.row0; r0 < h; r0 += U * lm.step) {
    float va[U], vb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int r = r0 + u * lm.step;
      va[u] = 0.f; vb[u] = 0.f;
      if (r < h) {
        const int ro = rmap[r];
        if ((ro | cx) >= 0) {
          va[u] = ld_io<IO>(io.xa, (size_t)(ro + cx));
          if (io.xb) vb[u] = ld_io<IO>(io.xb, (size_t)(ro + cx));
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int r = r0 + u * lm.step;
      if (r < h) tile[r * tp + lm.lc] = make_float2(va[u], vb[u]);
    }
  }
}

// tile[x][c] <-> S^T[x][y0 + c]
template <int LN_, int U>
CVB_HD void tile_rows_from_ws2(int tid, int nthr, float2* tile, int tp, int w, int nc, const float2* ST, int h,
                               int y0) {
  const LaneMap<LN_> lm(tid, nthr);
  if (lm.lc >= nc) return;
  const float2* src = ST + y0 + lm.lc;
  for (int x0 = lm.row0; x0 < w; x0 += U * lm.step) {
    float2 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int x = x0 + u * lm.step;
      v[u] = x < w ? src[(size_t)x * h] : make_float2(0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int x = x0 + u * lm.step;
      if (x < w) tile[x * tp + lm.lc] = v[u];
    }
  }
}
template <int LN_>
CVB_HD void tile_rows_to_ws2(int tid, int nthr, const float2* tile, int tp, int w, int nc, float2* ST, int h,
                             int y0) {
  const LaneMap<LN_> lm(tid, nthr);
  if (lm.lc >= nc) return;
  float2* dst = ST + y0 + lm.lc;
  for (int x = lm.row0; x < w; x += lm.step) dst[(size_t)x * h] = tile[x * tp + lm.lc];
}

// tile -> out, cropped (s == 1), optional GELU
template <typename IO, int LN_>
CVB_HD void tile_store_crop2(int tid, int nthr, const float2* tile, int tp, int nc, int x0, const FwdParams& P,
                             const IoArgs& io) {
  const LaneMap<LN_> lm(tid, nthr);
  const int ox = x0 + lm.lc - P.p;
  if (lm.lc >= nc || ox < 0 || ox >= P.W) return;
  for (int oy = lm.row0; oy < P.H; oy += lm.step) {
    const float2 v = tile[(oy + P.p) * tp + lm.lc];
    float va = v.x, vb = v.y;
    if (io.gelu) gelu_pair(va, vb);
    const size_t off = (size_t)oy * P.W + ox;
    st_io<IO>(io.oa, off, va);
    if (io.ob) st_io<IO>(io.ob, off, vb);
  }
}

CVB_HD void strip_maps(int tid, int nthr, int* rmap, int* cmap, int x0, int nc, const FwdParams& P) {
  for (int i = tid; i < P.h; i += nthr) {
    const int ry = pad_index(i - P.p, P.H, P.pad_mode);
    rmap[i] = ry < 0 ? -1 : ry * P.W;
  }
  for (int i = tid; i < nc; i += nthr) cmap[i] = pad_index(x0 + i - P.p, P.W, P.pad_mode);
}


// carve one block's shared memory
struct Strip2Smem {
  float2* cur;
  float2* oth;   // second tile buffer of a Rader plan
  float2* tw;
  float2* rtab;  // Rader tables
  int* rmap;
  int* cmap;
  float* wk;
};
CVB_HD Strip2Smem strip2_carve(float2* smem, int N, int lines, int k, int R0) {
  const int tp = lines | 1;
  const bool rad = strip2_rader(R0);
  Strip2Smem m;
  m.cur = smem;
  m.oth = rad ? smem + N * tp : smem;
  m.tw = m.oth + N * tp;
  m.rtab = m.tw + N;
  m.rmap = (int*)(m.rtab + (rad ? rader_floats2(R0) : 0));
  m.cmap = m.rmap + N;
  m.wk = (float*)((float2*)m.rmap + (N + lines + 1) / 2);
  return m;
}

// ---- A: column strip forward ----
template <typename IO, int R0, int R1, int S0, int S1>
__host__ __device__ void strip2_A_body(const StripParams& SP, int lp, int strip, float2* smem, int nthr_emu) {
  (void)nthr_emu;
  constexpr int h = R0 * R1;
  constexpr int LN = strip2_lines(h, R0);
  constexpr bool big = R0 > kMaxRegisterRadix;
  const FwdParams& P = SP.f;
  const int w = P.w;
  const int x0 = strip * LN;
  const int nc = (w - x0) < LN ? (w - x0) : LN;
  constexpr int tp = LN | 1;
  Strip2Smem m = strip2_carve(smem, h, LN, P.k, R0);
  const float2* blob = P.table + (size_t)P.C * h * w;
  int c;
  IoArgs io = strip_io<IO>(P, SP.pair0 + lp, c);
  io.rmap = m.rmap;
  io.cmap = m.cmap;
  float2* ST = SP.ws + (size_t)lp * h * w;
  const PassArgs a0 = strip_pass(m.cur, tp, nc, h, h, R1, m.tw);
  const PassArgs a1 = strip_pass(m.cur, tp, nc, h, R1, 1, m.tw);
  if constexpr (!big) {
    CVB_PHASE((copy_twiddles(tid, nthr, m.tw, blob, h), strip_maps(tid, nthr, m.rmap, m.cmap, x0, nc, P)));
    CVB_PHASE((fft_pass<R0, IO, h, h, R1, 0, PASS_SRC_GLOBAL>(tid, nthr, a0, io, 0)));
  } else {
    const RaderSmem rsm = rader_views(m.rtab, R0);
    CVB_PHASE(strip_maps(tid, nthr, m.rmap, m.cmap, x0, nc, P));
    CVB_PHASE((copy_twiddles(tid, nthr, m.tw, blob, h),
               copy_twiddles(tid, nthr, m.rtab, blob + h + w + SP.ry.off, rader_floats2(R0)),
               tile_load_maps<IO, LN, (h * LN + 255) / 256>(tid, nthr, m.cur, tp, nc, h, m.rmap, m.cmap, io)));
    CVB_RADER_STATIC(R0, R1, S0, S1, m.cur, m.oth, a0, SP.ry, rsm, false, 1.0f);
  }
  CVB_PHASE((fft_pass<R1, IO, h, R1, 1, 0, 0>(tid, nthr, a1, io, 0)));
  CVB_PHASE(tileT_to_ws<h>(tid, nthr, m.cur, tp, nc, ST, x0));
}

// ---- B: strip of pos_y values, row transform both ways with the transfer multiply ----
template <int R0, int R1, int S0, int S1>
__host__ __device__ void strip2_B_body(const StripParams& SP, int lp, int strip, float2* smem, int nthr_emu) {
  (void)nthr_emu;
  constexpr int w = R0 * R1;
  constexpr int LN = strip2_lines(w, R0);
  constexpr bool big = R0 > kMaxRegisterRadix;
  const FwdParams& P = SP.f;
  const int h = P.h;
  const int y0 = strip * LN;
  const int nc = (h - y0) < LN ? (h - y0) : LN;
  constexpr int tp = LN | 1;
  Strip2Smem m = strip2_carve(smem, w, LN, P.k, R0);
  const float2* blob = P.table + (size_t)P.C * h * w;
  int c;
  IoArgs io = strip_io<float>(P, SP.pair0 + lp, c);
  float2* ST = SP.ws + (size_t)lp * h * w;
  io.ws = ST + y0;   // line = pos_y - y0, element x at stride h
  io.wes = h;
  io.wls = 1;
  io.tab = io.tab + y0;  // table order [posx][posy]
  io.h = h;
  const PassArgs a0 = strip_pass(m.cur, tp, nc, w, w, R1, m.tw);
  const PassArgs a1 = strip_pass(m.cur, tp, nc, w, R1, 1, m.tw);
  if constexpr (!big) {
    CVB_PHASE(copy_twiddles(tid, nthr, m.tw, blob + h, w));
    CVB_PHASE((fft_pass<R0, float, w, w, R1, 0, PASS_SRC_WS>(tid, nthr, a0, io, 0)));
    CVB_PHASE((fft_pass<R1, float, w, R1, 1, 0, PASS_MID>(tid, nthr, a1, io, 0)));
    CVB_PHASE((fft_pass<R0, float, w, w, R1, 0, PASS_PRE | PASS_DST_WS>(tid, nthr, a0, io, 0)));
  } else {
    const RaderSmem rsm = rader_views(m.rtab, R0);
    CVB_PHASE((copy_twiddles(tid, nthr, m.tw, blob + h, w),
               copy_twiddles(tid, nthr, m.rtab, blob + h + w + SP.rx.off, rader_floats2(R0)),
               tile_rows_from_ws2<LN, (w * LN + 255) / 256>(tid, nthr, m.cur, tp, w, nc, ST, h, y0)));
    CVB_RADER_STATIC(R0, R1, S0, S1, m.cur, m.oth, a0, SP.rx, rsm, false, 1.0f);
    CVB_PHASE((fft_pass<R1, float, w, R1, 1, 0, PASS_MID>(tid, nthr, a1, io, 0)));
    CVB_RADER_STATIC(R0, R1, S0, S1, m.cur, m.oth, a0, SP.rx, rsm, true, 1.0f);
    CVB_PHASE(tile_rows_to_ws2<LN>(tid, nthr, m.cur, tp, w, nc, ST, h, y0));
  }
}

// ---- C: column strip inverse, crop / epilogue ----
template <typename IO, int R0, int R1, int S0, int S1>
__host__ __device__ void strip2_C_body(const StripParams& SP, int lp, int strip, float2* smem, int nthr_emu) {
  (void)nthr_emu;
  constexpr int h = R0 * R1;
  constexpr int LN = strip2_lines(h, R0);
  constexpr bool big = R0 > kMaxRegisterRadix;
  const FwdParams& P = SP.f;
  const int w = P.w;
  const int hl = P.s > 1 ? SP.halo_l : 0, hr = P.s > 1 ? SP.halo_r : 0;
  const int cw = LN - SP.halo_l - SP.halo_r;  // plane columns owned by a strip
  const int x0 = strip * cw;
  const int nc = (w - x0) < cw ? (w - x0) : cw;
  const int nt = nc + hl + hr;
  constexpr int tp = LN | 1;
  Strip2Smem m = strip2_carve(smem, h, LN, P.k, R0);
  const float2* blob = P.table + (size_t)P.C * h * w;
  int c;
  IoArgs io = strip_io<IO>(P, SP.pair0 + lp, c);
  io.xoff = x0;
  const float2* ST = SP.ws + (size_t)lp * h * w;
  const PassArgs a0 = strip_pass(m.cur, tp, nt, h, h, R1, m.tw);
  const PassArgs a1 = strip_pass(m.cur, tp, nt, h, R1, 1, m.tw);
  const float* gw = P.weight + (size_t)c * P.k * P.k;
  constexpr bool rad = strip2_rader(R0);
  CVB_PHASE((copy_twiddles(tid, nthr, m.tw, blob, h),
             copy_twiddles(tid, nthr, m.rtab, blob + h + w + SP.ry.off, rad ? rader_floats2(R0) : 0),
             copy_floats(tid, nthr, m.wk, gw, P.s > 1 ? P.k * P.k : 0),
             tileT_from_ws<h>(tid, nthr, m.cur, tp, nt, ST, w, x0 - hl)));
  CVB_PHASE((fft_pass<R1, float, h, R1, 1, 0, PASS_PRE>(tid, nthr, a1, io, 0)));
  if constexpr (!big) {
    if (P.s == 1) {
      CVB_PHASE((fft_pass<R0, IO, h, h, R1, 0, PASS_PRE | PASS_CONJ_OUT | PASS_DST_GLOBAL>(tid, nthr, a0, io, 0)));
    } else {
      CVB_PHASE((fft_pass<R0, IO, h, h, R1, 0, PASS_PRE | PASS_CONJ_OUT>(tid, nthr, a0, io, 0)));
      CVB_PHASE(tile_epilogue<IO>(tid, nthr, m.cur, tp, nc, x0, hl, m.wk, P, io));
    }
  } else {
    const RaderSmem rsm = rader_views(m.rtab, R0);
    CVB_RADER_STATIC(R0, R1, S0, S1, m.cur, m.oth, a0, SP.ry, rsm, true, -1.0f);
    if (P.s == 1) {
      CVB_PHASE((tile_store_crop2<IO, LN>(tid, nthr, m.cur, tp, nc, x0, P, io)));
    } else {
      CVB_PHASE(tile_epilogue<IO>(tid, nthr, m.cur, tp, nc, x0, hl, m.wk, P, io));
    }
  }
}

}  // namespace cvb
