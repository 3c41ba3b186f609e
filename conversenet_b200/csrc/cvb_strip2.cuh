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
#include "cvb_tcdft.cuh"

namespace cvb {

// Threads per block: a first radix that is a large prime runs on the tensor cores (cvb_tcdft.cuh)
// with one block of 512 threads per SM; the register-radix plans run two blocks of 256.
CVB_HD constexpr int strip2_threads(int R0) { return R0 > kMaxRegisterRadix ? 512 : 256; }
// lines per strip (columns for A / C, pos_y values for B): the widest of 32 / 16 / 8 whose
// tile stays under ~76 KB, so that three blocks share an SM; 32 (whole accumulator tiles of 128
// vectors) for the tensor-core plans
CVB_HD constexpr int strip2_lines(int N, int R0) {
  return R0 > kMaxRegisterRadix ? 32 : N * 33 * 8 <= 76 * 1024 ? 32 : N * 17 * 8 <= 76 * 1024 ? 16 : 8;
}

// shared memory (bytes) of one block: tile, twiddles, maps / taps, tensor-core operands
CVB_HD size_t strip2_smem(int N, int lines, int R0, int k) {
  const bool big = R0 > kMaxRegisterRadix;
  const size_t f2 = (size_t)N * (lines | 1) + N + (N + lines + 1) / 2 + (k * k + 1) / 2;
  return f2 * sizeof(float2) + (big ? tcdft::bytes(R0) + 128 : 0);
}

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
  float2* tw;
  int* rmap;
  int* cmap;
  float* wk;
  void* tc;   // tensor-core operands of a large-prime plan (128-byte aligned)
};
CVB_HD Strip2Smem strip2_carve(float2* smem, int N, int lines, int k) {
  const int tp = lines | 1;
  Strip2Smem m;
  m.cur = smem;
  m.tw = m.cur + N * tp;
  m.rmap = (int*)(m.tw + N);
  m.cmap = m.rmap + N;
  m.wk = (float*)((float2*)m.rmap + (N + lines + 1) / 2);
  m.tc = (void*)(((uintptr_t)(m.wk + 2 * ((k * k + 1) / 2)) + 127) & ~(uintptr_t)127);
  return m;
}

// one large-prime stage over the whole tile (all threads on the GPU; plain loops on the host)
#define CVB_TC_STAGE(R, R1_, LN_, ctx, cur, tp, tw, pre_, osg_) \
  tcdft::stage<R, R1_, LN_>(ctx, cur, tp, tw, pre_, osg_, nthr_emu)

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
  Strip2Smem m = strip2_carve(smem, h, LN, P.k);
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
    tcdft::Ctx tcx = tcdft::carve<R0>(m.tc, P.status);
    tcdft::setup<R0>(tcx);
    CVB_PHASE((copy_twiddles(tid, nthr, m.tw, blob, h), tile_load_x<IO>(tid, nthr, m.cur, tp, nc, x0, P, io)));
    CVB_TC_STAGE(R0, R1, LN, tcx, m.cur, tp, m.tw, false, 1.0f);
    CVB_PHASE((fft_pass<R1, IO, h, R1, 1, 0, 0>(tid, nthr, a1, io, 0)));
    CVB_PHASE(tileT_to_ws<h>(tid, nthr, m.cur, tp, nc, ST, x0));
    tcdft::finish(tcx);
    return;
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
  Strip2Smem m = strip2_carve(smem, w, LN, P.k);
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
    tcdft::Ctx tcx = tcdft::carve<R0>(m.tc, P.status);
    tcdft::setup<R0>(tcx);
    CVB_PHASE((copy_twiddles(tid, nthr, m.tw, blob + h, w), tile_rows_from_ws(tid, nthr, m.cur, tp, w, nc, ST, h, y0)));
    CVB_TC_STAGE(R0, R1, LN, tcx, m.cur, tp, m.tw, false, 1.0f);
    CVB_PHASE((fft_pass<R1, float, w, R1, 1, 0, PASS_MID>(tid, nthr, a1, io, 0)));
    CVB_TC_STAGE(R0, R1, LN, tcx, m.cur, tp, m.tw, true, 1.0f);
    CVB_PHASE(tile_rows_to_ws(tid, nthr, m.cur, tp, w, nc, ST, h, y0));
    tcdft::finish(tcx);
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
  Strip2Smem m = strip2_carve(smem, h, LN, P.k);
  const float2* blob = P.table + (size_t)P.C * h * w;
  int c;
  IoArgs io = strip_io<IO>(P, SP.pair0 + lp, c);
  io.xoff = x0;
  const float2* ST = SP.ws + (size_t)lp * h * w;
  const PassArgs a0 = strip_pass(m.cur, tp, nt, h, h, R1, m.tw);
  const PassArgs a1 = strip_pass(m.cur, tp, nt, h, R1, 1, m.tw);
  const float* gw = P.weight + (size_t)c * P.k * P.k;
  tcdft::Ctx tcx = tcdft::carve<big ? R0 : 3>(m.tc, P.status);
  if constexpr (big) tcdft::setup<R0>(tcx);
  CVB_PHASE((copy_twiddles(tid, nthr, m.tw, blob, h),
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
    CVB_TC_STAGE(R0, R1, LN, tcx, m.cur, tp, m.tw, true, -1.0f);
    if (P.s == 1) {
      CVB_PHASE(tile_store_crop<IO>(tid, nthr, m.cur, tp, nc, x0, P, io));
    } else {
      CVB_PHASE(tile_epilogue<IO>(tid, nthr, m.cur, tp, nc, x0, hl, m.wk, P, io));
    }
    tcdft::finish(tcx);
  }
}

}  // namespace cvb
