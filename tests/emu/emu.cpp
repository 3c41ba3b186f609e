// Host emulation of the CUDA block bodies -- TEST BUILD ONLY, never part of the product library.
// The kernels are written as per-thread phase functions; compiled for the host a phase
// is a loop over thread ids, so the index arithmetic of whole blocks (padding maps,
// digit-reversed table order, butterfly addressing, crop, epilogue taps) is
// checked against the oracle on a machine without a GPU.
#include <vector>
#include <cstdio>
#include "../../conversenet_b200/csrc/cvb_plan.h"
#include "../../conversenet_b200/csrc/cvb_strip2.cuh"
#include "../../conversenet_b200/csrc/cvb_block.cuh"

using namespace cvb;

template <typename FA, typename FB, typename FC>
static void run_strip2(StripParams& SP, int npairs, int chunk, std::vector<float2>& smem, int nthr, FA fa, FB fb,
                       FC fc, int lny, int lnx) {
  const FwdParams& P = SP.f;
  const int cwc = lny - SP.halo_l - SP.halo_r;
  const int nA = (P.w + lny - 1) / lny, nB = (P.h + lnx - 1) / lnx, nC = (P.w + cwc - 1) / cwc;
  for (int p0 = 0; p0 < npairs; p0 += chunk) {
    SP.pair0 = p0;
    SP.npair = (npairs - p0) < chunk ? (npairs - p0) : chunk;
    for (int lp = 0; lp < SP.npair; ++lp) for (int st = 0; st < nA; ++st) fa(SP, lp, st, smem.data(), nthr);
    for (int lp = 0; lp < SP.npair; ++lp) for (int st = 0; st < nB; ++st) fb(SP, lp, st, smem.data(), nthr);
    for (int lp = 0; lp < SP.npair; ++lp) for (int st = 0; st < nC; ++st) fc(SP, lp, st, smem.data(), nthr);
  }
}


extern "C" {

static int build_table(const float* weight, const float* bias, int C, int k, int s, int h, int w,
                       float eps, void* table, int kind) {
  TransferParams T;
  if (!make_plan(h, T.py) || !make_plan(w, T.px)) return -3;
  T.weight = weight; T.bias = bias; T.table = (float2*)table;
  T.C = C; T.k = k; T.s = s; T.h = h; T.w = w; T.eps = eps; T.kind = kind;
  if (s <= kFastMaxScale) {
    // tiled build, as the CUDA library launches it
    static TransferTileSmem S;
    const long long nblk = (long long)C * ((w + kTransferTile - 1) / kTransferTile);
    for (long long blk = 0; blk < nblk; ++blk) {
      switch (k * 10 + s) {
#define X(KK, SS) case KK * 10 + SS: transfer_tile_block<KK, SS>(T, blk, 64, S); break;
        CVB_TRANSFER_CASES(X)
#undef X
        default: transfer_tile_block<0, 0>(T, blk, 64, S); break;
      }
    }
  } else {
    for (int c = 0; c < C; ++c)
      for (int px = 0; px < w; ++px)
        for (int py = 0; py < h; ++py) transfer_entry(T, c, py, px);
  }
  for (int i = 0; i < h + w; ++i) twiddle_entry(T, i);
  rader_both(T.py, T.px, T.ry, T.rx);
  for (int i = 0; T.ry.R && i < T.ry.R - 1; ++i) rader_entry(T, T.ry, i);
  for (int i = 0; T.rx.R && i < T.rx.R - 1; ++i) rader_entry(T, T.rx, i);
  return 0;
}

int emu_build_transfer(const float* weight, const float* bias, int C, int k, int s, int h, int w,
                       float eps, void* table) {
  return build_table(weight, bias, C, k, s, h, w, eps, table, 0);
}
// the x0 term's table: 1 / (alias mean of |FK|^2 + lambda)
int emu_build_x0_table(const float* weight, const float* bias, int C, int k, int s, int h, int w,
                       float eps, void* table) {
  return build_table(weight, bias, C, k, s, h, w, eps, table, 1);
}

// variant: 0 = runtime-plan body, 1 = compile-time-plan body (only for the sizes instantiated below)
int emu_converse2d_fwd(const float* x, float* out, const void* table, const float* weight, int B, int C,
                       int H, int W, int k, int s, int p, int pad_mode, int fuse_gelu, int nthr,
                       int variant) {
  FwdParams P;
  P.x = x; P.out = out; P.table = (const float2*)table; P.weight = weight;
  P.B = B; P.C = C; P.H = H; P.W = W; P.k = k; P.s = s; P.p = p; P.pad_mode = pad_mode;
  P.fuse_gelu = fuse_gelu;
  P.h = H + 2 * p; P.w = W + 2 * p; P.pitch = P.w | 1;
  P.skip_mask = 0;
  P.ystash = (variant & 2) ? 0 : choose_ystash(P.h, P.w, k, s);
  if (!make_plan(P.h, P.py) || !make_plan(P.w, P.px)) return -3;
  std::vector<float2> smem(smem_bytes_for(P.h, P.w, k, 1) / sizeof(float2) + 16);
  const int pairs = C * ((B + 1) / 2);
  P.status = nullptr;
  if (variant & 4) {
    // persistent body: 3 emulated blocks share the pairs round-robin
    if (!(P.h == 68 && P.w == 68)) return -100;
    P.ystash = 0;
    std::vector<unsigned char> ps(persistent_smem_bytes(P.h, P.w, H, W, k, 4) + 256);
    unsigned char* base = (unsigned char*)(((size_t)ps.data() + 127) / 128 * 128);
    for (int b = 0; b < 3; ++b) smem_persistent_static<float, 17, 4, 17, 4, 272>(P, base, b, 3);
    return 0;
  }
  for (int pair = 0; pair < pairs; ++pair) {
    if ((variant & 1) == 0) {
      smem_block_dynamic<float>(P, pair, smem.data(), nthr);
    } else if (P.h == 68 && P.w == 68) {
      smem_block_static<float, 17, 4, 17, 4, 272>(P, pair, smem.data());
    } else if (P.h == 34 && P.w == 42) {
      smem_block_static<float, 17, 2, 7, 6, 96>(P, pair, smem.data());
    } else if (P.h == 36 && P.w == 44) {
      smem_block_static<float, 6, 6, 11, 4, 160>(P, pair, smem.data());
    } else {
      return -100;
    }
  }
  return 0;
}

// The multi-pass path: the three strip kernels run block by block over a host workspace.
int emu_converse2d_strip(const float* x, float* out, const void* table, const float* weight, int B, int C,
                         int H, int W, int k, int s, int p, int pad_mode, int fuse_gelu, int nthr) {
  FwdParams P;
  P.x = x; P.out = out; P.table = (const float2*)table; P.weight = weight;
  P.B = B; P.C = C; P.H = H; P.W = W; P.k = k; P.s = s; P.p = p; P.pad_mode = pad_mode;
  P.fuse_gelu = fuse_gelu;
  P.h = H + 2 * p; P.w = W + 2 * p; P.pitch = P.w | 1;
  P.skip_mask = 0; P.ystash = 0; P.status = nullptr;
  if (!make_plan(P.h, P.py) || !make_plan(P.w, P.px)) return -3;
  const int npairs = C * ((B + 1) / 2);
  StripGeo g = strip_geometry(P.h, P.w, k, s, npairs);
  if (g.chunk_pairs > 3) g.chunk_pairs = 3;  // exercise the chunk loop
  std::vector<float2> ws((size_t)g.chunk_pairs * P.h * P.w);
  std::vector<float2> smem((g.smem_col > g.smem_row ? g.smem_col : g.smem_row) / sizeof(float2) + 16);
  StripParams SP;
  SP.f = P; SP.ws = ws.data(); SP.cw = g.cw; SP.rh = g.rh; SP.halo_l = g.halo_l; SP.halo_r = g.halo_r;
  SP.big_y = plan_has_big(P.py) ? 1 : 0; SP.big_x = plan_has_big(P.px) ? 1 : 0;
  rader_both(P.py, P.px, SP.ry, SP.rx);
  if (nthr < 0) { nthr = -nthr; SP.ry.R = 0; SP.rx.R = 0; }  // negative thread count: direct large-prime butterflies
  const int ncs = (P.w + g.cw - 1) / g.cw, nrs = (P.h + g.rh - 1) / g.rh;
  for (int p0 = 0; p0 < npairs; p0 += g.chunk_pairs) {
    SP.pair0 = p0;
    SP.npair = (npairs - p0) < g.chunk_pairs ? (npairs - p0) : g.chunk_pairs;
    for (int lp = 0; lp < SP.npair; ++lp)
      for (int st = 0; st < ncs; ++st) strip_colfwd_body<float>(SP, lp, st, smem.data(), nthr);
    for (int lp = 0; lp < SP.npair; ++lp)
      for (int st = 0; st < nrs; ++st) strip_rowmid_body(SP, lp, st, smem.data(), nthr);
    for (int lp = 0; lp < SP.npair; ++lp)
      for (int st = 0; st < ncs; ++st) strip_colinv_body<float>(SP, lp, st, smem.data(), nthr);
  }
  return 0;
}

// The multi-pass path with compile-time axis plans (transposed workspace), for the two plane
// sizes instantiated here: 34 x 42 = (17*2) x (7*6) and 58 x 86 = (29*2) x (43*2) with Rader.
int emu_converse2d_strip2(const float* x, float* out, const void* table, const float* weight, int B, int C,
                          int H, int W, int k, int s, int p, int pad_mode, int fuse_gelu, int nthr) {
  FwdParams P;
  P.x = x; P.out = out; P.table = (const float2*)table; P.weight = weight;
  P.B = B; P.C = C; P.H = H; P.W = W; P.k = k; P.s = s; P.p = p; P.pad_mode = pad_mode;
  P.fuse_gelu = fuse_gelu;
  P.h = H + 2 * p; P.w = W + 2 * p; P.pitch = P.w | 1;
  P.skip_mask = 0; P.ystash = 0; P.status = nullptr;
  if (!make_plan(P.h, P.py) || !make_plan(P.w, P.px)) return -3;
  const int npairs = C * ((B + 1) / 2);
  StripGeo g = strip_geometry(P.h, P.w, k, s, npairs);
  std::vector<float2> ws((size_t)2 * P.h * P.w);
  std::vector<float2> smem((strip2_smem(128, 32, 127, k) + strip2_smem(128, 32, 43, k)) / sizeof(float2) + 64);
  StripParams SP;
  SP.f = P; SP.ws = ws.data(); SP.cw = g.cw; SP.rh = g.rh; SP.halo_l = g.halo_l; SP.halo_r = g.halo_r;
  SP.big_y = plan_has_big(P.py) ? 1 : 0; SP.big_x = plan_has_big(P.px) ? 1 : 0;
  rader_both(P.py, P.px, SP.ry, SP.rx);
  if (P.h == 34 && P.w == 42) {
    run_strip2(SP, npairs, 2, smem, nthr, strip2_A_body<float, 17, 2, 0, 0>, strip2_B_body<7, 6, 0, 0>,
               strip2_C_body<float, 17, 2, 0, 0>, strip2_lines(34, 17), strip2_lines(42, 7));
  } else if (P.h == 58 && P.w == 86) {
    run_strip2(SP, npairs, 2, smem, nthr, strip2_A_body<float, 29, 2, 7, 4>, strip2_B_body<43, 2, 7, 6>,
               strip2_C_body<float, 29, 2, 7, 4>, strip2_lines(58, 29), strip2_lines(86, 43));
  } else {
    return -100;
  }
  return 0;
}

// batch-summed cross spectrum: every (channel, segment) block in turn; `tw` = twiddles of h then w
int emu_cross_spectrum(const float* x, const float* q, const void* tw, void* out, int nseg, int B, int C, int H,
                       int W, int p, int pad_mode, int nthr, int direct) {
  XspecParams Q;
  Q.x = x; Q.q = q; Q.out = (float2*)out; Q.tw = (const float2*)tw;
  Q.B = B; Q.C = C; Q.H = H; Q.W = W; Q.p = p; Q.pad_mode = pad_mode;
  Q.h = H + 2 * p; Q.w = W + 2 * p; Q.pitch = Q.w | 1; Q.nseg = nseg;
  if (!make_plan(Q.h, Q.py) || !make_plan(Q.w, Q.px)) return -3;
  if (plan_has_big(Q.py) || plan_has_big(Q.px)) return -4;
  Q.direct = direct;
  std::vector<float2> smem(xspec_smem_bytes(Q.h, Q.w, direct) / sizeof(float2) + 16);
  for (int c = 0; c < C; ++c)
    for (int seg = 0; seg < nseg; ++seg) smem_block_xspec(Q, c, seg, smem.data(), nthr);
  return 0;
}

// the kernels' GELU on an array
int emu_gelu(const float* in, float* out, int n) {
  for (int i = 0; i < n; ++i) out[i] = gelu_erf(in[i]);
  return 0;
}

// Fused channel-mixing kernels of ConverseBlock, one emulated block of `nthr` threads at a time.
int emu_ln_pw_gelu(const float* x, float* out, const float* ln_w, const float* ln_b, float eps, const float* w,
                   const float* b, int B, int HW, int nthr) {
  BlockParams P;
  memset(&P, 0, sizeof(P));
  P.x = x; P.out = out; P.ln_w = ln_w; P.ln_b = ln_b; P.ln_eps = eps; P.w_a = w; P.b_a = b; P.B = B; P.HW = HW;
  std::vector<float> sm(kBlkC * kBlkM + kBlkM);
  for (int t = 0; t < nthr; ++t) k1_stage(t, nthr, P, sm.data(), sm.data() + kBlkC * kBlkM);
  const long long total = (long long)B * HW;
  for (long long blk = 0; blk * nthr * 2 < total; ++blk)
    for (int t = 0; t < nthr; ++t) {
      const long long pix0 = blk * nthr * 2 + t;
      if (pix0 < total) k1_pixels<float, 2>(P, sm.data(), sm.data() + kBlkC * kBlkM, pix0, nthr, total);
    }
  return 0;
}

int emu_pw_res_mlp(const float* t2, const float* x, float* out, const float* w2, const float* b2, const float* a1,
                   const float* ln_w, const float* ln_b, float eps, const float* w3, const float* b3,
                   const float* w4, const float* b4, const float* a2, int B, int HW, int nthr) {
  BlockParams P;
  memset(&P, 0, sizeof(P));
  P.t = t2; P.x = x; P.out = out; P.ln_w = ln_w; P.ln_b = ln_b; P.ln_eps = eps;
  P.w_a = w2; P.b_a = b2; P.w_b = w3; P.b_b = b3; P.w_c = w4; P.b_c = b4; P.alpha1 = a1; P.alpha2 = a2;
  P.B = B; P.HW = HW;
  std::vector<float> sm(k3_smem_floats());
  const K3Smem m = k3_carve(sm.data());
  for (int t = 0; t < nthr; ++t) k3_stage(t, nthr, P, m);
  for (long long pix = 0; pix < (long long)B * HW; ++pix) k3_pixel<float>(P, m, pix);
  return 0;
}

int emu_plan(int n, int* radices) {
  Plan1D pl;
  if (!make_plan(n, pl)) return 0;
  for (int i = 0; i < pl.nst; ++i) radices[i] = pl.radix[i];
  return pl.nst;
}
}
