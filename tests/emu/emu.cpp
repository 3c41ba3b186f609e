// Host emulation of the CUDA block bodies -- TEST BUILD ONLY, never part of the product library.
// The kernels are written as per-thread phase functions; compiled for the host a phase
// is a loop over thread ids, so the index arithmetic of whole blocks (padding maps,
// digit-reversed table order, butterfly addressing, crop, epilogue taps) is
// checked against the oracle on a machine without a GPU.
#include <vector>
#include <cstdio>
#include "../../conversenet_b200/csrc/cvb_plan.h"

using namespace cvb;

extern "C" {

int emu_build_transfer(const float* weight, const float* bias, int C, int k, int s, int h, int w,
                       float eps, void* table) {
  TransferParams T;
  if (!make_plan(h, T.py) || !make_plan(w, T.px)) return -3;
  T.weight = weight; T.bias = bias; T.table = (float2*)table;
  T.C = C; T.k = k; T.s = s; T.h = h; T.w = w; T.eps = eps;
  for (int c = 0; c < C; ++c)
    for (int px = 0; px < w; ++px)
      for (int py = 0; py < h; ++py) transfer_entry(T, c, py, px);
  for (int i = 0; i < h + w; ++i) twiddle_entry(T, i);
  return 0;
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

int emu_plan(int n, int* radices) {
  Plan1D pl;
  if (!make_plan(n, pl)) return 0;
  for (int i = 0; i < pl.nst; ++i) radices[i] = pl.radix[i];
  return pl.nst;
}
}
