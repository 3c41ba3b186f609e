// Host-side FFT plan selection, shared by the library and the host-emulation test build.
#pragma once
#include <cstdlib>
#include <cstring>
#include "cvb_kernels.cuh"

namespace cvb {

constexpr size_t kSmemLimit = 227 * 1024;

// ------------------------------------------------------------------ plans
// A short list of radices in fixed storage: plan selection allocates nothing (the entry point
// for callers that cannot allocate promises a heap-free host side).
struct RadixList {
  int v[32];
  int n = 0;
  void push(int r) { if (n < 32) v[n] = r; ++n; }   // n > 32 marks an overflow; callers reject it
  void pop() { --n; }
};

// Factor n into supported radices: fewest stages, then smallest largest radix,
// radices in descending order.  Returns false when n has a prime factor above
// the largest prime butterfly.
inline bool search(int n, int max_r, RadixList& cur, RadixList& best) {
  if (n == 1) {
    if (best.n == 0 || cur.n < best.n || (cur.n == best.n && cur.v[0] < best.v[0])) best = cur;
    return true;
  }
  if (best.n != 0 && cur.n + 1 > best.n) return false;
  if (cur.n >= kMaxStages) return false;
  bool any = false;
  for (int i = kNumRadices - 1; i >= 0; --i) {
    const int r = kRadices[i];
    if (r > max_r || n % r) continue;
    cur.push(r);
    any |= search(n / r, r, cur, best);
    cur.pop();
  }
  return any;
}

constexpr int kMaxBigPrime = 127;  // largest prime handled by the direct out-of-place butterfly

// Radices of n: prime factors above the register butterflies (each its own stage, only
// usable on the multi-pass path), then the fewest-stage factorisation of the rest.
inline bool make_plan(int n, Plan1D& pl, bool* has_big = nullptr) {
  memset(&pl, 0, sizeof(pl));
  if (has_big) *has_big = false;
  if (n < 2) return false;
  pl.n = n;
  RadixList big;   // ascending while collected, stored descending
  int rest = n;
  for (int f = 29; f <= kMaxBigPrime && f <= rest; f += 2) {
    bool prime = true;
    for (int d = 3; d * d <= f; d += 2) if (f % d == 0) { prime = false; break; }
    if (!prime) continue;
    while (rest % f == 0) { big.push(f); rest /= f; }
  }
  if (big.n > kMaxStages) return false;
  if (big.n > 0 && has_big) *has_big = true;
  RadixList best;
  if (rest > 1) {
    RadixList cur;
    search(rest, 1 << 30, cur, best);
    if (best.n == 0) return false;
  }
  if (big.n + best.n > kMaxStages) return false;
  pl.nst = big.n + best.n;
  int L = n;
  for (int i = 0; i < pl.nst; ++i) {
    const int r = i < big.n ? big.v[big.n - 1 - i] : best.v[i - big.n];
    pl.radix[i] = r;
    pl.L[i] = L;
    pl.M[i] = L / r;
    L /= r;
  }
  return true;
}

// ---- plans of the tensor-core multi-pass kernels: n = 4 * R0 with R0 in the registry ----
inline bool gemm_axis(int n) {
  if (n % 4) return false;
  static const int r0s[] = {
#define CVB_GEMM(r0) r0,
#include "gemm_registry.inc"
#undef CVB_GEMM
  };
  for (int r : r0s) if (n / 4 == r) return true;
  return false;
}
inline void make_gemm_plan(int n, Plan1D& pl) {
  memset(&pl, 0, sizeof(pl));
  pl.n = n; pl.nst = 2; pl.gemm = 1;
  pl.radix[0] = n / 4; pl.L[0] = n; pl.M[0] = 4;
  pl.radix[1] = 4; pl.L[1] = 4; pl.M[1] = 1;
}
inline bool gemm_disabled() {   // tuning builds: CVB_NO_GEMM=1 takes the register-FFT multi-pass kernels instead
#ifdef CVB_TUNING
  const char* v = getenv("CVB_NO_GEMM");
  return v && *v && *v != '0';
#else
  return false;
#endif
}
// Plans of both axes of a padded plane.  A plane whose two lengths are in the registry takes the
// tensor-core multi-pass kernels whatever its scale or tap count (the transfer table is laid out
// for the plan, so the choice may depend on nothing but h and w).
inline bool make_axis_plans(int h, int w, Plan1D& py, Plan1D& px, bool* big = nullptr) {
  if (big) *big = false;
  if (gemm_axis(h) && gemm_axis(w) && !gemm_disabled()) {
    make_gemm_plan(h, py);
    make_gemm_plan(w, px);
    if (big) *big = true;
    return true;
  }
  bool by = false, bx = false;
  if (!make_plan(h, py, &by) || !make_plan(w, px, &bx)) return false;
  if (big) *big = by || bx;
  return true;
}

// ---- Rader tables for a large prime in the first stage of an axis plan ----
inline int primitive_root(int R) {
  int fac[16], nfac = 0;
  int m = R - 1;
  for (int f = 2; f * f <= m; ++f)
    if (m % f == 0) { if (nfac < 16) fac[nfac++] = f; while (m % f == 0) m /= f; }
  if (m > 1 && nfac < 16) fac[nfac++] = m;
  for (int g = 2; g < R; ++g) {
    bool ok = true;
    for (int fi = 0; fi < nfac; ++fi) {
      const int f = fac[fi];
      long long r = 1, b = g; int e = (R - 1) / f;
      while (e) { if (e & 1) r = r * b % R; b = b * b % R; e >>= 1; }
      if (r == 1) { ok = false; break; }
    }
    if (ok) return g;
  }
  return 0;
}

// Rader applies when the first stage is a large prime R and R-1 factors into register radices.
inline RaderInfo rader_for(const Plan1D& pl, int off) {
  RaderInfo r;
  memset(&r, 0, sizeof(r));
  r.off = off;
  if (pl.nst < 1 || pl.radix[0] <= 26 || pl.gemm) return r;
  bool big = false;
  if (!make_plan(pl.radix[0] - 1, r.sub, &big) || big) return r;
  r.g = primitive_root(pl.radix[0]);
  if (r.g) r.R = pl.radix[0];
  return r;
}
// float2 slots one axis' tables take in the blob: bhat, twiddles, two int permutations
inline int rader_blob_float2(const RaderInfo& r) { return r.R ? 3 * (r.R - 1) : 0; }
// both axes: column tables first, then row tables
inline void rader_both(const Plan1D& py, const Plan1D& px, RaderInfo& ry, RaderInfo& rx) {
  ry = rader_for(py, 0);
  rx = rader_for(px, rader_blob_float2(ry));
}

// ---- multi-pass (strip) path geometry ----
#ifdef CVB_WS_TARGET_MB   // tuning builds
constexpr size_t kWorkspaceTarget = (size_t)CVB_WS_TARGET_MB << 20;
#else
constexpr size_t kWorkspaceTarget = 48u << 20;  // chunk workspace kept well inside the 126 MB L2
#endif

struct StripGeo {
  int cw, rh, halo_l, halo_r;
  size_t smem_col, smem_row;  // dynamic shared memory of the column / row kernels
  int chunk_pairs;
  size_t ws_bytes;
};

inline bool plan_has_big(const Plan1D& pl) {
  for (int i = 0; i < pl.nst; ++i)
    if (pl.radix[i] > 26) return true;
  return false;
}

// Shared memory of a column-strip block: one tile (two when a large prime needs the
// out-of-place butterfly), the column twiddles, the taps.
inline size_t strip_smem_col(int h, int cw, int halo, int k, bool big) {
  return ((size_t)(big ? 2 : 1) * h * ((cw + halo) | 1) + h + (big ? 3 * kMaxBigPrime : 0) + (k * k + 1) / 2) *
         sizeof(float2);
}
inline size_t strip_smem_row(int w, int rh, bool big) {
  return ((size_t)(big ? 2 : 1) * rh * (w | 1) + w + (big ? 3 * kMaxBigPrime : 0)) * sizeof(float2);
}

// Pairs per launch of the three multi-pass kernels.  Kernel i runs (pairs * n[i]) blocks, bpsm[i]
// of them resident per SM, so it takes ceil(blocks / (bpsm[i] * sms)) waves, each costing about
// bpsm[i] block times on an issue-bound SM.  Among the chunk sizes between half the cap and the
// cap this returns the cheapest in total (the largest on a tie), so that launches do not end on
// a nearly empty wave.
inline int balance_chunk(int npairs, int cap, const int n[3], const int bpsm[3], int sms) {
  if (cap <= 1 || sms < 1) return cap;
  long best_cost = -1;
  int best = cap;
  for (int c2 = cap; c2 >= (cap + 1) / 2; --c2) {
    long cost = 0;
    for (int p0 = 0; p0 < npairs; p0 += c2) {
      const long np = (npairs - p0) < c2 ? (npairs - p0) : c2;
      for (int i = 0; i < 3; ++i) {
        const long slots = (long)(bpsm[i] > 0 ? bpsm[i] : 1) * sms;
        cost += ((np * n[i] + slots - 1) / slots) * (bpsm[i] > 0 ? bpsm[i] : 1);
      }
    }
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = c2; }
  }
  return best;
}

inline StripGeo strip_geometry(int h, int w, int k, int s, int npairs, size_t ws_cap = kWorkspaceTarget,
                               bool at_least_one = true) {
  StripGeo g;
  const int c = k / 2;
  g.halo_l = s > 1 ? (c + s - 1) / s : 0;
  g.halo_r = s > 1 ? (s - 1 + k - 1 - c) / s : 0;
  Plan1D py, px;
  const bool bigy = make_plan(h, py) && plan_has_big(py);
  const bool bigx = make_plan(w, px) && plan_has_big(px);
  // widest strip that still lets three blocks share an SM, else the widest that fits at all
  const size_t want = kSmemLimit / 3;
  g.cw = 2;
  for (int cw : {32, 16, 8, 4, 2})
    if (strip_smem_col(h, cw, g.halo_l + g.halo_r, k, bigy) <= want) { g.cw = cw; break; }
  if (strip_smem_col(h, g.cw, g.halo_l + g.halo_r, k, bigy) > want)
    for (int cw : {16, 8, 4, 2})
      if (strip_smem_col(h, cw, g.halo_l + g.halo_r, k, bigy) <= kSmemLimit) { g.cw = cw; break; }
  g.rh = 1;
  for (int rh : {32, 16, 8, 4, 2, 1})
    if (strip_smem_row(w, rh, bigx) <= want) { g.rh = rh; break; }
  g.smem_col = strip_smem_col(h, g.cw, g.halo_l + g.halo_r, k, bigy);
  g.smem_row = strip_smem_row(w, g.rh, bigx);
  const size_t per_pair = (size_t)h * w * sizeof(float2);
  size_t cp = ws_cap / per_pair;
  if (cp < 1 && at_least_one) cp = 1;  // otherwise chunk_pairs == 0: one pair does not fit the cap
  if (cp > (size_t)npairs) cp = npairs;
  g.chunk_pairs = (int)cp;
  g.ws_bytes = cp * per_pair;
  return g;
}

inline size_t smem_bytes_for(int h, int w, int k, int ystash = 0) {
  return smem_layout(h, w, w | 1, k, ystash).bytes();
}

// Keep the padded input in shared memory for the s > 1 epilogue when two blocks
// per SM still fit with it (otherwise the epilogue re-reads x through L2).
inline int choose_ystash(int h, int w, int k, int s) {
  if (s <= 1) return 0;
  return smem_bytes_for(h, w, k, 1) <= kSmemLimit / 2 ? 1 : 0;
}


}  // namespace cvb
