// Host-side FFT plan selection, shared by the library and the host-emulation test build.
#pragma once
#include <cstring>
#include <vector>
#include "cvb_kernels.cuh"

namespace cvb {

constexpr size_t kSmemLimit = 227 * 1024;

// ------------------------------------------------------------------ plans
// Factor n into supported radices: fewest stages, then smallest largest radix,
// radices in descending order.  Returns false when n has a prime factor above
// the largest prime butterfly.
inline bool search(int n, int max_r, std::vector<int>& cur, std::vector<int>& best) {
  if (n == 1) {
    if (best.empty() || cur.size() < best.size() ||
        (cur.size() == best.size() && cur.front() < best.front())) {
      best = cur;
    }
    return true;
  }
  if (!best.empty() && cur.size() + 1 > best.size()) return false;
  bool any = false;
  for (int i = kNumRadices - 1; i >= 0; --i) {
    const int r = kRadices[i];
    if (r > max_r || n % r) continue;
    cur.push_back(r);
    any |= search(n / r, r, cur, best);
    cur.pop_back();
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
  std::vector<int> radices;
  int rest = n;
  for (int f = 29; f <= kMaxBigPrime && f <= rest; f += 2) {
    bool prime = true;
    for (int d = 3; d * d <= f; d += 2) if (f % d == 0) { prime = false; break; }
    if (!prime) continue;
    while (rest % f == 0) { radices.insert(radices.begin(), f); rest /= f; }
  }
  if (!radices.empty() && has_big) *has_big = true;
  if (rest > 1) {
    std::vector<int> cur, best;
    search(rest, 1 << 30, cur, best);
    if (best.empty()) return false;
    radices.insert(radices.end(), best.begin(), best.end());
  }
  if ((int)radices.size() > kMaxStages) return false;
  pl.nst = (int)radices.size();
  int L = n;
  for (int i = 0; i < pl.nst; ++i) {
    pl.radix[i] = radices[i];
    pl.L[i] = L;
    pl.M[i] = L / radices[i];
    L /= radices[i];
  }
  return true;
}

// ---- multi-pass (strip) path geometry ----
constexpr size_t kWorkspaceTarget = 48u << 20;  // chunk workspace kept well inside the 126 MB L2

struct StripGeo {
  int cw, rh, halo_l, halo_r;
  size_t smem_col, smem_row;  // dynamic shared memory of the column / row kernels
  int chunk_pairs;
  size_t ws_bytes;
};

inline StripGeo strip_geometry(int h, int w, int k, int s, int npairs, size_t ws_cap = kWorkspaceTarget,
                               bool at_least_one = true) {
  StripGeo g;
  const int c = k / 2;
  g.halo_l = s > 1 ? (c + s - 1) / s : 0;
  g.halo_r = s > 1 ? (s - 1 + k - 1 - c) / s : 0;
  g.cw = 16;
  g.rh = 8;
  const int tpc = (g.cw + g.halo_l + g.halo_r) | 1;
  g.smem_col = ((size_t)2 * h * tpc + h + (k * k + 1) / 2) * sizeof(float2);
  while (g.smem_col > kSmemLimit && g.cw > 2) {
    g.cw /= 2;
    g.smem_col = ((size_t)2 * h * ((g.cw + g.halo_l + g.halo_r) | 1) + h + (k * k + 1) / 2) * sizeof(float2);
  }
  g.smem_row = ((size_t)2 * g.rh * (w | 1) + w) * sizeof(float2);
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
