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

inline bool make_plan(int n, Plan1D& pl) {
  memset(&pl, 0, sizeof(pl));
  if (n < 1) return false;
  pl.n = n;
  if (n == 1) {
    pl.nst = 1; pl.radix[0] = 1; pl.L[0] = 1; pl.M[0] = 1;
    return false;  // a 1-wide axis is not a useful image; reject
  }
  std::vector<int> cur, best;
  search(n, 1 << 30, cur, best);
  if (best.empty() || (int)best.size() > kMaxStages) return false;
  pl.nst = (int)best.size();
  int L = n;
  for (int i = 0; i < pl.nst; ++i) {
    pl.radix[i] = best[i];
    pl.L[i] = L;
    pl.M[i] = L / best[i];
    L /= best[i];
  }
  return true;
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
