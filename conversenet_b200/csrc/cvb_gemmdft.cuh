// Multi-pass Converse2D for padded lengths N = 4 * R0: the R0-point transforms run as dense
// contractions on the 5th-generation tensor cores (tcgen05, accumulators in TMEM), the 4-point
// stage as register / warp-shuffle butterflies.  Four streaming kernels per chunk of plane pairs
// meet in the workspace S^T[pair][x][pos_y] (float2, pos_y fastest):
//
//   A   x (through the pad maps) --R0-point DFT along y--> twiddle --4-point--> S^T[x][pos_y]
//   B1  S^T --R0-point DFT along x--> twiddle --4-point--> . transfer table, conjugate
//           --4-point--> twiddle --> S^T (in place; slot x = 4k + j holds inner index j, frequency k)
//   B2  S^T --R0-point DFT along k--> S^T[x = 4q + j][pos_y] --4-point over pos_y = 4k' .. 4k' + 3-->
//           twiddle --> S^T (in place: the first step of the inverse column transform)
//   C   S^T --R0-point DFT along k'--> crop, GELU, store
//       (scale >= 2: the plane r goes back to S^T and a small epilogue kernel finishes)
//
// Index conventions are those of the register FFT (cvb_kernels.cuh): decimation in frequency
// forward, y = 4q + j --(R0 over q)--> (k, j) --(4 over j)--> position 4k + j2 = frequency
// k + R0 * j2; the inverse runs the same forward transforms on the conjugated spectrum in reverse
// order, so one constant operand serves all four contractions.
//
// One contraction: a tile is 128 "vectors" (32 lines x 4 inner indices) of R0 complex values.
// With C[k][q] = cos(2 pi k q / R0), S[k][q] = sin(..):
//     X[k]      = (C xr + S xi)[k] + i (C xi - S xr)[k]
//     X[R0 - k] = (C xr - S xi)[k] + i (C xi + S xr)[k],      k = 0 .. R0 / 2,
// i.e. two real GEMMs D0 = Xr B^T, D1 = Xi B^T (M = 128 vectors, N = NB columns: 2k = C[k],
// 2k + 1 = S[k]; K = q in chunks of 8), fp32 operands split into TF32 hi + lo, three MMAs per
// product (hi hi + hi lo + lo hi: fp32 accuracy).  A block has 256 staging / read-back threads (two
// per vector) and one warp that issues the MMAs.  A staging thread writes its four K values of a chunk
// (hi and lo of both parts) into a ring of 32-column slots in tensor memory behind the accumulators
// (tcgen05.st), the MMAs read that operand from TMEM -- no shared-memory operand ring and no
// generic-to-async proxy fence on the way; shared memory beside the constant operand holds the first
// chunks of the block's NEXT tile, which each thread requests with cp.async before it reads the current
// tile back, the remaining chunks are requested when the tile starts and land while the first ones are
// staged.  A chunk is signalled on a named barrier, the issuing warp issues its six MMAs and commits
// to the slot's mbarrier, which is what staging waits for before it reuses the slot.  After the last chunk every thread reads its TMEM lane 16 columns at a time, finishes the
// stage in registers (lane butterflies are branch-free warp shuffles) and stores.  Blocks are
// persistent over tiles; the constant operand (hi, lo) arrives once per block by a bulk copy (TMA).
// Every mbarrier wait is bounded: after a time-out a thread stops waiting and working but keeps
// arriving on the barriers, the block sets the status word, frees its TMEM and returns.
#pragma once
#include "cvb_strip.cuh"
#ifdef __CUDACC__
#include "cvb_tc.cuh"
#endif

namespace cvb {
namespace gd {

constexpr int kVec = 128;             // vectors per tile = MMA M
constexpr int kStageThreads = 256;    // staging / read-back threads: two per vector
constexpr int kThreads = 288;         // threads per block: those and the warp that issues the MMAs
constexpr int kLines = kVec / 4;      // lines per tile
constexpr int kChunk = 8;             // K per MMA (TF32)
constexpr int kWait = 1 << 20;        // polls of a bounded wait

enum { MODE_A = 0, MODE_B1 = 1, MODE_B2 = 2, MODE_C = 3 };

template <int R0>
struct Geo {
  static constexpr int N = 4 * R0;
  static constexpr int KH = R0 / 2;                                   // k = 0 .. KH computed, R0 - k mirrored
  static constexpr int NB = ((2 * (KH + 1) + 15) / 16) * 16;          // accumulator columns per GEMM
  static constexpr int KP = ((R0 + kChunk - 1) / kChunk) * kChunk;
  static constexpr int NCH = KP / kChunk;
  static constexpr int NG = (KH + 1 + 7) / 8;                         // read-back groups of 8 k
  static constexpr int B_LBO = (NB / 8) * 128, B_KSTEP = 2 * B_LBO;   // bytes
  static constexpr int B_FLOATS = NCH * (B_KSTEP / 4);                // one array (hi or lo)
  static constexpr int TMEM_COLS = 2 * NB <= 32 ? 32 : 2 * NB <= 64 ? 64 : 2 * NB <= 128 ? 128 : 2 * NB <= 256 ? 256 : 512;
};

// Ring slots of 32 columns (xr hi, xr lo, xi hi, xi lo: 8 each) behind the two accumulators.  Two: measured
// against three, four and seven slots, two were as fast (268) or faster (512, 516: 2 - 4 %).
template <int R0> CVB_HD constexpr int tmem_a_slots() { return 2; }

// Shared memory beside the constant operand holds the first chunks of a block's NEXT tile, fetched ahead
// (cp.async, 8 KB per chunk: 128 rows x 8 K x float2) while the current tile is read back: as many chunks
// as fit with the block count per SM unchanged.
template <int R0> CVB_HD constexpr int prefetch_chunks() {
  typedef Geo<R0> G;
  const long long blocks = 512 / G::TMEM_COLS;                                   // per SM, by tensor memory
  const long long room = 232448 / blocks - 1024 - (long long)(2 * G::B_FLOATS) * 4 - (long long)G::N * 12 - 512;
  const long long n = room / 8192;
  return (int)(n < 0 ? 0 : n > G::NCH ? G::NCH : n);
}
template <int R0> CVB_HD constexpr size_t ring_bytes(int) { return (size_t)prefetch_chunks<R0>() * 8192; }

// dynamic shared memory of one block
template <int R0>
CVB_HD constexpr size_t smem_bytes(int mode) {
  typedef Geo<R0> G;
  return (size_t)(2 * G::B_FLOATS) * 4 + ring_bytes<R0>(mode) + (size_t)G::N * 8 + (size_t)G::N * 4 + 8 * 8 + 64 + 128;
}

// float index of element (row, k) of the constant operand (K-major core matrices, no swizzle)
CVB_HD int b_index(int n, int k, int lbo_f, int kstep_f) {
  return (n >> 3) * 32 + (n & 7) * 4 + (k & 3) + ((k >> 2) & 1) * lbo_f + (k >> 3) * kstep_f;
}

struct Params {
  FwdParams f;
  float2* ws;          // S^T of this chunk of pairs
  const float* bmat;   // constant operand of the launching kernel's axis: hi then lo, operand layout
  int pair0, npair;
};

#ifdef __CUDACC__
// The constant operand for R0 (hi then lo), written once per device.
template <int R0>
__global__ void dft_matrix_kernel(float* out) {
#ifdef __CUDA_ARCH__
  typedef Geo<R0> G;
  constexpr int KH = G::KH, NB = G::NB, KP = G::KP, b_floats = G::B_FLOATS, lbo_f = G::B_LBO / 4, kstep_f = G::B_KSTEP / 4;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < NB * KP; i += gridDim.x * blockDim.x) {
    const int n = i / KP, q = i - n * KP;
    const int k = n >> 1;
    float v = 0.f;
    if (k <= KH && q < R0) {
      double sn, cs;
      sincospi(2.0 * (double)((k * q) % R0) / (double)R0, &sn, &cs);
      v = (float)((n & 1) ? sn : cs);
    }
    float hi, lo;
    tc::split_tf32(v, hi, lo);
    const int idx = b_index(n, q, lbo_f, kstep_f);
    out[idx] = hi;
    out[b_floats + idx] = lo;
  }
#endif
}
#endif

#ifdef __CUDACC__
__device__ __forceinline__ void tmem_ld16x2(uint32_t ta, uint32_t tb, float (&a)[16], float (&b)[16]) {
  uint32_t r[16], s[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(ta)
      : "memory");
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(s[0]), "=r"(s[1]), "=r"(s[2]), "=r"(s[3]), "=r"(s[4]), "=r"(s[5]), "=r"(s[6]), "=r"(s[7]),
        "=r"(s[8]), "=r"(s[9]), "=r"(s[10]), "=r"(s[11]), "=r"(s[12]), "=r"(s[13]), "=r"(s[14]), "=r"(s[15])
      : "r"(tb)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int j = 0; j < 16; ++j) { a[j] = __uint_as_float(r[j]); b[j] = __uint_as_float(s[j]); }
}

// v * conj(w): the twiddle of a forward-type stage
__device__ __forceinline__ float2 mul_conj(float2 v, float2 w) {
  return make_float2(fmaf(v.y, w.y, v.x * w.x), fmaf(-v.x, w.y, v.y * w.x));
}

// Per-thread constants of the two lane butterflies (branch-free: every lane runs the same instructions).
struct Lane4 {
  float s1;                  // first step: v = t + s1 a
  bool swap;                 // second step: p = swap ? v : t, q = swap ? t : v
  float cx, cy, dx, dy;      //   out = (p.x + cx q.x + cy q.y, p.y + dx q.x + dy q.y)
};
// 4-point forward DFT across the four lanes j = lane & 3 (lane j holds a_j).  Afterwards lane 0, 1,
// 2, 3 holds X_0, X_2, X_1, X_3: output index = bitrev2(lane & 3).
__device__ __forceinline__ Lane4 lane4_spread(int j) {
  Lane4 c;
  c.s1 = j < 2 ? 1.f : -1.f;                 // e = a + t (lanes 0, 1), o = t - a (lanes 2, 3)
  c.swap = j == 2;
  c.cx = j == 0 ? 1.f : j == 1 ? -1.f : 0.f; // 0: t + v   1: t - v   2: v - i t   3: t + i v
  c.dy = c.cx;
  c.cy = j == 2 ? 1.f : j == 3 ? -1.f : 0.f;
  c.dx = -c.cy;
  return c;
}
// The same transform for inputs stored the way the spread form leaves its outputs (lane 0, 1, 2, 3
// holds a_0, a_2, a_1, a_3); afterwards lane j holds X_j.
__device__ __forceinline__ Lane4 lane4_gather(int j) {
  Lane4 c;
  c.s1 = (j & 1) ? -1.f : 1.f;               // e0, o0, e1, o1 on lanes 0 .. 3
  c.swap = j == 1;
  c.cx = j == 0 ? 1.f : j == 2 ? -1.f : 0.f; // 0: t + v   1: v - i t   2: t - v   3: t + i v
  c.dy = c.cx;
  c.cy = j == 1 ? 1.f : j == 3 ? -1.f : 0.f;
  c.dx = -c.cy;
  return c;
}
template <int X1, int X2>
__device__ __forceinline__ float2 bfly4_lanes(float2 a, const Lane4& c) {
  const unsigned full = 0xffffffffu;
  float2 t = make_float2(__shfl_xor_sync(full, a.x, X1), __shfl_xor_sync(full, a.y, X1));
  const float2 v = make_float2(fmaf(c.s1, a.x, t.x), fmaf(c.s1, a.y, t.y));
  t = make_float2(__shfl_xor_sync(full, v.x, X2), __shfl_xor_sync(full, v.y, X2));
  const float2 p = c.swap ? v : t, q = c.swap ? t : v;
  return make_float2(fmaf(c.cy, q.y, fmaf(c.cx, q.x, p.x)), fmaf(c.dy, q.y, fmaf(c.dx, q.x, p.y)));
}
__device__ __forceinline__ float2 bfly4_spread(float2 a, const Lane4& c) { return bfly4_lanes<2, 1>(a, c); }
__device__ __forceinline__ float2 bfly4_gather(float2 a, const Lane4& c) { return bfly4_lanes<1, 2>(a, c); }
__device__ __forceinline__ int bitrev2(int j) { return ((j & 1) << 1) | (j >> 1); }

// one thread's unit of a K-chunk (row = its TMEM lane, four K values) staged in tensor memory: columns
// [0,8) xr hi, [8,16) xr lo, [16,24) xi hi, [24,32) xi lo of the slot; `taddr` = this thread's lane, the
// slot's first column + 4 * K half
__device__ __forceinline__ void stage_quad_ta(uint32_t taddr, const float (&re)[4], const float (&im)[4]) {
  float rh[4], rl[4], ih[4], il[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    tc::split_tf32(re[e], rh[e], rl[e]);
    tc::split_tf32(im[e], ih[e], il[e]);
  }
  tc::tmem_st4(taddr + 0, rh[0], rh[1], rh[2], rh[3]);
  tc::tmem_st4(taddr + 8, rl[0], rl[1], rl[2], rl[3]);
  tc::tmem_st4(taddr + 16, ih[0], ih[1], ih[2], ih[3]);
  tc::tmem_st4(taddr + 24, il[0], il[1], il[2], il[3]);
  tc::tmem_wait_st();
}

// the six MMAs of K-chunk `ch`, accumulating unless ch == 0; operand A in tensor memory (slot = 32 columns at
// `a_tmem`), the constant operand in shared memory
template <int R0>
__device__ __forceinline__ void issue_chunk_ta(uint32_t tmem, uint32_t a_tmem, const float* b_hi, const float* b_lo,
                                               int ch) {
  typedef Geo<R0> G;
  constexpr uint32_t idesc = tc::idesc_tf32(kVec, G::NB, false, false);
  const uint64_t bh = tc::smem_desc((const char*)b_hi + ch * G::B_KSTEP, G::B_LBO, 128);
  const uint64_t bl = tc::smem_desc((const char*)b_lo + ch * G::B_KSTEP, G::B_LBO, 128);
#pragma unroll
  for (int part = 0; part < 2; ++part) {
    const uint32_t ah = a_tmem + (uint32_t)(16 * part), al = ah + 8u;
    const uint32_t d = tmem + (uint32_t)(part * G::NB);
    tc::mma_tf32_ta(d, ah, bh, idesc, ch > 0 ? 1u : 0u);
    tc::mma_tf32_ta(d, ah, bl, idesc, 1u);
    tc::mma_tf32_ta(d, al, bh, idesc, 1u);
  }
}

// ---------------------------------------------------------------------------------------------
// Which line of which pair a thread serves in a tile, and where its data lives.
template <typename IO>
struct Ident {
  bool valid;
  int pos;            // x (modes A, C) or pos_y (B1, B2) of the line
  int c, pa, pb;      // channel and the two planes of the pair
  int cx;             // mode A: source column of x, -1 = zero padding
  float2* ST;         // S^T of the pair
  const IO* xa;
  const IO* xb;
};

template <int MODE, typename IO>
__device__ __forceinline__ Ident<IO> identify(const Params& P, int tile, int l, int other, long long nlines) {
  const FwdParams& F = P.f;
  Ident<IO> id;
  const long long line = (long long)tile * kLines + l;
  id.valid = line < nlines;
  const int lp = id.valid ? (int)(line / other) : 0;
  id.pos = id.valid ? (int)(line - (long long)lp * other) : 0;
  pair_planes(F, P.pair0 + lp, id.c, id.pa, id.pb);
  id.ST = P.ws + (size_t)lp * F.h * F.w;
  const size_t in_plane = (size_t)F.H * F.W;
  id.xa = (const IO*)F.x + (size_t)id.pa * in_plane;
  id.xb = id.pb >= 0 ? (const IO*)F.x + (size_t)id.pb * in_plane : nullptr;
  id.cx = (MODE == MODE_A) ? pad_index(id.pos - F.p, F.W, F.pad_mode) : 0;
  return id;
}

// the four values q = 8 ch + 4 hf .. + 3 of vector (line, j).  Modes B1, B2, C: `gp` = address of the
// vector's element q = 0 in S^T, `qs` = the stride between consecutive q (see vector_base)
template <int R0, int MODE, typename IO>
__device__ __forceinline__ void gather4(const Ident<IO>& id, int ch, int hf, int j, const float2* gp, size_t qs,
                                        const int* rmap, float (&gr)[4], float (&gi)[4]) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int q = ch * kChunk + 4 * hf + e;
    gr[e] = 0.f; gi[e] = 0.f;
    if (q < R0 && id.valid) {
      if (MODE == MODE_A) {
        const int ro = rmap[4 * q + j];
        if ((ro | id.cx) >= 0) {
          gr[e] = ld_io<IO>(id.xa, (size_t)(ro + id.cx));
          if (id.xb) gi[e] = ld_io<IO>(id.xb, (size_t)(ro + id.cx));
        }
      } else {
        const float2 v = gp[qs * q];
        gr[e] = v.x; gi[e] = v.y;
      }
    }
  }
}
// Where vector (line `id`, inner index j) starts in S^T[x][pos_y] and how far its elements are apart: B1 and
// B2 transform along x (element q at x = 4 q + j, line = pos_y), C along pos_y (element k at pos_y = 4 k + j,
// line = x).
template <int MODE, typename IO>
__device__ __forceinline__ const float2* vector_base(const Ident<IO>& id, int j, int h, size_t& qs) {
  if (MODE == MODE_C) {
    qs = 4;
    return id.ST + (size_t)id.pos * h + j;
  }
  qs = (size_t)4 * h;
  return id.ST + (size_t)j * h + id.pos;
}
// asynchronous copies global -> shared of 8 or 4 bytes; `ok` false writes zeros without reading
__device__ __forceinline__ void cp_async8(void* dst, const void* src, bool ok) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(ok ? 8 : 0) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src, bool ok) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(ok ? 4 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Named barriers between the 256 staging threads (arrive, never wait) and the issuing warp (sync).  The
// barrier number is an immediate: with a register operand the compiler reserves all sixteen barriers
// of the SM for one block.
template <int ID>
__device__ __forceinline__ void bar_arrive_imm() {
  asm volatile("bar.arrive %0, %1;" ::"n"(ID), "n"(kThreads) : "memory");
}
template <int ID>
__device__ __forceinline__ void bar_sync_imm() {
  asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(kThreads) : "memory");
}
__device__ __forceinline__ void bar_arrive(int id) {
  switch (id) {
    case 1: bar_arrive_imm<1>(); break;
    case 2: bar_arrive_imm<2>(); break;
    case 3: bar_arrive_imm<3>(); break;
    case 4: bar_arrive_imm<4>(); break;
    default: bar_arrive_imm<5>(); break;
  }
}
__device__ __forceinline__ void bar_sync(int id) {
  switch (id) {
    case 1: bar_sync_imm<1>(); break;
    case 2: bar_sync_imm<2>(); break;
    case 3: bar_sync_imm<3>(); break;
    case 4: bar_sync_imm<4>(); break;
    default: bar_sync_imm<5>(); break;
  }
}

// Block of 288 threads.  Warps 0-7 (256 threads) gather, stage and read back: thread tid serves operand
// row / TMEM lane m = tid & 127 (warps w and w + 4 share a TMEM quadrant) and takes half hf = tid >> 7
// of the work on it: K quad hf of every chunk when staging, read-back groups hf, hf + 2, ...  Warp 8
// issues the MMAs: it waits on the
// named barrier of a ring slot for the 256 arrivals of the chunk staged there, issues the chunk's six
// MMAs and commits them to the slot's mbarrier, which is what a staging thread waits for before it
// reuses the slot -- so staging never waits for the issue, only for the tensor cores one slot round back.
// Before the first chunk of a tile the issuing warp waits on one more named barrier until every thread
// has read the previous tile's accumulators, so a warp that has finished its read-back stages the next
// tile while the others still read.  After a time-out (ok == false) a thread stops waiting and working
// but keeps arriving on the barriers, so nobody is left waiting for it.
template <int R0, int MODE, typename IO>
__device__ void body(const Params& P, unsigned char* smem_raw) {
  typedef Geo<R0> G;
  constexpr int NS = tmem_a_slots<R0>();
  static_assert(NS >= 2, "operand ring needs two slots");
  constexpr uint32_t A_BASE = 2 * G::NB;     // first TMEM column of the operand ring
  // chunks of the next tile fetched ahead (fp32 tensors: 2-byte elements cannot be copied asynchronously one by one)
  constexpr int PF = (MODE == MODE_A && sizeof(IO) == 2) ? 0 : prefetch_chunks<R0>();
  constexpr int N = G::N;
  constexpr int BAR_FREE = NS + 1;           // named barrier "accumulators read"; slots use 1 .. NS
  const FwdParams& F = P.f;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool issuer = warp == kStageThreads / 32;
  const int m = tid & (kVec - 1), hf = (tid >> 7) & 1;
  const int h = F.h, w = F.w;
  // the axis this kernel transforms has length N; lines run along the other axis
  const int other = (MODE == MODE_A || MODE == MODE_C) ? w : h;
  const long long nlines = (long long)P.npair * other;
  const int ntiles = (int)((nlines + kLines - 1) / kLines);

  float* b_hi = (float*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  float* b_lo = b_hi + G::B_FLOATS;
  float* ring = b_lo + G::B_FLOATS;
  float2* tw = (float2*)((char*)ring + ring_bytes<R0>(MODE));
  int* rmap = (int*)(tw + N);
  uint64_t* mbar = (uint64_t*)(((uintptr_t)(rmap + N) + 7) & ~(uintptr_t)7);   // [NS] slots, [NS] = operand B
  uint32_t* holder = (uint32_t*)(mbar + NS + 1);
  // ---- set-up: barriers, constant operand, twiddles, pad map, TMEM ----
  if (tid == 0) {
    for (int i = 0; i <= NS; ++i) mbar_init(&mbar[i], 1);
    mbar_fence_init();
    mbar_expect_tx(&mbar[NS], 2 * G::B_FLOATS * 4);
    bulk_g2s(b_hi, P.bmat, 2 * G::B_FLOATS * 4, &mbar[NS]);
  }
  {
    const float2* blob = F.table + (size_t)F.C * h * w + ((MODE == MODE_A || MODE == MODE_C) ? 0 : h);
    for (int i = tid; i < N; i += kThreads) tw[i] = blob[i];
    if (MODE == MODE_A)
      for (int i = tid; i < N; i += kThreads) {
        const int ry = pad_index(i - F.p, F.H, F.pad_mode);
        rmap[i] = ry < 0 ? -1 : ry * F.W;
      }
  }
  if (warp == 0) tc::tmem_alloc(holder, G::TMEM_COLS);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = *holder;
  bool ok = true;
  // Ring bookkeeping: chunk number g (counted over the block's life) uses slot g % NS for the
  // (g / NS)-th time; that use may start once the commit of the use before it has arrived.
  uint32_t seq = 0;

  if (issuer) {
    // ---------------- the issuing warp ----------------
    bool first = true;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
      if (!first) bar_sync(BAR_FREE);   // the previous tile's accumulators have been read
      for (int ch = 0; ch < G::NCH; ++ch) {
        const uint32_t slot = seq % NS;
        bar_sync(1 + (int)slot);        // chunk staged
        tc::fence_after_sync();
        if (lane == 0) {
          if (first && ch == 0) ok = mbar_wait_bounded(&mbar[NS], 0, kWait);   // the constant operand has landed
          if (ok) issue_chunk_ta<R0>(tmem, tmem + A_BASE + slot * 32u, b_hi, b_lo, ch);
          tc::mma_commit(&mbar[slot]);
        }
        __syncwarp();
        seq += 1;
      }
      first = false;
    }
    if (lane == 0 && first) mbar_wait_bounded(&mbar[NS], 0, kWait);   // no tile: let the bulk copy land
    if (lane == 0 && !ok && F.status) atomicExch(F.status, 4);
  } else {
    // ---------------- the 256 staging / read-back threads ----------------
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    // row m = vector (line l = m / 4, inner index j = m % 4)
    const int l = m >> 2;
    const int j = m & 3;
    const size_t in_plane = (size_t)F.H * F.W;

    Ident<IO> id = identify<MODE, IO>(P, blockIdx.x, l, other, nlines);

    // TMEM-staged modes: request the first PF chunks of a tile into this thread's cells of the raw buffer,
    // [chunk][e][hf][m] float2 (m fastest: no bank conflicts either way)
    float2* raw = (float2*)ring;
    auto prefetch = [&](const Ident<IO>& pid) {
      size_t qs;
      const float2* gp = vector_base<MODE, IO>(pid, j, h, qs);
#pragma unroll 1
      for (int ch = 0; ch < PF; ++ch) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int q = ch * kChunk + 4 * hf + e;
          float2* dst = raw + (size_t)((ch * 4 + e) * 2 + hf) * kVec + m;
          const bool live = q < R0 && pid.valid;
          if (MODE == MODE_A) {
            const int ro = live ? rmap[4 * q + j] : -1;
            const bool in = live && (ro | pid.cx) >= 0;
            const size_t off = in ? (size_t)(ro + pid.cx) : 0;
            cp_async4(&dst->x, (const float*)pid.xa + off, in);
            cp_async4(&dst->y, (const float*)(pid.xb ? pid.xb : pid.xa) + off, in && pid.xb != nullptr);
          } else {
            cp_async8(dst, live ? (const void*)(gp + qs * q) : (const void*)P.ws, live);
          }
        }
      }
      cp_async_commit();
    };
    if (PF > 0 && blockIdx.x < ntiles) prefetch(id);

    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
      const int ntile = tile + gridDim.x;
      const Ident<IO> nid =
          identify<MODE, IO>(P, ntile < ntiles ? ntile : tile, l, other, ntile < ntiles ? nlines : 0);

      // ---- gather ahead, split, stage, signal: one K-chunk (two for mode C) per step ----
      {
        // Operand staged in tensor memory.  The first PF chunks of this tile were fetched into shared memory
        // by this thread while it read the previous tile back (cp.async; each thread reads only what it
        // copied itself, so a wait_group is all the ordering needed); the rest is requested now and lands
        // while those are staged.
        size_t qs;
        const float2* gp = vector_base<MODE, IO>(id, j, h, qs);
        constexpr int NR = G::NCH - PF;
        float vr[NR > 0 ? NR : 1][4], vi[NR > 0 ? NR : 1][4];
#pragma unroll
        for (int cb = 0; cb < NR; ++cb) gather4<R0, MODE, IO>(id, PF + cb, hf, j, gp, qs, rmap, vr[cb], vi[cb]);
        if (PF > 0) cp_async_wait_all();
#pragma unroll 1
        for (int ch = 0; ch < PF; ++ch) {
          const float2* rp = raw + (size_t)(ch * 8 + hf) * kVec + m;
          float re[4], im[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 v = rp[e * 2 * kVec];
            re[e] = v.x; im[e] = v.y;
          }
          const uint32_t slot = seq % NS, use = seq / NS;
          if (use > 0 && ok) ok = mbar_wait_bounded(&mbar[slot], (use - 1) & 1u, kWait);
          stage_quad_ta(lane_base + A_BASE + slot * 32u + 4u * (uint32_t)hf, re, im);
          tc::fence_before_sync();
          bar_arrive(1 + (int)slot);
          seq += 1;
        }
#pragma unroll
        for (int cb = 0; cb < NR; ++cb) {
          const uint32_t slot = seq % NS, use = seq / NS;
          if (use > 0 && ok) ok = mbar_wait_bounded(&mbar[slot], (use - 1) & 1u, kWait);
          stage_quad_ta(lane_base + A_BASE + slot * 32u + 4u * (uint32_t)hf, vr[cb], vi[cb]);
          tc::fence_before_sync();
          bar_arrive(1 + (int)slot);
          seq += 1;
        }
        if (PF > 0 && ntile < ntiles) prefetch(nid);   // the raw buffer is free again: next tile's first chunks
      }

      // ---- wait for the tile's last MMAs, read this thread's TMEM lane back, finish the stage ----
      {
        const uint32_t last = (seq - 1) % NS, use = (seq - 1) / NS;
        if (ok) ok = mbar_wait_bounded(&mbar[last], use & 1u, kWait);
      }
      tc::fence_after_sync();
      const float2* tab = F.table + (size_t)id.c * h * w;   // [pos_x][pos_y]
      const int jr = bitrev2(j);
      const Lane4 ls = lane4_spread(j), j4 = lane4_gather(j);
      const bool valid = id.valid && ok;
      const int pos = id.pos;
      float2* ST = id.ST;
      // output element i of a half-group hh of group g: k = 8 g + 4 hh + i / 2, mirrored (R0 - k) for odd i
      auto out_index = [&](int g, int hh, int i, bool& live) {
        const int k = 8 * g + 4 * hh + (i >> 1), mir = i & 1;
        live = k <= G::KH && !(mir && (k == 0 || 2 * k == R0));
        return live ? (mir ? R0 - k : k) : 0;
      };
      // mode B2 also runs the first step of the inverse column transform: the 4-point DFT over the four
      // pos_y = 4 k' .. 4 k' + 3 of a column (four consecutive lines = lanes 4 apart; tiles and planes start
      // at multiples of four lines) and its twiddle, so that kernel C gathers finished vectors.  Lane i4 of
      // the four ends up with output index bitrev2(i4), stored at pos_y = 4 k' + bitrev2(i4).
      const int i4 = l & 3, jy = bitrev2(i4), kprime = pos >> 2;
      const Lane4 lsy = lane4_spread(i4);
      float2 twy = make_float2(1.f, 0.f);
      if (MODE == MODE_B2) twy = (F.table + (size_t)F.C * h * w)[jy * kprime];   // y-axis twiddle (cos, sin)(2 pi jy k' / h)
      const float2* tabp = tab + (size_t)jr * h + pos;     // mode B1: element (4 kq + jr, pos) at tabp[4 h kq]
      float2 gn[8];                                        // mode B1: table values of the next half-group
      if (MODE == MODE_B1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          bool live;
          const int kq = out_index(hf, 0, i, live);
          gn[i] = make_float2(0.f, 0.f);
          if (valid && live) gn[i] = tabp[(size_t)4 * h * kq];
        }
      }
#pragma unroll 1
      for (int g = hf; g < G::NG; g += 2) {
        float d0[16], d1[16];
        tmem_ld16x2(lane_base + (uint32_t)(16 * g), lane_base + (uint32_t)(G::NB + 16 * g), d0, d1);
        // two halves of four k each: all loads first, then the arithmetic of the eight outputs (independent
        // chains), then the stores
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          float2 v[8], t1[8], gt[8];
          int kq[8];
          bool live[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            kq[i] = out_index(g, hh, i, live[i]);
            const int mir = i & 1;
            const float cxr = d0[8 * hh + 2 * (i >> 1)], sxr = d0[8 * hh + 2 * (i >> 1) + 1];
            const float cxi = d1[8 * hh + 2 * (i >> 1)], sxi = d1[8 * hh + 2 * (i >> 1) + 1];
            v[i] = mir ? make_float2(cxr - sxi, cxi + sxr) : make_float2(cxr + sxi, cxi - sxr);
            if (MODE == MODE_A || MODE == MODE_B1) t1[i] = tw[j * kq[i]];
            if (MODE == MODE_B1) gt[i] = gn[i];
          }
          if (MODE == MODE_B1) {   // request the next half-group's table values before this one's arithmetic
            const int g2 = hh ? g + 2 : g, h2 = hh ? 0 : 1;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              bool lv;
              const int kn = out_index(g2, h2, i, lv);
              gn[i] = make_float2(0.f, 0.f);
              if (valid && lv && g2 < G::NG) gn[i] = tabp[(size_t)4 * h * kn];
            }
          }
          if (MODE == MODE_A || MODE == MODE_B1) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = bfly4_spread(mul_conj(v[i], t1[i]), ls);
          }
          if (MODE == MODE_B2) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = mul_conj(bfly4_lanes<8, 4>(v[i], lsy), twy);
          }
          if (MODE == MODE_B1) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float2 u = make_float2(fmaf(-v[i].y, gt[i].y, v[i].x * gt[i].x),
                                           -fmaf(v[i].x, gt[i].y, v[i].y * gt[i].x));   // conj(v * g)
              v[i] = mul_conj(bfly4_gather(u, j4), t1[i]);
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (!(valid && live[i])) continue;
            if (MODE == MODE_A) {
              ST[(size_t)pos * h + 4 * kq[i] + jr] = v[i];
            } else if (MODE == MODE_B1) {
              ST[(size_t)(4 * kq[i] + j) * h + pos] = v[i];
            } else if (MODE == MODE_B2) {
              ST[(size_t)(4 * kq[i] + j) * h + 4 * kprime + jy] = v[i];
            } else {
              const int y = 4 * kq[i] + j;
              if (F.s > 1) {
                ST[(size_t)pos * h + y] = make_float2(v[i].x, -v[i].y);    // plane r for the epilogue kernel
              } else {
                const int oy = y - F.p, ox = pos - F.p;
                if (oy >= 0 && oy < F.H && ox >= 0 && ox < F.W) {
                  float va = v[i].x, vb = -v[i].y;
                  if (F.fuse_gelu) gelu_pair(va, vb);
                  const size_t off = (size_t)oy * F.W + ox;
                  st_io<IO>((IO*)F.out + (size_t)id.pa * in_plane, off, va);
                  if (id.pb >= 0) st_io<IO>((IO*)F.out + (size_t)id.pb * in_plane, off, vb);
                }
              }
            }
          }
        }
      }
      tc::fence_before_sync();
      if (ntile < ntiles) bar_arrive(BAR_FREE);   // this thread has read its share of the accumulators
      id = nid;
    }
    if (!ok && F.status) atomicExch(F.status, 4);
  }

  // ---- tear-down ----
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, G::TMEM_COLS);
}

// scale >= 2 after mode C left r in S^T: out = crop(nearest(y) + corr(K, zero_insert(r))); one thread per
// low-resolution cell (models/util_converse.py:171-173,185-190 collapsed, see cvb_kernels.cuh)
template <typename IO>
__device__ void epilogue_body(const Params& P) {
  const FwdParams& F = P.f;
  const int s = F.s, k = F.k, cc = F.k / 2, p = F.p, h = F.h, w = F.w;
  const long long cells = (long long)P.npair * F.H * F.W;
  const size_t in_plane = (size_t)F.H * F.W, out_plane = in_plane * s * s;
  const int oW = F.W * s;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < cells;
       i += (long long)gridDim.x * blockDim.x) {
    const int lp = (int)(i / (long long)in_plane);
    const int ci = (int)(i - (long long)lp * in_plane);
    const int my = ci / F.W, mx = ci - my * F.W;
    int c, pa, pb;
    pair_planes(F, P.pair0 + lp, c, pa, pb);
    const float2* ST = P.ws + (size_t)lp * h * w;
    const float* wk = F.weight + (size_t)c * k * k;
    const float ya = ld_io<IO>((const IO*)F.x + (size_t)pa * in_plane, (size_t)ci);
    const float yb = pb >= 0 ? ld_io<IO>((const IO*)F.x + (size_t)pb * in_plane, (size_t)ci) : 0.f;
    const int m = my + p, n = mx + p;
    for (int da = 0; da < s; ++da)
      for (int db = 0; db < s; ++db) {
        float acca = ya, accb = yb;
        for (int a = 0; a < k; ++a) {
          const int ii = da + a - cc;
          const int fi = floordiv(ii, s);
          if (ii - fi * s != 0) continue;
          int rm = (m + fi) % h; if (rm < 0) rm += h;
          for (int b = 0; b < k; ++b) {
            const int jj = db + b - cc;
            const int fj = floordiv(jj, s);
            if (jj - fj * s != 0) continue;
            int rn = (n + fj) % w; if (rn < 0) rn += w;
            const float2 rv = ST[(size_t)rn * h + rm];
            const float kv = wk[a * k + b];
            acca = fmaf(kv, rv.x, acca);
            accb = fmaf(kv, rv.y, accb);
          }
        }
        if (F.fuse_gelu) gelu_pair(acca, accb);
        const size_t off = (size_t)(my * s + da) * oW + (size_t)(mx * s + db);
        st_io<IO>((IO*)F.out + (size_t)pa * out_plane, off, acca);
        if (pb >= 0) st_io<IO>((IO*)F.out + (size_t)pb * out_plane, off, accb);
      }
  }
}
#endif  // __CUDACC__

}  // namespace gd
}  // namespace cvb
