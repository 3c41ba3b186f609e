// The channel-mixing parts of ConverseBlock (models/util_converse.py:278-293), fused per pixel.
//
//   K1  ln_pw_gelu :  t1 = GELU( W1 . LN1(x) + b1 )                          (C -> 2C)
//                     = conv1[0..2]: LayerNorm(channels_first) :60-68, Conv2d 1x1 :279, GELU :280
//   K3  pw_res_mlp :  x1  = x + a1 * ( W2 . t2 + b2 )                        (2C -> C, :283 + :291)
//                     out = x1 + a2 * ( W4 . GELU( W3 . LN2(x1) + b3 ) + b4 ) (conv2 :285-288 + :292)
//                     a1, a2 = alpha1 / alpha2 of ConverseBlockAlphaVariant (:321-322), or 1.
//
// Both are exact fp32 on the CUDA cores: a thread owns whole pixels (all channels in registers, so
// LayerNorm needs no cross-thread reduction), the weights sit in shared memory and are read as
// 16-byte broadcasts.  The LayerNorm affine is folded into the following 1x1 weights when a block
// stages them.  Tensors are NCHW, so for a fixed channel consecutive threads touch consecutive pixels.
#pragma once
#include "cvb_kernels.cuh"

namespace cvb {

constexpr int kBlkC = 64;         // channels of the block (the networks use num_features = 64)
constexpr int kBlkM = 2 * kBlkC;  // hidden width

struct BlockParams {
  const void* x;    // K1: (B,C,HW) input.  K3: (B,C,HW) block input (residual)
  const void* t;    // K3: (B,2C,HW) output of Converse2D + GELU
  void* out;        // K1: (B,2C,HW).  K3: (B,C,HW)
  const float* ln_w; const float* ln_b; float ln_eps;   // LN1 (K1) or LN2 (K3)
  const float* w_a; const float* b_a;   // K1: W1 (2C,C), b1 (2C).  K3: W2 (C,2C), b2 (C)
  const float* w_b; const float* b_b;   // K3: W3 (2C,C), b3 (2C)
  const float* w_c; const float* b_c;   // K3: W4 (C,2C), b4 (C)
  const float* alpha1; const float* alpha2;  // K3: (C) or null
  int B, HW;
};

// ---------------------------------------------------------------- weight staging
// K1: wt[ic][oc] = W1[oc][ic] * gamma[ic]; bf[oc] = b1[oc] + sum_ic W1[oc][ic] * beta[ic]
CVB_HD void k1_stage(int tid, int nthr, const BlockParams& P, float* wt, float* bf) {
  for (int i = tid; i < kBlkM * kBlkC; i += nthr) {
    const int oc = i / kBlkC, ic = i - oc * kBlkC;
    wt[ic * kBlkM + oc] = P.w_a[i] * P.ln_w[ic];
  }
  for (int oc = tid; oc < kBlkM; oc += nthr) {
    float s = P.b_a[oc];
    for (int ic = 0; ic < kBlkC; ++ic) s = fmaf(P.w_a[oc * kBlkC + ic], P.ln_b[ic], s);
    bf[oc] = s;
  }
}

// LayerNorm statistics of one pixel held in registers, as the reference computes them
// (mean, biased variance of the centred values, 1/sqrt(var + eps))
template <int N>
CVB_HD void ln_stats(const float (&v)[N], float eps, float& mean, float& rstd) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < N; ++i) s += v[i];
  mean = s * (1.0f / N);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < N; ++i) { const float d = v[i] - mean; q = fmaf(d, d, q); }
  rstd = 1.0f / sqrtf(q * (1.0f / N) + eps);
}

// K1 for PX pixels pix0, pix0 + stride, ... of the flattened (image, pixel) index; pixels at or
// beyond `total` are computed on a clamped address and not stored
template <typename IO, int PX>
CVB_HD void k1_pixels(const BlockParams& P, const float* wt, const float* bf, long long pix0, int stride,
                      long long total) {
  size_t xin[PX], xout[PX];
  bool valid[PX];
#pragma unroll
  for (int u = 0; u < PX; ++u) {
    long long pix = pix0 + (long long)u * stride;
    valid[u] = pix < total;
    if (!valid[u]) pix = total - 1;
    const int b = (int)(pix / P.HW);
    const int p0 = (int)(pix - (long long)b * P.HW);
    xin[u] = (size_t)b * kBlkC * P.HW + p0;
    xout[u] = (size_t)b * kBlkM * P.HW + p0;
  }
  float xn[PX][kBlkC];
#pragma unroll
  for (int ic = 0; ic < kBlkC; ++ic)
#pragma unroll
    for (int u = 0; u < PX; ++u) xn[u][ic] = ld_io<IO>(P.x, xin[u] + (size_t)ic * P.HW);
#pragma unroll
  for (int u = 0; u < PX; ++u) {
    float mean, rstd;
    ln_stats<kBlkC>(xn[u], P.ln_eps, mean, rstd);
#pragma unroll
    for (int ic = 0; ic < kBlkC; ++ic) xn[u][ic] = (xn[u][ic] - mean) * rstd;
  }
#pragma unroll 1
  for (int oc0 = 0; oc0 < kBlkM; oc0 += 8) {
    float acc[PX][8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int u = 0; u < PX; ++u) acc[u][j] = bf[oc0 + j];
#pragma unroll
    for (int ic = 0; ic < kBlkC; ++ic) {
      const float4 wa = *(const float4*)(wt + ic * kBlkM + oc0);
      const float4 wb = *(const float4*)(wt + ic * kBlkM + oc0 + 4);
      const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int u = 0; u < PX; ++u) acc[u][j] = fmaf(xn[u][ic], wv[j], acc[u][j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int u = 0; u < PX; ++u)
        if (valid[u]) st_io<IO>(P.out, xout[u] + (size_t)(oc0 + j) * P.HW, gelu_erf(acc[u][j]));
  }
}

// ---------------------------------------------------------------- K3
// staged weights: w2t[ic][oc] = W2[oc][ic];  w3f[mc][ic] = W3[mc][ic] * gamma[ic];
// b3f[mc] = b3[mc] + sum_ic W3[mc][ic] * beta[ic];  w4t[mc][oc] = W4[oc][mc]
struct K3Smem {
  float* w2t;  // [2C][C]
  float* w3f;  // [2C][C]
  float* w4t;  // [2C][C]
  float* b2;   // [C]
  float* b3f;  // [2C]
  float* b4;   // [C]
  float* a1;   // [C]
  float* a2;   // [C]
};
CVB_HD size_t k3_smem_floats() { return (size_t)3 * kBlkM * kBlkC + kBlkC * 4 + kBlkM; }
CVB_HD K3Smem k3_carve(float* s) {
  K3Smem m;
  m.w2t = s;
  m.w3f = m.w2t + kBlkM * kBlkC;
  m.w4t = m.w3f + kBlkM * kBlkC;
  m.b2 = m.w4t + kBlkM * kBlkC;
  m.b3f = m.b2 + kBlkC;
  m.b4 = m.b3f + kBlkM;
  m.a1 = m.b4 + kBlkC;
  m.a2 = m.a1 + kBlkC;
  return m;
}
CVB_HD void k3_stage(int tid, int nthr, const BlockParams& P, const K3Smem& m) {
  for (int i = tid; i < kBlkC * kBlkM; i += nthr) {
    const int oc = i / kBlkM, ic = i - oc * kBlkM;   // W2, W4: (C, 2C)
    m.w2t[ic * kBlkC + oc] = P.w_a[i];
    m.w4t[ic * kBlkC + oc] = P.w_c[i];
    const int mc = i / kBlkC, jc = i - mc * kBlkC;   // W3: (2C, C)
    m.w3f[i] = P.w_b[i] * P.ln_w[jc];
    (void)mc;
  }
  for (int mc = tid; mc < kBlkM; mc += nthr) {
    float s = P.b_b[mc];
    for (int ic = 0; ic < kBlkC; ++ic) s = fmaf(P.w_b[mc * kBlkC + ic], P.ln_b[ic], s);
    m.b3f[mc] = s;
  }
  for (int oc = tid; oc < kBlkC; oc += nthr) {
    m.b2[oc] = P.b_a[oc];
    m.b4[oc] = P.b_c[oc];
    m.a1[oc] = P.alpha1 ? P.alpha1[oc] : 1.0f;
    m.a2[oc] = P.alpha2 ? P.alpha2[oc] : 1.0f;
  }
}

template <typename IO>
CVB_HD void k3_pixel(const BlockParams& P, const K3Smem& m, long long pix) {
  const int b = (int)(pix / P.HW);
  const int p0 = (int)(pix - (long long)b * P.HW);
  const size_t tin = (size_t)b * kBlkM * P.HW + p0;
  const size_t xin = (size_t)b * kBlkC * P.HW + p0;
  // u = W2 . t + b2
  float u[kBlkC];
#pragma unroll
  for (int oc = 0; oc < kBlkC; ++oc) u[oc] = m.b2[oc];
#pragma unroll 1
  for (int ic0 = 0; ic0 < kBlkM; ic0 += 16) {
    float tv[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) tv[i] = ld_io<IO>(P.t, tin + (size_t)(ic0 + i) * P.HW);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float* wr = m.w2t + (ic0 + i) * kBlkC;
#pragma unroll
      for (int oc = 0; oc < kBlkC; oc += 4) {
        const float4 w4 = *(const float4*)(wr + oc);
        u[oc] = fmaf(w4.x, tv[i], u[oc]);
        u[oc + 1] = fmaf(w4.y, tv[i], u[oc + 1]);
        u[oc + 2] = fmaf(w4.z, tv[i], u[oc + 2]);
        u[oc + 3] = fmaf(w4.w, tv[i], u[oc + 3]);
      }
    }
  }
  // x1 = x + a1 * u ; LayerNorm 2
#pragma unroll
  for (int oc = 0; oc < kBlkC; ++oc) u[oc] = fmaf(m.a1[oc], u[oc], ld_io<IO>(P.x, xin + (size_t)oc * P.HW));
  float mean, rstd;
  ln_stats<kBlkC>(u, P.ln_eps, mean, rstd);
  const float sigma = 1.0f / rstd;
#pragma unroll
  for (int oc = 0; oc < kBlkC; ++oc) u[oc] = (u[oc] - mean) * rstd;   // u now holds the normalised x1
  // v = W4 . GELU(W3 . xn + b3) + b4, one hidden channel at a time
  float v[kBlkC];
#pragma unroll
  for (int oc = 0; oc < kBlkC; ++oc) v[oc] = m.b4[oc];
#pragma unroll 1
  for (int mc = 0; mc < kBlkM; ++mc) {
    const float* w3 = m.w3f + mc * kBlkC;
    float s0 = m.b3f[mc], s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
    for (int ic = 0; ic < kBlkC; ic += 4) {
      const float4 w4 = *(const float4*)(w3 + ic);
      s0 = fmaf(w4.x, u[ic], s0);
      s1 = fmaf(w4.y, u[ic + 1], s1);
      s2 = fmaf(w4.z, u[ic + 2], s2);
      s3 = fmaf(w4.w, u[ic + 3], s3);
    }
    const float g = gelu_erf((s0 + s1) + (s2 + s3));
    const float* w4r = m.w4t + mc * kBlkC;
#pragma unroll
    for (int oc = 0; oc < kBlkC; oc += 4) {
      const float4 w4 = *(const float4*)(w4r + oc);
      v[oc] = fmaf(w4.x, g, v[oc]);
      v[oc + 1] = fmaf(w4.y, g, v[oc + 1]);
      v[oc + 2] = fmaf(w4.z, g, v[oc + 2]);
      v[oc + 3] = fmaf(w4.w, g, v[oc + 3]);
    }
  }
  // out = x1 + a2 * v, with x1 = xn * sigma + mean
#pragma unroll
  for (int oc = 0; oc < kBlkC; ++oc) {
    const float x1 = fmaf(u[oc], sigma, mean);
    st_io<IO>(P.out, xin + (size_t)oc * P.HW, fmaf(m.a2[oc], v[oc], x1));
  }
}

}  // namespace cvb
