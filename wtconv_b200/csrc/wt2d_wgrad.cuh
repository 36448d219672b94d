// Parameter gradients of WTConv2d: the sub-band pyramid of a tensor and the correlation sums
// from which every parameter gradient follows.
//
// With S = un-normalised Haar sub-bands of the input x (level 0: x itself) and G = the same
// pyramid of the output gradient g (the adjoint of the synthesis cascade is the analysis
// cascade: the transform is orthogonal), the K x K correlation sums
//     stat[set][ky*K+kx][c] = sum over samples and positions p of  G_set[n,c,p] * S_set[n,c,p + (ky-r, kx-r)]
// (zero outside the plane) and stat[set][K*K][c] = sum of G_set give, per channel,
//     d base_conv.weight = base_scale * stat[base],   d base_conv.bias = base_scale * stat[base][K*K],
//     d base_scale = <base_conv.weight, stat[base]> + bias * stat[base][K*K],
//     d wavelet_convs[l].weight[4c+s] = wavelet_scale[l][4c+s] * gain_l * stat[1 + 4l + s],
//     d wavelet_scale[l][4c+s] = gain_l * <wavelet_convs[l].weight[4c+s], stat[1 + 4l + s]>,
// gain_l = (analysis tap * synthesis tap)^(l+1), which is what autograd computes for
// wtconv/wtconv2d.py:46-85 and what the reference CUDA backend computes with
// fused_haar_grad_weight_kernel / depthwise_grad_weight_kernel
// (fast_wtconv/cuda_haar/fused_haar_conv.cu:257-342, depthwise_grad.cu:32-101).
//
// Lanes run over 32 consecutive channels; a thread takes a tile of 4 x 8 positions of one
// (sample, channel) plane at a time: the G tile and the S window go to registers in one go,
// then K*K dot products of 32 terms.  Its sums stay in registers over all its tiles; the
// warps of a CTA meet in shared memory, the CTAs of a channel group in global memory
// (floating-point atomics: the summation order, like the reference's, is not fixed).
#pragma once

#include "wt_common.h"

namespace wt {

constexpr int kWgradThreads = 128;
constexpr int kWgradWarps = kWgradThreads / 32;
constexpr int kWgradTH = 4, kWgradTW = 8;

#ifdef __CUDA_ARCH__
#define WT_ATOMIC_ADD(ptr, v) atomicAdd((ptr), (v))
#else
#define WT_ATOMIC_ADD(ptr, v) (*(ptr) += (v))
#endif

// ---- pyramid: one level per launch, thread = (sample, position, channel), channel fastest
struct PyramidLevel {
  int B, C;
  int Hin, Win;              // plane read
  int Hs, Ws;                // positions written: (B, Hs, Ws, 4, C) floats
  long long in_s[4];         // element strides (n, c, row, col) of the plane read
};

template <typename T>
WT_HD void pyramid_item(const PyramidLevel& a, const T* __restrict__ in, float* __restrict__ S, long long i) {
  const int c = (int)(i % a.C);
  long long t = i / a.C;
  const int j = (int)(t % a.Ws);
  t /= a.Ws;
  const int ii = (int)(t % a.Hs);
  const long long n = t / a.Hs;
  const T* p = in + n * a.in_s[0] + c * a.in_s[1] + (long long)(2 * ii) * a.in_s[2] + (long long)(2 * j) * a.in_s[3];
  const bool right = 2 * j + 1 < a.Win, down = 2 * ii + 1 < a.Hin;    // zero extension of odd sizes
  const float va = Elem<T>::to_f(p[0]);
  const float vb = right ? Elem<T>::to_f(p[a.in_s[3]]) : 0.f;
  const float vc = down ? Elem<T>::to_f(p[a.in_s[2]]) : 0.f;
  const float vd = (right && down) ? Elem<T>::to_f(p[a.in_s[2] + a.in_s[3]]) : 0.f;
  const float pp = va + vb, qq = va - vb, uu = vc + vd, vv = vc - vd;
  float* o = S + (((n * a.Hs + ii) * a.Ws + j) * 4) * a.C + c;
  o[0] = pp + uu;                 // LL, LH, HL, HH (wavelet.py:62-67 without the taps)
  o[a.C] = pp - uu;
  o[2 * a.C] = qq + vv;
  o[3 * a.C] = qq - vv;
}

// ---- correlation sums of one set
struct WGradSet {
  int B, C;
  int h, w;                  // plane size of the set
  int tiles_y, tiles_x;
  int nsplit;                // CTAs that share the (sample, tile) items of a channel group
  long long s_s[4], g_s[4];  // element strides (n, c, row, col) of the S and G planes
};

template <typename T, int K>
WT_HD void wgrad_cta(const WGradSet& a, const T* __restrict__ S, const T* __restrict__ G, float* __restrict__ stat,
                     float* __restrict__ smem, int cg, int split) {
  constexpr int r = K / 2;
  constexpr int NA = K * K + 1;
  constexpr int TH = kWgradTH, TW = kWgradTW;
  const int nthr = kWgradThreads;
  const int c0 = cg * 32;

  // ---- phase 1: every thread sums over its tiles; the sums go to shared memory [warp][k][lane]
  WT_PHASE(nthr) {
    const int lane = tid & 31, warp = tid >> 5;
    const int c = imin(c0 + lane, a.C - 1);
    float acc[NA];
#pragma unroll
    for (int k = 0; k < NA; ++k) acc[k] = 0.f;
    const int ntiles = a.tiles_y * a.tiles_x;
    const long long nitems = (long long)a.B * ntiles;
    const int s2 = (int)a.s_s[2], s3 = (int)a.s_s[3], g2 = (int)a.g_s[2], g3 = (int)a.g_s[3];
    for (long long it = (long long)split * kWgradWarps + warp; it < nitems; it += (long long)a.nsplit * kWgradWarps) {
      const int n = (int)(it / ntiles);
      const int t = (int)(it - (long long)n * ntiles);
      const int ty = t / a.tiles_x, tx = t - ty * a.tiles_x;
      const int y0 = ty * TH, x0 = tx * TW;
      const T* sp = S + (long long)n * a.s_s[0] + (long long)c * a.s_s[1];
      const T* gp = G + (long long)n * a.g_s[0] + (long long)c * a.g_s[1];
      T sraw[TH + K - 1][TW + K - 1], graw[TH][TW];
#pragma unroll
      for (int wy = 0; wy < TH + K - 1; ++wy) {
        const int gy = imin(imax(y0 + wy - r, 0), a.h - 1);
#pragma unroll
        for (int wx = 0; wx < TW + K - 1; ++wx) sraw[wy][wx] = sp[gy * s2 + imin(imax(x0 + wx - r, 0), a.w - 1) * s3];
      }
#pragma unroll
      for (int i = 0; i < TH; ++i) {
        const int gy = imin(y0 + i, a.h - 1);
#pragma unroll
        for (int j = 0; j < TW; ++j) graw[i][j] = gp[gy * g2 + imin(x0 + j, a.w - 1) * g3];
      }
      float sw[TH + K - 1][TW + K - 1], gw[TH][TW];
#pragma unroll
      for (int wy = 0; wy < TH + K - 1; ++wy) {
        const bool rowok = y0 + wy - r >= 0 && y0 + wy - r < a.h;
#pragma unroll
        for (int wx = 0; wx < TW + K - 1; ++wx)
          sw[wy][wx] = (rowok && x0 + wx - r >= 0 && x0 + wx - r < a.w) ? Elem<T>::to_f(sraw[wy][wx]) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < TH; ++i)
#pragma unroll
        for (int j = 0; j < TW; ++j)
          gw[i][j] = (y0 + i < a.h && x0 + j < a.w) ? Elem<T>::to_f(graw[i][j]) : 0.f;
#pragma unroll
      for (int ky = 0; ky < K; ++ky)
#pragma unroll
        for (int kx = 0; kx < K; ++kx) {
          float v = acc[ky * K + kx];
#pragma unroll
          for (int i = 0; i < TH; ++i)
#pragma unroll
            for (int j = 0; j < TW; ++j) v = fmaf(gw[i][j], sw[i + ky][j + kx], v);
          acc[ky * K + kx] = v;
        }
      float sg = acc[K * K];
#pragma unroll
      for (int i = 0; i < TH; ++i)
#pragma unroll
        for (int j = 0; j < TW; ++j) sg += gw[i][j];
      acc[K * K] = sg;
    }
    float* dst = smem + (warp * NA) * 32 + lane;
#pragma unroll
    for (int k = 0; k < NA; ++k) dst[k * 32] = acc[k];
  }

  // ---- phase 2: warps of the CTA -> global sums of the channel group
  WT_PHASE(nthr) {
    for (int e = tid; e < NA * 32; e += nthr) {
      const int k = e >> 5, lane = e & 31;
      if (c0 + lane >= a.C) continue;
      float v = 0.f;
#pragma unroll
      for (int wq = 0; wq < kWgradWarps; ++wq) v += smem[(wq * NA + k) * 32 + lane];
      WT_ATOMIC_ADD(stat + (long long)k * a.C + c0 + lane, v);
    }
  }
}

}  // namespace wt
