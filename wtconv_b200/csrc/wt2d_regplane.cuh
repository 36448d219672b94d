// Register-resident kernel for very small planes (up to 8 x 8): one THREAD owns one
// (sample, channel) plane and runs the whole cascade for it in registers.
//
// The deepest planes of a WTConv pyramid are tiny (7x7 -> 4x4 -> 2x2 for every
// WTConvNeXt stage), and a CTA-wide phase structure spends its time in barriers and
// half-empty phases there.  Here nothing is shared between threads except the staged
// tap sets: the plane, its sub-bands (wtconv/util/wavelet.py:62-67), the scaled
// sub-band convolutions (wtconv/wtconv2d.py:57-58), the bottom-up reconstruction
// (wtconv2d.py:64-78, wavelet.py:70-75) and the base path (wtconv2d.py:81-82) are
// fully unrolled straight-line code with compile-time geometry, so zero padding of
// odd sizes and the 'same' padding of the convolutions cost nothing: taps that only
// see zeros are never issued.
//
// Lanes run over 32 consecutive channels (coalesced for channels-last tensors), warps
// over samples.  Used for a whole layer (BASE: reads x, writes y) or for the bottom of a
// larger pyramid: then the input is the un-normalised low-pass plane of level lvl0 (fp32
// planes made by the block-sum reduction) and the result is the reconstruction R of the
// levels below the cut, written as fp32 (B,C,PH,PW) planes for the next shallower launch.
#pragma once

#include "wt_common.h"

namespace wt {

constexpr int kRegPlaneThreads = 128;
constexpr int kRegPlaneWarps = kRegPlaneThreads / 32;

struct RegPlane {
  int B, C;
  int PH, PW;               // plane size of the stage (template parameters of the kernel)
  int K, nlev, lvl0;        // levels lvl0+1 .. lvl0+nlev of the layer
  int has_base;
  int wstride;              // packed floats per channel
  int wbeg, wlen, wpad;     // staged slice of a channel's packed block; its pitch in shared memory
  int samples_per_warp;
  int ngroups, nbatch;      // grid: channel groups of 32, sample blocks
  long long xs[4], ys[4];   // element strides (n,c,h,w) of the tensor read / of the layer output
  long long os[4];          // strides of the fp32 reconstruction written when there is no base path
};

// floats of one 2-D tap set (wt_common.h::tapset_floats) as a compile-time constant
template <int K> struct TapSet2d { static constexpr int value = (K * K + 1 + 3) / 4 * 4; };

// P[y][x] with zero outside the plane; indices are compile-time constants after unrolling
template <int H, int W>
WT_HD float plane_at(const float (&P)[H][W], int y, int x) {
  return (y >= 0 && y < H && x >= 0 && x < W) ? P[(y >= 0 && y < H) ? y : 0][(x >= 0 && x < W) ? x : 0] : 0.f;
}

// Un-normalised 2x2 analysis butterflies (sub-band order LL, LH, HL, HH), zero extension
template <int H, int W>
WT_HD void regplane_analyse(const float (&P)[H][W], float (&S)[4][(H + 1) / 2][(W + 1) / 2]) {
#pragma unroll
  for (int i = 0; i < (H + 1) / 2; ++i) {
#pragma unroll
    for (int j = 0; j < (W + 1) / 2; ++j) {
      const float a = plane_at<H, W>(P, 2 * i, 2 * j), b = plane_at<H, W>(P, 2 * i, 2 * j + 1);
      const float c = plane_at<H, W>(P, 2 * i + 1, 2 * j), d = plane_at<H, W>(P, 2 * i + 1, 2 * j + 1);
      const float pp = a + b, qq = a - b, uu = c + d, vv = c - d;
      S[0][i][j] = pp + uu;
      S[1][i][j] = pp - uu;
      S[2][i][j] = qq + vv;
      S[3][i][j] = qq - vv;
    }
  }
}

// Y += 'same' K x K correlation of S with the tap set at w (16-byte aligned, shared memory)
template <int K, int H, int W>
WT_HD void regplane_conv(const float (&S)[H][W], float (&Y)[H][W], const float* __restrict__ w) {
  constexpr int r = K / 2;
  constexpr int TS = TapSet2d<K>::value;
  float wt[TS];
#pragma unroll
  for (int q = 0; q < TS / 4; ++q) {
    const float4 v = *reinterpret_cast<const float4*>(w + 4 * q);
    wt[4 * q] = v.x; wt[4 * q + 1] = v.y; wt[4 * q + 2] = v.z; wt[4 * q + 3] = v.w;
  }
#pragma unroll
  for (int ky = 0; ky < K; ++ky) {
#pragma unroll
    for (int kx = 0; kx < K; ++kx) {
      const float wv = wt[ky * K + kx];
#pragma unroll
      for (int i = 0; i < H; ++i) {
#pragma unroll
        for (int j = 0; j < W; ++j) {
          const int sy = i + ky - r, sx = j + kx - r;
          if (sy >= 0 && sy < H && sx >= 0 && sx < W) Y[i][j] = fmaf(wv, S[sy][sx], Y[i][j]);
        }
      }
    }
  }
}

// acc (H x W) += reconstruction of NL levels below the plane P.  `w` points at the four tap
// sets of the first of them; deeper levels follow.
template <int K, int H, int W, int NL>
struct RegCascade {
  static constexpr int H1 = (H + 1) / 2, W1 = (W + 1) / 2;
  static WT_HD void run(const float (&P)[H][W], float (&acc)[H][W], const float* __restrict__ w) {
    constexpr int TS = TapSet2d<K>::value;
    float S[4][H1][W1];
    regplane_analyse<H, W>(P, S);
    float R[H1][W1];
#pragma unroll
    for (int i = 0; i < H1; ++i)
#pragma unroll
      for (int j = 0; j < W1; ++j) R[i][j] = 0.f;
    if constexpr (NL > 1) RegCascade<K, H1, W1, NL - 1>::run(S[0], R, w + 4 * TS);
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      float Y[H1][W1];
#pragma unroll
      for (int i = 0; i < H1; ++i)
#pragma unroll
        for (int j = 0; j < W1; ++j) Y[i][j] = (s == 0) ? R[i][j] : 0.f;   // wtconv2d.py:71
      regplane_conv<K, H1, W1>(S[s], Y, w + s * TS);
      // synthesis as signed accumulation, cropped to the plane (wtconv2d.py:76)
#pragma unroll
      for (int i = 0; i < H1; ++i) {
#pragma unroll
        for (int j = 0; j < W1; ++j) {
#pragma unroll
          for (int di = 0; di < 2; ++di) {
#pragma unroll
            for (int dj = 0; dj < 2; ++dj) {
              const int yy = 2 * i + di, xx = 2 * j + dj;
              if (yy < H && xx < W) {
                const bool neg = (s == 1 && di) || (s == 2 && dj) || (s == 3 && (di != dj));
                acc[yy][xx] = neg ? acc[yy][xx] - Y[i][j] : acc[yy][xx] + Y[i][j];
              }
            }
          }
        }
      }
    }
  }
};

// Body of one CTA: channel group `cg` (32 channels), sample block `nb`.
template <typename T, int K, int PH, int PW, int NLEV, bool BASE>
WT_HD void regplane_cta(const RegPlane& a, const T* __restrict__ x, T* __restrict__ y, float* __restrict__ rout,
                        const float* __restrict__ packed, float* __restrict__ smem, int cg, int nb) {
  constexpr int TS = TapSet2d<K>::value;
  const int nthr = kRegPlaneThreads;
  const int c0 = cg * 32;

  // ---- tap sets of the 32 channels -> shared memory (pitch wpad: odd multiple of 16 bytes,
  //      so the 128-bit reads of a quarter warp fall into eight different bank groups)
  WT_PHASE(nthr) {
    const int per = a.wlen / 4;
    for (int i = tid; i < 32 * per; i += nthr) {
      const int lc = i / per, k4 = i - lc * per;
      const int c = imin(c0 + lc, a.C - 1);
      async_copy16(smem + lc * a.wpad + 4 * k4, packed + (size_t)c * a.wstride + a.wbeg + 4 * k4);
    }
    async_wait_all();
  }

  WT_PHASE(nthr) {
    const int lane = tid & 31, warp = tid >> 5;
    const int c = c0 + lane;
    if (c >= a.C) continue;
    const float* w = smem + lane * a.wpad;
    const int xs2 = (int)a.xs[2], xs3 = (int)a.xs[3];
    for (int it = 0; it < a.samples_per_warp; ++it) {
      const int n = (nb * a.samples_per_warp + it) * kRegPlaneWarps + warp;
      if (n >= a.B) break;
      const T* xp = x + (long long)n * a.xs[0] + (long long)c * a.xs[1];

      float X[PH][PW];
#pragma unroll
      for (int yy = 0; yy < PH; ++yy)
#pragma unroll
        for (int xx = 0; xx < PW; ++xx) X[yy][xx] = Elem<T>::to_f(xp[yy * xs2 + xx * xs3]);

      float acc[PH][PW];
      const float* wl = w;
      if constexpr (BASE) {
        const float bias = w[K * K];
#pragma unroll
        for (int yy = 0; yy < PH; ++yy)
#pragma unroll
          for (int xx = 0; xx < PW; ++xx) acc[yy][xx] = bias;
        regplane_conv<K, PH, PW>(X, acc, w);
        wl = w + TS;
      } else {
#pragma unroll
        for (int yy = 0; yy < PH; ++yy)
#pragma unroll
          for (int xx = 0; xx < PW; ++xx) acc[yy][xx] = 0.f;
      }
      if constexpr (NLEV > 0) RegCascade<K, PH, PW, NLEV>::run(X, acc, wl);

      if constexpr (BASE) {
        T* yp = y + (long long)n * a.ys[0] + (long long)c * a.ys[1];
        const int ys2 = (int)a.ys[2], ys3 = (int)a.ys[3];
#pragma unroll
        for (int yy = 0; yy < PH; ++yy)
#pragma unroll
          for (int xx = 0; xx < PW; ++xx) yp[yy * ys2 + xx * ys3] = Elem<T>::from_f(acc[yy][xx]);
      } else {
        float* rp = rout + (long long)n * a.os[0] + (long long)c * a.os[1];
        const int os2 = (int)a.os[2], os3 = (int)a.os[3];
#pragma unroll
        for (int yy = 0; yy < PH; ++yy)
#pragma unroll
          for (int xx = 0; xx < PW; ++xx) rp[yy * os2 + xx * os3] = acc[yy][xx];
      }
    }
  }
}

}  // namespace wt
