// Fused multi-level WTConv1d forward for one CTA (sm_100a).
//
// Replaces the whole body of the reference forward (wtconv/wtconv1d.py:38-87):
// right zero padding of odd lengths, 2-tap Haar analysis of every level, the
// 2C-channel depthwise K-tap convolution and scale of every level, the
// bottom-up inverse transform with low-pass accumulation, the base depthwise
// convolution with scale and bias, the final add and the average-pool stride.
//
// A CTA owns G channels of one sample and a tile of TX output samples; every
// level of the cascade is computed on chip from one staged input segment (tile
// plus a halo of (K/2)*2^L samples per side, clipped to the signal).  Shared
// memory is fp32 and row-major per channel:
//   X0[g]            input segment with zero border
//   S_j[g][s]        un-normalised sub-bands of level j, s = low, high
//   R_j[g]           reconstruction accumulated at level j
#pragma once

#include "wt2d_plan.h"

namespace wt {

struct Plan1d {
  int B, C, N;
  int K, r, rb;
  int nlev;
  int out_stride, Nout;
  int wstride, tapset;
  int G, TX, ntile, ngroups, nthreads;
  int Nj[kMaxFused + 1];
  int pitch[kMaxFused + 1], off[kMaxFused + 1];
  int rpitch[kMaxFused + 1], roff[kMaxFused + 1];
  int woff, smem_floats;
  long long xs[3], ys[3];
};

constexpr int kTile1d = 8;   // outputs per thread of the 1-D convolution tile

// K-tap cross-correlation of TW consecutive outputs; `src` is the first sample
// of the (TW+K-1)-sample window, 16-byte aligned.
template <int K, int TW>
WT_HD void conv_row(const float* __restrict__ src, const float* __restrict__ wts, float (&acc)[TW]) {
  constexpr int WIN = TW + K - 1;
  constexpr int NV = (WIN + 3) / 4;
  constexpr int NW = (K + 3) / 4;
  float w[NW * 4], row[NV * 4];
#pragma unroll
  for (int v = 0; v < NW; ++v) {
    const float4 t = reinterpret_cast<const float4*>(wts)[v];
    w[4 * v + 0] = t.x; w[4 * v + 1] = t.y; w[4 * v + 2] = t.z; w[4 * v + 3] = t.w;
  }
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const float4 t = reinterpret_cast<const float4*>(src)[v];
    row[4 * v + 0] = t.x; row[4 * v + 1] = t.y; row[4 * v + 2] = t.z; row[4 * v + 3] = t.w;
  }
#pragma unroll
  for (int j = 0; j < K; ++j)
#pragma unroll
    for (int o = 0; o < TW; ++o) acc[o] = fmaf(w[j], row[o + j], acc[o]);
}

template <typename T, int K>
WT_HD void wt1d_cta(const Plan1d& p, const T* __restrict__ x, T* __restrict__ y,
                    const float* __restrict__ packed, float* smem, int bid) {
  constexpr int TW = kTile1d;
  const int nthr = p.nthreads;
  const int d = p.nlev, r = p.r;
  const int tile = bid % p.ntile;
  int rest = bid / p.ntile;
  const int cg = rest % p.ngroups;
  const int nb = rest / p.ngroups;
  const int c0 = cg * p.G;
  const int gc = imin(p.G, p.C - c0);

  Axis ax;
  axis_geometry(d, r, p.rb, 1, p.Nj, tile * p.TX, imin(p.N, (tile + 1) * p.TX), 4, ax);

  // ---- clear, stage weights
  WT_PHASE(nthr) {
    float4* z = reinterpret_cast<float4*>(smem);
    const int n4 = p.smem_floats / 4;
    for (int i = tid; i < n4; i += nthr) z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  WT_PHASE(nthr) {
    const int n4 = gc * p.wstride / 4;
    const float4* src = reinterpret_cast<const float4*>(packed + (size_t)c0 * p.wstride);
    float4* dst = reinterpret_cast<float4*>(smem + p.woff);
    for (int i = tid; i < n4; i += nthr) dst[i] = src[i];
    // ---- input segment (zero outside the signal, wtconv1d.py:49-51)
    const int x0 = imax(ax.lo[0], 0), x1 = imin(ax.hi[0], p.N);
    const int nc = x1 - x0;
    const int total = gc * nc;
    const T* xb = x + (size_t)nb * p.xs[0] + (size_t)c0 * p.xs[1];
    for (int i = tid; i < total; i += nthr) {
      const int g = i / nc, xx = i - g * nc;
      smem[p.off[0] + g * p.pitch[0] + (x0 + xx - ax.org[0])] =
          Elem<T>::to_f(xb[(size_t)g * p.xs[1] + (size_t)(x0 + xx) * p.xs[2]]);
    }
  }

  // ---- analysis (wavelet.py:46-51); the raw low band feeds the next level
  for (int j = 1; j <= d; ++j) {
    WT_PHASE(nthr) {
      const int x0 = imax(ax.lo[j], 0), x1 = imin(ax.hi[j], p.Nj[j]);
      const int nc = x1 - x0;
      const int total = gc * nc;
      const int sns = (j == 1) ? 1 : 2;
      for (int i = tid; i < total; i += nthr) {
        const int g = i / nc, xx = i - g * nc;
        const float* s = smem + p.off[j - 1] + (g * sns) * p.pitch[j - 1] + (2 * (x0 + xx) - ax.org[j - 1]);
        float* o = smem + p.off[j] + (g * 2) * p.pitch[j] + (x0 + xx - ax.org[j]);
        const float a = s[0], b = s[1];
        o[0] = a + b;
        o[p.pitch[j]] = a - b;
      }
    }
  }

  // ---- bottom-up: sub-band convolutions, low-pass accumulation, synthesis (wtconv1d.py:64-78)
  for (int j = d; j >= 1; --j) {
    WT_PHASE(nthr) {
      const int ntx = cdiv(ax.n[j], TW);
      const int total = gc * ntx;
      const bool has_r = (j < d);
      for (int i = tid; i < total; i += nthr) {
        const int g = i / ntx, ix = i - g * ntx;
        const int wx = ax.a[j] + ix * TW - r - ax.org[j];
        float lo[TW], hi[TW];
#pragma unroll
        for (int o = 0; o < TW; ++o) { lo[o] = 0.f; hi[o] = 0.f; }
        const float* wts = smem + p.woff + g * p.wstride + p.tapset * (1 + 2 * (j - 1));
        conv_row<K, TW>(smem + p.off[j] + (g * 2) * p.pitch[j] + wx, wts, lo);
        conv_row<K, TW>(smem + p.off[j] + (g * 2 + 1) * p.pitch[j] + wx, wts + p.tapset, hi);
        if (has_r) {
          const float* rj = smem + p.roff[j] + g * p.rpitch[j] + ix * TW;
#pragma unroll
          for (int o = 0; o < TW; ++o) lo[o] += rj[o];
        }
        float* out = smem + p.roff[j - 1] + g * p.rpitch[j - 1];
        const int ncol = ax.n[j - 1];
#pragma unroll
        for (int o = 0; o < TW; ++o) {
          const int ox = 2 * (ix * TW + o);
          if (ox < ncol) out[ox] = lo[o] + hi[o];
          if (ox + 1 < ncol) out[ox + 1] = lo[o] - hi[o];
        }
      }
    }
  }

  // ---- base convolution + bias on top of R_0 (wtconv1d.py:81-82)
  WT_PHASE(nthr) {
    const int ntx = cdiv(ax.n[0], TW);
    const int total = gc * ntx;
    for (int i = tid; i < total; i += nthr) {
      const int g = i / ntx, ix = i - g * ntx;
      const int wx = ax.t0 + ix * TW - r - ax.org[0];
      float* r0 = smem + p.roff[0] + g * p.rpitch[0] + ix * TW;
      const float* wts = smem + p.woff + g * p.wstride;
      const float bias = wts[K];
      float acc[TW];
#pragma unroll
      for (int o = 0; o < TW; ++o) acc[o] = r0[o] + bias;
      conv_row<K, TW>(smem + p.off[0] + g * p.pitch[0] + wx, wts, acc);
#pragma unroll
      for (int o = 0; o < TW; ++o) r0[o] = acc[o];
    }
  }

  // ---- store; stride > 1 is an average pool of `stride` samples (wtconv1d.py:34)
  WT_PHASE(nthr) {
    const int s = p.out_stride;
    const int o0 = ax.t0 / s;                       // TX is a multiple of the stride
    const int o1 = imin(ax.t1 / s, p.Nout);
    const int nc = o1 - o0;
    const int total = gc * nc;
    T* yb = y + (size_t)nb * p.ys[0] + (size_t)c0 * p.ys[1];
    for (int i = tid; i < total; i += nthr) {
      const int g = i / nc, xx = i - g * nc;
      const float* src = smem + p.roff[0] + g * p.rpitch[0] + ((o0 + xx) * s - ax.t0);
      float v = src[0];
      if (s > 1) {
        for (int k = 1; k < s; ++k) v += src[k];
        v /= (float)s;
      }
      yb[(size_t)g * p.ys[1] + (size_t)(o0 + xx) * p.ys[2]] = Elem<T>::from_f(v);
    }
  }
}

}  // namespace wt
