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
// plus a halo of (K/2)*2^L samples per side, clipped to the signal), so every
// sample crosses HBM once in and once out.  Shared memory is fp32, one row per
// channel (row pitches padded so that lanes working on different channels hit
// different bank groups):
//   X0[g]            input segment with zero border
//   S_j[g][s]        un-normalised sub-bands of level j, s = low, high
//   R_j[g]           reconstruction accumulated at level j
// Every cell of X0 / S_j is written by the staging phases (values, or zeros
// outside the signal), so nothing is cleared.  The top level is fused with the
// base convolution in registers: one item = 8 positions of level 1 = 16 output
// samples, stored straight to global memory.
#pragma once

#include "wt2d_fused.cuh"

namespace wt {

struct Plan1d {
  int B, C, N;
  int K, r, rb;
  int nlev;
  int out_stride, Nout;
  int wstride, tapset, wsm;
  int G, g_shift, TX, ntile, ngroups, nthreads;
  int Nj[kMaxFused + 1];
  int pitch[kMaxFused + 1], off[kMaxFused + 1];     // X0 / S_j rows: floats per row, offset
  int rpitch[kMaxFused + 1], roff[kMaxFused + 1];   // R_j rows (j = 0 only with a pooling stride)
  int woff, smem_floats;
  long long xs[3], ys[3];
};

constexpr int kTile1d = 8;   // level positions per item

// K-tap cross-correlation of TW consecutive outputs; `src` is the first sample
// of the (TW+K-1)-sample window, 16-byte aligned.
// K = 0 is the generic instance: the kernel size `kdyn` is a run-time value (any odd size up to kMaxK).
template <int K, int TW>
WT_HD void conv_row(const float* __restrict__ src, const float* __restrict__ wts, float (&acc)[TW], int kdyn) {
  if constexpr (K == 0) {
    for (int j = 0; j < kdyn; ++j) {
      const float w = wts[j];
#pragma unroll
      for (int o = 0; o < TW; ++o) acc[o] = fmaf(w, src[o + j], acc[o]);
    }
  } else {
  (void)kdyn;
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
}

struct Smem1d {
  float* base;
  const Plan1d* p;
  WT_HD float* x0(int g) const { return base + p->off[0] + g * p->pitch[0]; }
  WT_HD float* sub(int j, int g, int s) const { return base + p->off[j] + (s * p->G + g) * p->pitch[j]; }
  WT_HD float* rec(int j, int g) const { return base + p->roff[j] + g * p->rpitch[j]; }
  // tap set of level j (1-based), sub-band s; j = 0: base set
  WT_HD const float* taps(int g, int j, int s) const {
    return base + p->woff + g * p->wsm + p->tapset * (j == 0 ? 0 : 1 + 2 * (j - 1) + s);
  }
};

// Level item: both scaled sub-band convolutions of 8 positions of level j, low-pass
// accumulation (wtconv1d.py:71) and synthesis (wavelet.py:54-59): 16 values of level j-1.
template <int K>
WT_HD void level_item_1d(const Plan1d& p, const Smem1d& sm, int j, int g, int ix, int wx, bool has_r,
                         float (&out)[2 * kTile1d]) {
  constexpr int TW = kTile1d;
  float lo[TW], hi[TW];
#pragma unroll
  for (int o = 0; o < TW; ++o) { lo[o] = 0.f; hi[o] = 0.f; }
  conv_row<K, TW>(sm.sub(j, g, 0) + wx, sm.taps(g, j, 0), lo, p.K);
  conv_row<K, TW>(sm.sub(j, g, 1) + wx, sm.taps(g, j, 1), hi, p.K);
  if (has_r) {
    const float* rj = sm.rec(j, g) + ix * TW;
#pragma unroll
    for (int v = 0; v < TW / 4; ++v) {
      float t[4];
      load4(rj + 4 * v, t);
      lo[4 * v + 0] += t[0]; lo[4 * v + 1] += t[1]; lo[4 * v + 2] += t[2]; lo[4 * v + 3] += t[3];
    }
  }
#pragma unroll
  for (int o = 0; o < TW; ++o) { out[2 * o] = lo[o] + hi[o]; out[2 * o + 1] = lo[o] - hi[o]; }
}

// 16 finished consecutive output samples of one channel -> global memory (no pooling stride)
template <typename T>
WT_HD void store_run16(T* __restrict__ dst, long long s2, const float (&v)[2 * kTile1d], int nvalid) {
  const bool vec = (s2 == 1) && nvalid >= 16 && ((reinterpret_cast<uintptr_t>(dst) & (4 * sizeof(T) - 1)) == 0);
  if (vec) {
#pragma unroll
    for (int q = 0; q < 4; ++q) store4(dst + 4 * q, v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  } else {
#pragma unroll
    for (int o = 0; o < 16; ++o)
      if (o < nvalid) dst[(size_t)o * s2] = Elem<T>::from_f(v[o]);
  }
}

template <typename T, int K>
WT_HD void wt1d_cta(const Plan1d& p, const T* __restrict__ x, T* __restrict__ y,
                    const float* __restrict__ packed, float* smem, int tile, int cg, int nb) {
  constexpr int TW = kTile1d;
  const int nthr = p.nthreads;
  const int d = p.nlev, r = p.r;
  const int c0 = cg * p.G;
  const int gc = imin(p.G, p.C - c0);
  const int gsh = p.g_shift;
  const int t0 = tile * p.TX, t1 = imin(p.N, t0 + p.TX);
  Smem1d sm{smem, &p};
  const T* xb = x + (size_t)nb * p.xs[0] + (size_t)c0 * p.xs[1];
  T* yb = y + (size_t)nb * p.ys[0] + (size_t)c0 * p.ys[1];

  // ---- phase 0: tap sets (asynchronous copies) and the input segment; cells outside the
  //      signal are written as zeros (wtconv1d.py:49-51 and the 'same' padding)
  WT_PHASE(nthr) {
    {
      const int per = p.wsm >> 2;
      const RowWalk w(per, tid, nthr);
      for (int g = w.row0; g < gc; g += w.step) {
        const float4* src = reinterpret_cast<const float4*>(packed + (size_t)(c0 + g) * p.wstride);
        float4* dst = reinterpret_cast<float4*>(smem + p.woff + g * p.wsm);
        for (int k = w.col0; k < per; k += 32) async_copy16(dst + k, src + k);
      }
    }
    const LevelGeo g0 = level_geo(d, r, p.rb, 0, p.N, t0, t1, 3);
    const int xlo = imax(g0.lo, 0), xhi = imin(g0.hi, p.N);
    const int pitch = p.pitch[0];
    const int warp = tid >> 5, lane = tid & 31, nwarp = nthr >> 5;
    const int nblk = (pitch + 127) >> 7;               // 128-sample blocks per row
    const int nvrow = gc * nblk;
    if (warp < nvrow) {
      int g = warp / nblk, b = warp - g * nblk;
      const int dg = nwarp / nblk, db = nwarp - dg * nblk;
      for (int vr = warp; vr < nvrow; vr += nwarp) {
        const T* row = xb + (size_t)g * p.xs[1];
        float* dst = sm.x0(g) + (b << 7);
        const int px_blk = g0.org + (b << 7);
        // 128-bit path: fp32 rows whose block start is 16-byte aligned in global memory
        const bool vec = sizeof(T) == 4 && p.xs[2] == 1 && px_blk >= xlo && px_blk + 127 < xhi &&
                         (b << 7) + 127 < pitch &&
                         ((reinterpret_cast<uintptr_t>(row + px_blk) & 15) == 0);
        if (vec) {
          async_copy16(dst + 4 * lane, reinterpret_cast<const float*>(row) + px_blk + 4 * lane);
        } else if constexpr (sizeof(T) == 4) {
          // coalesced 4-byte asynchronous copies: lane i takes samples i, i+32, i+64, i+96 of the
          // block; cells outside the signal are zero-filled by the copy itself
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int px = px_blk + lane + 32 * k;
            const int col = (b << 7) + lane + 32 * k;
            if (col < pitch)
              async_copy4_zfill(dst + lane + 32 * k, row + (size_t)imin(imax(px, 0), p.N - 1) * p.xs[2],
                                px >= xlo && px < xhi);
          }
        } else {
          // 16-bit activations are converted on the way: clamped loads, zeroed by a select
          float v[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int px = px_blk + lane + 32 * k;
            v[k] = Elem<T>::to_f(row[(size_t)imin(imax(px, 0), p.N - 1) * p.xs[2]]);
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int px = px_blk + lane + 32 * k;
            const int col = (b << 7) + lane + 32 * k;
            if (col < pitch) dst[lane + 32 * k] = (px >= xlo && px < xhi) ? v[k] : 0.f;
          }
        }
        g += dg; b += db;
        if (b >= nblk) { b -= nblk; ++g; }
      }
    }
    async_wait_all();
  }

  // ---- analysis (wavelet.py:46-51); the raw low band feeds the next level.  One item = four
  //      positions; positions outside the signal or without their source pair are zeros.
  for (int j = 1; j <= d; ++j) {
    WT_PHASE(nthr) {
      const int oj = level_geo(d, r, p.rb, j, p.Nj[j], t0, t1, 3).org;
      const int os = level_geo(d, r, p.rb, j - 1, p.Nj[j - 1], t0, t1, 3).org;
      const int pitch = p.pitch[j], sp = p.pitch[j - 1];
      const int ngrp = pitch >> 2;
      const int Nj = p.Nj[j];
      const int dstep = p.G * pitch;
      const RowWalk w(ngrp, tid, nthr);
      for (int g = w.row0; g < gc; g += w.step) {
        const float* s0 = (j == 1) ? sm.x0(g) : sm.sub(j - 1, g, 0);
        float* o0 = sm.sub(j, g, 0);
        for (int gq = w.col0; gq < ngrp; gq += 32) {
          const int px0 = oj + 4 * gq;
          const int sx0 = 2 * px0 - os;
          float lo[4], hi[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int px = px0 + k, sx = sx0 + 2 * k;
            const bool ok = px >= 0 && px < Nj && sx >= 0 && sx + 1 < sp;
            const int cx = imin(imax(sx, 0), sp - 2);
            float a, b;
            if (K != 0 && (K / 2) % 2 == 0) load2(s0 + (cx & ~1), a, b);
            else { a = s0[cx]; b = s0[cx + 1]; }
            lo[k] = ok ? a + b : 0.f;
            hi[k] = ok ? a - b : 0.f;
          }
          store4(o0 + 4 * gq, lo[0], lo[1], lo[2], lo[3]);
          store4(o0 + dstep + 4 * gq, hi[0], hi[1], hi[2], hi[3]);
        }
      }
    }
  }

  // ---- deep levels bottom-up (wtconv1d.py:64-78): 8 positions per item -> 16 values of R_{j-1}
  for (int j = d; j >= 2; --j) {
    WT_PHASE(nthr) {
      const LevelGeo lj = level_geo(d, r, p.rb, j, p.Nj[j], t0, t1, 3);
      const int ncol = level_geo(d, r, p.rb, j - 1, p.Nj[j - 1], t0, t1, 3).n;
      const int ntx = cdiv(lj.n, TW);
      const int total = p.G * ntx;
      const int wbase = lj.a - r - lj.org;
      for (int i = tid; i < total; i += nthr) {
        int ix, g;
        if (gsh >= 0) { ix = i >> gsh; g = i & (p.G - 1); }
        else { ix = i / p.G; g = i - ix * p.G; }
        if (g >= gc) continue;
        float out[2 * TW];
        level_item_1d<K>(p, sm, j, g, ix, wbase + ix * TW, j < d, out);
        float* dst = sm.rec(j - 1, g) + 2 * ix * TW;
        if (2 * ix * TW + 2 * TW <= ncol) {
#pragma unroll
          for (int q = 0; q < 4; ++q) store4(dst + 4 * q, out[4 * q], out[4 * q + 1], out[4 * q + 2], out[4 * q + 3]);
        } else {
#pragma unroll
          for (int o = 0; o < 2 * TW; ++o)
            if (2 * ix * TW + o < ncol) dst[o] = out[o];
        }
      }
    }
  }

  // ---- top level + base convolution + bias (wtconv1d.py:81-82), 16 output samples per item
  WT_PHASE(nthr) {
    const LevelGeo g0 = level_geo(d, r, p.rb, 0, p.N, t0, t1, 3);
    const int n0 = t1 - t0;
    const int ntx = cdiv(n0, 2 * TW);
    const int total = p.G * ntx;
    const int wx0 = g0.a - r - g0.org;
    int w1base = 0;
    if (d >= 1) {
      const LevelGeo g1 = level_geo(d, r, p.rb, 1, p.Nj[1], t0, t1, 3);
      w1base = g1.a - r - g1.org;
    }
    for (int i = tid; i < total; i += nthr) {
      int ix, g;
      if (gsh >= 0) { ix = i >> gsh; g = i & (p.G - 1); }
      else { ix = i / p.G; g = i - ix * p.G; }
      if (g >= gc) continue;
      float acc[2 * TW];
      if (d >= 1) level_item_1d<K>(p, sm, 1, g, ix, w1base + ix * TW, d > 1, acc);
      else {
#pragma unroll
        for (int o = 0; o < 2 * TW; ++o) acc[o] = 0.f;
      }
      const float* wts = sm.taps(g, 0, 0);
      const float bias = wts[p.K];
#pragma unroll
      for (int o = 0; o < 2 * TW; ++o) acc[o] += bias;
      conv_row<K, 2 * TW>(sm.x0(g) + wx0 + ix * 2 * TW, wts, acc, p.K);
      const int nvalid = n0 - ix * 2 * TW;
      if (p.out_stride == 1) {
        store_run16<T>(yb + (size_t)g * p.ys[1] + (size_t)(t0 + ix * 2 * TW) * p.ys[2], p.ys[2], acc, nvalid);
      } else {
        float* dst = sm.rec(0, g) + ix * 2 * TW;     // pooled in the next phase
#pragma unroll
        for (int q = 0; q < 4; ++q) store4(dst + 4 * q, acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
      }
    }
  }

  // ---- pooling stride: average of `stride` consecutive samples (wtconv1d.py:34)
  if (p.out_stride > 1) {
    WT_PHASE(nthr) {
      const int s = p.out_stride;
      const int o0 = t0 / s;                          // TX is a multiple of the stride
      const int o1 = imin(t1 / s, p.Nout);
      const int nc = o1 - o0;
      const int total = gc * nc;
      for (int i = tid; i < total; i += nthr) {
        const int g = i / nc, xx = i - g * nc;
        const float* src = sm.rec(0, g) + xx * s;
        float v = src[0];
        for (int k = 1; k < s; ++k) v += src[k];
        v /= (float)s;
        yb[(size_t)g * p.ys[1] + (size_t)(o0 + xx) * p.ys[2]] = Elem<T>::from_f(v);
      }
    }
  }
}

}  // namespace wt
