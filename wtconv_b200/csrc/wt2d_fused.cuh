// Fused multi-level WTConv2d forward for one CTA (sm_100a).
//
// Replaces, for the tile a CTA owns, the whole body of the reference forward
// (wtconv/wtconv2d.py:38-87): zero padding of odd sizes, Haar analysis of every
// level, the 4C-channel depthwise KxK convolution and scale of every level, the
// bottom-up inverse transform with the low-pass accumulation, the base
// depthwise convolution with its scale and bias, the final add and the stride.
//
// Shared-memory data layout (planar per channel g, planes padded so that the
// eight lanes of a quarter warp, which work on eight different channels, hit
// eight different 16-byte bank groups):
//   X0[g]            input tile with zero border; kept in the activation type when it
//                    is 16-bit and comes straight from x, fp32 otherwise
//   S_j[s][g]        fp32  un-normalised Haar sub-bands of level j, s = LL,LH,HL,HH
//   Y[s][g]          fp32  scaled sub-band convolutions of one deep level (scratch)
//   R_j[g]           fp32  reconstruction accumulated at level j
//   OUT[g]           T     finished output tile, staged for coalesced stores
// The Haar taps are not applied here: the packed parameters carry the product
// of the analysis and synthesis taps of each depth, so analysis and synthesis
// are pure add/sub butterflies on un-normalised coefficients.
//
// Work split inside the CTA:
//   * the top level of the stage (the largest one, ~86 % of the FMAs together
//     with the base convolution) runs as register-tiled items of 2x4 positions:
//     four sub-band convolutions, the synthesis butterfly and the 4x8-pixel base
//     convolution all stay in registers, 64 accumulators per thread;
//   * deeper levels are small: one item is one sub-band of a 2x4 / 4x4 tile, the
//     four sub-bands meet again in shared memory for the synthesis butterfly;
//   * staging phases (load, analysis, store) move four pixels per step with
//     128-bit accesses and write every cell of their arrays, so nothing is cleared.
#pragma once

#include "wt2d_plan.h"

namespace wt {

template <bool B, typename A, typename C> struct Select { typedef A type; };
template <typename A, typename C> struct Select<false, A, C> { typedef C type; };

// four consecutive elements of a shared-memory row
WT_HD void load4(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <typename H>
WT_HD void load4(const H* p, float (&v)[4]) {
  Chunk<H, 8> c;
  c.raw = *reinterpret_cast<const uint2*>(p);
#pragma unroll
  for (int e = 0; e < 4; ++e) v[e] = Elem<H>::to_f(c.get(e));
}
WT_HD void store4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <typename H>
WT_HD void store4(H* p, float a, float b, float c, float d) {
  Chunk<H, 8> k;
  k.set(0, Elem<H>::from_f(a)); k.set(1, Elem<H>::from_f(b));
  k.set(2, Elem<H>::from_f(c)); k.set(3, Elem<H>::from_f(d));
  *reinterpret_cast<uint2*>(p) = k.raw;
}
// two consecutive elements (8-byte / 4-byte aligned)
WT_HD void load2(const float* p, float& a, float& b) {
  const float2 t = *reinterpret_cast<const float2*>(p);
  a = t.x; b = t.y;
}
template <typename H>
WT_HD void load2(const H* p, float& a, float& b) {
  Chunk<H, 4> c;
  c.raw = *reinterpret_cast<const unsigned int*>(p);
  a = Elem<H>::to_f(c.get(0)); b = Elem<H>::to_f(c.get(1));
}

// ---------------------------------------------------------------------------
// Register-tiled depthwise KxK cross-correlation of a TH x TW tile.
// `src` points at the top-left element of the (TH+K-1) x (TW+K-1) window, aligned
// to four elements; rows are `pitch` elements apart (pitch % 4 == 0).  One input
// row at a time is read with 128-bit (fp32) / 64-bit (16-bit source) loads and
// applied to all output rows it contributes to, so each loaded element feeds
// about K*min(K,TH)*TW/(TW+K-1) FMAs.
// ---------------------------------------------------------------------------
// K = 0 is the generic instance: the kernel size `kdyn` is a run-time value, taps and window
// elements are read one by one (any odd size up to kMaxK; slower than the unrolled sizes).
template <int K, int TH, int TW, typename ST>
WT_HD void conv_tile(const ST* __restrict__ src, int pitch, const float* __restrict__ wts,
                     float (&acc)[TH][TW], int kdyn) {
  if constexpr (K == 0) {
    for (int i = 0; i < kdyn; ++i)
      for (int j = 0; j < kdyn; ++j) {
        const float w = wts[i * kdyn + j];
#pragma unroll
        for (int oh = 0; oh < TH; ++oh)
#pragma unroll
          for (int ow = 0; ow < TW; ++ow)
            acc[oh][ow] = fmaf(w, Elem<ST>::to_f(src[(oh + i) * pitch + ow + j]), acc[oh][ow]);
      }
  } else {
  (void)kdyn;
  constexpr int WIN = TW + K - 1;
  constexpr int NV = (WIN + 3) / 4;
  constexpr int NW = (K * K + 3) / 4;
  float w[NW * 4];
#pragma unroll
  for (int v = 0; v < NW; ++v) {
    const float4 t = reinterpret_cast<const float4*>(wts)[v];
    w[4 * v + 0] = t.x; w[4 * v + 1] = t.y; w[4 * v + 2] = t.z; w[4 * v + 3] = t.w;
  }
#pragma unroll
  for (int rr = 0; rr < TH + K - 1; ++rr) {
    float row[NV * 4];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      float t[4];
      load4(src + rr * pitch + 4 * v, t);
      row[4 * v + 0] = t[0]; row[4 * v + 1] = t[1]; row[4 * v + 2] = t[2]; row[4 * v + 3] = t[3];
    }
#pragma unroll
    for (int i = 0; i < K; ++i) {
      const int oh = rr - i;
      if (oh >= 0 && oh < TH) {
#pragma unroll
        for (int j = 0; j < K; ++j) {
#pragma unroll
          for (int ow = 0; ow < TW; ++ow) acc[oh][ow] = fmaf(w[i * K + j], row[ow + j], acc[oh][ow]);
        }
      }
    }
  }
  }
}

struct Smem2d {
  float* base;
  const Plan2d* p;
  template <typename XT> WT_HD XT* x0(int g) const { return reinterpret_cast<XT*>(base + p->off[0]) + g * p->plane[0]; }
  WT_HD float* sub(int j, int g, int s) const { return base + p->off[j] + (s * p->G + g) * p->plane[j]; }
  WT_HD float* rec(int j, int g) const { return base + p->roff[j] + g * p->rplane[j]; }
  WT_HD float* ybuf(int g, int s) const { return base + p->yoff + (s * p->G + g) * p->yplane; }
  // tap set of level j (1-based within the stage), sub-band s; j = 0: base set
  WT_HD const float* taps(int g, int j, int s) const {
    return base + p->woff + g * p->wsm + p->tapset * (j == 0 ? 0 : p->has_base + 4 * (j - 1) + s);
  }
};

// Synthesis butterfly of one position (wavelet.py:70-75, taps folded on the host)
WT_HD void synth4(float ll, float lh, float hl, float hh, float& o00, float& o01, float& o10, float& o11) {
  const float pp = ll + lh, qq = ll - lh, uu = hl + hh, vv = hl - hh;
  o00 = pp + uu; o01 = pp - uu; o10 = qq + vv; o11 = qq - vv;
}

// Geometry of the CTA's tile: the two tile ranges plus what level_geo needs.  Levels are
// evaluated on demand (closed form, registers only).
struct TileGeo {
  int d, r, rb;
  int ty0, ty1, tx0, tx1;
  const int* Hj;
  const int* Wj;
  WT_HD LevelGeo y(int j) const { return level_geo(d, r, rb, j, Hj[j], ty0, ty1, 0); }
  WT_HD LevelGeo x(int j) const { return level_geo(d, r, rb, j, Wj[j], tx0, tx1, 3); }
};

// ---------------------------------------------------------------------------
// Top-level item: 2 x 4 positions of level 1 of this stage for one channel.
// Four scaled sub-band convolutions, low-pass accumulation of the deeper
// reconstruction (wtconv2d.py:71) and the synthesis butterfly give the 4 x 8
// block of R_0 in registers.  With FUSE_BASE the base convolution and bias
// (wtconv2d.py:81-82) are accumulated on top and the finished block goes to the
// OUT staging tile; otherwise the block is written to R_0 (cropped).
// (wy1, wx1) / (wy0, wx0): array coordinates of the item's level-1 / level-0 window.
// ---------------------------------------------------------------------------
template <typename T, typename XT, int K, bool FUSE_BASE>
WT_HD void top_item(const Plan2d& p, const Smem2d& sm, int g, int iy, int ix, int wy1, int wx1, int wy0, int wx0,
                    int nrow0, int ncol0, bool has_r, T* __restrict__ out_tile, T* __restrict__ ytile,
                    float* __restrict__ rtile) {
  constexpr int TH = 2, TW = 4;
  float acc[2 * TH][2 * TW];
  {
    // the 2x2 block of a position starts from the deeper reconstruction (it enters all four
    // outputs with a plus sign, like the low-pass band)
#pragma unroll
    for (int i = 0; i < TH; ++i) {
      float t[4] = {0.f, 0.f, 0.f, 0.f};
      if (has_r) load4(sm.rec(1, g) + (iy * TH + i) * p.rpitch[1] + ix * TW, t);
#pragma unroll
      for (int q = 0; q < TW; ++q) {
        acc[2 * i][2 * q] = t[q]; acc[2 * i][2 * q + 1] = t[q];
        acc[2 * i + 1][2 * q] = t[q]; acc[2 * i + 1][2 * q + 1] = t[q];
      }
    }
    // one pass per sub-band (kept as a loop: four times less code to fetch); the synthesis
    // butterfly (wavelet.py:70-75) is applied as signed accumulation: LH flips the odd row,
    // HL the odd column, HH both
    const int pitch = p.pitch[1];
    const int sstep = p.G * p.plane[1];
    const float* sb = sm.sub(1, g, 0) + wy1 * pitch + wx1;
    const float* tp = sm.taps(g, 1, 0);
#pragma unroll 1
    for (int s = 0; s < 4; ++s) {
      float y[TH][TW];
#pragma unroll
      for (int i = 0; i < TH; ++i)
#pragma unroll
        for (int q = 0; q < TW; ++q) y[i][q] = 0.f;
      conv_tile<K, TH, TW, float>(sb + s * sstep, pitch, tp + s * p.tapset, y, p.K);
      const float fy = (s & 1) ? -1.f : 1.f, fx = (s & 2) ? -1.f : 1.f, fxy = fx * fy;
#pragma unroll
      for (int i = 0; i < TH; ++i)
#pragma unroll
        for (int q = 0; q < TW; ++q) {
          acc[2 * i][2 * q] += y[i][q];
          acc[2 * i][2 * q + 1] = fmaf(fx, y[i][q], acc[2 * i][2 * q + 1]);
          acc[2 * i + 1][2 * q] = fmaf(fy, y[i][q], acc[2 * i + 1][2 * q]);
          acc[2 * i + 1][2 * q + 1] = fmaf(fxy, y[i][q], acc[2 * i + 1][2 * q + 1]);
        }
    }
  }
  if (FUSE_BASE) {
    const int pitch = p.pitch[0];
    const float* wts = sm.taps(g, 0, 0);
    const float bias = wts[p.K * p.K];
#pragma unroll
    for (int i = 0; i < 2 * TH; ++i)
#pragma unroll
      for (int q = 0; q < 2 * TW; ++q) acc[i][q] += bias;
    conv_tile<K, 2 * TH, 2 * TW, XT>(sm.x0<XT>(g) + wy0 * pitch + wx0, pitch, wts, acc, p.K);
    if (p.direct_store) {
      // finished pixels -> y: `ytile` is the tile's first pixel of the group's first channel
      const int ys2 = (int)p.ys[2], ys3 = (int)p.ys[3];
      T* o = ytile + g + (iy * 2 * TH) * ys2 + (ix * 2 * TW) * ys3;
#pragma unroll
      for (int i = 0; i < 2 * TH; ++i) {
        if (iy * 2 * TH + i >= nrow0) continue;
#pragma unroll
        for (int q = 0; q < 2 * TW; ++q)
          if (ix * 2 * TW + q < ncol0) o[i * ys2 + q * ys3] = Elem<T>::from_f(acc[i][q]);
      }
    } else {
      // finished pixels -> OUT[g]; the tile is allocated with the overhang of partial items
      T* o = out_tile + g * p.oplane + (iy * 2 * TH) * p.opitch + ix * 2 * TW;
#pragma unroll
      for (int i = 0; i < 2 * TH; ++i) {
        store4(o + i * p.opitch, acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        store4(o + i * p.opitch + 4, acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
      }
    }
  } else {
    if (p.direct_store) {
      // reconstruction block -> the fp32 planes in global memory: `rtile` is the tile's first
      // element of the group's first channel; rows of eight floats, 128-bit stores when whole
      float* out = rtile + (size_t)g * ((size_t)p.H * p.W) + (size_t)(iy * 2 * TH) * p.W + ix * 2 * TW;
      const bool whole = (ix * 2 * TW + 2 * TW <= ncol0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) && ((p.W & 3) == 0);
#pragma unroll
      for (int i = 0; i < 2 * TH; ++i) {
        if (iy * 2 * TH + i >= nrow0) continue;
        float* orow = out + (size_t)i * p.W;
        if (whole) {
          store4(orow, acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
          store4(orow + 4, acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
        } else {
#pragma unroll
          for (int q = 0; q < 2 * TW; ++q)
            if (ix * 2 * TW + q < ncol0) orow[q] = acc[i][q];
        }
      }
    } else {
      float* out = sm.rec(0, g);
      const int opitch = p.rpitch[0];
#pragma unroll
      for (int i = 0; i < 2 * TH; ++i) {
        const int oy = iy * 2 * TH + i;
#pragma unroll
        for (int q = 0; q < 2 * TW; ++q) {
          const int ox = ix * 2 * TW + q;
          if (oy < nrow0 && ox < ncol0) out[oy * opitch + ox] = acc[i][q];
        }
      }
    }
  }
}

// Base-only layer (no wavelet level in this stage): OUT = bias + base conv.
template <typename T, typename XT, int K>
WT_HD void base_item(const Plan2d& p, const Smem2d& sm, int g, int iy, int ix, int wy0, int wx0,
                     T* __restrict__ out_tile) {
  constexpr int BH = 4, BW = 8;
  const int pitch = p.pitch[0];
  const float* wts = sm.taps(g, 0, 0);
  const float bias = wts[p.K * p.K];
  float acc[BH][BW];
#pragma unroll
  for (int i = 0; i < BH; ++i)
#pragma unroll
    for (int q = 0; q < BW; ++q) acc[i][q] = bias;
  conv_tile<K, BH, BW, XT>(sm.x0<XT>(g) + wy0 * pitch + wx0, pitch, wts, acc, p.K);
  T* o = out_tile + g * p.oplane + (iy * BH) * p.opitch + ix * BW;
#pragma unroll
  for (int i = 0; i < BH; ++i) {
    store4(o + i * p.opitch, acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    store4(o + i * p.opitch + 4, acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
  }
}

// Deep-level item: one sub-band s of a TH x 4 tile of level j -> Y[s][g]
template <int K, int TH>
WT_HD void deep_item(const Plan2d& p, const Smem2d& sm, int j, int g, int s, int iy, int ix, int wy, int wx) {
  const int pitch = p.pitch[j];
  float y[TH][4];
#pragma unroll
  for (int i = 0; i < TH; ++i)
#pragma unroll
    for (int q = 0; q < 4; ++q) y[i][q] = 0.f;
  conv_tile<K, TH, 4, float>(sm.sub(j, g, s) + wy * pitch + wx, pitch, sm.taps(g, j, s), y, p.K);
  float* o = sm.ybuf(g, s) + (iy * TH) * p.ypitch + ix * 4;
#pragma unroll
  for (int i = 0; i < TH; ++i) store4(o + i * p.ypitch, y[i][0], y[i][1], y[i][2], y[i][3]);
}

// ---------------------------------------------------------------------------
// Row walker of the staging phases.  A phase moves `nrows` rows of `ncols` items;
// P2 = 2^shift >= min(ncols, 32) lanes share a row, so thread t starts at row
// t >> shift, column t & (P2-1), and steps nthr >> shift rows: no division in the
// loops.  Rows that are flattened (channel, row) pairs are split with one division
// per thread and phase, then advanced incrementally.
// ---------------------------------------------------------------------------
struct RowWalk {
  int shift, col0, row0, step;
  WT_HD RowWalk(int ncols, int tid, int nthr) {
    shift = lane_shift(ncols);
    col0 = tid & ((1 << shift) - 1);
    row0 = tid >> shift;
    step = nthr >> shift;
  }
};

// ---------------------------------------------------------------------------
// Staging of the input tile.  Every cell of the X0 arrays is written: pixels of
// the plane that the tile needs get their value, everything else (the zero
// extension of wtconv2d.py:49-51, the 'same' padding, the overhang of partial
// thread tiles) gets 0 -- so shared memory never has to be cleared.  One item is
// four consecutive columns; all global loads of an item are issued before
// their first use.
// ---------------------------------------------------------------------------
struct FillRange {   // valid source range in plane coordinates and the array origin
  int ylo, yhi, xlo, xhi, orgy, orgx;
};

// Channels-last: one item = four pixels x CB bytes of consecutive channels.  All loads are
// unconditional (clamped to a valid pixel) so that they issue back to back -- two rows, eight
// loads per thread in flight -- and pixels the tile must not take from the plane are zeroed by
// a select afterwards.
template <typename T, typename XT, int CB>
WT_HD void fill_x0_chunks(const Plan2d& p, const T* __restrict__ src, XT* __restrict__ dst, const FillRange& fr,
                          int tid, int nthr) {
  constexpr int VEC = Chunk<T, CB>::VEC;
  if (VEC < 1) return;
  constexpr int V = VEC > 0 ? VEC : 1;
  constexpr int U = 2;                            // rows in flight per thread
  typedef typename RawChunk<CB>::type Raw;
  const int rows = p.rows[0], pitch = p.pitch[0], plane = p.plane[0];
  const int nch = p.G / V;                        // power of two (G and V are)
  const int nsh = lane_shift(nch);
  const int ncols = (pitch >> 2) * nch;
  const int xs2 = (int)p.xs[2], xs3 = (int)p.xs[3];
  const RowWalk w(ncols, tid, nthr);
  for (int rr0 = w.row0; rr0 < rows; rr0 += U * w.step) {
    for (int ci = w.col0; ci < ncols; ci += 32) {
      const int gq = ci >> nsh, ch = ci & (nch - 1);
      const int px0 = fr.orgx + 4 * gq;
      Chunk<T, CB> c[U][4];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int py = fr.orgy + rr0 + u * w.step;
        const T* s0 = src + imin(imax(py, 0), p.Hsrc - 1) * xs2 + ch * V;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          c[u][k].raw = *reinterpret_cast<const Raw*>(s0 + imin(imax(px0 + k, 0), p.Wsrc - 1) * xs3);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int rr = rr0 + u * w.step;
        if (rr >= rows) break;
        const int py = fr.orgy + rr;
        const bool rowok = py >= fr.ylo && py < fr.yhi;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const bool ok = rowok && (px0 + k) >= fr.xlo && (px0 + k) < fr.xhi;
          if (!ok) c[u][k].raw = Raw();           // zero bits = 0.0 in every activation type
        }
        XT* dd = dst + (ch * V) * plane + rr * pitch + 4 * gq;
        if constexpr (sizeof(XT) == 2) {
          // X0 keeps the 16-bit activation type: a pure 4 x V transpose, no conversion
#pragma unroll
          for (int e = 0; e < V; ++e) {
            Chunk<T, 8> q;
            q.set(0, c[u][0].get(e)); q.set(1, c[u][1].get(e)); q.set(2, c[u][2].get(e)); q.set(3, c[u][3].get(e));
            *reinterpret_cast<uint2*>(dd + e * plane) = q.raw;
          }
        } else {
#pragma unroll
          for (int e = 0; e < V; ++e)
            store4(dd + e * plane, Elem<T>::to_f(c[u][0].get(e)), Elem<T>::to_f(c[u][1].get(e)),
                   Elem<T>::to_f(c[u][2].get(e)), Elem<T>::to_f(c[u][3].get(e)));
        }
      }
    }
  }
}

// Channels-last with reduction: every destination pixel is the sum of an EDGE x EDGE block of
// source pixels (the low-pass input of a deep stage, wtconv2d.py:49-54, formed straight from x).
// 4*EDGE*EDGE unconditional loads per item, then predicated accumulation.
template <typename T, int CB, int EDGE>
WT_HD void fill_x0_chunks_reduced(const Plan2d& p, const T* __restrict__ src, float* __restrict__ dst,
                                  const FillRange& fr, int tid, int nthr) {
  constexpr int VEC = Chunk<T, CB>::VEC;
  if (VEC < 1) return;
  constexpr int V = VEC > 0 ? VEC : 1;
  typedef typename RawChunk<CB>::type Raw;
  const int rows = p.rows[0], pitch = p.pitch[0], plane = p.plane[0];
  const int nch = p.G / V;
  const int nsh = lane_shift(nch);
  const int ncols = (pitch >> 2) * nch;
  const int xs2 = (int)p.xs[2], xs3 = (int)p.xs[3];
  const RowWalk w(ncols, tid, nthr);
  for (int rr = w.row0; rr < rows; rr += w.step) {
    const int py = fr.orgy + rr;
    const bool rowok = py >= fr.ylo && py < fr.yhi;
    for (int ci = w.col0; ci < ncols; ci += 32) {
      const int gq = ci >> nsh, ch = ci & (nch - 1);
      const int px0 = fr.orgx + 4 * gq;
      Chunk<T, CB> c[4][EDGE * EDGE];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int px = imax(px0 + k, 0);
#pragma unroll
        for (int b = 0; b < EDGE * EDGE; ++b) {
          const int sy = imin(imax(py, 0) * EDGE + b / EDGE, p.Hsrc - 1);
          const int sx = imin(px * EDGE + b % EDGE, p.Wsrc - 1);
          c[k][b].raw = *reinterpret_cast<const Raw*>(src + sy * xs2 + sx * xs3 + ch * V);
        }
      }
      float v[4][V];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int px = px0 + k;
        const bool pok = rowok && px >= fr.xlo && px < fr.xhi;
#pragma unroll
        for (int e = 0; e < V; ++e) v[k][e] = 0.f;
#pragma unroll
        for (int by = 0; by < EDGE; ++by) {
          float racc[V];
#pragma unroll
          for (int e = 0; e < V; ++e) racc[e] = 0.f;
#pragma unroll
          for (int bx = 0; bx < EDGE; ++bx) {
            const bool ok = pok && (py * EDGE + by) < p.Hsrc && (px * EDGE + bx) < p.Wsrc;
#pragma unroll
            for (int e = 0; e < V; ++e) racc[e] += ok ? Elem<T>::to_f(c[k][by * EDGE + bx].get(e)) : 0.f;
          }
#pragma unroll
          for (int e = 0; e < V; ++e) v[k][e] += racc[e];
        }
      }
      float* dd = dst + (ch * V) * plane + rr * pitch + 4 * gq;
#pragma unroll
      for (int e = 0; e < V; ++e) store4(dd + e * plane, v[0][e], v[1][e], v[2][e], v[3][e]);
    }
  }
}

// Any layout, any reduction edge: one item = four consecutive pixels of one channel.
// Lanes walk along a row, so NCHW rows are read coalesced (128-bit when aligned).
template <typename T, typename XT>
WT_HD void fill_x0_planar(const Plan2d& p, const T* __restrict__ src, XT* __restrict__ dst, const FillRange& fr,
                          int gc, int tid, int nthr) {
  const int rows = p.rows[0], pitch = p.pitch[0], plane = p.plane[0];
  const int ngrp = pitch >> 2;
  const int nrows = gc * rows;
  const int edge = 1 << p.in_shift;
  const bool vec_ok = (edge == 1) && p.xs[3] == 1 && (sizeof(T) == 4) && ((p.xs[2] & 3) == 0) &&
                      ((p.xs[1] & 3) == 0) && ((p.xs[0] & 3) == 0) &&
                      ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
  const RowWalk w(ngrp, tid, nthr);
  if (w.row0 >= nrows) return;
  int g = w.row0 / rows, rr = w.row0 - g * rows;
  const int dg = w.step / rows, drr = w.step - dg * rows;
  for (int row = w.row0; row < nrows; row += w.step) {
    const int py = fr.orgy + rr;
    const bool rowok = py >= fr.ylo && py < fr.yhi;
    const T* sb = src + (size_t)g * p.xs[1];
    for (int gq = w.col0; gq < ngrp; gq += 32) {
      const int px0 = fr.orgx + 4 * gq;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (rowok) {
        if (vec_ok && px0 >= fr.xlo && px0 + 3 < fr.xhi && (px0 & 3) == 0) {
          const float4 t = *reinterpret_cast<const float4*>(sb + (size_t)py * p.xs[2] + px0);
          v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else if (edge == 1) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            if (px0 + k >= fr.xlo && px0 + k < fr.xhi)
              v[k] = Elem<T>::to_f(sb[(size_t)py * p.xs[2] + (size_t)(px0 + k) * p.xs[3]]);
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int px = px0 + k;
            if (px >= fr.xlo && px < fr.xhi) {
              float acc = 0.f;
              for (int by = 0; by < edge; ++by) {
                const int sy = py * edge + by;
                if (sy >= p.Hsrc) break;
                float racc = 0.f;
                for (int bx = 0; bx < edge; ++bx) {
                  const int sx = px * edge + bx;
                  if (sx >= p.Wsrc) break;
                  racc += Elem<T>::to_f(sb[(size_t)sy * p.xs[2] + (size_t)sx * p.xs[3]]);
                }
                acc += racc;
              }
              v[k] = acc;
            }
          }
        }
      }
      store4(dst + g * plane + rr * pitch + 4 * gq, v[0], v[1], v[2], v[3]);
    }
    g += dg; rr += drr;
    if (rr >= rows) { rr -= rows; ++g; }
  }
}

// ---------------------------------------------------------------------------
// Haar analysis of one level for the whole array extent (wavelet.py:62-67, raw
// LL feeds the next level): one item = four consecutive positions of one
// channel -> four 128-bit stores (LL, LH, HL, HH).  Positions outside the plane,
// or whose 2x2 source block is not held on chip, are written as zeros.
// `src0` is the first source plane (channel 0), `splane` the channel stride;
// (oy, ox) / (soy, sox) are the array origins of this level / the source level.
// ---------------------------------------------------------------------------
template <int K, typename ST>
WT_HD void analysis_level(const Plan2d& p, const Smem2d& sm, int j, int oy, int ox, int soy, int sox,
                          const ST* __restrict__ src0, int splane, int gc, int tid, int nthr) {
  const int rows = p.rows[j], pitch = p.pitch[j];
  const int ngrp = pitch >> 2;
  const int nrows = gc * rows;
  const int sp = p.pitch[j - 1], srows = p.rows[j - 1];
  const int dstep = p.G * p.plane[j];                    // distance between sub-band groups
  const int Hj = p.Hj[j], Wj = p.Wj[j];
  const RowWalk w(ngrp, tid, nthr);
  if (w.row0 >= nrows) return;
  int g = w.row0 / rows, rr = w.row0 - g * rows;
  const int dg = w.step / rows, drr = w.step - dg * rows;
  for (int row = w.row0; row < nrows; row += w.step) {
    const int py = oy + rr;
    const int sy = 2 * py - soy;
    const bool rowok = py >= 0 && py < Hj && sy >= 0 && sy + 1 < srows;
    // rows / columns whose source block is not on chip read a clamped (valid) address and
    // are zeroed by a select, so that the loop has no divergent branch
    const ST* s0 = src0 + g * splane + imin(imax(sy, 0), srows - 2) * sp;
    float* orow = sm.sub(j, g, 0) + rr * pitch;
    for (int gq = w.col0; gq < ngrp; gq += 32) {
      const int px0 = ox + 4 * gq;
      const int sx0 = 2 * px0 - sox;
      float o[4][4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int px = px0 + k, sx = sx0 + 2 * k;
        const bool ok = rowok && px >= 0 && px < Wj && sx >= 0 && sx + 1 < sp;
        const int cx = imin(imax(sx, 0), sp - 2);
        float a0, a1, b0, b1;
        if (K != 0 && (K / 2) % 2 == 0) {          // even radius: source column pairs are aligned
          load2(s0 + (cx & ~1), a0, a1);
          load2(s0 + sp + (cx & ~1), b0, b1);
        } else {
          a0 = Elem<ST>::to_f(s0[cx]); a1 = Elem<ST>::to_f(s0[cx + 1]);
          b0 = Elem<ST>::to_f(s0[sp + cx]); b1 = Elem<ST>::to_f(s0[sp + cx + 1]);
        }
        const float ab = a0 + a1, cd = b0 + b1, amb = a0 - a1, cmd = b0 - b1;
        o[0][k] = ok ? ab + cd : 0.f;
        o[1][k] = ok ? ab - cd : 0.f;
        o[2][k] = ok ? amb + cmd : 0.f;
        o[3][k] = ok ? amb - cmd : 0.f;
      }
      float* od = orow + 4 * gq;
#pragma unroll
      for (int s = 0; s < 4; ++s) store4(od + s * dstep, o[s][0], o[s][1], o[s][2], o[s][3]);
    }
    g += dg; rr += drr;
    if (rr >= rows) { rr -= rows; ++g; }
  }
}

// ---------------------------------------------------------------------------
// Channels-last store of the finished tile: one item = two adjacent pixels x CB
// bytes of consecutive channels, gathered from the planar OUT tile.
// ---------------------------------------------------------------------------
template <typename T, int CB>
WT_HD void store_chunks(const Plan2d& p, T* __restrict__ dst, const T* __restrict__ src, int nr, int nc,
                        int s, int tid, int nthr) {
  constexpr int VEC = Chunk<T, CB>::VEC;
  if (VEC < 1) return;
  constexpr int V = VEC > 0 ? VEC : 1;
  typedef typename RawChunk<CB>::type Raw;
  const int op = p.opitch, oplane = p.oplane;
  const int nch = p.G / V;
  const int nsh = lane_shift(nch);
  const int ncols = ((nc + 1) >> 1) * nch;
  const int ys2 = (int)p.ys[2], ys3 = (int)p.ys[3];
  const RowWalk w(ncols, tid, nthr);
  for (int yy = w.row0; yy < nr; yy += w.step) {
    for (int ci = w.col0; ci < ncols; ci += 32) {
      const int pq = ci >> nsh, ch = ci & (nch - 1);
      const int xx = 2 * pq;
      const bool two = xx + 1 < nc;
      const T* ss = src + (ch * V) * oplane + (yy * s) * op + xx * s;
      Chunk<T, CB> c0, c1;
      if (s == 1 && sizeof(T) == 2) {          // two adjacent 16-bit pixels per 32-bit load
#pragma unroll
        for (int e = 0; e < V; ++e) {
          Chunk<T, 4> t;
          t.raw = *reinterpret_cast<const unsigned int*>(ss + e * oplane);
          c0.set(e, t.get(0)); c1.set(e, t.get(1));
        }
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) c0.set(e, ss[e * oplane]);
        if (two) {
#pragma unroll
          for (int e = 0; e < V; ++e) c1.set(e, ss[e * oplane + s]);
        }
      }
      T* dd = dst + yy * ys2 + xx * ys3 + ch * V;
      *reinterpret_cast<Raw*>(dd) = c0.raw;
      if (two) *reinterpret_cast<Raw*>(dd + ys3) = c1.raw;
    }
  }
}

// Any layout: one item = four consecutive output pixels of one channel.
template <typename T>
WT_HD void store_planar(const Plan2d& p, T* __restrict__ dst, const T* __restrict__ src, int gc, int nr, int nc,
                        int s, int tid, int nthr) {
  const int op = p.opitch, oplane = p.oplane;
  const int ngrp = (nc + 3) >> 2;
  const int nrows = gc * nr;
  const RowWalk w(ngrp, tid, nthr);
  if (w.row0 >= nrows) return;
  int g = w.row0 / nr, yy = w.row0 - g * nr;
  const int dg = w.step / nr, dyy = w.step - dg * nr;
  for (int row = w.row0; row < nrows; row += w.step) {
    for (int gq = w.col0; gq < ngrp; gq += 32) {
      const T* ss = src + g * oplane + (yy * s) * op + (4 * gq) * s;
      T* dd = dst + (size_t)g * p.ys[1] + (size_t)yy * p.ys[2] + (size_t)(4 * gq) * p.ys[3];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (4 * gq + k < nc) dd[(size_t)k * p.ys[3]] = ss[k * s];
    }
    g += dg; yy += dyy;
    if (yy >= nr) { yy -= nr; ++g; }
  }
}

// fp32 plane rows between global memory and shared memory (R_in load, deep-stage output):
// `nrows` flattened (channel, row) pairs of `ncols` floats, 128-bit when `vec_ok`.
template <bool LOAD>
WT_HD void move_plane_rows(float* __restrict__ gmem, int gplane, int gpitch, float* __restrict__ smem_arr,
                           int splane, int spitch, int gc, int nr, int nc, bool vec_ok, int tid, int nthr) {
  const int ngrp = (nc + 3) >> 2;
  const int nrows = gc * nr;
  const RowWalk w(ngrp, tid, nthr);
  if (w.row0 >= nrows) return;
  int g = w.row0 / nr, yy = w.row0 - g * nr;
  const int dg = w.step / nr, dyy = w.step - dg * nr;
  for (int row = w.row0; row < nrows; row += w.step) {
    for (int gq = w.col0; gq < ngrp; gq += 32) {
      float* gp = gmem + (size_t)g * gplane + (size_t)yy * gpitch + 4 * gq;
      float* sp = smem_arr + g * splane + yy * spitch + 4 * gq;
      const bool whole = vec_ok && 4 * gq + 3 < nc;
      if (LOAD) {
        if (whole) async_copy16(sp, gp);
        else {
          float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
          if (4 * gq + 0 < nc) t.x = gp[0];
          if (4 * gq + 1 < nc) t.y = gp[1];
          if (4 * gq + 2 < nc) t.z = gp[2];
          if (4 * gq + 3 < nc) t.w = gp[3];
          *reinterpret_cast<float4*>(sp) = t;
        }
      } else {
        const float4 t = *reinterpret_cast<const float4*>(sp);
        if (whole) *reinterpret_cast<float4*>(gp) = t;
        else {
          if (4 * gq + 0 < nc) gp[0] = t.x;
          if (4 * gq + 1 < nc) gp[1] = t.y;
          if (4 * gq + 2 < nc) gp[2] = t.z;
          if (4 * gq + 3 < nc) gp[3] = t.w;
        }
      }
    }
    g += dg; yy += dyy;
    if (yy >= nr) { yy -= nr; ++g; }
  }
}

// ---------------------------------------------------------------------------
// The CTA body for block (channel group cg, tile bx/by, sample nb).
//   FINAL = true : last stage of a layer: reads x (type T), adds the base
//                  convolution and writes y (type T).  X0 is kept in T when T is
//                  a 16-bit type.
//   FINAL = false: deep stage: reads either x (type T, low-pass block sums formed
//                  while loading) or fp32 planes from scratch (T = float), and
//                  writes fp32 (B,C,h,w)-contiguous planes of its reconstruction.
// `rin` / `rout` are the fp32 planes that connect the stages of one layer.
// ---------------------------------------------------------------------------
template <typename T, int K, bool FINAL>
WT_HD void wt2d_cta(const Plan2d& p, const T* __restrict__ x, T* __restrict__ y,
                    const float* __restrict__ packed, const float* __restrict__ rin,
                    float* __restrict__ rout, float* smem, int cg, int bx, int by, int nb) {
  typedef typename Select<FINAL && sizeof(T) == 2, T, float>::type XT;
  const int nthr = p.nthreads;
  const int d = p.nlev;
  const int c0 = cg * p.G;
  const int gc = imin(p.G, p.C - c0);   // channels actually present in this group
  const int gsh = p.g_shift;            // log2(G) when G is a power of two, else -1

  TileGeo tg;
  tg.d = d; tg.r = p.r; tg.rb = p.rb;
  tg.ty0 = by * p.TY; tg.ty1 = imin(p.H, tg.ty0 + p.TY);
  tg.tx0 = bx * p.TX; tg.tx1 = imin(p.W, tg.tx0 + p.TX);
  tg.Hj = p.Hj; tg.Wj = p.Wj;
  Smem2d sm{smem, &p};
  T* out_tile = reinterpret_cast<T*>(smem + p.ooff);

  // ---- phase 0: stage the tap sets this stage uses, the input tile and the deeper reconstruction
  WT_PHASE(nthr) {
    {
      // per channel: [base set (if any)] [4 sets per level of this stage]
      const int per = p.wsm >> 2;                      // float4 per channel in shared memory
      const int nbase = p.has_base ? (p.tapset >> 2) : 0;
      const int skip = (p.tapset >> 2) * (1 + 4 * p.lvl0) - nbase;
      const RowWalk w(per, tid, nthr);
      for (int g = w.row0; g < gc; g += w.step) {
        const float4* src = reinterpret_cast<const float4*>(packed + (size_t)(c0 + g) * p.wstride);
        float4* dst = reinterpret_cast<float4*>(smem + p.woff + g * p.wsm);
        for (int k = w.col0; k < per; k += 32) async_copy16(dst + k, src + (k < nbase ? k : k + skip));
      }
    }
    // reconstruction of the deeper levels, produced by an earlier launch: asynchronous copies,
    // in flight while the input tile is loaded below
    if (p.has_rin) {
      const LevelGeo dy = tg.y(d), dx = tg.x(d);
      const int Hd = p.Hj[d], Wd = p.Wj[d];
      float* rb = const_cast<float*>(rin) + ((size_t)nb * p.C + c0) * (size_t)(Hd * Wd) + (size_t)dy.a * Wd + dx.a;
      const bool vec_ok = ((Wd & 3) == 0) && ((dx.a & 3) == 0) && (((Hd * Wd) & 3) == 0);
      move_plane_rows<true>(rb, Hd * Wd, Wd, smem + p.roff[d], p.rplane[d], p.rpitch[d], gc, dy.n, dx.n, vec_ok,
                            tid, nthr);
    }
    // input tile -> X0; everything the tile does not take from the plane is zero
    const LevelGeo gy = tg.y(0), gx = tg.x(0);
    FillRange fr;
    fr.ylo = imax(gy.lo, 0); fr.yhi = imin(gy.hi, p.H);
    fr.xlo = imax(gx.lo, 0); fr.xhi = imin(gx.hi, p.W);
    fr.orgy = gy.org; fr.orgx = gx.org;
    const T* xb = x + (size_t)nb * p.xs[0] + (size_t)c0 * p.xs[1];
    XT* x0arr = sm.x0<XT>(0);
    if (p.x_vec && gc == p.G && p.in_shift == 0) {
      if (p.x_vec == 16) fill_x0_chunks<T, XT, 16>(p, xb, x0arr, fr, tid, nthr);
      else if (p.x_vec == 8) fill_x0_chunks<T, XT, 8>(p, xb, x0arr, fr, tid, nthr);
      else fill_x0_chunks<T, XT, 4>(p, xb, x0arr, fr, tid, nthr);
    } else if (!FINAL && p.x_vec && gc == p.G && p.in_shift == 1) {
      float* xf = reinterpret_cast<float*>(x0arr);      // deep stages keep X0 in fp32
      if (p.x_vec == 16) fill_x0_chunks_reduced<T, 16, 2>(p, xb, xf, fr, tid, nthr);
      else if (p.x_vec == 8) fill_x0_chunks_reduced<T, 8, 2>(p, xb, xf, fr, tid, nthr);
      else fill_x0_chunks_reduced<T, 4, 2>(p, xb, xf, fr, tid, nthr);
    } else {
      fill_x0_planar<T, XT>(p, xb, x0arr, fr, gc, tid, nthr);
    }
    async_wait_all();
  }

  // ---- phase 1: Haar analysis, level by level (wavelet.py:62-67; raw LL feeds the next level)
  for (int j = 1; j <= d; ++j) {
    WT_PHASE(nthr) {
      const int oy = tg.y(j).org, ox = tg.x(j).org, soy = tg.y(j - 1).org, sox = tg.x(j - 1).org;
      if (j == 1) analysis_level<K, XT>(p, sm, 1, oy, ox, soy, sox, sm.x0<XT>(0), p.plane[0], gc, tid, nthr);
      else analysis_level<K, float>(p, sm, j, oy, ox, soy, sox, sm.sub(j - 1, 0, 0), p.plane[j - 1], gc, tid, nthr);
    }
  }

  // ---- phase 2: deep levels bottom-up: per-sub-band convolutions into Y, then the
  //      low-pass accumulation and synthesis butterfly into R_{j-1}
  for (int j = d; j >= 2; --j) {
    WT_PHASE(nthr) {
      const LevelGeo ly = tg.y(j), lx = tg.x(j);
      const int th = p.th[j];
      const int nty = cdiv(ly.n, th), ntx = cdiv(lx.n, 4);
      const int wy_base = ly.a - p.r - ly.org, wx_base = lx.a - p.r - lx.org;
      const int per = p.G * 4;                 // channel fastest, then sub-band, then tile
      const int total = per * nty * ntx;
      for (int i = tid; i < total; i += nthr) {
        int t, gs;
        if (gsh >= 0) { t = i >> (gsh + 2); gs = i & (per - 1); }
        else { t = i / per; gs = i - t * per; }
        int s, g;
        if (gsh >= 0) { s = gs >> gsh; g = gs & (p.G - 1); }
        else { s = gs / p.G; g = gs - s * p.G; }
        if (g >= gc) continue;
        const int iy = t / ntx, ix = t - iy * ntx;
        if (th == 4) deep_item<K, 4>(p, sm, j, g, s, iy, ix, wy_base + iy * 4, wx_base + ix * 4);
        else deep_item<K, 2>(p, sm, j, g, s, iy, ix, wy_base + iy * 2, wx_base + ix * 4);
      }
    }
    WT_PHASE(nthr) {
      const LevelGeo ly = tg.y(j), lx = tg.x(j);
      const int hn = ly.n, wn = lx.n;
      const bool has_r = (j < d) || p.has_rin;
      const int ystep = p.G * p.yplane;
      const int nrow = tg.y(j - 1).n, ncol = tg.x(j - 1).n;
      const int opitch = p.rpitch[j - 1];
      const int nrows = gc * hn;
      const RowWalk w(wn, tid, nthr);
      if (w.row0 < nrows) {
        int g = w.row0 / hn, yy = w.row0 - g * hn;
        const int dg = w.step / hn, dyy = w.step - dg * hn;
        for (int row = w.row0; row < nrows; row += w.step) {
          for (int xx = w.col0; xx < wn; xx += 32) {
            const float* yb = sm.ybuf(g, 0) + yy * p.ypitch + xx;
            float ll = yb[0];
            if (has_r) ll += sm.rec(j, g)[yy * p.rpitch[j] + xx];
            float o00, o01, o10, o11;
            synth4(ll, yb[ystep], yb[2 * ystep], yb[3 * ystep], o00, o01, o10, o11);
            float* out = sm.rec(j - 1, g) + (2 * yy) * opitch + 2 * xx;
            const bool c1 = 2 * xx + 1 < ncol;
            out[0] = o00;                                  // (2yy, 2xx) is always inside
            if (c1) out[1] = o01;
            if (2 * yy + 1 < nrow) {
              out[opitch] = o10;
              if (c1) out[opitch + 1] = o11;
            }
          }
          g += dg; yy += dyy;
          if (yy >= hn) { yy -= hn; ++g; }
        }
      }
    }
  }

  T* ytile = nullptr;
  float* rtile = nullptr;
  if (FINAL && p.direct_store)
    ytile = y + (size_t)nb * p.ys[0] + (size_t)c0 * p.ys[1] + (size_t)tg.ty0 * p.ys[2] + (size_t)tg.tx0 * p.ys[3];
  if (!FINAL && p.direct_store)
    rtile = rout + ((size_t)nb * p.C + c0) * (size_t)(p.H * p.W) + (size_t)tg.ty0 * p.W + tg.tx0;
  // ---- phase 3: top level of the stage (+ base convolution and bias); lanes run over the
  //      channels of the group first, so a quarter warp touches eight different planes
  WT_PHASE(nthr) {
    const LevelGeo y0 = tg.y(0), x0g = tg.x(0);
    if (d >= 1) {
      const LevelGeo y1 = tg.y(1), x1 = tg.x(1);
      const int nty = cdiv(y1.n, 2), ntx = cdiv(x1.n, 4);
      const int total = p.G * nty * ntx;
      const bool has_r = (d > 1) || p.has_rin;
      const int wy1 = y1.a - p.r - y1.org, wx1 = x1.a - p.r - x1.org;
      const int wy0 = y0.a - p.r - y0.org, wx0 = x0g.a - p.r - x0g.org;
      for (int i = tid; i < total; i += nthr) {
        int t, g;
        if (gsh >= 0) { t = i >> gsh; g = i & (p.G - 1); }
        else { t = i / p.G; g = i - t * p.G; }
        if (g >= gc) continue;
        const int iy = t / ntx, ix = t - iy * ntx;
        top_item<T, XT, K, FINAL>(p, sm, g, iy, ix, wy1 + iy * 2, wx1 + ix * 4, wy0 + iy * 4, wx0 + ix * 8,
                                  y0.n, x0g.n, has_r, out_tile, ytile, rtile);
      }
    } else if (FINAL) {
      const int nty = cdiv(y0.n, 4), ntx = cdiv(x0g.n, 8);
      const int total = p.G * nty * ntx;
      const int wy0 = y0.a - p.r - y0.org, wx0 = x0g.a - p.r - x0g.org;
      for (int i = tid; i < total; i += nthr) {
        int t, g;
        if (gsh >= 0) { t = i >> gsh; g = i & (p.G - 1); }
        else { t = i / p.G; g = i - t * p.G; }
        if (g >= gc) continue;
        const int iy = t / ntx, ix = t - iy * ntx;
        base_item<T, XT, K>(p, sm, g, iy, ix, wy0 + iy * 4, wx0 + ix * 8, out_tile);
      }
    }
  }

  // ---- phase 4: write the tile (unless the items of phase 3 stored their pixels themselves)
  if (p.direct_store && d >= 1) return;
  WT_PHASE(nthr) {
    const int hn = tg.ty1 - tg.ty0, wn = tg.tx1 - tg.tx0;
    if (!FINAL) {
      float* ob = rout + ((size_t)nb * p.C + c0) * (size_t)(p.H * p.W) + (size_t)tg.ty0 * p.W + tg.tx0;
      const bool vec_ok = ((p.W & 3) == 0) && ((tg.tx0 & 3) == 0) && (((p.H * p.W) & 3) == 0);
      move_plane_rows<false>(ob, p.H * p.W, p.W, smem + p.roff[0], p.rplane[0], p.rpitch[0], gc, hn, wn, vec_ok,
                             tid, nthr);
    } else {
      const int s = p.out_stride;
      const int oy0 = cdiv(tg.ty0, s), oy1 = cdiv(tg.ty1, s);
      const int ox0 = cdiv(tg.tx0, s), ox1 = cdiv(tg.tx1, s);
      const int nr = oy1 - oy0, nc = ox1 - ox0;
      T* yb = y + (size_t)nb * p.ys[0] + (size_t)c0 * p.ys[1] + (size_t)oy0 * p.ys[2] + (size_t)ox0 * p.ys[3];
      const T* o0 = out_tile + (oy0 * s - tg.ty0) * p.opitch + (ox0 * s - tg.tx0);
      if (p.y_vec && gc == p.G) {
        if (p.y_vec == 16) store_chunks<T, 16>(p, yb, o0, nr, nc, s, tid, nthr);
        else if (p.y_vec == 8) store_chunks<T, 8>(p, yb, o0, nr, nc, s, tid, nthr);
        else store_chunks<T, 4>(p, yb, o0, nr, nc, s, tid, nthr);
      } else {
        store_planar<T>(p, yb, o0, gc, nr, nc, s, tid, nthr);
      }
    }
  }
}

}  // namespace wt
