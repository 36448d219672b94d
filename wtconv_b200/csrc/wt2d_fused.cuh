// Fused multi-level WTConv2d forward for one CTA (sm_100a).
//
// Replaces, for the tile a CTA owns, the whole body of the reference forward
// (wtconv/wtconv2d.py:38-87): zero padding of odd sizes, Haar analysis of every
// level, the 4C-channel depthwise KxK convolution and scale of every level, the
// bottom-up inverse transform with the low-pass accumulation, the base
// depthwise convolution with its scale and bias, the final add and the stride.
//
// Shared-memory data layout (planar per channel g):
//   X0[g]            fp32  input tile with zero border (level 0)
//   S_j[g][s]        fp32  un-normalised Haar sub-bands of level j, s = LL,LH,HL,HH
//   Y[g][s]          fp32  scaled sub-band convolutions of one deep level (scratch)
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
//     four sub-bands meet again in shared memory for the synthesis butterfly.
#pragma once

#include "wt2d_plan.h"

namespace wt {

// ---------------------------------------------------------------------------
// Register-tiled depthwise KxK cross-correlation of a TH x TW tile.
// `src` points at the top-left element of the (TH+K-1) x (TW+K-1) window, 16-byte
// aligned; rows are `pitch` floats apart (pitch % 4 == 0).  The window is read
// with 128-bit shared-memory loads, one input row at a time, and every row is
// applied to all output rows it contributes to, so each loaded float feeds
// about K*min(K,TH)*TW/(TW+K-1) FMAs.
// ---------------------------------------------------------------------------
template <int K, int TH, int TW>
WT_HD void conv_tile(const float* __restrict__ src, int pitch, const float* __restrict__ wts,
                     float (&acc)[TH][TW]) {
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
    const float4* p4 = reinterpret_cast<const float4*>(src + rr * pitch);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const float4 t = p4[v];
      row[4 * v + 0] = t.x; row[4 * v + 1] = t.y; row[4 * v + 2] = t.z; row[4 * v + 3] = t.w;
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

struct Smem2d {
  float* base;
  const Plan2d* p;
  // sub-band array s of channel g at level j (j = 0 has a single array, s = 0)
  WT_HD float* arr(int j, int g, int s) const {
    const int ns = (j == 0) ? 1 : 4;
    return base + p->off[j] + (g * ns + s) * (p->rows[j] * p->pitch[j]);
  }
  WT_HD float* rec(int j, int g) const { return base + p->roff[j] + g * (p->rrows[j] * p->rpitch[j]); }
  WT_HD float* ybuf(int g, int s) const { return base + p->yoff + (g * 4 + s) * (p->yrows * p->ypitch); }
  WT_HD float* weights(int g) const { return base + p->woff + g * p->wsm; }
  // tap set of level j (1-based within the stage), sub-band s; j = 0: base set
  WT_HD const float* taps(int g, int j, int s) const {
    return weights(g) + p->tapset * (j == 0 ? 0 : p->has_base + 4 * (j - 1) + s);
  }
};

// Synthesis butterfly of one position (wavelet.py:70-75, taps folded on the host)
WT_HD void synth4(float ll, float lh, float hl, float hh, float& o00, float& o01, float& o10, float& o11) {
  const float pp = ll + lh, qq = ll - lh, uu = hl + hh, vv = hl - hh;
  o00 = pp + uu; o01 = pp - uu; o10 = qq + vv; o11 = qq - vv;
}

// ---------------------------------------------------------------------------
// Top-level item: TH x TW positions of level 1 of this stage for one channel.
// Four scaled sub-band convolutions, low-pass accumulation of the deeper
// reconstruction (wtconv2d.py:71) and the synthesis butterfly give the
// 2TH x 2TW block of R_0 in registers.  With FUSE_BASE the base convolution and
// bias (wtconv2d.py:81-82) are accumulated on top and the finished block goes to
// the OUT staging tile; otherwise the block is written to R_0 (cropped).
// ---------------------------------------------------------------------------
template <typename T, int K, int TH, int TW, bool FUSE_BASE>
WT_HD void top_item(const Plan2d& p, const Smem2d& sm, const Axis& ay, const Axis& ax, int g, int iy, int ix,
                    bool has_r, T* __restrict__ out_tile) {
  const int r = p.r;
  float acc[2 * TH][2 * TW];
  {
    const int pitch = p.pitch[1];
    const int wy = ay.a[1] + iy * TH - r - ay.org[1];   // window origin in array coordinates
    const int wx = ax.a[1] + ix * TW - r - ax.org[1];
    float y[4][TH][TW];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
#pragma unroll
      for (int i = 0; i < TH; ++i)
#pragma unroll
        for (int q = 0; q < TW; ++q) y[s][i][q] = 0.f;
      conv_tile<K, TH, TW>(sm.arr(1, g, s) + wy * pitch + wx, pitch, sm.taps(g, 1, s), y[s]);
    }
    if (has_r) {
      const float* rj = sm.rec(1, g) + (iy * TH) * p.rpitch[1] + ix * TW;
#pragma unroll
      for (int i = 0; i < TH; ++i) {
        const float4 t = *reinterpret_cast<const float4*>(rj + i * p.rpitch[1]);
        static_assert(TW == 4, "top items are four positions wide");
        y[0][i][0] += t.x; y[0][i][1] += t.y; y[0][i][2] += t.z; y[0][i][3] += t.w;
      }
    }
#pragma unroll
    for (int i = 0; i < TH; ++i)
#pragma unroll
      for (int q = 0; q < TW; ++q)
        synth4(y[0][i][q], y[1][i][q], y[2][i][q], y[3][i][q], acc[2 * i][2 * q], acc[2 * i][2 * q + 1],
               acc[2 * i + 1][2 * q], acc[2 * i + 1][2 * q + 1]);
  }
  if (FUSE_BASE) {
    const int pitch = p.pitch[0];
    const int wy = ay.t0 + iy * 2 * TH - r - ay.org[0];
    const int wx = ax.t0 + ix * 2 * TW - r - ax.org[0];
    const float* wts = sm.taps(g, 0, 0);
    const float bias = wts[K * K];
#pragma unroll
    for (int i = 0; i < 2 * TH; ++i)
#pragma unroll
      for (int q = 0; q < 2 * TW; ++q) acc[i][q] += bias;
    conv_tile<K, 2 * TH, 2 * TW>(sm.arr(0, g, 0) + wy * pitch + wx, pitch, wts, acc);
    // finished pixels -> OUT[g] (type T); the tile is allocated with the overhang of
    // partial items, so no predicate is needed
    T* o = out_tile + (size_t)g * (p.orows * p.opitch) + (iy * 2 * TH) * p.opitch + ix * 2 * TW;
#pragma unroll
    for (int i = 0; i < 2 * TH; ++i)
#pragma unroll
      for (int q = 0; q < 2 * TW; ++q) o[i * p.opitch + q] = Elem<T>::from_f(acc[i][q]);
  } else {
    float* out = sm.rec(0, g);
    const int opitch = p.rpitch[0];
    const int nrow = ay.n[0], ncol = ax.n[0];
#pragma unroll
    for (int i = 0; i < 2 * TH; ++i) {
      const int oy = iy * 2 * TH + i;
#pragma unroll
      for (int q = 0; q < 2 * TW; ++q) {
        const int ox = ix * 2 * TW + q;
        if (oy < nrow && ox < ncol) out[oy * opitch + ox] = acc[i][q];
      }
    }
  }
}

// Base-only layer (wt_levels == 0 in this stage): OUT = bias + base conv.
template <typename T, int K, int BH, int BW>
WT_HD void base_item(const Plan2d& p, const Smem2d& sm, const Axis& ay, const Axis& ax, int g, int iy, int ix,
                     T* __restrict__ out_tile) {
  const int r = p.r;
  const int pitch = p.pitch[0];
  const int wy = ay.t0 + iy * BH - r - ay.org[0];
  const int wx = ax.t0 + ix * BW - r - ax.org[0];
  const float* wts = sm.taps(g, 0, 0);
  const float bias = wts[K * K];
  float acc[BH][BW];
#pragma unroll
  for (int i = 0; i < BH; ++i)
#pragma unroll
    for (int q = 0; q < BW; ++q) acc[i][q] = bias;
  conv_tile<K, BH, BW>(sm.arr(0, g, 0) + wy * pitch + wx, pitch, wts, acc);
  T* o = out_tile + (size_t)g * (p.orows * p.opitch) + (iy * BH) * p.opitch + ix * BW;
#pragma unroll
  for (int i = 0; i < BH; ++i)
#pragma unroll
    for (int q = 0; q < BW; ++q) o[i * p.opitch + q] = Elem<T>::from_f(acc[i][q]);
}

// Deep-level item: one sub-band s of a TH x 4 tile of level j -> Y[g][s]
template <int K, int TH>
WT_HD void deep_item(const Plan2d& p, const Smem2d& sm, const Axis& ay, const Axis& ax, int j, int g, int s,
                     int iy, int ix) {
  const int r = p.r;
  const int pitch = p.pitch[j];
  const int wy = ay.a[j] + iy * TH - r - ay.org[j];
  const int wx = ax.a[j] + ix * 4 - r - ax.org[j];
  float y[TH][4];
#pragma unroll
  for (int i = 0; i < TH; ++i)
#pragma unroll
    for (int q = 0; q < 4; ++q) y[i][q] = 0.f;
  conv_tile<K, TH, 4>(sm.arr(j, g, s) + wy * pitch + wx, pitch, sm.taps(g, j, s), y);
  float* o = sm.ybuf(g, s) + (iy * TH) * p.ypitch + ix * 4;
#pragma unroll
  for (int i = 0; i < TH; ++i)
    *reinterpret_cast<float4*>(o + i * p.ypitch) = make_float4(y[i][0], y[i][1], y[i][2], y[i][3]);
}

// ---------------------------------------------------------------------------
// Channels-last staging: every thread moves CB-byte chunks (CB/sizeof(T)
// consecutive channels of one pixel) between global memory and planar arrays.
// Pixels are walked with an incremental (row, col) counter: no division in the loop.
// ---------------------------------------------------------------------------
template <typename T, int CB>
WT_HD void load_chunks(const Plan2d& p, const T* __restrict__ src, float* __restrict__ dst, int nr, int nc,
                       int pitch, int plane, int tid, int nthr) {
  constexpr int VEC = Chunk<T, CB>::VEC;
  if (VEC < 1) return;
  const int nch = p.G / (VEC > 0 ? VEC : 1);
  const int total = nr * nc * nch;
  if (tid >= total) return;
  // item i = pix * nch + ch
  int ch = tid % nch, pix = tid / nch;
  int yy = pix / nc, xx = pix - yy * nc;
  const int dch = nthr % nch, dpix = nthr / nch;
  const int dy = dpix / nc, dx = dpix - dy * nc;
  for (int i = tid; i < total; i += nthr) {
    Chunk<T, CB> c;
    c.raw = *reinterpret_cast<const typename RawChunk<CB>::type*>(src + (size_t)yy * p.xs[2] + (size_t)xx * p.xs[3] + ch * VEC);
    float* dd = dst + (ch * VEC) * plane + yy * pitch + xx;
#pragma unroll
    for (int e = 0; e < VEC; ++e) dd[e * plane] = Elem<T>::to_f(c.get(e));
    ch += dch; xx += dx; yy += dy;
    if (ch >= nch) { ch -= nch; ++xx; }
    if (xx >= nc) { xx -= nc; ++yy; }
    if (xx >= nc) { xx -= nc; ++yy; }
  }
}

// Same walk, but every destination cell is the sum of an edge x edge block of source pixels
// (the low-pass input of a deep stage formed directly from the layer input).
template <typename T, int CB>
WT_HD void load_chunks_reduced(const Plan2d& p, const T* __restrict__ src, float* __restrict__ dst, int y0, int x0,
                               int nr, int nc, int pitch, int plane, int edge, int tid, int nthr) {
  constexpr int VEC = Chunk<T, CB>::VEC;
  if (VEC < 1) return;
  const int nch = p.G / (VEC > 0 ? VEC : 1);
  const int total = nr * nc * nch;
  if (tid >= total) return;
  int ch = tid % nch, pix = tid / nch;
  int yy = pix / nc, xx = pix - yy * nc;
  const int dch = nthr % nch, dpix = nthr / nch;
  const int dy = dpix / nc, dx = dpix - dy * nc;
  for (int i = tid; i < total; i += nthr) {
    float acc[VEC > 0 ? VEC : 1];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
    for (int by = 0; by < edge; ++by) {
      const int sy = (y0 + yy) * edge + by;
      if (sy >= p.Hsrc) break;
      float racc[VEC > 0 ? VEC : 1];
#pragma unroll
      for (int e = 0; e < VEC; ++e) racc[e] = 0.f;
      for (int bx = 0; bx < edge; ++bx) {
        const int sx = (x0 + xx) * edge + bx;
        if (sx >= p.Wsrc) break;
        Chunk<T, CB> c;
        c.raw = *reinterpret_cast<const typename RawChunk<CB>::type*>(src + (size_t)sy * p.xs[2] + (size_t)sx * p.xs[3] + ch * VEC);
#pragma unroll
        for (int e = 0; e < VEC; ++e) racc[e] += Elem<T>::to_f(c.get(e));
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] += racc[e];
    }
    float* dd = dst + (ch * VEC) * plane + yy * pitch + xx;
#pragma unroll
    for (int e = 0; e < VEC; ++e) dd[e * plane] = acc[e];
    ch += dch; xx += dx; yy += dy;
    if (ch >= nch) { ch -= nch; ++xx; }
    if (xx >= nc) { xx -= nc; ++yy; }
    if (xx >= nc) { xx -= nc; ++yy; }
  }
}

template <typename T, int CB>
WT_HD void store_chunks(const Plan2d& p, T* __restrict__ dst, const T* __restrict__ src, int nr, int nc,
                        int op, int oplane, int s, int tid, int nthr) {
  constexpr int VEC = Chunk<T, CB>::VEC;
  if (VEC < 1) return;
  const int nch = p.G / (VEC > 0 ? VEC : 1);
  const int total = nr * nc * nch;
  if (tid >= total) return;
  int ch = tid % nch, pix = tid / nch;
  int yy = pix / nc, xx = pix - yy * nc;
  const int dch = nthr % nch, dpix = nthr / nch;
  const int dy = dpix / nc, dx = dpix - dy * nc;
  for (int i = tid; i < total; i += nthr) {
    const T* ss = src + (ch * VEC) * oplane + (yy * s) * op + xx * s;
    Chunk<T, CB> c;
#pragma unroll
    for (int e = 0; e < VEC; ++e) c.set(e, ss[e * oplane]);
    *reinterpret_cast<typename RawChunk<CB>::type*>(dst + (size_t)yy * p.ys[2] + (size_t)xx * p.ys[3] + ch * VEC) = c.raw;
    ch += dch; xx += dx; yy += dy;
    if (ch >= nch) { ch -= nch; ++xx; }
    if (xx >= nc) { xx -= nc; ++yy; }
    if (xx >= nc) { xx -= nc; ++yy; }
  }
}

// Clears the cells of one level's arrays that lie outside the plane (the zero
// extension of wtconv2d.py:49-51 and the 'same' padding of the convolutions).
// One (array, row) pair per step; interior tiles have nothing to clear.
WT_HD void clear_border(float* __restrict__ arrs, int narr, int rows, int pitch, int orgy, int orgx, int H, int W,
                        int tid, int nthr) {
  const bool rows_inside = orgy >= 0 && orgy + rows <= H;
  const bool cols_inside = orgx >= 0 && orgx + pitch <= W;
  if (rows_inside && cols_inside) return;
  const int total = narr * rows;
  const int left = imin(imax(-orgx, 0), pitch);           // columns [0,left) are outside
  const int right = imax(imin(W - orgx, pitch), 0);       // columns [right,pitch) are outside
  for (int i = tid; i < total; i += nthr) {
    const int rr = i % rows;
    float* row = arrs + (size_t)i * pitch;
    const int py = orgy + rr;
    if (py < 0 || py >= H) {
      float4* r4 = reinterpret_cast<float4*>(row);
      for (int v = 0; v < pitch / 4; ++v) r4[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
      for (int c = 0; c < left; ++c) row[c] = 0.f;
      for (int c = right; c < pitch; ++c) row[c] = 0.f;
    }
  }
}

// ---------------------------------------------------------------------------
// The CTA body.  `bid` is the linear block index; x / y are the launch's input
// and output, `rin` / `rout` fp32 (B,C,h,w)-contiguous planes used by the
// multi-launch path for planes that do not fit on chip.
// ---------------------------------------------------------------------------
template <typename T, int K>
WT_HD void wt2d_cta(const Plan2d& p, const T* __restrict__ x, T* __restrict__ y,
                    const float* __restrict__ packed, const float* __restrict__ rin,
                    float* __restrict__ rout, float* smem, int bid) {
  const int nthr = p.nthreads;
  const int d = p.nlev;
  // block -> (channel group, tile x, tile y, sample); the group index runs fastest so
  // that CTAs sharing the 32-byte sectors of a channels-last pixel are scheduled together
  const int cg = bid % p.ngroups;
  int rest = bid / p.ngroups;
  const int bx = rest % p.ntile_x;
  rest /= p.ntile_x;
  const int by = rest % p.ntile_y;
  const int nb = rest / p.ntile_y;
  const int c0 = cg * p.G;
  const int gc = imin(p.G, p.C - c0);   // channels actually present in this group

  Axis ay, ax;
  axis_geometry(d, p.r, p.rb, p.has_base, p.Hj, by * p.TY, imin(p.H, (by + 1) * p.TY), 1, ay);
  axis_geometry(d, p.r, p.rb, p.has_base, p.Wj, bx * p.TX, imin(p.W, (bx + 1) * p.TX), 4, ax);
  Smem2d sm{smem, &p};
  T* out_tile = reinterpret_cast<T*>(smem + p.ooff);

  // ---- phase 0: zero borders, stage the tap sets this stage uses, load the input tile
  WT_PHASE(nthr) {
    for (int j = 0; j <= d; ++j)
      clear_border(smem + p.off[j], gc * (j == 0 ? 1 : 4), p.rows[j], p.pitch[j], ay.org[j], ax.org[j], p.Hj[j],
                   p.Wj[j], tid, nthr);
    {
      // per channel: [base set (if any)] [4 sets per level of this stage]
      const int per = p.wsm / 4;                       // float4 per channel in shared memory
      const int nbase = p.has_base ? p.tapset / 4 : 0;
      const int total = gc * per;
      for (int i = tid; i < total; i += nthr) {
        const int g = i / per, k = i - g * per;
        const float4* src = reinterpret_cast<const float4*>(packed + (size_t)(c0 + g) * p.wstride);
        const int sk = (k < nbase) ? k : (p.tapset / 4) * (1 + 4 * p.lvl0) + (k - nbase);
        reinterpret_cast<float4*>(smem + p.woff)[i] = src[sk];
      }
    }
    // input tile -> X0 (fp32); cells outside the plane stay zero (wtconv2d.py:49-51)
    const int y0 = imax(ay.lo[0], 0), y1 = imin(ay.hi[0], p.H);
    const int x0 = imax(ax.lo[0], 0), x1 = imin(ax.hi[0], p.W);
    const int nr = y1 - y0, nc = x1 - x0;
    const int pitch = p.pitch[0];
    const int plane = p.rows[0] * pitch;
    float* dst0 = smem + p.off[0] + (y0 - ay.org[0]) * pitch + (x0 - ax.org[0]);
    const T* xb = x + (size_t)nb * p.xs[0] + (size_t)c0 * p.xs[1];
    if (p.in_shift > 0) {
      // low-pass input formed on the fly: un-normalised sum of the 2^q x 2^q source block,
      // zero outside the source plane (wtconv2d.py:49-54 applied q times, taps folded)
      const int q = p.in_shift, edge = 1 << q;
      if (p.x_vec && gc == p.G) {
        const T* xo = xb;
        if (p.x_vec == 16) load_chunks_reduced<T, 16>(p, xo, dst0, y0, x0, nr, nc, pitch, plane, edge, tid, nthr);
        else if (p.x_vec == 8) load_chunks_reduced<T, 8>(p, xo, dst0, y0, x0, nr, nc, pitch, plane, edge, tid, nthr);
        else load_chunks_reduced<T, 4>(p, xo, dst0, y0, x0, nr, nc, pitch, plane, edge, tid, nthr);
      } else {
        const int total = nr * nc * gc;
        const bool cl = p.x_cl != 0;
        for (int i = tid; i < total; i += nthr) {
          int g, yy, xx;
          if (cl) { g = i % gc; const int pix = i / gc; yy = pix / nc; xx = pix - yy * nc; }
          else { xx = i % nc; const int t = i / nc; yy = t % nr; g = t / nr; }
          const T* sb = xb + (size_t)g * p.xs[1];
          float acc = 0.f;
          for (int dy = 0; dy < edge; ++dy) {
            const int sy = (y0 + yy) * edge + dy;
            if (sy >= p.Hsrc) break;
            float racc = 0.f;
            for (int dx = 0; dx < edge; ++dx) {
              const int sx = (x0 + xx) * edge + dx;
              if (sx >= p.Wsrc) break;
              racc += Elem<T>::to_f(sb[(size_t)sy * p.xs[2] + (size_t)sx * p.xs[3]]);
            }
            acc += racc;
          }
          dst0[g * plane + yy * pitch + xx] = acc;
        }
      }
    } else if (p.x_vec && gc == p.G) {
      const T* xo = xb + (size_t)y0 * p.xs[2] + (size_t)x0 * p.xs[3];
      if (p.x_vec == 16) load_chunks<T, 16>(p, xo, dst0, nr, nc, pitch, plane, tid, nthr);
      else if (p.x_vec == 8) load_chunks<T, 8>(p, xo, dst0, nr, nc, pitch, plane, tid, nthr);
      else load_chunks<T, 4>(p, xo, dst0, nr, nc, pitch, plane, tid, nthr);
    } else if (p.x_cl) {
      const int total = nr * nc * gc;
      for (int i = tid; i < total; i += nthr) {
        const int g = i % gc;
        const int pix = i / gc;
        const int yy = pix / nc, xx = pix - yy * nc;
        dst0[g * plane + yy * pitch + xx] =
            Elem<T>::to_f(xb[(size_t)g * p.xs[1] + (size_t)(y0 + yy) * p.xs[2] + (size_t)(x0 + xx) * p.xs[3]]);
      }
    } else {
      const int total = nr * nc * gc;
      for (int i = tid; i < total; i += nthr) {
        const int xx = i % nc;
        const int t = i / nc;
        const int yy = t % nr, g = t / nr;
        dst0[g * plane + yy * pitch + xx] =
            Elem<T>::to_f(xb[(size_t)g * p.xs[1] + (size_t)(y0 + yy) * p.xs[2] + (size_t)(x0 + xx) * p.xs[3]]);
      }
    }
    // reconstruction of the deeper levels, produced by an earlier launch
    if (p.has_rin) {
      const int hn = ay.n[d], wn = ax.n[d];
      const int total = gc * hn * wn;
      const float* rb = rin + ((size_t)nb * p.C + c0) * (size_t)(p.Hj[d] * p.Wj[d]);
      for (int i = tid; i < total; i += nthr) {
        const int xx = i % wn;
        const int t = i / wn;
        const int yy = t % hn, g = t / hn;
        sm.rec(d, g)[yy * p.rpitch[d] + xx] =
            rb[(size_t)g * (p.Hj[d] * p.Wj[d]) + (size_t)(ay.a[d] + yy) * p.Wj[d] + (ax.a[d] + xx)];
      }
    }
  }

  // ---- phase 1: Haar analysis, level by level (wavelet.py:62-67; raw LL feeds the next level)
  for (int j = 1; j <= d; ++j) {
    WT_PHASE(nthr) {
      const int y0 = imax(ay.lo[j], 0), y1 = imin(ay.hi[j], p.Hj[j]);
      const int x0 = imax(ax.lo[j], 0), x1 = imin(ax.hi[j], p.Wj[j]);
      const int nr = y1 - y0, nc = x1 - x0;
      const int total = gc * nr * nc;
      const int sp = p.pitch[j - 1], dp = p.pitch[j];
      const int dplane = p.rows[j] * dp;
      if (tid < total) {
        int xx = tid % nc, t = tid / nc;
        int yy = t % nr, g = t / nr;
        const int dx = nthr % nc, dt = nthr / nc;
        const int dy = dt % nr, dg = dt / nr;
        for (int i = tid; i < total; i += nthr) {
          const float* s = sm.arr(j - 1, g, 0) + (2 * (y0 + yy) - ay.org[j - 1]) * sp + (2 * (x0 + xx) - ax.org[j - 1]);
          const float a = s[0], b = s[1], c = s[sp], e = s[sp + 1];
          float* o = sm.arr(j, g, 0) + (y0 + yy - ay.org[j]) * dp + (x0 + xx - ax.org[j]);
          const float ab = a + b, cd = c + e, amb = a - b, cmd = c - e;
          o[0] = ab + cd;            // LL
          o[dplane] = ab - cd;       // LH
          o[2 * dplane] = amb + cmd; // HL
          o[3 * dplane] = amb - cmd; // HH
          xx += dx; yy += dy; g += dg;
          if (xx >= nc) { xx -= nc; ++yy; }
          if (yy >= nr) { yy -= nr; ++g; }
          if (yy >= nr) { yy -= nr; ++g; }
        }
      }
    }
  }

  // ---- phase 2: deep levels bottom-up: per-sub-band convolutions into Y, then the
  //      low-pass accumulation and synthesis butterfly into R_{j-1}
  for (int j = d; j >= 2; --j) {
    WT_PHASE(nthr) {
      const int th = p.th[j];
      const int nty = cdiv(ay.n[j], th), ntx = cdiv(ax.n[j], 4);
      const int per = nty * ntx;
      const int total = gc * 4 * per;
      for (int i = tid; i < total; i += nthr) {
        const int t = i % per;
        const int gs = i / per;
        const int s = gs & 3, g = gs >> 2;
        const int iy = t / ntx, ix = t - iy * ntx;
        if (th == 4) deep_item<K, 4>(p, sm, ay, ax, j, g, s, iy, ix);
        else deep_item<K, 2>(p, sm, ay, ax, j, g, s, iy, ix);
      }
    }
    WT_PHASE(nthr) {
      const int hn = ay.n[j], wn = ax.n[j];
      const int total = gc * hn * wn;
      const bool has_r = (j < d) || p.has_rin;
      const int yplane = p.yrows * p.ypitch;
      const int nrow = ay.n[j - 1], ncol = ax.n[j - 1];
      const int opitch = p.rpitch[j - 1];
      for (int i = tid; i < total; i += nthr) {
        const int xx = i % wn;
        const int t = i / wn;
        const int yy = t % hn, g = t / hn;
        const float* yb = sm.ybuf(g, 0) + yy * p.ypitch + xx;
        float ll = yb[0];
        if (has_r) ll += sm.rec(j, g)[yy * p.rpitch[j] + xx];
        float o00, o01, o10, o11;
        synth4(ll, yb[yplane], yb[2 * yplane], yb[3 * yplane], o00, o01, o10, o11);
        float* out = sm.rec(j - 1, g) + (2 * yy) * opitch + 2 * xx;
        const bool c1 = 2 * xx + 1 < ncol;
        out[0] = o00;                                  // (2yy, 2xx) is always inside
        if (c1) out[1] = o01;
        if (2 * yy + 1 < nrow) {
          out[opitch] = o10;
          if (c1) out[opitch + 1] = o11;
        }
      }
    }
  }

  // ---- phase 3: top level of the stage (+ base convolution and bias)
  WT_PHASE(nthr) {
    if (d >= 1) {
      const int nty = cdiv(ay.n[1], 2), ntx = cdiv(ax.n[1], 4);
      const int per = nty * ntx;
      const int total = gc * per;
      const bool has_r = (d > 1) || p.has_rin;
      for (int i = tid; i < total; i += nthr) {
        const int g = i / per;
        const int t = i - g * per;
        const int iy = t / ntx, ix = t - iy * ntx;
        if (p.has_base) top_item<T, K, 2, 4, true>(p, sm, ay, ax, g, iy, ix, has_r, out_tile);
        else top_item<T, K, 2, 4, false>(p, sm, ay, ax, g, iy, ix, has_r, out_tile);
      }
    } else {
      const int nty = cdiv(ay.n[0], 4), ntx = cdiv(ax.n[0], 8);
      const int per = nty * ntx;
      const int total = gc * per;
      for (int i = tid; i < total; i += nthr) {
        const int g = i / per;
        const int t = i - g * per;
        const int iy = t / ntx, ix = t - iy * ntx;
        base_item<T, K, 4, 8>(p, sm, ay, ax, g, iy, ix, out_tile);
      }
    }
  }

  // ---- phase 4: write the tile
  WT_PHASE(nthr) {
    if (p.out_planes) {
      const int rp = p.rpitch[0];
      const int rplane = p.rrows[0] * rp;
      const float* r0 = smem + p.roff[0];
      const int hn = ay.n[0], wn = ax.n[0];
      const int total = gc * hn * wn;
      float* ob = rout + ((size_t)nb * p.C + c0) * (size_t)(p.H * p.W);
      for (int i = tid; i < total; i += nthr) {
        const int xx = i % wn;
        const int t = i / wn;
        const int yy = t % hn, g = t / hn;
        ob[(size_t)g * (p.H * p.W) + (size_t)(ay.t0 + yy) * p.W + (ax.t0 + xx)] = r0[g * rplane + yy * rp + xx];
      }
    } else {
      const int op = p.opitch;
      const int oplane = p.orows * op;
      const int s = p.out_stride;
      const int oy0 = cdiv(ay.t0, s), oy1 = cdiv(ay.t1, s);
      const int ox0 = cdiv(ax.t0, s), ox1 = cdiv(ax.t1, s);
      const int nr = oy1 - oy0, nc = ox1 - ox0;
      T* yb = y + (size_t)nb * p.ys[0] + (size_t)c0 * p.ys[1];
      const T* o0 = out_tile + (oy0 * s - ay.t0) * op + (ox0 * s - ax.t0);
      if (p.y_vec && gc == p.G) {
        T* yo = yb + (size_t)oy0 * p.ys[2] + (size_t)ox0 * p.ys[3];
        if (p.y_vec == 16) store_chunks<T, 16>(p, yo, o0, nr, nc, op, oplane, s, tid, nthr);
        else if (p.y_vec == 8) store_chunks<T, 8>(p, yo, o0, nr, nc, op, oplane, s, tid, nthr);
        else store_chunks<T, 4>(p, yo, o0, nr, nc, op, oplane, s, tid, nthr);
      } else if (p.y_cl) {
        const int total = nr * nc * gc;
        for (int i = tid; i < total; i += nthr) {
          const int g = i % gc;
          const int pix = i / gc;
          const int yy = pix / nc, xx = pix - yy * nc;
          yb[(size_t)g * p.ys[1] + (size_t)(oy0 + yy) * p.ys[2] + (size_t)(ox0 + xx) * p.ys[3]] =
              o0[g * oplane + (yy * s) * op + xx * s];
        }
      } else {
        const int total = nr * nc * gc;
        for (int i = tid; i < total; i += nthr) {
          const int xx = i % nc;
          const int t = i / nc;
          const int yy = t % nr, g = t / nr;
          yb[(size_t)g * p.ys[1] + (size_t)(oy0 + yy) * p.ys[2] + (size_t)(ox0 + xx) * p.ys[3]] =
              o0[g * oplane + (yy * s) * op + xx * s];
        }
      }
    }
  }
}

}  // namespace wt
