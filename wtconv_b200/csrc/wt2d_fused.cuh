// Fused multi-level WTConv2d forward for one CTA (sm_100a).
//
// Replaces, for the tile a CTA owns, the whole body of the reference forward
// (wtconv/wtconv2d.py:38-87): zero padding of odd sizes, Haar analysis of every
// level, the 4C-channel depthwise KxK convolution and scale of every level, the
// bottom-up inverse transform with the low-pass accumulation, the base
// depthwise convolution with its scale and bias, the final add and the stride.
//
// Shared-memory data layout (all fp32, planar per channel):
//   level 0            X0[g]            input tile with zero border
//   level j = 1..d     S_j[g][s]        un-normalised Haar sub-bands s = LL,LH,HL,HH
//   R_j,  j = 0..d     R_j[g]           reconstruction accumulated at level j
// The Haar taps are not applied here: the packed parameters carry the product
// of the analysis and synthesis taps of each depth, so analysis and synthesis
// are pure add/sub butterflies on un-normalised coefficients.
#pragma once

#include "wt2d_plan.h"

namespace wt {

// ---------------------------------------------------------------------------
// Register-tiled depthwise KxK cross-correlation of a TH x TW tile.
// `src` points at the top-left element of the (TH+K-1) x (TW+K-1) window, 16-byte
// aligned; rows are `pitch` floats apart (pitch % 4 == 0).  The window is read
// with 128-bit shared-memory loads, one input row at a time, and every row is
// applied to all output rows it contributes to, so each loaded float feeds
// K*min(K,TH)*TW/(TW+K-1) FMAs.
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
  WT_HD float* weights(int g) const { return base + p->woff + g * p->wstride; }
};

// ---------------------------------------------------------------------------
// One level of sub-band convolution + inverse butterfly for one thread tile.
// Computes the four scaled sub-band convolutions of level j on TH x TW
// positions, adds the reconstruction of the deeper levels to the low-pass
// band (wtconv2d.py:71), applies the 2x2 synthesis butterfly (wavelet.py:70-75)
// and writes the 2TH x 2TW block of R_{j-1}, cropped to the level's true size
// (wtconv2d.py:76).
// ---------------------------------------------------------------------------
template <int K, int TH, int TW>
WT_HD void level_item(const Plan2d& p, const Smem2d& sm, const Axis& ay, const Axis& ax, int j, int g,
                      int iy, int ix, bool has_r) {
  const int r = p.r;
  const int pitch = p.pitch[j];
  const int wy = ay.a[j] + iy * TH - r - ay.org[j];   // window origin in array coordinates
  const int wx = ax.a[j] + ix * TW - r - ax.org[j];
  float y[4][TH][TW];
#pragma unroll
  for (int s = 0; s < 4; ++s) {
#pragma unroll
    for (int i = 0; i < TH; ++i)
#pragma unroll
      for (int q = 0; q < TW; ++q) y[s][i][q] = 0.f;
    const float* wts = sm.weights(g) + p.tapset * (1 + 4 * (p.lvl0 + j - 1) + s);
    conv_tile<K, TH, TW>(sm.arr(j, g, s) + wy * pitch + wx, pitch, wts, y[s]);
  }
  if (has_r) {
    const float* rj = sm.rec(j, g) + (iy * TH) * p.rpitch[j] + ix * TW;
#pragma unroll
    for (int i = 0; i < TH; ++i)
#pragma unroll
      for (int q = 0; q < TW; ++q) y[0][i][q] += rj[i * p.rpitch[j] + q];
  }
  // synthesis butterfly into R_{j-1}
  float* out = sm.rec(j - 1, g);
  const int opitch = p.rpitch[j - 1];
  const int nrow = ay.n[j - 1], ncol = ax.n[j - 1];
#pragma unroll
  for (int i = 0; i < TH; ++i) {
    const int oy = 2 * (iy * TH + i);
#pragma unroll
    for (int q = 0; q < TW; ++q) {
      const int ox = 2 * (ix * TW + q);
      const float pp = y[0][i][q] + y[1][i][q], qq = y[0][i][q] - y[1][i][q];
      const float uu = y[2][i][q] + y[3][i][q], vv = y[2][i][q] - y[3][i][q];
      if (oy < nrow) {
        if (ox < ncol) out[oy * opitch + ox] = pp + uu;
        if (ox + 1 < ncol) out[oy * opitch + ox + 1] = pp - uu;
      }
      if (oy + 1 < nrow) {
        if (ox < ncol) out[(oy + 1) * opitch + ox] = qq + vv;
        if (ox + 1 < ncol) out[(oy + 1) * opitch + ox + 1] = qq - vv;
      }
    }
  }
}

// Base depthwise convolution of one BH x BW output tile, accumulated in place on
// R_0 (wtconv2d.py:81-82: base_scale*(conv+bias) + x_tag, scale folded on the host).
template <int K, int BH, int BW>
WT_HD void base_item(const Plan2d& p, const Smem2d& sm, const Axis& ay, const Axis& ax, int g, int iy, int ix) {
  const int r = p.r;
  const int pitch = p.pitch[0];
  const int wy = ay.t0 + iy * BH - r - ay.org[0];
  const int wx = ax.t0 + ix * BW - r - ax.org[0];
  float* r0 = sm.rec(0, g) + (iy * BH) * p.rpitch[0] + ix * BW;
  const float* wts = sm.weights(g);
  const float bias = wts[K * K];
  float acc[BH][BW];
#pragma unroll
  for (int i = 0; i < BH; ++i)
#pragma unroll
    for (int q = 0; q < BW; ++q) acc[i][q] = r0[i * p.rpitch[0] + q] + bias;
  conv_tile<K, BH, BW>(sm.arr(0, g, 0) + wy * pitch + wx, pitch, wts, acc);
#pragma unroll
  for (int i = 0; i < BH; ++i)
#pragma unroll
    for (int q = 0; q < BW; ++q) r0[i * p.rpitch[0] + q] = acc[i][q];
}

template <int K>
WT_HD void level_dispatch(const Plan2d& p, const Smem2d& sm, const Axis& ay, const Axis& ax, int j, int g,
                          int iy, int ix, bool has_r) {
  const int code = p.th[j] * 16 + p.tw[j];
  switch (code) {
    case 4 * 16 + 4: level_item<K, 4, 4>(p, sm, ay, ax, j, g, iy, ix, has_r); break;
    case 2 * 16 + 4: level_item<K, 2, 4>(p, sm, ay, ax, j, g, iy, ix, has_r); break;
    default: level_item<K, 1, 4>(p, sm, ay, ax, j, g, iy, ix, has_r); break;
  }
}

template <int K>
WT_HD void base_dispatch(const Plan2d& p, const Smem2d& sm, const Axis& ay, const Axis& ax, int g, int iy, int ix) {
  const int code = p.th[0] * 16 + p.tw[0];
  switch (code) {
    case 8 * 16 + 4: base_item<K, 8, 4>(p, sm, ay, ax, g, iy, ix); break;
    case 4 * 16 + 4: base_item<K, 4, 4>(p, sm, ay, ax, g, iy, ix); break;
    default: base_item<K, 2, 4>(p, sm, ay, ax, g, iy, ix); break;
  }
}

// Channels-last staging: every thread moves CB-byte chunks (CB/sizeof(T) consecutive
// channels of one pixel) between global memory and the planar fp32 arrays.
template <typename T, int CB>
WT_HD void load_chunks(const Plan2d& p, const T* __restrict__ src, float* __restrict__ dst, int nr, int nc,
                       int pitch, int plane, int tid, int nthr) {
  constexpr int VEC = Chunk<T, CB>::VEC;
  if (VEC < 1) return;
  const int nch = p.G / (VEC > 0 ? VEC : 1);
  const int total = nr * nc * nch;
  for (int i = tid; i < total; i += nthr) {
    const int ch = i % nch;
    const int pix = i / nch;
    const int yy = pix / nc, xx = pix - yy * nc;
    Chunk<T, CB> c;
    c.raw = *reinterpret_cast<const typename RawChunk<CB>::type*>(src + (size_t)yy * p.xs[2] + (size_t)xx * p.xs[3] + ch * VEC);
    float* dd = dst + (ch * VEC) * plane + yy * pitch + xx;
#pragma unroll
    for (int e = 0; e < VEC; ++e) dd[e * plane] = Elem<T>::to_f(c.get(e));
  }
}

template <typename T, int CB>
WT_HD void store_chunks(const Plan2d& p, T* __restrict__ dst, const float* __restrict__ src, int nr, int nc,
                        int rp, int rplane, int s, int tid, int nthr) {
  constexpr int VEC = Chunk<T, CB>::VEC;
  if (VEC < 1) return;
  const int nch = p.G / (VEC > 0 ? VEC : 1);
  const int total = nr * nc * nch;
  for (int i = tid; i < total; i += nthr) {
    const int ch = i % nch;
    const int pix = i / nch;
    const int yy = pix / nc, xx = pix - yy * nc;
    const float* ss = src + (ch * VEC) * rplane + (yy * s) * rp + xx * s;
    Chunk<T, CB> c;
#pragma unroll
    for (int e = 0; e < VEC; ++e) c.set(e, Elem<T>::from_f(ss[e * rplane]));
    *reinterpret_cast<typename RawChunk<CB>::type*>(dst + (size_t)yy * p.ys[2] + (size_t)xx * p.ys[3] + ch * VEC) = c.raw;
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

  // ---- phase 0: clear the arrays (borders and out-of-plane cells stay zero), stage weights
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

    // ---- phase 1: input tile -> X0 (fp32), zero outside the plane (wtconv2d.py:49-51)
    const int y0 = imax(ay.lo[0], 0), y1 = imin(ay.hi[0], p.H);
    const int x0 = imax(ax.lo[0], 0), x1 = imin(ax.hi[0], p.W);
    const int nr = y1 - y0, nc = x1 - x0;
    const int pitch = p.pitch[0];
    const int plane = p.rows[0] * pitch;
    float* dst0 = smem + p.off[0] + (y0 - ay.org[0]) * pitch + (x0 - ax.org[0]);
    const T* xb = x + (size_t)nb * p.xs[0] + (size_t)c0 * p.xs[1];
    if (p.x_vec && gc == p.G) {
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

  // ---- phase 2: Haar analysis, level by level (wavelet.py:62-67; raw LL feeds the next level)
  for (int j = 1; j <= d; ++j) {
    WT_PHASE(nthr) {
      const int y0 = imax(ay.lo[j], 0), y1 = imin(ay.hi[j], p.Hj[j]);
      const int x0 = imax(ax.lo[j], 0), x1 = imin(ax.hi[j], p.Wj[j]);
      const int nr = y1 - y0, nc = x1 - x0;
      const int total = gc * nr * nc;
      const int sp = p.pitch[j - 1], dp = p.pitch[j];
      const int dplane = p.rows[j] * dp;
      for (int i = tid; i < total; i += nthr) {
        const int xx = i % nc;
        const int t = i / nc;
        const int yy = t % nr, g = t / nr;
        const float* s = sm.arr(j - 1, g, 0) + (2 * (y0 + yy) - ay.org[j - 1]) * sp + (2 * (x0 + xx) - ax.org[j - 1]);
        const float a = s[0], b = s[1], c = s[sp], e = s[sp + 1];
        float* o = sm.arr(j, g, 0) + (y0 + yy - ay.org[j]) * dp + (x0 + xx - ax.org[j]);
        const float ab = a + b, cd = c + e, amb = a - b, cmd = c - e;
        o[0] = ab + cd;            // LL
        o[dplane] = ab - cd;       // LH
        o[2 * dplane] = amb + cmd; // HL
        o[3 * dplane] = amb - cmd; // HH
      }
    }
  }

  // ---- phase 3: bottom-up: sub-band convolutions, low-pass accumulation, synthesis
  for (int j = d; j >= 1; --j) {
    WT_PHASE(nthr) {
      const int nty = cdiv(ay.n[j], p.th[j]), ntx = cdiv(ax.n[j], p.tw[j]);
      const int per = nty * ntx;
      const int total = gc * per;
      const bool has_r = (j < d) || p.has_rin;
      for (int i = tid; i < total; i += nthr) {
        const int g = i / per;
        const int t = i - g * per;
        const int iy = t / ntx, ix = t - iy * ntx;
        level_dispatch<K>(p, sm, ay, ax, j, g, iy, ix, has_r);
      }
    }
  }

  // ---- phase 4: base depthwise convolution + bias, accumulated onto R_0
  if (p.has_base) {
    WT_PHASE(nthr) {
      const int nty = cdiv(ay.n[0], p.th[0]), ntx = cdiv(ax.n[0], p.tw[0]);
      const int per = nty * ntx;
      const int total = gc * per;
      for (int i = tid; i < total; i += nthr) {
        const int g = i / per;
        const int t = i - g * per;
        const int iy = t / ntx, ix = t - iy * ntx;
        base_dispatch<K>(p, sm, ay, ax, g, iy, ix);
      }
    }
  }

  // ---- phase 5: write the tile
  WT_PHASE(nthr) {
    const int rp = p.rpitch[0];
    const int rplane = p.rrows[0] * rp;
    const float* r0 = smem + p.roff[0];
    if (p.out_planes) {
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
      const int s = p.out_stride;
      const int oy0 = cdiv(ay.t0, s), oy1 = cdiv(ay.t1, s);
      const int ox0 = cdiv(ax.t0, s), ox1 = cdiv(ax.t1, s);
      const int nr = oy1 - oy0, nc = ox1 - ox0;
      T* yb = y + (size_t)nb * p.ys[0] + (size_t)c0 * p.ys[1];
      if (p.y_vec && gc == p.G) {
        T* yo = yb + (size_t)oy0 * p.ys[2] + (size_t)ox0 * p.ys[3];
        const float* ro = r0 + (oy0 * s - ay.t0) * rp + (ox0 * s - ax.t0);
        if (p.y_vec == 16) store_chunks<T, 16>(p, yo, ro, nr, nc, rp, rplane, s, tid, nthr);
        else if (p.y_vec == 8) store_chunks<T, 8>(p, yo, ro, nr, nc, rp, rplane, s, tid, nthr);
        else store_chunks<T, 4>(p, yo, ro, nr, nc, rp, rplane, s, tid, nthr);
      } else if (p.y_cl) {
        const int total = nr * nc * gc;
        for (int i = tid; i < total; i += nthr) {
          const int g = i % gc;
          const int pix = i / gc;
          const int yy = pix / nc, xx = pix - yy * nc;
          yb[(size_t)g * p.ys[1] + (size_t)(oy0 + yy) * p.ys[2] + (size_t)(ox0 + xx) * p.ys[3]] =
              Elem<T>::from_f(r0[g * rplane + ((oy0 + yy) * s - ay.t0) * rp + ((ox0 + xx) * s - ax.t0)]);
        }
      } else {
        const int total = nr * nc * gc;
        for (int i = tid; i < total; i += nthr) {
          const int xx = i % nc;
          const int t = i / nc;
          const int yy = t % nr, g = t / nr;
          yb[(size_t)g * p.ys[1] + (size_t)(oy0 + yy) * p.ys[2] + (size_t)(ox0 + xx) * p.ys[3]] =
              Elem<T>::from_f(r0[g * rplane + ((oy0 + yy) * s - ay.t0) * rp + ((ox0 + xx) * s - ax.t0)]);
        }
      }
    }
  }
}

}  // namespace wt
