// Launch plan and tile geometry of the fused 2-D WTConv kernel.
//
// One launch handles one "stage": an input plane set x (B,C,H,W), `nlev`
// wavelet levels computed on chip, optionally the reconstruction R_in of the
// deeper levels (fp32 planes from an earlier launch), optionally the base
// depthwise convolution, and one output (the layer output, or fp32 planes of
// R_0 for the next shallower launch).
//
// A CTA owns one (sample, channel group, output tile).  Everything a tile
// needs is derived from the zero-extension property of the reference cascade
// (wtconv/wtconv2d.py:49-51 pads right/bottom only and the 2x2 blocks are
// origin aligned): treat every level as zero outside [0,H_j)x[0,W_j), then
//   * level-j convolutions are needed on  [a_j, b_j) = tile >> j,
//   * their inputs (sub-bands of level j) on [a_j - r, b_j + r),
//   * the low-pass plane of level j additionally wherever level j+1 needs
//     its 2x2 sources, i.e. on 2*need_{j+1},
// all clipped to the plane plus a border of zeros.  With a single tile that
// covers the plane the clipping makes every halo the constant r (= K/2), which
// is the whole-plane-on-chip mode used for planes up to about 56x56.
#pragma once

#include "wt_common.h"

namespace wt {

struct Plan2d {
  // problem of this launch
  int B, C, H, W;
  int K, r, rb;          // kernel size, K/2, zero border max(r,1)
  int nlev;              // levels fused in this launch (d)
  int lvl0;              // index of the first of them in the packed parameters
  int has_base;          // add base conv + bias (final launch)
  int has_rin;           // R_d is read from `rin` (fp32 planes) instead of being zero
  int out_planes;        // output is fp32 (B,C,H,W)-contiguous planes (deep launch)
  int out_stride;        // spatial subsampling of the output (final launch only)
  int in_shift;          // q > 0: the stage's input plane is the 2^q x 2^q block sum of x, formed while loading
  int Hsrc, Wsrc;        // size of the tensor x actually read (== H, W when in_shift == 0)
  int Hout, Wout;
  // packed parameters
  int wstride;           // floats per channel
  int tapset;            // floats per tap set
  // tiling
  int G;                 // channels per CTA
  int g_shift;           // log2(G) when G is a power of two, else -1
  int TY, TX;            // output tile (multiples of 2^nlev unless a single tile)
  int ntile_y, ntile_x, ngroups;
  int nthreads;
  int elem_size;         // bytes per element of T (the launch's input / output type)
  // per-level extents, j = 0 (input plane) .. nlev
  int Hj[kMaxFused + 1], Wj[kMaxFused + 1];
  // arrays of level j: rows x pitch elements per channel (and sub-band), `plane` elements
  // apart (padded for bank spreading), starting `off` floats into shared memory
  int rows[kMaxFused + 1], pitch[kMaxFused + 1], plane[kMaxFused + 1], off[kMaxFused + 1];
  int rrows[kMaxFused + 1], rpitch[kMaxFused + 1], rplane[kMaxFused + 1], roff[kMaxFused + 1];
  int th[kMaxFused + 1], tw[kMaxFused + 1];   // thread tile per level (j=0: base conv tile)
  int woff, wsm;         // staged tap sets: offset, floats per channel
  int yoff, yrows, ypitch, yplane;   // Y scratch of the deep levels (4 sub-band arrays per channel)
  int ooff, orows, opitch, oplane;   // OUT staging tile: offset in floats; rows / pitch / plane in elements of T
  int x0_bytes;              // element size of X0: the activation size when 16-bit and final, else 4
  int smem_floats;
  // tensor strides in elements (n,c,h,w)
  long long xs[4], ys[4];
  int x_cl, y_cl;        // channel is the fastest-varying dimension
  int x_vec, y_vec;      // 16-byte channel chunks are legal for x / y
  int direct_store;      // final stage, channels-last y, no stride: top-level items store their pixels themselves
};

// Geometry of one level along one axis for the tile [t0,t1), all in closed form so
// that device code can evaluate just the levels it needs in registers:
//   a    first position whose convolution output the tile needs   (t0 >> j)
//   n    number of such positions
//   lo   first position of the level that must hold data: the halo grows by a factor
//        two per level going up, a - (K/2)*2^(d-j), clipped to the zero border
//   hi   one past the last such position: (b_d + K/2) * 2^(d-j), clipped likewise
//   org  position stored at array index 0: lo shifted left so that the first window
//        (position a - K/2) starts on a multiple of (vmask+1) elements
struct LevelGeo {
  int a, n, lo, hi, org;
};

WT_HD LevelGeo level_geo(int d, int r, int rb, int j, int size_j, int t0, int t1, int vmask) {
  LevelGeo g;
  g.a = t0 >> j;
  g.n = ((t1 + (1 << j) - 1) >> j) - g.a;
  const int bd = (t1 + (1 << d) - 1) >> d;
  g.lo = imax(g.a - (r << (d - j)), -rb);
  g.hi = imin((bd + r) << (d - j), size_j + rb);
  g.org = g.lo - ((g.lo - (g.a - r)) & vmask);
  return g;
}

// Per-CTA geometry along one axis, all levels (host-side planning and the 1-D kernel).
struct Axis {
  int t0, t1;                     // output range of the tile
  int a[kMaxFused + 1];           // first position whose convolution is needed at level j
  int n[kMaxFused + 1];           // number of such positions (b_j - a_j)
  int lo[kMaxFused + 1];          // first position of level j that must hold data
  int hi[kMaxFused + 1];          // one past the last such position
  int org[kMaxFused + 1];         // position stored at array index 0
};

// Fills `ax` for the tile [t0,t1) of an axis whose level sizes are `size[j]`.
// `vec_align` is 4 along x (window starts must be 16-byte aligned) and 1 along y.
WT_HD void axis_geometry(int d, int r, int rb, int has_base, const int* size, int t0, int t1, int vec_align,
                         Axis& ax) {
  (void)has_base;
  ax.t0 = t0;
  ax.t1 = t1;
  for (int j = 0; j <= d; ++j) {
    const LevelGeo g = level_geo(d, r, rb, j, size[j], t0, t1, vec_align - 1);
    ax.a[j] = g.a; ax.n[j] = g.n; ax.lo[j] = g.lo; ax.hi[j] = g.hi; ax.org[j] = g.org;
  }
}

// Extent (in positions) the array of level j must have along this axis: data
// range plus the overhang of the last, partially filled thread tile.
WT_HD int axis_extent(int r, int has_base, const Axis& ax, int j, int tile) {
  int last = ax.hi[j];
  const bool has_conv = (j >= 1) || has_base;
  if (has_conv) last = imax(last, ax.a[j] + round_up(ax.n[j], tile) + r);
  return last - ax.org[j];
}

}  // namespace wt
