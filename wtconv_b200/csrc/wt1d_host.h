// Host-side planner of the fused 1-D WTConv launch.
#pragma once

#include "wt1d_fused.cuh"

namespace wt {

constexpr int kThreads1d = 256;
constexpr int kSmemLimit1d = 232448;
constexpr int kSmemTwoPerSm1d = 75 * 1024;   // three CTAs per SM

struct Layer1d {
  int B, C, N, K, L, stride;
  long long xs[3], ys[3];
};

inline long long layout_1d(Plan1d& p) {
  const int d = p.nlev;
  p.r = p.K / 2;
  p.rb = imax(p.r, 1);
  p.tapset = tapset_floats(p.K, 1);
  p.wsm = p.wstride;                          // all tap sets of a channel are staged
  p.nthreads = kThreads1d;
  p.Nj[0] = p.N;
  for (int j = 1; j <= d; ++j) p.Nj[j] = (p.Nj[j - 1] + 1) / 2;
  p.ntile = cdiv(p.N, p.TX);
  p.ngroups = cdiv(p.C, p.G);
  p.g_shift = -1;
  for (int k = 0; k < 8; ++k) if ((1 << k) == p.G) p.g_shift = k;
  int ext[kMaxFused + 1] = {0}, rext[kMaxFused + 1] = {0};
  for (int t = 0; t < p.ntile; ++t) {
    if (t >= 2 && t < p.ntile - 2) continue;   // interior tiles are all alike
    Axis ax;
    axis_geometry(d, p.r, p.rb, 1, p.Nj, t * p.TX, imin(p.N, (t + 1) * p.TX), 4, ax);
    for (int j = 0; j <= d; ++j) {
      // items cover 16 samples at level 0 and 8 positions at the levels above
      ext[j] = imax(ext[j], axis_extent(p.r, 1, ax, j, j == 0 ? 2 * kTile1d : kTile1d));
      rext[j] = imax(rext[j], round_up(ax.n[j], j == 0 ? 2 * kTile1d : kTile1d));
    }
  }
  // row pitches padded so that consecutive channels start in different bank groups
  const int lanes_g = imin(p.G, 8);
  const int want = (lanes_g > 1) ? 4 * (8 / lanes_g) : 0;
  auto pad = [&](int words) {
    words = round_up(words, 4);
    if (lanes_g > 1) while (words % 32 != want) words += 4;
    return words;
  };
  long long off = 0;
  p.woff = 0;
  off += (long long)p.G * p.wsm;
  for (int j = 0; j <= d; ++j) {
    p.pitch[j] = pad(ext[j] + 4);             // +4: windows may over-read three floats
    p.off[j] = (int)off;
    off += (long long)p.G * (j == 0 ? 1 : 2) * p.pitch[j];
  }
  for (int j = 0; j <= d; ++j) {
    // R_j feeds the level-j items; R_0 exists only when the output is pooled
    const bool needed = (j == 0) ? (p.out_stride > 1) : (j < d);
    p.rpitch[j] = needed ? pad(rext[j]) : 0;
    p.roff[j] = (int)off;
    off += (long long)p.G * p.rpitch[j];
  }
  off = (off + 3) / 4 * 4 + 4;
  p.smem_floats = (int)off;
  return off * 4;
}

// Returns 0 or a negative status.
inline int plan_1d(Plan1d& p, long long& smem, const Layer1d& ly, int force_tx = 0, int force_g = 0) {
  if (ly.L > kMaxFused) return -3;
  p = Plan1d();
  p.B = ly.B; p.C = ly.C; p.N = ly.N; p.K = ly.K; p.nlev = ly.L;
  p.out_stride = ly.stride;
  p.Nout = ly.N / ly.stride;
  p.wstride = packed_channel_floats(ly.K, 1, ly.L);
  for (int i = 0; i < 3; ++i) { p.xs[i] = ly.xs[i]; p.ys[i] = ly.ys[i]; }
  // tile: a multiple of 2^L (level alignment), of the pooling stride and of the thread tile
  long long unit = (1LL << ly.L) * kTile1d;
  if (ly.stride > 1) unit *= ly.stride;
  int TX;
  if (unit >= ly.N || unit > 8192) TX = ly.N;           // one tile spans the signal
  else {
    long long t = (1024 / unit) * unit;
    if (t == 0) t = unit;
    TX = (int)(t >= ly.N ? ly.N : t);
  }
  if (force_tx > 0) TX = (int)imin((long long)ly.N, round_up(force_tx, (int)unit));
  p.TX = TX;
  static const int cand[4] = {8, 4, 2, 1};
  int best = 0;
  for (int i = 0; i < 4; ++i) {
    p.G = cand[i];
    if (p.G > ly.C && p.G != 1) continue;
    const long long bytes = layout_1d(p);
    if (bytes <= kSmemTwoPerSm1d) { best = p.G; break; }
    if (!best && bytes <= kSmemLimit1d && p.G == 1) best = 1;
  }
  if (!best) {
    // fall back to a shorter tile for very long halos
    p.G = 1;
    while (p.TX > (int)unit && layout_1d(p) > kSmemLimit1d) p.TX = (int)(((p.TX / 2) / unit) * unit > 0 ? ((p.TX / 2) / unit) * unit : unit);
    if (layout_1d(p) > kSmemLimit1d) return -6;
    best = 1;
  }
  p.G = force_g > 0 ? force_g : best;
  smem = layout_1d(p);
  if (smem > kSmemLimit1d) return -6;
  return 0;
}

}  // namespace wt
