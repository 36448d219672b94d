// Host-side planner of the fused 2-D WTConv launches: picks the channel group,
// the thread tiles and the shared-memory layout of a stage, and splits layers
// whose planes do not fit on chip into a short chain of stages that hand a
// coarse fp32 pyramid to one another through caller-provided scratch memory.
#pragma once

#include <vector>

#include "wt2d_plan.h"

namespace wt {

constexpr int kSmemLimitBytes = 232448;    // 227 KB opt-in dynamic shared memory per CTA on sm_100
constexpr int kSmemTwoPerSm = 113 * 1024;  // budget that lets two CTAs share one SM
constexpr int kThreads2d = 256;
constexpr int kTiledLevels = 2;            // levels fused per stage when a plane has to be tiled
constexpr int kTiledEdge = 64;             // output tile edge of a tiled stage

// thread-tile height for `n` rows out of a menu (largest first): cheapest padded
// row count, with a small penalty for short tiles (they reuse fewer loaded rows)
inline int pick_tile(int n, const int* menu, int nmenu, double small_penalty) {
  int best = menu[0];
  double best_cost = 1e30;
  for (int i = 0; i < nmenu; ++i) {
    const int t = menu[i];
    const double cost = round_up(n, t) * (1.0 + small_penalty * ((double)menu[0] / t - 1.0));
    if (cost < best_cost - 1e-9) { best_cost = cost; best = t; }
  }
  return best;
}

// Fills level sizes, thread tiles, extents, offsets and the shared-memory size
// of `p`.  Problem, flags, K, nlev, G, TY/TX and wstride must already be set.
// Returns the dynamic shared memory in bytes.
inline long long layout_stage(Plan2d& p) {
  const int d = p.nlev;
  p.r = p.K / 2;
  p.rb = imax(p.r, 1);
  p.tapset = tapset_floats(p.K, 2);
  p.nthreads = kThreads2d;
  p.Hj[0] = p.H;
  p.Wj[0] = p.W;
  for (int j = 1; j <= d; ++j) {
    p.Hj[j] = (p.Hj[j - 1] + 1) / 2;
    p.Wj[j] = (p.Wj[j - 1] + 1) / 2;
  }
  p.ntile_y = cdiv(p.H, p.TY);
  p.ntile_x = cdiv(p.W, p.TX);
  p.ngroups = cdiv(p.C, p.G);

  static const int lvl_menu[3] = {4, 2, 1};
  static const int base_menu[3] = {8, 4, 2};
  const int ny0 = imin(p.TY, p.H);
  for (int j = 0; j <= d; ++j) {
    const int nyj = (ny0 + (1 << j) - 1) >> j;
    p.th[j] = (j == 0) ? pick_tile(nyj, base_menu, 3, 0.10) : pick_tile(nyj, lvl_menu, 3, 0.15);
    p.tw[j] = 4;
  }

  // static extents = maximum over all tiles of the per-CTA extents
  int ext[2][kMaxFused + 1], rext[2][kMaxFused + 1];
  for (int a = 0; a < 2; ++a)
    for (int j = 0; j <= kMaxFused; ++j) ext[a][j] = rext[a][j] = 0;
  for (int axis = 0; axis < 2; ++axis) {
    const int ntile = axis ? p.ntile_x : p.ntile_y;
    const int T = axis ? p.TX : p.TY;
    const int size0 = axis ? p.W : p.H;
    const int* sizes = axis ? p.Wj : p.Hj;
    for (int t = 0; t < ntile; ++t) {
      Axis ax;
      axis_geometry(d, p.r, p.rb, p.has_base, sizes, t * T, imin(size0, (t + 1) * T), axis ? 4 : 1, ax);
      for (int j = 0; j <= d; ++j) {
        const int tile = axis ? p.tw[j] : p.th[j];
        ext[axis][j] = imax(ext[axis][j], axis_extent(p.r, p.has_base, ax, j, tile));
        const bool tiled = (j >= 1) || p.has_base;
        rext[axis][j] = imax(rext[axis][j], tiled ? round_up(ax.n[j], tile) : ax.n[j]);
      }
    }
  }
  long long off = 0;
  p.woff = (int)off;
  off += (long long)p.G * p.wstride;
  for (int j = 0; j <= d; ++j) {
    p.rows[j] = ext[0][j];
    p.pitch[j] = round_up(ext[1][j], 4);
    p.off[j] = (int)off;
    off += (long long)p.G * (j == 0 ? 1 : 4) * p.rows[j] * p.pitch[j];
  }
  for (int j = 0; j <= d; ++j) {
    const bool needed = (j < d) || (j == 0) || p.has_rin;
    p.rrows[j] = needed ? rext[0][j] : 0;
    p.rpitch[j] = needed ? round_up(rext[1][j], 4) : 0;
    p.roff[j] = (int)off;
    off += (long long)p.G * p.rrows[j] * p.rpitch[j];
  }
  off += 4;                       // the last window may over-read up to three floats
  off = (off + 3) / 4 * 4;
  p.smem_floats = (int)off;
  return off * 4;
}

struct Stage2d {
  Plan2d plan;
  long long xin_off;   // fp32 low-pass planes read as input (floats into scratch), -1: the layer input
  long long rin_off;   // reconstruction of the deeper levels read, -1: none
  long long rout_off;  // fp32 planes written, -1: the layer output
  long long smem_bytes;
};

// Low-pass reduction x (or a coarser plane set) -> sums over 2^q x 2^q blocks
struct Reduce2d {
  long long in_off;    // -1: the layer input
  long long out_off;
  int Hin, Win, Hout, Wout, shift;
};

struct Chain2d {
  std::vector<Reduce2d> reduces;   // run first, in order
  std::vector<Stage2d> stages;     // run next, in order (deepest first)
  long long scratch_floats = 0;
  int status = 0;
};

struct Layer2d {
  int B, C, H, W, K, L, stride, elem_size;
  long long xs[4], ys[4];
  int x_align, y_align;   // largest power of two (<= 16) dividing the base addresses
};

inline int vec_bytes(const long long* s, int G, int elem_size, int ptr_align) {
  // channel-fastest tensors are read/written in per-pixel chunks of 16, 8 or 4 bytes
  if (s[1] != 1) return 0;
  for (int cb = 16; cb >= 4; cb /= 2) {
    const int vec = cb / elem_size;
    if (vec < 1 || (G % vec) != 0) continue;
    if ((s[0] % vec) || (s[2] % vec) || (s[3] % vec)) continue;
    if (ptr_align < cb) continue;
    if (vec == 1) return 0;       // a one-element chunk is the scalar path
    return cb;
  }
  return 0;
}

// Plan one stage with a fixed tiling; returns smem bytes
inline long long plan_stage(Plan2d& p, const Layer2d& ly, int H, int W, int first_level, int nlev,
                            bool final_stage, bool has_rin, int G, int TY, int TX) {
  p = Plan2d();
  p.B = ly.B; p.C = ly.C; p.H = H; p.W = W; p.K = ly.K;
  p.nlev = nlev;
  p.lvl0 = first_level;
  p.has_base = final_stage ? 1 : 0;
  p.has_rin = has_rin ? 1 : 0;
  p.out_planes = final_stage ? 0 : 1;
  p.out_stride = final_stage ? ly.stride : 1;
  p.Hout = final_stage ? cdiv(H, ly.stride) : H;
  p.Wout = final_stage ? cdiv(W, ly.stride) : W;
  p.wstride = packed_channel_floats(ly.K, 2, ly.L);
  p.G = G; p.TY = TY; p.TX = TX;
  if (first_level == 0) {
    for (int i = 0; i < 4; ++i) p.xs[i] = ly.xs[i];
    p.x_cl = (ly.xs[1] == 1 && ly.C > 1) ? 1 : 0;
    p.x_vec = vec_bytes(ly.xs, G, ly.elem_size, ly.x_align);
  } else {   // fp32 planes from scratch
    p.xs[0] = (long long)ly.C * H * W; p.xs[1] = (long long)H * W; p.xs[2] = W; p.xs[3] = 1;
    p.x_cl = 0; p.x_vec = 0;
  }
  if (final_stage) {
    for (int i = 0; i < 4; ++i) p.ys[i] = ly.ys[i];
    p.y_cl = (ly.ys[1] == 1 && ly.C > 1) ? 1 : 0;
    p.y_vec = vec_bytes(ly.ys, G, ly.elem_size, ly.y_align);
  }
  return layout_stage(p);
}

// Whole-plane stage: single tile, all `nlev` levels on chip.  Picks G; returns false if
// even one channel does not fit.
inline bool plan_whole_plane(Plan2d& p, long long& smem, const Layer2d& ly, int H, int W, int first_level,
                             int nlev, bool final_stage, int forced_group = 0) {
  if (nlev > kMaxFused) return false;
  if (forced_group > 0) {
    smem = plan_stage(p, ly, H, W, first_level, nlev, final_stage, false, forced_group, imax(H, 1), imax(W, 1));
    return smem <= kSmemLimitBytes;
  }
  static const int cand[5] = {16, 8, 4, 2, 1};
  const int TY = imax(H, 1), TX = imax(W, 1);
  int fit_two = 0, fit_one = 0;
  for (int i = 0; i < 5; ++i) {
    const int G = cand[i];
    if (G > ly.C && G != 1) continue;
    Plan2d q;
    const long long bytes = plan_stage(q, ly, H, W, first_level, nlev, final_stage, false, G, TY, TX);
    if (!fit_two && bytes <= kSmemTwoPerSm) fit_two = G;
    if (!fit_one && bytes <= kSmemLimitBytes) fit_one = G;
  }
  int G = 0;
  if (fit_two >= 4) G = fit_two;
  else if (fit_one) G = imin(fit_one, 4) > fit_two ? imin(fit_one, 4) : fit_two;
  if (G == 0) return false;
  smem = plan_stage(p, ly, H, W, first_level, nlev, final_stage, false, G, TY, TX);
  if (smem > kSmemLimitBytes) {   // imin(fit_one,4) is a candidate that fits by construction
    return false;
  }
  return true;
}

// Optional planner overrides (all zero = automatic).  Used by tuning sweeps and by
// the tests to exercise the tiled multi-stage path on small planes.
struct Tuning2d {
  int force_tiled = 0;   // never use the whole-plane mode
  int tile_edge = 0;     // output tile edge of tiled stages
  int tile_levels = 0;   // levels fused per tiled stage
  int group = 0;         // channels per CTA
};

// Builds the launch chain of one layer.
inline Chain2d plan_layer(const Layer2d& ly, const Tuning2d& tune = Tuning2d()) {
  Chain2d ch;
  const int tiled_levels = tune.tile_levels > 0 ? imin(tune.tile_levels, kMaxFused) : kTiledLevels;
  const int tiled_edge = tune.tile_edge > 0 ? round_up(tune.tile_edge, 1 << tiled_levels) : kTiledEdge;
  // level sizes of the whole pyramid
  std::vector<int> Hl(ly.L + 1), Wl(ly.L + 1);
  Hl[0] = ly.H; Wl[0] = ly.W;
  for (int j = 1; j <= ly.L; ++j) { Hl[j] = (Hl[j - 1] + 1) / 2; Wl[j] = (Wl[j - 1] + 1) / 2; }

  // top-down: decide the stage boundaries
  struct Cut { int first, nlev; bool whole; };
  std::vector<Cut> cuts;
  int q = 0;
  while (true) {
    const int remaining = ly.L - q;
    Plan2d tmp; long long bytes = 0;
    if (!tune.force_tiled && remaining <= kMaxFused &&
        plan_whole_plane(tmp, bytes, ly, Hl[q], Wl[q], q, remaining, q == 0, tune.group)) {
      cuts.push_back({q, remaining, true});
      break;
    }
    const int nlev = imin(remaining, tiled_levels);
    cuts.push_back({q, nlev, false});
    q += nlev;
    if (q == ly.L) break;   // also ends a base-only layer (nlev == 0)
  }
  // scratch: for every cut after the first, low-pass planes of its input level and
  // the reconstruction it hands up
  long long off = 0;
  std::vector<long long> xoff(cuts.size(), -1), roff(cuts.size(), -1);
  for (size_t i = 1; i < cuts.size(); ++i) {
    const long long n = (long long)ly.B * ly.C * Hl[cuts[i].first] * Wl[cuts[i].first];
    xoff[i] = off; off += (n + 3) / 4 * 4;
    roff[i] = off; off += (n + 3) / 4 * 4;
  }
  ch.scratch_floats = off;
  for (size_t i = 1; i < cuts.size(); ++i) {
    Reduce2d rd;
    const int from = cuts[i - 1].first, to = cuts[i].first;
    rd.in_off = xoff[i - 1];
    rd.out_off = xoff[i];
    rd.Hin = Hl[from]; rd.Win = Wl[from]; rd.Hout = Hl[to]; rd.Wout = Wl[to];
    rd.shift = to - from;
    ch.reduces.push_back(rd);
  }
  for (int i = (int)cuts.size() - 1; i >= 0; --i) {
    Stage2d st;
    const Cut& c = cuts[i];
    const bool final_stage = (c.first == 0);
    const bool has_rin = (i + 1 < (int)cuts.size());
    if (c.whole) {
      if (!plan_whole_plane(st.plan, st.smem_bytes, ly, Hl[c.first], Wl[c.first], c.first, c.nlev, final_stage,
                            tune.group)) {
        ch.status = -6; return ch;
      }
    } else {
      int G = 4;
      const int cb_chunk = (ly.elem_size == 2) ? 8 : 4;
      if (final_stage && ly.xs[1] == 1 && ly.C % cb_chunk == 0) G = cb_chunk;
      if (tune.group > 0) G = tune.group;
      while (true) {
        st.smem_bytes = plan_stage(st.plan, ly, Hl[c.first], Wl[c.first], c.first, c.nlev, final_stage, has_rin,
                                   G, tiled_edge, tiled_edge);
        if (st.smem_bytes <= kSmemLimitBytes || G == 1) break;
        G /= 2;
      }
      if (st.smem_bytes > kSmemLimitBytes) { ch.status = -6; return ch; }
    }
    st.xin_off = xoff[i];
    st.rin_off = has_rin ? roff[i + 1] : -1;
    st.rout_off = final_stage ? -1 : roff[i];
    ch.stages.push_back(st);
  }
  return ch;
}

}  // namespace wt
