// Host-side planner of the fused 2-D WTConv launches: picks the channel group,
// the thread tiles and the shared-memory layout of a stage, and splits layers
// whose planes do not fit on chip into a short chain of stages that hand a
// coarse fp32 pyramid to one another through caller-provided scratch memory.
#pragma once

#include <vector>

#include "wt2d_cl_host.h"
#include "wt2d_plan.h"
#include "wt2d_quad.cuh"
#include "wt2d_regplane.cuh"

namespace wt {

constexpr int kSmemLimitBytes = 232448;    // 227 KB opt-in dynamic shared memory per CTA on sm_100
constexpr int kSmemTwoPerSm = 113 * 1024;  // budget that lets two CTAs share one SM
constexpr int kThreads2d = 256;
constexpr int kTiledLevels = 2;            // levels fused per stage when a plane has to be tiled

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
  p.Hj[0] = p.H;
  p.Wj[0] = p.W;
  for (int j = 1; j <= d; ++j) {
    p.Hj[j] = (p.Hj[j - 1] + 1) / 2;
    p.Wj[j] = (p.Wj[j - 1] + 1) / 2;
  }
  p.ntile_y = cdiv(p.H, p.TY);
  p.ntile_x = cdiv(p.W, p.TX);
  p.ngroups = cdiv(p.C, p.G);
  p.g_shift = -1;
  for (int k = 0; k < 8; ++k) if ((1 << k) == p.G) p.g_shift = k;

  // thread tiles: the top level runs 2x4-position items (fused with a 4x8-pixel base
  // tile); deeper levels run one sub-band of a 4x4 or 2x4 tile per item
  static const int deep_menu[2] = {4, 2};
  const int ny0 = imin(p.TY, p.H);
  for (int j = 0; j <= d; ++j) {
    const int nyj = (ny0 + (1 << j) - 1) >> j;
    p.th[j] = (j == 0) ? 4 : (j == 1) ? 2 : pick_tile(nyj, deep_menu, 2, 0.15);
    p.tw[j] = (j == 0) ? 8 : 4;
  }

  // static extents = maximum over all tiles of the per-CTA extents
  int ext[2][kMaxFused + 1], rext[2][kMaxFused + 1], yext[2] = {0, 0};
  for (int a = 0; a < 2; ++a)
    for (int j = 0; j <= kMaxFused; ++j) ext[a][j] = rext[a][j] = 0;
  for (int axis = 0; axis < 2; ++axis) {
    const int ntile = axis ? p.ntile_x : p.ntile_y;
    const int T = axis ? p.TX : p.TY;
    const int size0 = axis ? p.W : p.H;
    const int* sizes = axis ? p.Wj : p.Hj;
    for (int t = 0; t < ntile; ++t) {
      if (t >= 2 && t < ntile - 2) continue;   // interior tiles are all alike
      Axis ax;
      axis_geometry(d, p.r, p.rb, p.has_base, sizes, t * T, imin(size0, (t + 1) * T), axis ? 4 : 1, ax);
      for (int j = 0; j <= d; ++j) {
        const int tile = axis ? p.tw[j] : p.th[j];
        ext[axis][j] = imax(ext[axis][j], axis_extent(p.r, p.has_base, ax, j, tile));
        // R_1 is read by whole top-level items, R_0 (deep stages only) and R_j, j>=2 element-wise
        rext[axis][j] = imax(rext[axis][j], (j == 1) ? round_up(ax.n[j], tile) : ax.n[j]);
        if (j >= 2) yext[axis] = imax(yext[axis], round_up(ax.n[j], tile));
      }
    }
  }
  // Planes are padded so that consecutive channels start 16*(8/min(G,8)) bytes further in
  // the bank pattern: the lanes of a quarter warp work on different channels of one tile.
  const int lanes_g = imin(p.G, 8);
  const int want_words = (lanes_g > 1) ? 4 * (8 / lanes_g) : 0;     // plane size mod 32 words
  auto pad_words = [&](long long words) {
    words = (words + 3) / 4 * 4;
    if (lanes_g > 1) while (words % 32 != want_words) words += 4;
    return words;
  };
  long long off = 0;
  p.woff = (int)off;
  p.wsm = p.tapset * (p.has_base + 4 * d);
  off += (long long)p.G * p.wsm;
  p.x0_bytes = (p.has_base && p.elem_size == 2) ? 2 : 4;
  for (int j = 0; j <= d; ++j) {
    p.rows[j] = ext[0][j];
    p.pitch[j] = round_up(ext[1][j], 4);
    p.off[j] = (int)off;
    const int esz = (j == 0) ? p.x0_bytes : 4;
    const long long words = pad_words(((long long)p.rows[j] * p.pitch[j] * esz + 3) / 4);
    p.plane[j] = (int)(words * 4 / esz);
    off += (long long)p.G * (j == 0 ? 1 : 4) * words;
  }
  p.yrows = yext[0];
  p.ypitch = round_up(yext[1], 4);
  p.yplane = (int)pad_words((long long)p.yrows * p.ypitch);
  p.yoff = (int)off;
  off += (long long)p.G * 4 * p.yplane;
  for (int j = 0; j <= d; ++j) {
    // R_0 only exists in stages without a base convolution (their output); R_d only when
    // an earlier launch provides it
    const bool needed = (j == 0) ? (!p.has_base && !p.direct_store) : ((j < d) || p.has_rin);
    p.rrows[j] = needed ? rext[0][j] : 0;
    p.rpitch[j] = needed ? round_up(rext[1][j], 4) : 0;
    p.rplane[j] = needed ? (int)pad_words((long long)p.rrows[j] * p.rpitch[j]) : 0;
    p.roff[j] = (int)off;
    off += (long long)p.G * p.rplane[j];
  }
  p.ooff = (int)off;
  p.orows = p.opitch = p.oplane = 0;
  if (p.has_base && !p.direct_store) {     // OUT staging tile (not needed when the items store to y themselves)
    const int tile_y = imin(p.TY, p.H), tile_x = imin(p.TX, p.W);
    p.orows = round_up(tile_y, 4);
    p.opitch = round_up(tile_x, 8);
    const long long words = pad_words(((long long)p.orows * p.opitch * p.elem_size + 3) / 4);
    p.oplane = (int)(words * 4 / p.elem_size);
    off += (long long)p.G * words;
  }
  off += 4;                       // the last window may over-read up to three floats
  off = (off + 3) / 4 * 4;
  p.smem_floats = (int)off;
  // threads: enough for one top-level item each, at least four warps
  {
    const int tile_y = imin(p.TY, p.H), tile_x = imin(p.TX, p.W);
    const int items = (d >= 1) ? p.G * cdiv((tile_y + 1) / 2, 2) * cdiv((tile_x + 1) / 2, 4)
                               : p.G * cdiv(tile_y, 4) * cdiv(tile_x, 8);
    p.nthreads = imin(256, imax(128, round_up(items, 32)));
    // 16-bit activations: an eighth warp that takes no item still shortens the staging phases
    // (measured -1 % / -3 % on 56x56 / 28x28 planes; with fp32 activations it costs 4 % at 56x56)
    if (p.elem_size == 2 && p.nthreads > 192) p.nthreads = 256;
  }
  return off * 4;
}

// Combinations of the register-resident small-plane kernel that are compiled in
inline bool regplane_supported(int K, int PH, int PW, int nlev) {
  return K == 5 && PH == 7 && PW == 7 && nlev >= 1 && nlev <= 3;
}

// Launch description of a register-resident stage: levels q+1 .. q+nlev on the PH x PW plane of
// level q.  q = 0: the layer itself (tensor strides xs / ys, base path included); q > 0: the
// plane set is the fp32 block-sum reduction of the layer input, (B,C,PH,PW)-contiguous.
inline long long plan_regplane(RegPlane& a, int B, int C, int K, int L, int q, int nlev, int PH, int PW,
                               const long long* xs, const long long* ys, bool reduced_cl) {
  a = RegPlane();
  a.B = B; a.C = C; a.PH = PH; a.PW = PW;
  a.K = K; a.nlev = nlev; a.lvl0 = q; a.has_base = (q == 0) ? 1 : 0;
  a.wstride = packed_channel_floats(K, 2, L);
  const int ts = tapset_floats(K, 2);
  a.wbeg = a.has_base ? 0 : ts * (1 + 4 * q);
  a.wlen = ts * (a.has_base + 4 * nlev);
  a.wpad = a.wlen + (((a.wlen / 4) % 2 == 0) ? 4 : 0);
  a.ngroups = cdiv(C, 32);
  // about one wave of CTAs (three per SM), so the tap sets are staged once per resident CTA
  const long long warp_tasks = (long long)B * a.ngroups;
  a.samples_per_warp = (int)imax(1, (int)((warp_tasks + kRegPlaneWarps * 444 - 1) / (kRegPlaneWarps * 444)));
  a.nbatch = cdiv(B, kRegPlaneWarps * a.samples_per_warp);
  const long long planar[4] = {(long long)C * PH * PW, (long long)PH * PW, PW, 1};
  const long long chlast[4] = {(long long)C * PH * PW, 1, (long long)PW * C, C};
  for (int i = 0; i < 4; ++i) {
    a.xs[i] = (q == 0) ? xs[i] : (reduced_cl ? chlast[i] : planar[i]);
    a.ys[i] = (q == 0) ? ys[i] : 0;
    a.os[i] = planar[i];
  }
  return (long long)32 * a.wpad * 4;
}

// The four-warp level kernel handles planes of 13 or 14 rows / columns (7 x 7 sub-bands), K = 5
inline bool quad_supported(int K, int H, int W) {
  return K == 5 && (H == 13 || H == 14) && (W == 13 || W == 14);
}

// Launch description of the four-warp kernel for level q+1 on the Hp x Wp plane of level q.
// q = 0: the layer itself (tensor strides xs / ys, base path included); q > 0: the plane set is
// a channel-fastest fp32 reduction and the reconstruction is written as (B,C,Hp,Wp) planes.
inline long long plan_quad(QuadPlane& a, int B, int C, int K, int L, int q, int Hp, int Wp, const long long* xs,
                           const long long* ys) {
  a = QuadPlane();
  a.B = B; a.C = C; a.Hp = Hp; a.Wp = Wp; a.K = K; a.lvl0 = q;
  a.has_base = (q == 0) ? 1 : 0;
  a.has_rin = 1;
  a.wstride = packed_channel_floats(K, 2, L);
  const int ts = tapset_floats(K, 2);
  a.wbeg = a.has_base ? 0 : ts * (1 + 4 * q);
  a.wlen = ts * (a.has_base + 4);
  a.wpad = a.wlen + (((a.wlen / 4) % 2 == 0) ? 4 : 0);
  a.ngroups = cdiv(C, 32);
  // about one wave of CTAs (three per SM): the tap sets are staged once per CTA
  const long long tasks = (long long)B * a.ngroups;
  a.samples_per_cta = (int)imax(1, (int)((tasks + 443) / 444));
  a.nbatch = cdiv(B, a.samples_per_cta);
  const long long chlast[4] = {(long long)C * Hp * Wp, 1, (long long)Wp * C, C};
  const long long rcl[4] = {(long long)C * kQuadP * kQuadP, 1, (long long)kQuadP * C, C};
  for (int i = 0; i < 4; ++i) {
    a.xs[i] = (q == 0) ? xs[i] : chlast[i];
    a.ys[i] = (q == 0) ? ys[i] : 0;
    a.rs[i] = rcl[i];
  }
  return (long long)(32 * a.wpad + kQuadSmemFloats) * 4;
}

struct Stage2d {
  // 0: CTA-tile kernel (plan), 1: register-resident small-plane kernel (reg),
  // 2: four-warp 14 x 14 level kernel (quad), 3: channels-last level stage (cl),
  // 4: channels-last deep stage (deep), 5: channels-last sub-band pyramid, 6: channels-last low-pass
  // planes (5 and 6 read the layer input or a low-pass plane set of cl.H x cl.W; 6 writes one
  // level down to rout_off and, if rin_off >= 0, two levels down there)
  int kind = 0;
  RegPlane reg;
  QuadPlane quad;
  ClStage cl;
  ClDeepArgs deep;
  Plan2d plan = Plan2d();
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
  int out_cl = 0;      // 1: the sums are stored channel-fastest, (B,Hout,Wout,C)
  int in_cl = 0;       // 1: the input is such a channel-fastest fp32 array in scratch
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

// Plan one stage with a fixed tiling; returns smem bytes.  `in_shift` > 0: the stage reads
// the layer input and forms its low-pass plane of level `first_level` while loading.
inline long long plan_stage(Plan2d& p, const Layer2d& ly, int H, int W, int first_level, int nlev,
                            bool final_stage, bool has_rin, int G, int TY, int TX, int in_shift = 0) {
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
  p.in_shift = in_shift;
  p.Hsrc = in_shift ? ly.H : H;
  p.Wsrc = in_shift ? ly.W : W;
  const bool from_x = (first_level == 0) || in_shift > 0;
  p.elem_size = from_x ? ly.elem_size : 4;
  p.G = G; p.TY = TY; p.TX = TX;
  if (from_x) {
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
    // one barrier-separated phase less per tile: the quarter warp of an item (eight channels of
    // one pixel) writes 16 contiguous bytes, neighbouring channel groups fill the sector in L2
    // (tiles across the whole plane width only: with narrower tiles the scattered stores of a large
    // plane were measured 2.5x slower than the staged, coalesced ones)
    p.direct_store = (nlev >= 1 && ly.stride == 1 && p.y_vec == 16 && (ly.C % G) == 0 &&
                      TX >= W) ? 1 : 0;
  } else {
    // deep stages: the reconstruction block of an item goes straight to the fp32 planes
    p.direct_store = (nlev >= 1 && TX >= W) ? 1 : 0;
  }
  return layout_stage(p);
}

// Optional planner overrides (all zero = automatic).  The shared library always plans with
// the defaults; the host-emulation test library uses them to exercise the tiled multi-stage
// path on small planes.
struct Tuning2d {
  int force_tiled = 0;   // 1: never use the whole-plane mode for the top stage; 2: for no stage
  int tile_y = 0;        // output tile of tiled stages
  int tile_x = 0;
  int tile_levels = 0;   // levels fused per tiled stage
  int group = 0;         // channels per CTA
  int regplane = 0;      // -1: never use the register-level kernels at the bottom; 1: also with other overrides
  int deep_group = 0;    // channel group of whole-plane stages below the top (0: automatic)
  int cl = 0;            // -1: never use the channels-last kernels (they have no host form)
};

// Whole-plane stage: single tile, all `nlev` levels on chip.  Picks the largest channel
// group that lets two CTAs share an SM (or the forced one).  `good` tells whether that
// group still moves at least 8 bytes per pixel of a channels-last tensor.
inline bool plan_whole_plane(Plan2d& p, long long& smem, bool& good, const Layer2d& ly, int H, int W,
                             int first_level, int nlev, bool final_stage, int in_shift, int forced_group = 0,
                             bool has_rin = false) {
  good = false;
  if (nlev > kMaxFused) return false;
  const int TY = imax(H, 1), TX = imax(W, 1);
  if (forced_group > 0) {
    smem = plan_stage(p, ly, H, W, first_level, nlev, final_stage, has_rin, forced_group, TY, TX, in_shift);
    good = smem <= kSmemLimitBytes;
    return good;
  }
  static const int cand[5] = {16, 8, 4, 2, 1};
  int fit_two = 0, fit_one = 0;
  for (int i = 0; i < 5; ++i) {
    const int G = cand[i];
    if (G > ly.C && G != 1) continue;
    Plan2d q;
    const long long bytes = plan_stage(q, ly, H, W, first_level, nlev, final_stage, has_rin, G, TY, TX, in_shift);
    if (!fit_two && bytes <= kSmemTwoPerSm) fit_two = G;
    if (!fit_one && bytes <= kSmemLimitBytes) fit_one = G;
  }
  const int G = fit_two ? fit_two : fit_one;
  if (G == 0) return false;
  smem = plan_stage(p, ly, H, W, first_level, nlev, final_stage, has_rin, G, TY, TX, in_shift);
  const bool from_x = (first_level == 0) || in_shift > 0;
  const bool channels_last = from_x && ly.xs[1] == 1 && ly.C > 1;
  good = fit_two > 0 && (!channels_last || G * ly.elem_size >= 8 || G >= ly.C);
  return true;
}

// The channels-last kernels (wt2d_cl.cuh) read the layer input through a tensor map: channel
// stride 1, every other stride and the base address multiples of 16 bytes.
inline bool cl_stage_supported(const Layer2d& ly) {
  if (ly.K != 5 || ly.stride != 1 || ly.C < 8) return false;
  if ((long long)ly.B * ly.C * ly.H * ly.W >= (1LL << 35)) return false;   // 32-bit item indices in the pyramid kernels
  if (ly.xs[1] != 1 || ly.ys[1] != 1) return false;
  if (ly.x_align < 16) return false;
  for (int i = 0; i < 4; ++i)
    if (i != 1 && ((ly.xs[i] * ly.elem_size) % 16 != 0)) return false;
  return true;
}

// Tile configuration of the channels-last level stage for a W-wide plane (see launch_shape)
inline int cl_config(int W) {
  if (W <= 8) return 3;
  if (W <= 16) return 2;
  if (W <= 32) return 1;
  return 0;
}

// Bands (CTAs per plane slot) of the level stage on an H x W plane; they travel in grid.y
inline long long cl_bands(int H, int W) {
  static const int rows[4] = {4 * kClRH, 7 * kClRH, 4 * kClRH, 2 * kClRH}, cols[4] = {7 * kClCW, 4 * kClCW, 2 * kClCW, 1 * kClCW};
  const int cfg = cl_config(W);
  return (long long)cdiv((H + 1) / 2, rows[cfg]) * cdiv((W + 1) / 2, cols[cfg]);
}

// Description of a channels-last level stage.  level 0 with the base path finishes the layer
// (input x, output y); a deeper level reads the low-pass plane of the level above from scratch
// (dense channels-last, the layer's type) and writes an fp32 reconstruction.
inline void plan_cl_level(ClStage& s, const Layer2d& ly, int level, int H, int W, bool rin_channels_last,
                          float rin_scale) {
  const bool final_stage = (level == 0);
  s.B = ly.B; s.C = ly.C; s.H = H; s.W = W; s.K = ly.K;
  s.level = level; s.has_base = final_stage ? 1 : 0;
  s.config = cl_config(W);
  s.nlevels = ly.L;
  s.cl_off = cl_param_offset(ly.C, ly.K, ly.L);
  const int Hh = (H + 1) / 2, Wh = (W + 1) / 2;
  const long long dense[4] = {(long long)H * W * ly.C, 1, (long long)W * ly.C, ly.C};
  for (int k = 0; k < 4; ++k) {
    s.xs[k] = final_stage ? ly.xs[k] : dense[k];
    s.os[k] = final_stage ? ly.ys[k] : dense[k];
  }
  if (rin_channels_last) {
    s.rs[0] = (long long)Hh * Wh * ly.C; s.rs[1] = 1; s.rs[2] = (long long)Wh * ly.C; s.rs[3] = ly.C;
    s.rin_vec = (ly.C % 2 == 0) ? 1 : 0;
  } else {
    s.rs[0] = (long long)ly.C * Hh * Wh; s.rs[1] = (long long)Hh * Wh; s.rs[2] = Wh; s.rs[3] = 1;
    s.rin_vec = 0;
  }
  s.rin_scale = rin_scale;
  s.pdl = 0;
  s.x_vec = final_stage ? ((ly.x_align >= 2 * ly.elem_size && (ly.xs[0] % 2) == 0 && (ly.xs[2] % 2) == 0 && (ly.xs[3] % 2) == 0) ? 1 : 0)
                        : ((ly.C % 2 == 0) ? 1 : 0);
  if (final_stage) {
    const int pair_bytes = 2 * ly.elem_size;
    s.out_vec = (ly.y_align >= pair_bytes && (ly.ys[0] % 2) == 0 && (ly.ys[2] % 2) == 0 && (ly.ys[3] % 2) == 0) ? 1 : 0;
  } else {
    s.out_vec = (ly.C % 2 == 0) ? 1 : 0;
  }
}

// Builds the launch chain of one layer.
inline Chain2d plan_layer(const Layer2d& ly, const Tuning2d& tune = Tuning2d()) {
  Chain2d ch;
  // level sizes of the whole pyramid
  std::vector<int> Hl(ly.L + 1), Wl(ly.L + 1);
  Hl[0] = ly.H; Wl[0] = ly.W;
  for (int j = 1; j <= ly.L; ++j) { Hl[j] = (Hl[j - 1] + 1) / 2; Wl[j] = (Wl[j - 1] + 1) / 2; }

  // Bottom of the pyramid: when the plane of some level q is small enough for the
  // register-resident kernel (channels-last tensors, every remaining level), that kernel
  // takes levels q+1..L; the CTA-tile stages above it cover levels 1..q only.
  const bool use_cl = tune.cl >= 0 && cl_stage_supported(ly) && cl_bands(ly.H, ly.W) <= 65535;
  // Channels-last tensors larger than 16 x 16 (smaller planes are faster in the register-level
  // kernels below): the sub-band pyramid kernel and a deep stage (whole
  // planes on chip) for the levels below the top one, then the level stage of the top level with
  // the base path.
  if (use_cl && ly.L >= 1 && (ly.H > 16 || ly.W > 16)) {
    // The level stage takes the top nl levels one launch each (the first nl-1 of them read low-pass
    // planes that a reduction kernel writes); the deep stage takes the rest, whose sub-bands must
    // fit on chip.  nl is as small as the shared memory allows: 1 for planes up to about 64 x 64.
    const bool tma_rows = (ly.C * ly.elem_size) % 16 == 0;     // dense planes in scratch feed tensor maps too
    const int groups = cdiv(ly.C, kClGroup);
    Stage2d deep;
    int nl = 0;
    for (int n = 1; n <= ly.L && !nl; ++n) {
      const int rest = ly.L - n;                               // levels left to the deep stage
      if (rest == 0) { nl = n; break; }
      if (!tma_rows) break;
      // slots per CTA: as many as let two CTAs share an SM (their phases overlap) and still leave
      // four CTAs per SM in the grid; failing that, the largest number that fits at all
      static const int cand[4] = {8, 4, 2, 1};
      for (int pass = 0; pass < 2 && !nl; ++pass)
        for (int i = 0; i < 4 && !nl; ++i) {
          const int ns = cand[i];
          const long long bytes = plan_cl_deep(deep.deep, ly.B, ly.C, Hl[n - 1], Wl[n - 1], ly.K, rest + 1, ly.elem_size, ns);
          if (bytes < 0 || bytes > (pass == 0 ? kSmemTwoPerSm : kSmemLimitBytes)) continue;
          const bool enough = (long long)cdiv(ly.B, ns) * groups >= 4 * 148 || ns == 1;
          if (enough) nl = n;
        }
    }
    if (nl > 1 && !tma_rows) nl = 0;
    if (nl) {
      const bool has_deep = ly.L > nl;
      auto align4 = [](long long v) { return (v + 3) / 4 * 4; };
      auto elems_as_floats = [&](long long elems) { return align4((elems * ly.elem_size + 3) / 4); };
      // scratch: reconstructions read by levels 1..nl (fp32), low-pass planes 1..nl-1 and the deep
      // stage's sub-bands (the layer's type)
      std::vector<long long> roff(nl + 1, -1), poff(nl, -1);
      long long off = 0;
      for (int jl = 1; jl <= nl; ++jl)
        if (jl < nl || has_deep) { roff[jl] = off; off += align4((long long)ly.B * Hl[jl] * Wl[jl] * ly.C); }
      for (int jl = 1; jl < nl; ++jl) { poff[jl] = off; off += elems_as_floats((long long)ly.B * Hl[jl] * Wl[jl] * ly.C); }
      long long soff = -1;
      if (has_deep) { soff = off; off += elems_as_floats((long long)ly.B * 4 * Hl[nl + 1] * Wl[nl + 1] * ly.C); }
      ch.scratch_floats = off;
      // low-pass planes, two levels per launch
      for (int jl = 1; jl < nl; jl += 2) {
        Stage2d lp;
        lp.kind = 6;
        lp.cl.H = Hl[jl - 1]; lp.cl.W = Wl[jl - 1];
        lp.xin_off = (jl == 1) ? -1 : poff[jl - 1];
        lp.rout_off = poff[jl];
        lp.rin_off = (jl + 1 < nl) ? poff[jl + 1] : -1;        // second output, if wanted
        lp.smem_bytes = 0;
        ch.stages.push_back(lp);
      }
      if (has_deep) {
        Stage2d pyr;
        pyr.kind = 5;
        pyr.cl.H = Hl[nl - 1]; pyr.cl.W = Wl[nl - 1];
        pyr.xin_off = (nl == 1) ? -1 : poff[nl - 1];
        pyr.rin_off = -1; pyr.rout_off = soff;                 // sub-bands of level nl+1, in the layer's type
        pyr.smem_bytes = 0;
        ch.stages.push_back(pyr);
        deep.kind = 4;
        deep.deep.cl_off = cl_param_offset(ly.C, ly.K, ly.L);
        deep.deep.nlevels = ly.L;
        deep.deep.lvl0 = nl - 1;
        deep.deep.pdl = 1;                                     // the pyramid kernel is the launch before it
        deep.xin_off = soff; deep.rin_off = -1; deep.rout_off = roff[nl];
        deep.smem_bytes = deep.deep.smem_bytes;
        ch.stages.push_back(deep);
      }
      for (int jl = nl; jl >= 1; --jl) {
        Stage2d st;
        st.kind = 3;
        plan_cl_level(st.cl, ly, jl - 1, Hl[jl - 1], Wl[jl - 1], true, 0.5f);
        st.cl.pdl = 1;                                         // its reconstruction comes from the launch before it
        st.smem_bytes = 0;
        st.xin_off = (jl == 1) ? -1 : poff[jl - 1];
        st.rin_off = roff[jl];
        st.rout_off = (jl == 1) ? -1 : roff[jl - 1];
        ch.stages.push_back(st);
      }
      return ch;
    }
  }
  int qreg = -1;
  const bool untuned = !tune.force_tiled && !tune.tile_y && !tune.tile_x && !tune.tile_levels && !tune.group;
  if ((untuned || tune.regplane > 0) && tune.regplane >= 0 && ly.xs[1] == 1 && ly.C > 1) {
    for (int q = 0; q < ly.L; ++q) {
      if (!regplane_supported(ly.K, Hl[q], Wl[q], ly.L - q)) continue;
      if (q == 0 && (ly.stride != 1 || ly.ys[1] != 1)) continue;
      qreg = q;
      break;
    }
  }
  if (qreg == 0) {
    Stage2d st;
    st.kind = 1;
    st.smem_bytes = plan_regplane(st.reg, ly.B, ly.C, ly.K, ly.L, 0, ly.L, Hl[0], Wl[0], ly.xs, ly.ys, false);
    st.xin_off = -1; st.rin_off = -1; st.rout_off = -1;
    ch.stages.push_back(st);
    return ch;
  }
  // The level whose sub-bands are those 7 x 7 planes goes to the four-warp kernel.
  int qquad = -1;
  if (qreg >= 1 && tune.regplane >= 0 && quad_supported(ly.K, Hl[qreg - 1], Wl[qreg - 1]) &&
      (qreg > 1 || (ly.stride == 1 && ly.ys[1] == 1)))
    qquad = qreg - 1;
  // Scratch of the register-level stages: low-pass planes (channel-fastest) and reconstructions
  long long off = 0;
  const long long n7 = qreg > 0 ? ((long long)ly.B * ly.C * Hl[qreg] * Wl[qreg] + 3) / 4 * 4 : 0;
  const long long n14 = qquad >= 0 ? ((long long)ly.B * ly.C * Hl[qquad] * Wl[qquad] + 3) / 4 * 4 : 0;
  long long x14_off = -1, x7_off = -1, r7_off = -1, r14_off = -1;
  if (qquad > 0) { x14_off = off; off += n14; }
  if (qreg > 0) { x7_off = off; off += n7; r7_off = off; off += n7; }
  if (qquad > 0) { r14_off = off; off += n14; }
  if (qreg > 0) {
    if (qquad > 0) {                   // x -> 14 x 14 planes -> 7 x 7 planes
      Reduce2d ra;
      ra.in_off = -1; ra.out_off = x14_off;
      ra.Hin = ly.H; ra.Win = ly.W; ra.Hout = Hl[qquad]; ra.Wout = Wl[qquad];
      ra.shift = qquad; ra.out_cl = 1;
      ch.reduces.push_back(ra);
      Reduce2d rb;
      rb.in_off = x14_off; rb.out_off = x7_off;
      rb.Hin = Hl[qquad]; rb.Win = Wl[qquad]; rb.Hout = Hl[qreg]; rb.Wout = Wl[qreg];
      rb.shift = 1; rb.out_cl = 1; rb.in_cl = 1;
      ch.reduces.push_back(rb);
    } else {                           // low-pass plane of level qreg straight from the layer input
      Reduce2d rd;
      rd.in_off = -1; rd.out_off = x7_off;
      rd.Hin = ly.H; rd.Win = ly.W; rd.Hout = Hl[qreg]; rd.Wout = Wl[qreg];
      rd.shift = qreg; rd.out_cl = 1;
      ch.reduces.push_back(rd);
    }
    Stage2d st;
    st.kind = 1;
    st.smem_bytes = plan_regplane(st.reg, ly.B, ly.C, ly.K, ly.L, qreg, ly.L - qreg, Hl[qreg], Wl[qreg], nullptr,
                                  nullptr, true);
    if (qquad >= 0)                    // the four-warp kernel reads the reconstruction channel-fastest
      for (int i = 0; i < 4; ++i) st.reg.os[i] = st.reg.xs[i];
    st.xin_off = x7_off; st.rin_off = -1; st.rout_off = r7_off;
    ch.stages.push_back(st);
  }
  if (qquad >= 0) {
    Stage2d st;
    st.kind = 2;
    st.smem_bytes = plan_quad(st.quad, ly.B, ly.C, ly.K, ly.L, qquad, Hl[qquad], Wl[qquad], ly.xs, ly.ys);
    st.xin_off = qquad == 0 ? -1 : x14_off;
    st.rin_off = r7_off;
    st.rout_off = qquad == 0 ? -1 : r14_off;
    ch.stages.push_back(st);
    if (qquad == 0) { ch.scratch_floats = off; return ch; }
  }
  const int qbelow = qquad > 0 ? qquad : qreg;   // level whose reconstruction the stages above read
  const long long rbelow_off = qquad > 0 ? r14_off : r7_off;
  const int Ltop = qbelow > 0 ? qbelow : ly.L;   // levels handled by CTA-tile stages
  const bool below = qbelow > 0;                 // their deepest stage reads a reconstruction from below

  // top-down: decide the stage boundaries.  A stage is "whole" (its plane and every
  // deeper level stay on chip) or "tiled" (a few levels on halo tiles, the rest below).
  struct Cut { int first, nlev; bool whole; };
  std::vector<Cut> cuts;
  int q = 0;
  while (true) {
    const int remaining = Ltop - q;
    Plan2d tmp; long long bytes = 0; bool good = false;
    const bool fits = !(tune.force_tiled == 2 && remaining > 0) && !(tune.force_tiled && q == 0) &&
                      remaining <= kMaxFused &&
                      plan_whole_plane(tmp, bytes, good, ly, Hl[q], Wl[q], q, remaining, q == 0, 0, tune.group, below);
    // the top stage is taken only if it is efficient (two CTAs per SM, wide enough channel group);
    // a deep stage also when only one CTA fits, as long as its plane is small: a large plane held
    // whole by one CTA per SM loses more to idle SMs than its tiled split costs
    const bool small_plane = (long long)Hl[q] * Wl[q] <= 64 * 64;
    if (fits && (good || (q > 0 && small_plane) || remaining == 0)) {
      cuts.push_back({q, remaining, true});
      break;
    }
    int nlev = tune.tile_levels > 0 ? imin(tune.tile_levels, kMaxFused)
                                    : ((Hl[q] > 128 || Wl[q] > 128) ? kTiledLevels : 1);
    if (use_cl && q == 0) nlev = 1;    // the channels-last stage takes exactly the top level
    nlev = imin(remaining, nlev);
    if (fits && nlev == remaining) {   // nothing to split off below: keep the whole-plane stage
      cuts.push_back({q, remaining, true});
      break;
    }
    cuts.push_back({q, nlev, false});
    q += nlev;
    if (q == Ltop) break;   // also ends a base-only layer (nlev == 0)
  }
  // With exactly one deep CTA-tile stage it reads the layer input itself and forms its low-pass
  // plane while loading; with more, the low-pass planes are materialised in scratch.
  const bool direct = (cuts.size() == 2);
  std::vector<long long> xoff(cuts.size(), -1), roff(cuts.size() + 1, -1);
  for (size_t i = 1; i < cuts.size(); ++i) {
    const long long n = (long long)ly.B * ly.C * Hl[cuts[i].first] * Wl[cuts[i].first];
    if (!direct) { xoff[i] = off; off += (n + 3) / 4 * 4; }
    roff[i] = off; off += (n + 3) / 4 * 4;
  }
  roff[cuts.size()] = rbelow_off;
  ch.scratch_floats = off;
  if (!direct) {
    for (size_t i = 1; i < cuts.size(); ++i) {
      Reduce2d rd;
      const int from = cuts[i - 1].first, to = cuts[i].first;
      rd.in_off = xoff[i - 1];
      rd.out_off = xoff[i];
      rd.Hin = Hl[from]; rd.Win = Wl[from]; rd.Hout = Hl[to]; rd.Wout = Wl[to];
      rd.shift = to - from;
      ch.reduces.push_back(rd);
    }
  }
  for (int i = (int)cuts.size() - 1; i >= 0; --i) {
    Stage2d st;
    const Cut& c = cuts[i];
    const bool final_stage = (c.first == 0);
    const bool has_rin = (i + 1 < (int)cuts.size()) || below;
    const int in_shift = (direct && i == 1) ? c.first : 0;
    const int H = Hl[c.first], W = Wl[c.first];
    if (use_cl && final_stage && c.nlev == 1) {
      st.kind = 3;
      plan_cl_level(st.cl, ly, 0, ly.H, ly.W, false, 1.0f);
      st.smem_bytes = 0;
      st.xin_off = -1;
      st.rin_off = has_rin ? roff[i + 1] : -1;
      st.rout_off = -1;
      ch.stages.push_back(st);
      continue;
    }
    if (c.whole) {
      bool good = false;
      if (!plan_whole_plane(st.plan, st.smem_bytes, good, ly, H, W, c.first, c.nlev, final_stage, in_shift,
                            final_stage ? tune.group : tune.deep_group, has_rin)) {
        ch.status = -6; return ch;
      }
    } else {
      // tile: a band across the plane when it is narrow, else a square; the channel group is
      // one 16-byte chunk of a channels-last tensor
      const bool from_x = final_stage || in_shift > 0;
      const int unit = 1 << (c.nlev + 1);                  // tiles start on top-item boundaries
      int TX = tune.tile_x > 0 ? tune.tile_x : (W <= 64 ? W : 64);
      int TY = tune.tile_y > 0 ? tune.tile_y : (W <= 64 ? 16 : 32);
      TY = round_up(TY, unit);
      if (TX < W) TX = round_up(TX, imax(unit, 8));
      int G = 4;
      const int chunk = 16 / ly.elem_size;
      if (from_x && ly.xs[1] == 1 && ly.C % chunk == 0) G = chunk;
      if (tune.group > 0) G = tune.group;
      while (true) {
        st.smem_bytes = plan_stage(st.plan, ly, H, W, c.first, c.nlev, final_stage, has_rin, G, TY, TX, in_shift);
        if (st.smem_bytes <= kSmemTwoPerSm || G == 1) break;
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
