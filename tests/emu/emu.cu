// TEST INFRASTRUCTURE: host emulation of the WTConv CTA bodies.
//
// Compiles the very same kernel bodies, planners and per-element helpers as
// libwtconv_b200.so, but for the host: WT_PHASE becomes a loop over thread ids,
// so one CTA is executed sequentially with the identical index arithmetic and
// shared-memory layout.  The CPU test-suite uses it to check tiling, halos,
// cropping and strides against the oracle without a GPU.  It is built only by
// the tests, exports emu_* symbols only, and is never loaded by the package.
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/wtconv_b200.h"
#include "../../wtconv_b200/csrc/wt1d_host.h"
#include "../../wtconv_b200/csrc/wt2d_fused.cuh"
#include "../../wtconv_b200/csrc/wt2d_quad.cuh"
#include "../../wtconv_b200/csrc/wt2d_wgrad.cuh"
#include "../../wtconv_b200/csrc/wt2d_host.h"
#include "../../wtconv_b200/csrc/wt_aux.h"

using namespace wt;

namespace {

struct AlignedBuf {
  float* p;
  explicit AlignedBuf(size_t floats) { p = static_cast<float*>(aligned_alloc(64, (floats * 4 + 63) / 64 * 64)); }
  ~AlignedBuf() { free(p); }
};

template <typename T, int K>
void run2d(const Plan2d& p, const void* x, void* y, const float* packed, const float* rin, float* rout) {
  AlignedBuf smem(p.smem_floats + 16);
  for (int nb = 0; nb < p.B; ++nb)
    for (int by = 0; by < p.ntile_y; ++by)
      for (int bx = 0; bx < p.ntile_x; ++bx)
        for (int cg = 0; cg < p.ngroups; ++cg) {
          // poison the buffer so that a cell the kernel forgets to write shows up
          for (int i = 0; i < p.smem_floats + 16; ++i) smem.p[i] = 1.0e30f;
          if (p.has_base)
            wt2d_cta<T, K, true>(p, static_cast<const T*>(x), static_cast<T*>(y), packed, rin, rout, smem.p, cg, bx, by, nb);
          else
            wt2d_cta<T, K, false>(p, static_cast<const T*>(x), static_cast<T*>(y), packed, rin, rout, smem.p, cg, bx, by, nb);
        }
}

template <int K>
void run2d_k(const Plan2d& p, int dtype, const void* x, void* y, const float* packed, const float* rin, float* rout) {
  if (dtype == 0) run2d<float, K>(p, x, y, packed, rin, rout);
  else if (dtype == 1) run2d<__nv_bfloat16, K>(p, x, y, packed, rin, rout);
  else run2d<__half, K>(p, x, y, packed, rin, rout);
}

// register-resident small-plane kernel: one call per CTA of its grid
template <typename T, int NLEV, bool BASE>
void run_regplane_lev(const RegPlane& a, const void* x, void* y, float* rout, const float* packed) {
  AlignedBuf smem(32 * a.wpad + 16);
  for (int nb = 0; nb < a.nbatch; ++nb)
    for (int cg = 0; cg < a.ngroups; ++cg) {
      for (int i = 0; i < 32 * a.wpad + 16; ++i) smem.p[i] = 1.0e30f;
      regplane_cta<T, 5, 7, 7, NLEV, BASE>(a, static_cast<const T*>(x), static_cast<T*>(y), rout, packed, smem.p, cg, nb);
    }
}

template <typename T, bool BASE>
void run_regplane_t(const RegPlane& a, const void* x, void* y, float* rout, const float* packed) {
  if (a.nlev == 1) run_regplane_lev<T, 1, BASE>(a, x, y, rout, packed);
  else if (a.nlev == 2) run_regplane_lev<T, 2, BASE>(a, x, y, rout, packed);
  else run_regplane_lev<T, 3, BASE>(a, x, y, rout, packed);
}

void run_regplane(const RegPlane& a, int dtype, const void* x, void* y, float* rout, const float* packed) {
  if (!a.has_base) run_regplane_t<float, false>(a, x, y, rout, packed);
  else if (dtype == 0) run_regplane_t<float, true>(a, x, y, rout, packed);
  else if (dtype == 1) run_regplane_t<__nv_bfloat16, true>(a, x, y, rout, packed);
  else run_regplane_t<__half, true>(a, x, y, rout, packed);
}

// four-warp 14 x 14 level kernel
template <typename T, bool BASE>
void run_quad_t(const QuadPlane& a, const void* x, void* y, const float* rin, float* rout, const float* packed) {
  const int floats = 32 * a.wpad + kQuadSmemFloats + 16;
  AlignedBuf smem(floats);
  for (int nb = 0; nb < a.nbatch; ++nb)
    for (int cg = 0; cg < a.ngroups; ++cg) {
      for (int i = 0; i < floats; ++i) smem.p[i] = 1.0e30f;
      quad_cta<T, 5, BASE>(a, static_cast<const T*>(x), static_cast<T*>(y), rin, rout, packed, smem.p, cg, nb);
    }
}

void run_quad(const QuadPlane& a, int dtype, const void* x, void* y, const float* rin, float* rout, const float* packed) {
  if (!a.has_base) run_quad_t<float, false>(a, x, nullptr, rin, rout, packed);
  else if (dtype == 0) run_quad_t<float, true>(a, x, y, rin, rout, packed);
  else if (dtype == 1) run_quad_t<__nv_bfloat16, true>(a, x, y, rin, rout, packed);
  else run_quad_t<__half, true>(a, x, y, rin, rout, packed);
}

template <typename T, int K>
void run1d(const Plan1d& p, const void* x, void* y, const float* packed) {
  AlignedBuf smem(p.smem_floats + 16);
  for (int nb = 0; nb < p.B; ++nb)
    for (int cg = 0; cg < p.ngroups; ++cg)
      for (int tile = 0; tile < p.ntile; ++tile) {
        for (int i = 0; i < p.smem_floats + 16; ++i) smem.p[i] = 1.0e30f;
        wt1d_cta<T, K>(p, static_cast<const T*>(x), static_cast<T*>(y), packed, smem.p, tile, cg, nb);
      }
}

template <int K>
void run1d_k(const Plan1d& p, int dtype, const void* x, void* y, const float* packed) {
  if (dtype == 0) run1d<float, K>(p, x, y, packed);
  else if (dtype == 1) run1d<__nv_bfloat16, K>(p, x, y, packed);
  else run1d<__half, K>(p, x, y, packed);
}

// parameter-gradient kernels
template <typename T>
void run_pyramid_level(const PyramidLevel& a, const void* in, float* S) {
  const long long total = (long long)a.B * a.Hs * a.Ws * a.C;
  for (long long i = 0; i < total; ++i) pyramid_item<T>(a, static_cast<const T*>(in), S, i);
}

template <typename T, int K>
void run_wgrad(const WGradSet& a, int nsub, const void* S, const void* G, float* stat, long long sub_s, long long sub_g,
               long long sub_stat) {
  AlignedBuf smem(kWgradWarps * (K * K + 1) * 32 + 16);
  for (int sb = 0; sb < nsub; ++sb)
    for (int split = 0; split < a.nsplit; ++split)
      for (int cg = 0; cg < (a.C + 31) / 32; ++cg) {
        for (int i = 0; i < kWgradWarps * (K * K + 1) * 32 + 16; ++i) smem.p[i] = 1.0e30f;
        wgrad_cta<T, K>(a, static_cast<const T*>(S) + sb * sub_s, static_cast<const T*>(G) + sb * sub_g,
                        stat + sb * sub_stat, smem.p, cg, split);
      }
}

template <typename T>
void run_wgrad_k(const WGradSet& a, int K, int nsub, const void* S, const void* G, float* stat, long long sub_s,
                 long long sub_g, long long sub_stat) {
  if (K == 1) run_wgrad<T, 1>(a, nsub, S, G, stat, sub_s, sub_g, sub_stat);
  else if (K == 3) run_wgrad<T, 3>(a, nsub, S, G, stat, sub_s, sub_g, sub_stat);
  else if (K == 5) run_wgrad<T, 5>(a, nsub, S, G, stat, sub_s, sub_g, sub_stat);
  else run_wgrad<T, 7>(a, nsub, S, G, stat, sub_s, sub_g, sub_stat);
}

int ptr_align(const void* p) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  int al = 16;
  while (al > 1 && (a % al)) al /= 2;
  return al;
}

}  // namespace

extern "C" {

int emu_pack_params(int ndim, int C, int K, int L, int param_dtype, double ana_tap, double syn_tap,
                    const void* base_w, const void* base_b, const void* base_scale, const void* const* wavelet_w,
                    const void* const* wavelet_scale, float* packed, int adjoint) {
  PackArgs a;
  a.C = C; a.L = L; a.adjoint = adjoint;
  a.taps = (ndim == 2) ? K * K : K;
  a.tapset = tapset_floats(K, ndim);
  a.subbands = (ndim == 2) ? 4 : 2;
  a.base_w = base_w; a.base_b = base_b; a.base_scale = base_scale;
  a.cl_off = 0;
  double g = 1.0;
  for (int l = 0; l < L; ++l) {
    a.wavelet_w[l] = wavelet_w[l];
    a.wavelet_scale[l] = wavelet_scale[l];
    g *= ana_tap * syn_tap;
    a.gain[l] = g;
  }
  const long long total = (long long)C * a.tapset * (1 + a.subbands * L);
  for (long long i = 0; i < total; ++i) {
    packed[i] = param_dtype == 0 ? pack_value<float>(a, i)
              : param_dtype == 1 ? pack_value<__nv_bfloat16>(a, i) : pack_value<__half>(a, i);
  }
  return 0;
}

// Planner overrides for the following emu_* calls: edge > 0 forces the tiled
// multi-stage path with this tile edge and `levels` levels per stage (exercises halos
// and the stage chain on small planes); group > 0 forces the channels per CTA; mode 2 tiles
// every stage, which makes chains of three and more stages with materialised low-pass planes.
static int g_force_edge = 0, g_force_levels = 0, g_force_group = 0, g_force_mode = 1, g_force_regplane = 0;
// -1: plan without the register-resident small-plane kernel, 0: automatic
int emu_regplane(int mode) { g_force_regplane = mode; return 0; }
int emu_force(int edge, int levels, int group, int mode) {
  g_force_edge = edge; g_force_levels = levels; g_force_group = group; g_force_mode = mode ? mode : 1;
  return 0;
}

int emu_wtconv2d_forward(const void* x, void* y, const float* packed, int B, int C, int H, int W, int K, int L,
                         int stride, int dtype, const long long* xs, const long long* ys, int* info) {
  Layer2d ly;
  ly.B = B; ly.C = C; ly.H = H; ly.W = W; ly.K = K; ly.L = L; ly.stride = stride;
  ly.elem_size = dtype == 0 ? 4 : 2;
  for (int i = 0; i < 4; ++i) { ly.xs[i] = xs[i]; ly.ys[i] = ys[i]; }
  ly.x_align = ptr_align(x);
  ly.y_align = ptr_align(y);
  Tuning2d tune;
  tune.force_tiled = g_force_edge > 0 ? g_force_mode : 0;
  tune.tile_y = g_force_edge;
  tune.tile_x = g_force_edge;
  tune.tile_levels = g_force_levels;
  tune.group = g_force_group;
  tune.regplane = g_force_regplane;
  tune.cl = -1;   // the TMA-fed channels-last stage has no host form; the emulation covers the other kernels
  Chain2d ch = plan_layer(ly, tune);
  if (ch.status) return ch.status;
  std::vector<float> ws((size_t)ch.scratch_floats + 4, 1.0e30f);
  for (const Reduce2d& rd : ch.reduces) {
    const long long total = (long long)B * C * rd.Hout * rd.Wout;
    float* out = ws.data() + rd.out_off;
    if (rd.in_off < 0) {
      for (long long i = 0; i < total; ++i) {
        out[rd.out_cl ? reduce_cl_index(i, C, rd.Hout, rd.Wout) : i] = dtype == 0 ? reduce_value<float>(static_cast<const float*>(x), i, C, rd.Hin, rd.Win, rd.Hout, rd.Wout, rd.shift, xs[0], xs[1], xs[2], xs[3])
               : dtype == 1 ? reduce_value<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(x), i, C, rd.Hin, rd.Win, rd.Hout, rd.Wout, rd.shift, xs[0], xs[1], xs[2], xs[3])
                            : reduce_value<__half>(static_cast<const __half*>(x), i, C, rd.Hin, rd.Win, rd.Hout, rd.Wout, rd.shift, xs[0], xs[1], xs[2], xs[3]);
      }
    } else {
      const float* in = ws.data() + rd.in_off;
      const long long s1 = rd.in_cl ? 1 : (long long)rd.Hin * rd.Win, s2 = rd.in_cl ? (long long)rd.Win * C : rd.Win,
                      s3 = rd.in_cl ? C : 1;
      for (long long i = 0; i < total; ++i)
        out[rd.out_cl ? reduce_cl_index(i, C, rd.Hout, rd.Wout) : i] =
            reduce_value<float>(in, i, C, rd.Hin, rd.Win, rd.Hout, rd.Wout, rd.shift, (long long)C * rd.Hin * rd.Win, s1, s2, s3);
    }
  }
  if (info) {
    info[0] = (int)ch.stages.size(); info[1] = (int)ch.reduces.size(); info[2] = ch.stages.back().plan.G;
    info[3] = (int)ch.stages.back().smem_bytes;
    info[4] = 0;
    info[5] = 0;
    for (const Stage2d& sg : ch.stages) { info[4] += sg.kind == 1; info[5] += sg.kind == 2; }
  }
  for (const Stage2d& sg : ch.stages) {
    const bool from_x = sg.xin_off < 0;
    const bool final_stage = sg.rout_off < 0;
    const void* xin = from_x ? x : static_cast<const void*>(ws.data() + sg.xin_off);
    const float* rin = sg.rin_off < 0 ? nullptr : ws.data() + sg.rin_off;
    float* rout = final_stage ? nullptr : ws.data() + sg.rout_off;
    const int dt = from_x ? dtype : 0;
    if (sg.kind == 1) {
      run_regplane(sg.reg, dt, xin, final_stage ? y : nullptr, rout, packed);
      continue;
    }
    if (sg.kind == 2) {
      run_quad(sg.quad, dt, xin, final_stage ? y : nullptr, rin, rout, packed);
      continue;
    }
    switch (K) {
      case 1: run2d_k<1>(sg.plan, dt, xin, final_stage ? y : nullptr, packed, rin, rout); break;
      case 3: run2d_k<3>(sg.plan, dt, xin, final_stage ? y : nullptr, packed, rin, rout); break;
      case 5: run2d_k<5>(sg.plan, dt, xin, final_stage ? y : nullptr, packed, rin, rout); break;
      case 7: run2d_k<7>(sg.plan, dt, xin, final_stage ? y : nullptr, packed, rin, rout); break;
      default: run2d_k<0>(sg.plan, dt, xin, final_stage ? y : nullptr, packed, rin, rout); break;   // run-time kernel size
    }
  }
  return 0;
}

// Parameter-gradient kernels: pyramid of a tensor (levels concatenated, (B,H_l,W_l,4,C) each)
int emu_wtconv2d_pyramid(const void* t, float* pyramid, int B, int C, int H, int W, int L, int dtype,
                         const long long* strides) {
  PyramidLevel a;
  a.B = B; a.C = C;
  int h = H, w = W;
  const void* src = t;
  int sdt = dtype;
  long long in_s[4] = {strides[0], strides[1], strides[2], strides[3]};
  float* out = pyramid;
  for (int l = 0; l < L; ++l) {
    a.Hin = h; a.Win = w; a.Hs = (h + 1) / 2; a.Ws = (w + 1) / 2;
    for (int i = 0; i < 4; ++i) a.in_s[i] = in_s[i];
    if (sdt == 0) run_pyramid_level<float>(a, src, out);
    else if (sdt == 1) run_pyramid_level<__nv_bfloat16>(a, src, out);
    else run_pyramid_level<__half>(a, src, out);
    src = out; sdt = 0;
    h = a.Hs; w = a.Ws;
    in_s[0] = (long long)h * w * 4 * C; in_s[1] = 1; in_s[2] = (long long)w * 4 * C; in_s[3] = 4LL * C;
    out += (size_t)B * h * w * 4 * C;
  }
  return 0;
}

// `nsplit` CTAs per channel group share the items, as on the device
int emu_wtconv2d_weight_grad_stats(const void* x, const void* gy, const float* xp, const float* gp, float* stats, int B,
                                   int C, int H, int W, int K, int L, int dtype, const long long* xs,
                                   const long long* gs, int nsplit) {
  const int per_set = (K * K + 1) * C;
  for (long long i = 0; i < (long long)(1 + 4 * L) * per_set; ++i) stats[i] = 0.f;
  WGradSet a;
  a.B = B; a.C = C; a.h = H; a.w = W;
  a.tiles_y = cdiv(H, kWgradTH); a.tiles_x = cdiv(W, kWgradTW); a.nsplit = nsplit;
  for (int i = 0; i < 4; ++i) { a.s_s[i] = xs[i]; a.g_s[i] = gs[i]; }
  if (dtype == 0) run_wgrad_k<float>(a, K, 1, x, gy, stats, 0, 0, 0);
  else if (dtype == 1) run_wgrad_k<__nv_bfloat16>(a, K, 1, x, gy, stats, 0, 0, 0);
  else run_wgrad_k<__half>(a, K, 1, x, gy, stats, 0, 0, 0);
  int h = H, w = W;
  size_t off = 0;
  for (int l = 0; l < L; ++l) {
    h = (h + 1) / 2; w = (w + 1) / 2;
    a.h = h; a.w = w; a.tiles_y = cdiv(h, kWgradTH); a.tiles_x = cdiv(w, kWgradTW);
    const long long ps[4] = {(long long)h * w * 4 * C, 1, (long long)w * 4 * C, 4LL * C};
    for (int i = 0; i < 4; ++i) { a.s_s[i] = ps[i]; a.g_s[i] = ps[i]; }
    run_wgrad_k<float>(a, K, 4, xp + off, gp + off, stats + (size_t)(1 + 4 * l) * per_set, C, C, per_set);
    off += (size_t)B * h * w * 4 * C;
  }
  return 0;
}

int emu_param_grads(int ndim, int C, int K, int L, double ana_tap, double syn_tap, const float* stats,
                    const void* base_w, const void* base_b, const void* base_scale, const void* const* wavelet_w,
                    const void* const* wavelet_scale, void* g_base_w, void* g_base_b, void* g_base_scale,
                    void* const* g_wavelet_w, void* const* g_wavelet_scale) {
  GradArgs a;
  a.ndim = ndim; a.C = C; a.K = K; a.L = L; a.stats = stats;
  a.base_w = base_w; a.base_b = base_b; a.base_scale = base_scale;
  a.g_base_w = g_base_w; a.g_base_b = g_base_b; a.g_base_scale = g_base_scale;
  double g = 1.0;
  for (int l = 0; l < L; ++l) {
    a.wavelet_w[l] = wavelet_w[l]; a.wavelet_scale[l] = wavelet_scale[l];
    a.g_wavelet_w[l] = g_wavelet_w[l]; a.g_wavelet_scale[l] = g_wavelet_scale[l];
    g *= ana_tap * syn_tap;
    a.gain[l] = g;
  }
  const int nsub = ndim == 2 ? 4 : 2;
  for (long long i = 0; i < (long long)(1 + nsub * L) * C; ++i) param_grad_item<float>(a, i);
  return 0;
}

int emu_wtconv1d_forward(const void* x, void* y, const float* packed, int B, int C, int N, int K, int L, int stride,
                         int dtype, const long long* xs, const long long* ys, int* info) {
  Layer1d ly;
  ly.B = B; ly.C = C; ly.N = N; ly.K = K; ly.L = L; ly.stride = stride;
  for (int i = 0; i < 3; ++i) { ly.xs[i] = xs[i]; ly.ys[i] = ys[i]; }
  if (N / stride == 0) return 0;
  Plan1d p;
  long long smem = 0;
  const int st = plan_1d(p, smem, ly);
  if (st) return st;
  if (g_force_edge) { p.TX = g_force_edge; if (g_force_group) p.G = g_force_group; smem = layout_1d(p); }
  if (info) { info[0] = p.ntile; info[1] = p.G; info[2] = p.TX; info[3] = (int)smem; }
  switch (K) {
    case 1: run1d_k<1>(p, dtype, x, y, packed); break;
    case 3: run1d_k<3>(p, dtype, x, y, packed); break;
    case 5: run1d_k<5>(p, dtype, x, y, packed); break;
    case 7: run1d_k<7>(p, dtype, x, y, packed); break;
    default: run1d_k<0>(p, dtype, x, y, packed); break;   // run-time kernel size
  }
  return 0;
}

}  // extern "C"
