// extern "C" entry points of libwtconv_b200.so (see include/wtconv_b200.h).
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <vector>

#include "../../include/wtconv_b200.h"
#include "wt1d_host.h"
#include "wt1d_warp.cuh"
#include "wt2d_host.h"
#include "wt2d_wgrad.cuh"
#include "wt_aux.h"

using namespace wt;

namespace {

inline bool valid_dtype(int d) { return d == WTCONV_F32 || d == WTCONV_BF16 || d == WTCONV_F16; }
inline int elem_size(int d) { return d == WTCONV_F32 ? 4 : 2; }
inline bool unrolled_k(int K) { return K == 1 || K == 3 || K == 5 || K == 7; }   // other odd sizes up to kMaxK take the run-time instance
inline int ptr_align(const void* p) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  int al = 16;
  while (al > 1 && (a % al)) al /= 2;
  return al;
}

cudaError_t launch_wt2d(const Plan2d& p, int dtype, const void* x, void* y, const float* packed, const float* rin,
                        float* rout, size_t smem, cudaStream_t st) {
  switch (p.K) {
    case 1: return launch_wt2d_k<1>(p, dtype, x, y, packed, rin, rout, smem, st);
    case 3: return launch_wt2d_k<3>(p, dtype, x, y, packed, rin, rout, smem, st);
    case 5: return launch_wt2d_k<5>(p, dtype, x, y, packed, rin, rout, smem, st);
    case 7: return launch_wt2d_k<7>(p, dtype, x, y, packed, rin, rout, smem, st);
    default: return launch_wt2d_k<0>(p, dtype, x, y, packed, rin, rout, smem, st);
  }
}

cudaError_t launch_wt1d(const Plan1d& p, int dtype, const void* x, void* y, const float* packed, size_t smem,
                        cudaStream_t st) {
  switch (p.K) {
    case 1: return launch_wt1d_k<1>(p, dtype, x, y, packed, smem, st);
    case 3: return launch_wt1d_k<3>(p, dtype, x, y, packed, smem, st);
    case 5: return launch_wt1d_k<5>(p, dtype, x, y, packed, smem, st);
    case 7: return launch_wt1d_k<7>(p, dtype, x, y, packed, smem, st);
    default: return launch_wt1d_k<0>(p, dtype, x, y, packed, smem, st);
  }
}

// Set by the TMA-fed kernels when one of their bounded mbarrier waits gives up (see wt2d_cl.cuh);
// read and cleared by wtconv_device_status().  One word per device that loads the library.
__device__ int g_wait_status;

int* wait_status_address() {
  void* p = nullptr;
  return cudaGetSymbolAddress(&p, g_wait_status) == cudaSuccess ? static_cast<int*>(p) : nullptr;
}

int check_common(int C, int K, int L, int dtype) {
  if (C <= 0 || !valid_dtype(dtype)) return WTCONV_ERR_BAD_ARG;
  if (K < 1 || (K % 2) == 0 || K > kMaxK) return WTCONV_ERR_BAD_KERNEL_SIZE;
  if (L < 0 || L > kMaxLevels) return WTCONV_ERR_BAD_LEVELS;
  return WTCONV_OK;
}

int make_layer2d(Layer2d& ly, const void* x, const void* y, int B, int C, int H, int W, int K, int L, int stride,
                 int dtype, const long long* xs, const long long* ys) {
  const int st = check_common(C, K, L, dtype);
  if (st) return st;
  if (B <= 0 || H <= 0 || W <= 0 || stride < 1) return WTCONV_ERR_BAD_ARG;
  if ((long long)B * C * H * W >= (1LL << 40) || H > (1 << 20) || W > (1 << 20) || B > 65535 ||
      (long long)C * H * W >= (1LL << 31))
    return WTCONV_ERR_TOO_LARGE;   // grid.z carries the sample index; per-sample offsets are 32-bit
  ly.B = B; ly.C = C; ly.H = H; ly.W = W; ly.K = K; ly.L = L; ly.stride = stride;
  ly.elem_size = elem_size(dtype);
  const int Ho = cdiv(H, stride), Wo = cdiv(W, stride);
  const long long dx[4] = {(long long)C * H * W, (long long)H * W, W, 1};
  const long long dy[4] = {(long long)C * Ho * Wo, (long long)Ho * Wo, Wo, 1};
  for (int i = 0; i < 4; ++i) {
    ly.xs[i] = xs ? xs[i] : dx[i];
    ly.ys[i] = ys ? ys[i] : dy[i];
    if (ly.xs[i] < 0 || ly.ys[i] < 0) return WTCONV_ERR_BAD_ARG;
  }
  ly.x_align = ptr_align(x);
  ly.y_align = ptr_align(y);
  return WTCONV_OK;
}

// Launch chains are pure functions of the layer description; the last few are kept so that a
// model that calls the same layers step after step does not re-plan them.
std::shared_ptr<const Chain2d> cached_chain(const Layer2d& ly) {
  struct Entry { Layer2d key; std::shared_ptr<const Chain2d> chain; };
  static std::mutex mu;
  static std::vector<Entry> entries;
  static size_t next = 0;
  constexpr size_t kCapacity = 64;
  Layer2d key;
  memset(&key, 0, sizeof(key));          // padding bytes take part in the comparison
  key.B = ly.B; key.C = ly.C; key.H = ly.H; key.W = ly.W; key.K = ly.K; key.L = ly.L; key.stride = ly.stride;
  key.elem_size = ly.elem_size; key.x_align = ly.x_align; key.y_align = ly.y_align;
  for (int i = 0; i < 4; ++i) { key.xs[i] = ly.xs[i]; key.ys[i] = ly.ys[i]; }
  {
    std::lock_guard<std::mutex> lock(mu);
    for (const Entry& e : entries)
      if (memcmp(&e.key, &key, sizeof(key)) == 0) return e.chain;
  }
  auto chain = std::make_shared<const Chain2d>(plan_layer(ly));
  std::lock_guard<std::mutex> lock(mu);
  if (entries.size() < kCapacity) entries.push_back({key, chain});
  else { entries[next] = {key, chain}; next = (next + 1) % kCapacity; }
  return chain;
}

}  // namespace

extern "C" {

int wtconv_query(int what) {
  switch (what) {
    case WTCONV_QUERY_VERSION: return 1;
    case WTCONV_QUERY_MAX_KERNEL_SIZE: return kMaxK;
    case WTCONV_QUERY_MAX_LEVELS: return kMaxLevels;
    case WTCONV_QUERY_SM_ARCH: return 100;
    default: return WTCONV_ERR_BAD_ARG;
  }
}

const char* wtconv_status_string(int status) {
  switch (status) {
    case WTCONV_OK: return "ok";
    case WTCONV_ERR_BAD_ARG: return "invalid argument (null pointer, non-positive size, negative stride or unknown dtype code)";
    case WTCONV_ERR_BAD_KERNEL_SIZE: return "kernel_size must be odd and at most 29 (parameter gradients: 1, 3, 5 or 7)";
    case WTCONV_ERR_BAD_LEVELS: return "wt_levels is negative or larger than this build supports";
    case WTCONV_ERR_WORKSPACE: return "workspace pointer missing or smaller than wtconv2d_workspace_bytes()";
    case WTCONV_ERR_MISALIGNED: return "a tensor pointer is not aligned to its element size";
    case WTCONV_ERR_TOO_LARGE: return "problem too large for the on-chip plan (dimension or shared-memory limit)";
    case WTCONV_ERR_NO_DEVICE: return "no usable sm_100 CUDA device";
    case WTCONV_ERR_DEVICE_WAIT: return "a kernel gave up waiting for one of its on-chip copies; the outputs of calls since the last status check are invalid";
    case WTCONV_ERR_SCRATCH_LIMIT:
      return "problem needs more scratch than the library's built-in array (WTCONV_STATIC_SCRATCH_BYTES); "
             "use wtconv2d_forward with a caller-provided workspace";
    default: break;
  }
  if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
  return "unknown wtconv status";
}

size_t wtconv_packed_param_floats(int ndim, int C, int K, int L) {
  if ((ndim != 1 && ndim != 2) || C <= 0 || K < 1 || L < 0) return 0;
  if (ndim == 2) return (size_t)(cl_param_offset(C, K, L) + cl_param_floats(C, K, L));
  return (size_t)C * packed_channel_floats(K, ndim, L);
}

static int pack_params_impl(int adjoint, int ndim, int C, int K, int L, int param_dtype, double ana_tap, double syn_tap,
                       const void* base_w, const void* base_b, const void* base_scale,
                       const void* const* wavelet_w, const void* const* wavelet_scale, float* packed,
                       void* stream) {
  if (ndim != 1 && ndim != 2) return WTCONV_ERR_BAD_ARG;
  const int st = check_common(C, K, L, param_dtype);
  if (st) return st;
  if (!base_w || !base_scale || !packed || (L > 0 && (!wavelet_w || !wavelet_scale))) return WTCONV_ERR_BAD_ARG;
  PackArgs a;
  a.C = C; a.L = L; a.adjoint = adjoint;
  a.taps = (ndim == 2) ? K * K : K;
  a.tapset = tapset_floats(K, ndim);
  a.subbands = (ndim == 2) ? 4 : 2;
  a.base_w = base_w; a.base_b = base_b; a.base_scale = base_scale;
  a.cl_off = (ndim == 2) ? cl_param_offset(C, K, L) : 0;
  double g = 1.0;
  for (int l = 0; l < kMaxLevels; ++l) {
    a.wavelet_w[l] = nullptr; a.wavelet_scale[l] = nullptr; a.gain[l] = 0.0;
  }
  for (int l = 0; l < L; ++l) {
    if (!wavelet_w[l] || !wavelet_scale[l]) return WTCONV_ERR_BAD_ARG;
    a.wavelet_w[l] = wavelet_w[l];
    a.wavelet_scale[l] = wavelet_scale[l];
    g *= ana_tap * syn_tap;
    a.gain[l] = g;
  }
  return (int)launch_pack(a, param_dtype, packed, static_cast<cudaStream_t>(stream));
}

int wtconv_pack_params(int ndim, int C, int K, int L, int param_dtype, double ana_tap, double syn_tap,
                       const void* base_w, const void* base_b, const void* base_scale,
                       const void* const* wavelet_w, const void* const* wavelet_scale, float* packed,
                       void* stream) {
  return pack_params_impl(0, ndim, C, K, L, param_dtype, ana_tap, syn_tap, base_w, base_b, base_scale, wavelet_w,
                          wavelet_scale, packed, stream);
}

int wtconv_pack_params_adjoint(int ndim, int C, int K, int L, int param_dtype, double ana_tap, double syn_tap,
                               const void* base_w, const void* base_b, const void* base_scale,
                               const void* const* wavelet_w, const void* const* wavelet_scale, float* packed,
                               void* stream) {
  return pack_params_impl(1, ndim, C, K, L, param_dtype, ana_tap, syn_tap, base_w, base_b, base_scale, wavelet_w,
                          wavelet_scale, packed, stream);
}

size_t wtconv2d_pyramid_floats(int B, int C, int H, int W, int L) {
  if (B <= 0 || C <= 0 || H <= 0 || W <= 0 || L < 0 || L > kMaxLevels) return 0;
  size_t total = 0;
  int h = H, w = W;
  for (int l = 0; l < L; ++l) {
    h = (h + 1) / 2; w = (w + 1) / 2;
    total += (size_t)B * h * w * 4 * C;
  }
  return total;
}

int wtconv2d_pyramid(const void* t, float* pyramid, int B, int C, int H, int W, int L, int dtype,
                     const long long* strides, void* stream) {
  if (!t || (!pyramid && L > 0)) return WTCONV_ERR_BAD_ARG;
  if (B <= 0 || C <= 0 || H <= 0 || W <= 0 || !valid_dtype(dtype)) return WTCONV_ERR_BAD_ARG;
  if (L < 0 || L > kMaxLevels) return WTCONV_ERR_BAD_LEVELS;
  if ((long long)B * C * H * W >= (1LL << 40)) return WTCONV_ERR_TOO_LARGE;
  const long long dflt[4] = {(long long)C * H * W, (long long)H * W, W, 1};
  PyramidLevel a;
  a.B = B; a.C = C;
  int h = H, w = W;
  const void* src = t;
  int src_dtype = dtype;
  long long in_s[4];
  for (int i = 0; i < 4; ++i) in_s[i] = strides ? strides[i] : dflt[i];
  float* out = pyramid;
  for (int l = 0; l < L; ++l) {
    a.Hin = h; a.Win = w;
    a.Hs = (h + 1) / 2; a.Ws = (w + 1) / 2;
    for (int i = 0; i < 4; ++i) a.in_s[i] = in_s[i];
    const cudaError_t e = launch_pyramid_level(a, src_dtype, src, out, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return (int)e;
    // the next level reads the low-pass sub-band just written: (B, Hs, Ws, 4, C), sub-band 0
    src = out; src_dtype = WTCONV_F32;
    h = a.Hs; w = a.Ws;
    in_s[0] = (long long)h * w * 4 * C; in_s[1] = 1; in_s[2] = (long long)w * 4 * C; in_s[3] = 4LL * C;
    out += (size_t)B * h * w * 4 * C;
  }
  return WTCONV_OK;
}

size_t wtconv2d_weight_grad_stat_floats(int C, int K, int L) {
  if (C <= 0 || K < 1 || L < 0) return 0;
  return (size_t)(1 + 4 * L) * (K * K + 1) * C;
}

int wtconv2d_weight_grad_stats(const void* x, const void* gy, const float* x_pyramid, const float* g_pyramid,
                               float* stats, int B, int C, int H, int W, int K, int L, int dtype,
                               const long long* x_strides, const long long* g_strides, void* stream) {
  if (!x || !gy || !stats || (L > 0 && (!x_pyramid || !g_pyramid))) return WTCONV_ERR_BAD_ARG;
  const int st = check_common(C, K, L, dtype);
  if (st) return st;
  if (!unrolled_k(K)) return WTCONV_ERR_BAD_KERNEL_SIZE;      // the correlation kernels exist for 1, 3, 5, 7 only
  if (B <= 0 || H <= 0 || W <= 0) return WTCONV_ERR_BAD_ARG;
  if ((long long)B * C * H * W >= (1LL << 40) || (long long)C * H * W >= (1LL << 31)) return WTCONV_ERR_TOO_LARGE;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const size_t nstat = wtconv2d_weight_grad_stat_floats(C, K, L);
  cudaError_t e = cudaMemsetAsync(stats, 0, nstat * sizeof(float), cs);
  if (e != cudaSuccess) return (int)e;
  const long long dflt[4] = {(long long)C * H * W, (long long)H * W, W, 1};
  const int per_set = (K * K + 1) * C;
  auto geometry = [&](WGradSet& a, int h, int w, int nsub) {
    a.B = B; a.C = C; a.h = h; a.w = w;
    a.tiles_y = cdiv(h, kWgradTH); a.tiles_x = cdiv(w, kWgradTW);
    const long long items = (long long)B * a.tiles_y * a.tiles_x;
    const long long want = cdiv(888, imax(1, cdiv(C, 32) * nsub));            // about two waves of CTAs
    const long long most = (items + kWgradWarps - 1) / kWgradWarps;
    a.nsplit = (int)imax(1, (int)(want < most ? want : most));
  };
  WGradSet a;
  geometry(a, H, W, 1);
  for (int i = 0; i < 4; ++i) { a.s_s[i] = x_strides ? x_strides[i] : dflt[i]; a.g_s[i] = g_strides ? g_strides[i] : dflt[i]; }
  e = launch_wgrad(a, K, dtype, 1, x, gy, stats, 0, 0, 0, cs);
  if (e != cudaSuccess) return (int)e;
  int h = H, w = W;
  size_t off = 0;
  for (int l = 0; l < L; ++l) {
    h = (h + 1) / 2; w = (w + 1) / 2;
    geometry(a, h, w, 4);
    const long long ps[4] = {(long long)h * w * 4 * C, 1, (long long)w * 4 * C, 4LL * C};
    for (int i = 0; i < 4; ++i) { a.s_s[i] = ps[i]; a.g_s[i] = ps[i]; }
    e = launch_wgrad(a, K, WTCONV_F32, 4, x_pyramid + off, g_pyramid + off, stats + (size_t)(1 + 4 * l) * per_set, C, C,
                     per_set, cs);
    if (e != cudaSuccess) return (int)e;
    off += (size_t)B * h * w * 4 * C;
  }
  return WTCONV_OK;
}

int wtconv_param_grads(int ndim, int C, int K, int L, int param_dtype, double ana_tap, double syn_tap,
                       const float* stats, const void* base_w, const void* base_b, const void* base_scale,
                       const void* const* wavelet_w, const void* const* wavelet_scale, void* g_base_w,
                       void* g_base_b, void* g_base_scale, void* const* g_wavelet_w, void* const* g_wavelet_scale,
                       void* stream) {
  if (ndim != 1 && ndim != 2) return WTCONV_ERR_BAD_ARG;
  const int st = check_common(C, K, L, param_dtype);
  if (st) return st;
  if (!stats || !base_w || !base_scale || !g_base_w || !g_base_scale || (base_b && !g_base_b) ||
      (L > 0 && (!wavelet_w || !wavelet_scale || !g_wavelet_w || !g_wavelet_scale)))
    return WTCONV_ERR_BAD_ARG;
  GradArgs a;
  a.ndim = ndim; a.C = C; a.K = K; a.L = L;
  a.stats = stats;
  a.base_w = base_w; a.base_b = base_b; a.base_scale = base_scale;
  a.g_base_w = g_base_w; a.g_base_b = g_base_b; a.g_base_scale = g_base_scale;
  double g = 1.0;
  for (int l = 0; l < kMaxLevels; ++l) {
    a.wavelet_w[l] = nullptr; a.wavelet_scale[l] = nullptr; a.g_wavelet_w[l] = nullptr; a.g_wavelet_scale[l] = nullptr;
    a.gain[l] = 0.0;
  }
  for (int l = 0; l < L; ++l) {
    if (!wavelet_w[l] || !wavelet_scale[l] || !g_wavelet_w[l] || !g_wavelet_scale[l]) return WTCONV_ERR_BAD_ARG;
    a.wavelet_w[l] = wavelet_w[l]; a.wavelet_scale[l] = wavelet_scale[l];
    a.g_wavelet_w[l] = g_wavelet_w[l]; a.g_wavelet_scale[l] = g_wavelet_scale[l];
    g *= ana_tap * syn_tap;
    a.gain[l] = g;
  }
  return (int)launch_param_grads(a, param_dtype, static_cast<cudaStream_t>(stream));
}

int wtconv_device_status(void* stream) {
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  int word = 0;
  cudaError_t e = cudaMemcpyFromSymbolAsync(&word, g_wait_status, sizeof(int), 0, cudaMemcpyDeviceToHost, cs);
  if (e == cudaSuccess) e = cudaStreamSynchronize(cs);
  if (e != cudaSuccess) return (int)e;
  if (word == 0) return WTCONV_OK;
  const int zero = 0;
  e = cudaMemcpyToSymbolAsync(g_wait_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, cs);
  if (e == cudaSuccess) e = cudaStreamSynchronize(cs);
  return e == cudaSuccess ? WTCONV_ERR_DEVICE_WAIT : (int)e;
}

int wtconv2d_workspace_bytes(int B, int C, int H, int W, int K, int L, int dtype, const long long* x_strides,
                             const long long* y_strides, size_t* bytes) {
  if (!bytes) return WTCONV_ERR_BAD_ARG;
  Layer2d ly;
  // The stage chain depends on the strides and on whether the base addresses are 16-byte aligned
  // (the tensor maps of the channels-last kernels need that).  The size reported is the larger of
  // both cases, so it holds for any pair of pointers with these strides.
  const int st = make_layer2d(ly, nullptr, nullptr, B, C, H, W, K, L, 1, dtype, x_strides, y_strides);
  if (st) return st;
  long long floats = 0;
  for (int variant = 0; variant < 2; ++variant) {
    ly.x_align = ly.y_align = variant ? ly.elem_size : 16;
    const std::shared_ptr<const Chain2d> chp = cached_chain(ly);
    if (chp->status) return chp->status;
    if (chp->scratch_floats > floats) floats = chp->scratch_floats;
  }
  *bytes = (size_t)floats * sizeof(float);
  return WTCONV_OK;
}

int wtconv2d_launch_count(int B, int C, int H, int W, int K, int L, int stride, int dtype,
                          const long long* x_strides, const long long* y_strides, int* launches) {
  if (!launches) return WTCONV_ERR_BAD_ARG;
  Layer2d ly;
  const int st = make_layer2d(ly, nullptr, nullptr, B, C, H, W, K, L, stride, dtype, x_strides, y_strides);
  if (st) return st;
  const std::shared_ptr<const Chain2d> chp = cached_chain(ly);
  if (chp->status) return chp->status;
  *launches = (int)(chp->reduces.size() + chp->stages.size());
  return WTCONV_OK;
}

int wtconv2d_forward(const void* x, void* y, const float* packed, void* workspace, size_t workspace_bytes, int B,
                     int C, int H, int W, int K, int L, int stride, int dtype, const long long* x_strides,
                     const long long* y_strides, void* stream) {
  if (!x || !y || !packed) return WTCONV_ERR_BAD_ARG;
  Layer2d ly;
  const int st = make_layer2d(ly, x, y, B, C, H, W, K, L, stride, dtype, x_strides, y_strides);
  if (st) return st;
  if (ly.x_align < ly.elem_size || ly.y_align < ly.elem_size || ptr_align(packed) < 16) return WTCONV_ERR_MISALIGNED;
  const std::shared_ptr<const Chain2d> chp = cached_chain(ly);
  const Chain2d& ch = *chp;
  if (ch.status) return ch.status;
  float* ws = static_cast<float*>(workspace);
  if (ch.scratch_floats > 0) {
    if (!ws || workspace_bytes < (size_t)ch.scratch_floats * sizeof(float)) return WTCONV_ERR_WORKSPACE;
    if (ptr_align(ws) < 16) return WTCONV_ERR_MISALIGNED;
  }
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  int* wait_status = nullptr;
  for (const Reduce2d& rd : ch.reduces) {
    cudaError_t e;
    if (rd.in_off < 0) {
      e = launch_reduce(dtype, x, ws + rd.out_off, B, C, rd.Hin, rd.Win, rd.Hout, rd.Wout, rd.shift, ly.xs, rd.out_cl, cs);
    } else {
      const long long planar[4] = {(long long)C * rd.Hin * rd.Win, (long long)rd.Hin * rd.Win, rd.Win, 1};
      const long long chlast[4] = {(long long)C * rd.Hin * rd.Win, 1, (long long)rd.Win * C, C};
      const long long* s = rd.in_cl ? chlast : planar;
      e = launch_reduce(WTCONV_F32, ws + rd.in_off, ws + rd.out_off, B, C, rd.Hin, rd.Win, rd.Hout, rd.Wout,
                        rd.shift, s, rd.out_cl, cs);
    }
    if (e != cudaSuccess) return (int)e;
  }
  for (const Stage2d& sg : ch.stages) {
    const bool from_x = sg.xin_off < 0;          // the layer input (directly, or reduced while loading)
    const bool final_stage = sg.rout_off < 0;
    const void* xin = from_x ? x : static_cast<const void*>(ws + sg.xin_off);
    const float* rin = sg.rin_off < 0 ? nullptr : ws + sg.rin_off;
    float* rout = final_stage ? nullptr : ws + sg.rout_off;
    const int in_dtype = from_x ? dtype : WTCONV_F32;
    if ((sg.kind == 3 || sg.kind == 4) && !wait_status) wait_status = wait_status_address();
    cudaError_t e;
    switch (sg.kind) {
      case 1:
        e = launch_regplane(sg.reg, in_dtype, xin, final_stage ? y : nullptr, rout, packed, (size_t)sg.smem_bytes, cs);
        break;
      case 2:
        e = launch_quad(sg.quad, in_dtype, xin, final_stage ? y : nullptr, rin, rout, packed, (size_t)sg.smem_bytes, cs);
        break;
      case 3:   // input: the layer input or a low-pass plane in the layer's type; output: y or fp32 planes
        e = launch_cl_level(sg.cl, dtype, xin, rin, final_stage ? y : static_cast<void*>(rout), packed, wait_status, cs);
        break;
      case 4:   // input: the sub-bands of level 2 in the layer's type
        e = launch_cl_deep(sg.deep, ly.K, dtype, xin, packed, rout, wait_status, cs);
        break;
      case 5:     // sub-bands two levels below the plane set read (layer input or a dense low-pass plane set)
      case 6: {   // low-pass planes one and two levels below it
        const long long dense[4] = {(long long)sg.cl.H * sg.cl.W * ly.C, 1, (long long)sg.cl.W * ly.C, ly.C};
        const long long* s = from_x ? ly.xs : dense;
        // 2: four channels of a pixel may be moved as one 8- / 16-byte access, 1: pairs as one word, 0: neither
        int xv;
        if (from_x) {
          auto mult = [&](int m) { return ly.x_align >= m * ly.elem_size && (ly.xs[0] % m) == 0 && (ly.xs[2] % m) == 0 && (ly.xs[3] % m) == 0; };
          xv = mult(4) ? 2 : (mult(2) ? 1 : 0);
        } else {
          xv = (ly.C % 4 == 0) ? 2 : ((ly.C % 2 == 0) ? 1 : 0);
        }
        if (sg.kind == 5) e = launch_cl_pyramid(dtype, xin, s, xv, ly.B, ly.C, sg.cl.H, sg.cl.W, rout, cs);
        else e = launch_cl_lowpass(dtype, xin, s, xv, ly.B, ly.C, sg.cl.H, sg.cl.W, rout,
                                   sg.rin_off < 0 ? nullptr : static_cast<void*>(ws + sg.rin_off), cs);
        break;
      }
      default:
        e = launch_wt2d(sg.plan, in_dtype, xin, final_stage ? y : nullptr, packed, rin, rout, (size_t)sg.smem_bytes, cs);
        break;
    }
    if (e != cudaSuccess) return (int)e;
  }
  return WTCONV_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Allocation-free variant: the scratch planes live in the library image.
// ---------------------------------------------------------------------------
namespace {

// Part of every context that loads the library; 256-byte aligned so that the fp32 planes and
// their 128-bit accesses are aligned whatever the offsets inside it.
static __device__ __align__(256) unsigned char g_static_scratch[WTCONV_STATIC_SCRATCH_BYTES];

// `g_static_scratch` is only a host-side handle here: kernels need the device address, which
// differs per device and does not survive a cudaDeviceReset.  It is therefore asked for on every
// call (a table lookup in the runtime), with the caller's device current.
int static_scratch_address(void** out) {
  void* ptr = nullptr;
  const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
  if (e != cudaSuccess) return (int)e;
  if (!ptr) return WTCONV_ERR_NO_DEVICE;
  *out = ptr;
  return WTCONV_OK;
}

}  // namespace

extern "C" {

int wtconv2d_forward_noalloc(const void* x, void* y, const float* packed, int B, int C, int H, int W, int K, int L,
                             int stride, int dtype, const long long* x_strides, const long long* y_strides,
                             void* stream) {
  // size check first, with the chain these very pointers and strides get: reject before touching the device
  if (!x || !y || !packed) return WTCONV_ERR_BAD_ARG;
  Layer2d ly;
  const int st = make_layer2d(ly, x, y, B, C, H, W, K, L, stride, dtype, x_strides, y_strides);
  if (st) return st;
  {
    const std::shared_ptr<const Chain2d> chp = cached_chain(ly);
    if (chp->status) return chp->status;
    if ((size_t)chp->scratch_floats * sizeof(float) > (size_t)WTCONV_STATIC_SCRATCH_BYTES) return WTCONV_ERR_SCRATCH_LIMIT;
  }
  void* scratch = nullptr;
  const int sa = static_scratch_address(&scratch);
  if (sa) return sa;
  return wtconv2d_forward(x, y, packed, scratch, (size_t)WTCONV_STATIC_SCRATCH_BYTES, B, C, H, W, K, L, stride, dtype,
                          x_strides, y_strides, stream);
}

int wtconv1d_forward(const void* x, void* y, const float* packed, int B, int C, int N, int K, int L, int stride,
                     int dtype, const long long* x_strides, const long long* y_strides, void* stream) {
  if (!x || !y || !packed) return WTCONV_ERR_BAD_ARG;
  const int st = check_common(C, K, L, dtype);
  if (st) return st;
  if (B <= 0 || N <= 0 || stride < 1) return WTCONV_ERR_BAD_ARG;
  if (L > kMaxFused) return WTCONV_ERR_BAD_LEVELS;
  // grid.z carries the sample index, grid.y the channel group; offsets inside a sample are 32-bit
  if (B > 65535 || (long long)C * N >= (1LL << 31) || (long long)B * C * N >= (1LL << 40)) return WTCONV_ERR_TOO_LARGE;
  if (ptr_align(x) < elem_size(dtype) || ptr_align(y) < elem_size(dtype) || ptr_align(packed) < 16)
    return WTCONV_ERR_MISALIGNED;
  if (N / stride == 0) return WTCONV_OK;   // empty output
  Layer1d ly;
  ly.B = B; ly.C = C; ly.N = N; ly.K = K; ly.L = L; ly.stride = stride;
  const int No = N / stride;
  const long long dx[3] = {(long long)C * N, N, 1}, dy[3] = {(long long)C * No, No, 1};
  for (int i = 0; i < 3; ++i) {
    ly.xs[i] = x_strides ? x_strides[i] : dx[i];
    ly.ys[i] = y_strides ? y_strides[i] : dy[i];
    if (ly.xs[i] < 0 || ly.ys[i] < 0) return WTCONV_ERR_BAD_ARG;
  }
  if (wt1d_warp_supported(K, L, stride, ly.xs[2], ly.ys[2])) {
    // time-contiguous signals, stride 1, up to four levels: the register-resident kernel
    Warp1dArgs wa;
    wa.x = x; wa.y = y; wa.packed = packed;
    wa.B = B; wa.C = C; wa.N = N;
    wa.wstride = packed_channel_floats(K, 1, L);
    wa.nseg = 0; wa.nwarps = 0;
    wa.xs0 = ly.xs[0]; wa.xs1 = ly.xs[1]; wa.ys0 = ly.ys[0]; wa.ys1 = ly.ys[1];
    const cudaError_t e = launch_wt1d_warp(wa, K, L, dtype, static_cast<cudaStream_t>(stream));
    if (e != cudaErrorNotSupported) return (int)e;     // more than 2^31 warps: the CTA-tile kernel below
  }
  Plan1d p;
  long long smem = 0;
  const int ps = plan_1d(p, smem, ly);
  if (ps) return ps;
  if (p.ngroups > 65535) return WTCONV_ERR_TOO_LARGE;
  return (int)launch_wt1d(p, dtype, x, y, packed, (size_t)smem, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
