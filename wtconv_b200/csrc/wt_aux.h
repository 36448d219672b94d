// Parameter folding and low-pass plane reduction: per-element bodies (shared
// by the CUDA kernels and the host emulation used in the CPU tests) and the
// launcher declarations used by the C-ABI translation unit.
#pragma once

#include <cuda_runtime.h>

#include "wt_common.h"

namespace wt {

struct Plan2d;
struct Plan1d;
struct RegPlane;
struct QuadPlane;
struct PyramidLevel;
struct WGradSet;

struct PackArgs {
  int C, L, taps, tapset, subbands;
  const void* base_w;
  const void* base_b;
  const void* base_scale;
  const void* wavelet_w[kMaxLevels];
  const void* wavelet_scale[kMaxLevels];
  double gain[kMaxLevels];   // (analysis tap * synthesis tap)^(level+1)
  int adjoint;               // 1: reversed tap sets and no bias (block of the adjoint layer)
  long long cl_off;          // 2-D: floats from the start of the block to its channels-last copy (0: none)
};

// Value of float `i` of the channels-last copy: [group][set][tap 0..taps][16 channels].  The
// channels-last kernels keep every sub-band and reconstruction at the reference's scale (their
// butterflies carry the factor 1/2 of a 2 x 2 Haar step themselves, which also keeps 16-bit
// storage in range at deep levels), so the sub-band taps of level l are the per-channel values
// times 4^(l+1) / 2: an exact power of two on top of the folded tap magnitudes.
template <typename P> WT_HD float pack_value(const PackArgs& a, long long i);
template <typename P>
WT_HD float pack_value_cl(const PackArgs& a, long long i) {
  const int ts1 = a.taps + 1;
  const int nset = 1 + a.subbands * a.L;
  const int ch = (int)(i % 16);
  long long t = i / 16;
  const int tap = (int)(t % ts1);
  t /= ts1;
  const int set = (int)(t % nset);
  const int g = (int)(t / nset);
  const int c = g * 16 + ch;
  if (c >= a.C) return 0.f;
  if (tap == a.taps && set != 0) return 0.f;
  const int per_c = a.tapset * nset;
  const float v = pack_value<P>(a, (long long)c * per_c + (long long)set * a.tapset + tap);
  if (set == 0) return v;
  const int l = (set - 1) / a.subbands;
  float up = 2.f;                       // 4^(l+1) / 2
  for (int k = 0; k < l; ++k) up *= 4.f;
  return v * up;
}

// Value of packed float `i`.  Layout per channel c (ts = tap-set floats):
//   [0, ts)                      base taps * base_scale[c]; slot K^d holds bias * base_scale[c]
//   [ts*(1 + S*l + s), +ts)      level l, sub-band s taps * wavelet_scale_l[S*c+s] * gain[l]
// The reference applies the same factors as separate tensor ops:
// wtconv/wtconv2d.py:58 (wavelet_scale), :81 (base_scale, bias included),
// wtconv/util/wavelet.py:62-75 (one analysis and one synthesis tap per level).
template <typename P>
WT_HD float pack_value(const PackArgs& a, long long i) {
  const int ts = a.tapset, sub = a.subbands, taps = a.taps;
  const int per_c = ts * (1 + sub * a.L);
  const int c = (int)(i / per_c);
  const int rem = (int)(i - (long long)c * per_c);
  const int set = rem / ts;
  int k = rem - set * ts;
  const bool is_tap = k < taps;
  if (a.adjoint && is_tap) k = taps - 1 - k;          // reversed taps = kernel flipped in every direction
  float v = 0.f;
  if (set == 0) {
    const float sc = Elem<P>::to_f(static_cast<const P*>(a.base_scale)[c]);
    if (is_tap) v = sc * Elem<P>::to_f(static_cast<const P*>(a.base_w)[(size_t)c * taps + k]);
    else if (k == taps && a.base_b && !a.adjoint) v = sc * Elem<P>::to_f(static_cast<const P*>(a.base_b)[c]);
  } else if (is_tap) {
    const int l = (set - 1) / sub, s = (set - 1) - l * sub;
    const int oc = sub * c + s;
    const float sc = Elem<P>::to_f(static_cast<const P*>(a.wavelet_scale[l])[oc]);
    const float w = Elem<P>::to_f(static_cast<const P*>(a.wavelet_w[l])[(size_t)oc * taps + k]);
    v = (float)((double)sc * (double)w * a.gain[l]);
  }
  return v;
}

// Parameter gradients from the correlation sums (see wt2d_wgrad.cuh): one item per
// (output set, channel).  Output set 0 is the base path, 1 + S*l + s sub-band s of level l
// (S = 4 in 2-D, 2 in 1-D).  1-D layers were summed as one-row images: their band s lives in
// 2-D set 1 + 4l + 2s and their K taps in the middle row of the K x K sums.
struct GradArgs {
  int ndim, C, K, L;
  const float* stats;            // (1+4L, K*K+1, C)
  const void* base_w;
  const void* base_b;            // may be null
  const void* base_scale;
  const void* wavelet_w[kMaxLevels];
  const void* wavelet_scale[kMaxLevels];
  void* g_base_w;
  void* g_base_b;
  void* g_base_scale;
  void* g_wavelet_w[kMaxLevels];
  void* g_wavelet_scale[kMaxLevels];
  double gain[kMaxLevels];       // (analysis tap * synthesis tap)^(level+1)
};

template <typename P>
WT_HD void param_grad_item(const GradArgs& a, long long idx) {
  const int nsub = (a.ndim == 2) ? 4 : 2;
  const int taps = (a.ndim == 2) ? a.K * a.K : a.K;
  const int kk1 = a.K * a.K + 1;
  const int c = (int)(idx % a.C);
  const int oset = (int)(idx / a.C);
  const int tap0 = (a.ndim == 2) ? 0 : (a.K / 2) * a.K;            // first of the taps in the K x K sums
  if (oset == 0) {
    const float* st = a.stats + c;
    const float sc = Elem<P>::to_f(static_cast<const P*>(a.base_scale)[c]);
    const P* w = static_cast<const P*>(a.base_w) + (size_t)c * taps;
    P* gw = static_cast<P*>(a.g_base_w) + (size_t)c * taps;
    float dot = 0.f;
    for (int t = 0; t < taps; ++t) {
      const float corr = st[(size_t)(tap0 + t) * a.C];
      gw[t] = Elem<P>::from_f(sc * corr);
      dot = fmaf(Elem<P>::to_f(w[t]), corr, dot);
    }
    const float sum_g = st[(size_t)(a.K * a.K) * a.C];
    if (a.base_b) {
      static_cast<P*>(a.g_base_b)[c] = Elem<P>::from_f(sc * sum_g);
      dot = fmaf(Elem<P>::to_f(static_cast<const P*>(a.base_b)[c]), sum_g, dot);
    }
    static_cast<P*>(a.g_base_scale)[c] = Elem<P>::from_f(dot);
  } else {
    const int l = (oset - 1) / nsub, s = (oset - 1) - l * nsub;
    const int set2d = 1 + 4 * l + ((a.ndim == 2) ? s : 2 * s);
    const float* st = a.stats + (size_t)set2d * kk1 * a.C + c;
    const int oc = nsub * c + s;
    const float g = (float)a.gain[l];
    const float sc = Elem<P>::to_f(static_cast<const P*>(a.wavelet_scale[l])[oc]);
    const P* w = static_cast<const P*>(a.wavelet_w[l]) + (size_t)oc * taps;
    P* gw = static_cast<P*>(a.g_wavelet_w[l]) + (size_t)oc * taps;
    float dot = 0.f;
    for (int t = 0; t < taps; ++t) {
      const float corr = st[(size_t)(tap0 + t) * a.C];
      gw[t] = Elem<P>::from_f(sc * g * corr);
      dot = fmaf(Elem<P>::to_f(w[t]), corr, dot);
    }
    static_cast<P*>(a.g_wavelet_scale[l])[oc] = Elem<P>::from_f(g * dot);
  }
}

cudaError_t launch_param_grads(const GradArgs& a, int param_dtype, cudaStream_t stream);

// out[n][c][yo][xo] = sum of the 2^shift x 2^shift block of `in`, zero outside the
// plane: the un-normalised low-pass plane `shift` levels further down
// (wtconv/wtconv2d.py:49-54 applied `shift` times, taps folded into the parameters).
template <typename T>
WT_HD float reduce_value(const T* __restrict__ in, long long i, int C, int Hin, int Win, int Hout, int Wout,
                         int shift, long long s0, long long s1, long long s2, long long s3) {
  const int edge = 1 << shift;
  const int xo = (int)(i % Wout);
  long long t = i / Wout;
  const int yo = (int)(t % Hout);
  t /= Hout;
  const int c = (int)(t % C), n = (int)(t / C);
  const T* base = in + n * s0 + c * s1;
  float acc = 0.f;
  for (int dy = 0; dy < edge; ++dy) {
    const int yy = yo * edge + dy;
    if (yy >= Hin) break;
    // pairwise order of the butterflies: (a+b)+(c+d) at every level
    float racc = 0.f;
    for (int dx = 0; dx < edge; ++dx) {
      const int xx = xo * edge + dx;
      if (xx >= Win) break;
      racc += Elem<T>::to_f(base[yy * s2 + xx * s3]);
    }
    acc += racc;
  }
  return acc;
}

cudaError_t launch_pack(const PackArgs& a, int param_dtype, float* packed, cudaStream_t stream);

// out_cl: store the sums channel-fastest, (B,Hout,Wout,C), instead of as (B,C,Hout,Wout) planes
cudaError_t launch_reduce(int dtype, const void* in, float* out, int B, int C, int Hin, int Win, int Hout,
                          int Wout, int shift, const long long* strides, int out_cl, cudaStream_t stream);

// index of element (n,c,yo,xo) of the plane-major index i in the channel-fastest output
WT_HD long long reduce_cl_index(long long i, int C, int Hout, int Wout) {
  const int xo = (int)(i % Wout);
  long long t = i / Wout;
  const int yo = (int)(t % Hout);
  t /= Hout;
  const int c = (int)(t % C);
  const long long n = t / C;
  return ((n * Hout + yo) * Wout + xo) * C + c;
}

template <int K>
cudaError_t launch_wt2d_k(const Plan2d& p, int dtype, const void* x, void* y, const float* packed,
                          const float* rin, float* rout, size_t smem_bytes, cudaStream_t stream);

cudaError_t launch_regplane(const RegPlane& a, int dtype, const void* x, void* y, float* rout,
                            const float* packed, size_t smem_bytes, cudaStream_t stream);

cudaError_t launch_quad(const QuadPlane& a, int dtype, const void* x, void* y, const float* rin, float* rout,
                        const float* packed, size_t smem_bytes, cudaStream_t stream);

cudaError_t launch_pyramid_level(const PyramidLevel& a, int dtype, const void* in, float* S, cudaStream_t stream);

cudaError_t launch_wgrad(const WGradSet& a, int K, int dtype, int nsub, const void* S, const void* G, float* stat,
                         long long sub_s, long long sub_g, long long sub_stat, cudaStream_t stream);

template <int K>
cudaError_t launch_wt1d_k(const Plan1d& p, int dtype, const void* x, void* y, const float* packed,
                          size_t smem_bytes, cudaStream_t stream);

}  // namespace wt
