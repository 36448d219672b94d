// One wavelet level on 14 x 14 planes (13 or 14 rows / columns), four warps per plane set.
//
// The 7 x 7 sub-band planes of such a level are small enough for the register-resident
// convolution of wt2d_regplane.cuh, but the plane itself is not.  So the plane is split into
// its four polyphase components X[2i+di][2j+dj] (7 x 7 each): warp q = (di,dj) of a CTA owns
// component q for 32 consecutive channels (lanes), for one sample at a time.
//   phase 1  every warp loads its component (coalesced over channels) and publishes it in
//            shared memory, [component][position][lane]; the reconstruction of the deeper
//            levels is staged alongside, a quarter per warp;
//   phase 2  warp s forms sub-band s from the four components (wavelet.py:62-67: the 2x2
//            butterfly is a signed sum over components), convolves it in registers with its
//            scaled taps (wtconv2d.py:57-58; warp 0 adds the reconstruction of the deeper
//            levels, wtconv2d.py:71) and publishes the result;
//   phase 3  warp q forms component q of the reconstruction (wavelet.py:70-75, again a signed
//            sum), adds the base convolution of the plane for its component (wtconv2d.py:81-82)
//            and stores it to the layer output; without a base path the components are
//            gathered in shared memory and leave as whole (B,C,Hp,Wp) planes (phase 4).
// In component form a K x K 'same' convolution of the plane is a sum over the four source
// components of small convolutions with shifts -1, 0, +1; which tap belongs to a shift
// depends on the parity of the warp's own component, so the taps are fetched from shared
// memory with a computed index and shifts without a tap are skipped by a branch that is
// uniform over the warp.  One code path for all four warps keeps the kernel small enough
// for the instruction cache.
#pragma once

#include "wt2d_regplane.cuh"
#include "wt_common.h"

namespace wt {

constexpr int kQuadThreads = 128;
constexpr int kQuadP = 7;                          // component / sub-band size
constexpr int kQuadCells = kQuadP * kQuadP * 32;   // floats of one published component
// shared memory after the tap sets: XS (four components; reused as the planar output tile, whose
// planes are padded to an odd pitch), YS (four convolved sub-bands), RS (deeper reconstruction)
constexpr int kQuadXsFloats = 4 * kQuadCells + 64;
constexpr int kQuadSmemFloats = kQuadXsFloats + 4 * kQuadCells + kQuadCells;

struct QuadPlane {
  int B, C;
  int Hp, Wp;               // plane size (13 or 14 each)
  int K, lvl0;              // the level handled is lvl0 + 1 of the layer
  int has_base, has_rin;
  int wstride, wbeg, wlen, wpad;
  int samples_per_cta;
  int ngroups, nbatch;
  long long xs[4];          // strides (n,c,h,w) of the plane read (elements of its type)
  long long ys[4];          // has_base: strides of the layer output
  long long rs[4];          // strides of the fp32 reconstruction of the deeper levels (7 x 7)
};

// sign of component (py,px) in sub-band s, which is also the sign of sub-band s in component
// (py,px) of the synthesis (sub-band order LL, LH, HL, HH)
WT_HD float quad_sign(int s, int py, int px) {
  const bool neg = (s == 1 && py) || (s == 2 && px) || (s == 3 && (py != px));
  return neg ? -1.f : 1.f;
}

template <typename T, int K, bool BASE>
WT_HD void quad_cta(const QuadPlane& a, const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ rin,
                    float* __restrict__ rout, const float* __restrict__ packed, float* __restrict__ smem, int cg,
                    int nb) {
  constexpr int P = kQuadP;
  constexpr int TS = TapSet2d<K>::value;
  constexpr int r = K / 2;
  const int nthr = kQuadThreads;
  const int c0 = cg * 32;
  float* XS = smem + 32 * a.wpad;
  float* YS = XS + kQuadXsFloats;
  float* RS = YS + 4 * kQuadCells;

  WT_PHASE(nthr) {
    const int per = a.wlen / 4;
    for (int i = tid; i < 32 * per; i += nthr) {
      const int lc = i / per, k4 = i - lc * per;
      const int c = imin(c0 + lc, a.C - 1);
      async_copy16(smem + lc * a.wpad + 4 * k4, packed + (size_t)c * a.wstride + a.wbeg + 4 * k4);
    }
    async_wait_all();
  }

  for (int it = 0; it < a.samples_per_cta; ++it) {
    const int n = nb * a.samples_per_cta + it;
    if (n >= a.B) break;                            // uniform over the CTA

    // ---- phase 1: polyphase component of the plane -> XS
    WT_PHASE(nthr) {
      const int lane = tid & 31, q = tid >> 5;
      const int di = q >> 1, dj = q & 1;
      const int c = imin(c0 + lane, a.C - 1);
      const T* xp = x + (long long)n * a.xs[0] + (long long)c * a.xs[1];
      const int xs2 = (int)a.xs[2], xs3 = (int)a.xs[3];
      T raw[P][P];
      float* dst = XS + q * kQuadCells + lane;
      if (a.Hp == 2 * P && a.Wp == 2 * P) {
        // full 14 x 14 plane: no clamping, the component is a plain strided view
        const T* xq = xp + di * xs2 + dj * xs3;
        const int rs = 2 * xs2, cs = 2 * xs3;
#pragma unroll
        for (int i = 0; i < P; ++i)
#pragma unroll
          for (int j = 0; j < P; ++j) raw[i][j] = xq[i * rs + j * cs];
#pragma unroll
        for (int i = 0; i < P; ++i)
#pragma unroll
          for (int j = 0; j < P; ++j) dst[(i * P + j) * 32] = Elem<T>::to_f(raw[i][j]);
      } else {
#pragma unroll
        for (int i = 0; i < P; ++i)
#pragma unroll
          for (int j = 0; j < P; ++j)
            raw[i][j] = xp[imin(2 * i + di, a.Hp - 1) * xs2 + imin(2 * j + dj, a.Wp - 1) * xs3];
#pragma unroll
        for (int i = 0; i < P; ++i)
#pragma unroll
          for (int j = 0; j < P; ++j) {
            const bool ok = 2 * i + di < a.Hp && 2 * j + dj < a.Wp;     // zero extension of odd sizes
            dst[(i * P + j) * 32] = ok ? Elem<T>::to_f(raw[i][j]) : 0.f;
          }
      }
      if (a.has_rin) {
        const float* rp = rin + (long long)n * a.rs[0] + (long long)c * a.rs[1];
        const int rs2 = (int)a.rs[2], rs3 = (int)a.rs[3];
        for (int e = q; e < P * P; e += 4) RS[e * 32 + lane] = rp[(e / P) * rs2 + (e % P) * rs3];
      }
    }

    // ---- phase 2: sub-band s of warp s, its convolution -> YS
    WT_PHASE(nthr) {
      const int lane = tid & 31, s = tid >> 5;
      float S[P][P];
#pragma unroll
      for (int i = 0; i < P; ++i)
#pragma unroll
        for (int j = 0; j < P; ++j) S[i][j] = 0.f;
#pragma unroll 1                                   // rolled: four times less code to fetch
      for (int comp = 0; comp < 4; ++comp) {
        const float sg = quad_sign(s, comp >> 1, comp & 1);
        const float* src = XS + comp * kQuadCells + lane;
#pragma unroll
        for (int i = 0; i < P; ++i)
#pragma unroll
          for (int j = 0; j < P; ++j) S[i][j] = fmaf(sg, src[(i * P + j) * 32], S[i][j]);
      }
      float Y[P][P];
      if (s == 0 && a.has_rin) {
#pragma unroll
        for (int i = 0; i < P; ++i)
#pragma unroll
          for (int j = 0; j < P; ++j) Y[i][j] = RS[(i * P + j) * 32 + lane];
      } else {
#pragma unroll
        for (int i = 0; i < P; ++i)
#pragma unroll
          for (int j = 0; j < P; ++j) Y[i][j] = 0.f;
      }
      regplane_conv<K, P, P>(S, Y, smem + lane * a.wpad + (BASE ? TS : 0) + s * TS);
      float* dst = YS + s * kQuadCells + lane;
#pragma unroll
      for (int i = 0; i < P; ++i)
#pragma unroll
        for (int j = 0; j < P; ++j) dst[(i * P + j) * 32] = Y[i][j];
    }

    // ---- phase 3: component q of the output: synthesis (+ base convolution) -> global
    WT_PHASE(nthr) {
      const int lane = tid & 31, q = tid >> 5;
      const int di = q >> 1, dj = q & 1;
      const int c = c0 + lane;
      float acc[P][P];
      const float* w = smem + lane * a.wpad;
      if constexpr (BASE) {
        const float bias = w[K * K];
#pragma unroll
        for (int i = 0; i < P; ++i)
#pragma unroll
          for (int j = 0; j < P; ++j) acc[i][j] = bias;
        // source component (py,px), shifted by (su,sv): source pixel row 2(i+su)+py must equal
        // 2i+di+ky-r, i.e. ky = 2su + py - di + r (likewise kx); no such tap -> nothing to add
#pragma unroll 1
        for (int comp = 0; comp < 4; ++comp) {
          const int py = comp >> 1, px = comp & 1;
          const float* src = XS + comp * kQuadCells + lane;
          float V[P][P];
#pragma unroll
          for (int i = 0; i < P; ++i)
#pragma unroll
            for (int j = 0; j < P; ++j) V[i][j] = src[(i * P + j) * 32];
#pragma unroll
          for (int su = -1; su <= 1; ++su) {
            const int ky = 2 * su + py - di + r;
            const bool kyok = ky >= 0 && ky < K;
#pragma unroll
            for (int sv = -1; sv <= 1; ++sv) {
              const int kx = 2 * sv + px - dj + r;
              if (!(kyok && kx >= 0 && kx < K)) continue;       // uniform over the warp
              const float wv = w[ky * K + kx];
#pragma unroll
              for (int i = 0; i < P; ++i) {
                if (i + su < 0 || i + su >= P) continue;
#pragma unroll
                for (int j = 0; j < P; ++j) {
                  if (j + sv < 0 || j + sv >= P) continue;
                  acc[i][j] = fmaf(wv, V[i + su][j + sv], acc[i][j]);
                }
              }
            }
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < P; ++i)
#pragma unroll
          for (int j = 0; j < P; ++j) acc[i][j] = 0.f;
      }
#pragma unroll 1
      for (int s = 0; s < 4; ++s) {
        const float sg = quad_sign(s, di, dj);
        const float* src = YS + s * kQuadCells + lane;
#pragma unroll
        for (int i = 0; i < P; ++i)
#pragma unroll
          for (int j = 0; j < P; ++j) acc[i][j] = fmaf(sg, src[(i * P + j) * 32], acc[i][j]);
      }
      if (c < a.C) {
        if constexpr (BASE) {
          T* yp = y + (long long)n * a.ys[0] + (long long)c * a.ys[1];
          const int ys2 = (int)a.ys[2], ys3 = (int)a.ys[3];
          if (a.Hp == 2 * P && a.Wp == 2 * P) {
            T* yq = yp + di * ys2 + dj * ys3;
            const int rs = 2 * ys2, cs = 2 * ys3;
#pragma unroll
            for (int i = 0; i < P; ++i)
#pragma unroll
              for (int j = 0; j < P; ++j) yq[i * rs + j * cs] = Elem<T>::from_f(acc[i][j]);
          } else {
#pragma unroll
            for (int i = 0; i < P; ++i)
#pragma unroll
              for (int j = 0; j < P; ++j)
                if (2 * i + di < a.Hp && 2 * j + dj < a.Wp)
                  yp[(2 * i + di) * ys2 + (2 * j + dj) * ys3] = Elem<T>::from_f(acc[i][j]);
          }
        }
      }
      if constexpr (!BASE) {
        // XS is not read in this phase without a base path: gather the planes there
        float* tile = XS + lane * (a.Hp * a.Wp + 1);
#pragma unroll
        for (int i = 0; i < P; ++i)
#pragma unroll
          for (int j = 0; j < P; ++j)
            if (2 * i + di < a.Hp && 2 * j + dj < a.Wp) tile[(2 * i + di) * a.Wp + (2 * j + dj)] = acc[i][j];
      }
    }

    // ---- phase 4 (no base path): the planes of the 32 channels are contiguous in the
    //      (B,C,Hp,Wp) reconstruction array: one coalesced copy
    if constexpr (!BASE) {
      WT_PHASE(nthr) {
        const int hw = a.Hp * a.Wp;
        const int nch = imin(32, a.C - c0);
        float* dst = rout + ((long long)n * a.C + c0) * hw;
        for (int e = tid; e < nch * hw; e += nthr) {
          const int ch = e / hw;
          dst[e] = XS[ch * (hw + 1) + (e - ch * hw)];
        }
      }
    }
  }
}

}  // namespace wt
