// Register-resident WTConv1d forward for time-contiguous signals (sm_100a).
//
// Same arithmetic as the CTA-tile kernel of wt1d_fused.cuh (reference: wtconv/wtconv1d.py:38-87,
// wtconv/util/wavelet.py:46-59) for the common case: stride 1, at most four levels, samples of a
// row contiguous in memory.  Nothing but the staging of unaligned rows goes through shared memory:
//
//   * a thread owns 16 consecutive samples of one row (one channel of one sample), so the whole
//     analysis cascade of up to four levels (2-tap Haar steps, un-normalised: the tap magnitudes
//     are folded into the packed taps) is local to the thread;
//   * the K-tap sub-band convolutions and the base convolution need K/2 neighbours per side and
//     level: they come from the neighbouring lanes by warp shuffles;
//   * the low-pass accumulation (wtconv1d.py:71) and the synthesis are pointwise, hence local;
//   * a warp therefore handles 32 x 16 consecutive samples of which the outer HL lanes per side
//     only supply neighbours (HL = ceil((K/2) * 2^L / 16): two lanes for K = 5, L = 4); consecutive
//     warps of a row overlap by those lanes.  Samples outside the signal are zeros, which is both
//     the right-hand zero padding of odd lengths at every level (wtconv1d.py:49-51) and the
//     'same' padding of the convolutions;
//   * the taps of the row's channel are the same for the whole warp: it copies them (at most 18
//     128-bit words) into shared memory while its samples are on their way and reads them back
//     as broadcasts.
//
// Rows that start on a 16-byte boundary are read and written with 128-bit accesses (every byte of
// a touched sector is used by the same lane); other rows are staged through a 2.5 KB per-warp
// buffer with coalesced element-wise accesses.
#pragma once

#include "wt_common.h"

namespace wt {

constexpr int kWarp1dSpt = 16;        // samples per thread
constexpr int kWarp1dPitch = 20;      // floats between the runs of two threads in the staging buffer
constexpr int kWarp1dWarps = 8;       // warps per CTA
constexpr int kWarp1dMaxLevels = 4;   // 2^4 = samples per thread

struct Warp1dArgs {
  const void* x;
  void* y;
  const float* packed;
  int B, C, N;
  int wstride;            // floats per channel in the packed block
  int nseg;               // warps per row
  long long nwarps;       // rows * nseg
  long long xs0, xs1;     // element strides of sample and channel (time stride is 1)
  long long ys0, ys1;
};

#ifdef __CUDA_ARCH__
// ext[i] = value at position i - R of this thread's NJ positions, neighbours from the lanes beside it
template <int NJ, int R>
__device__ __forceinline__ void warp1d_extend(const float (&v)[NJ], float (&ext)[NJ + 2 * R]) {
  constexpr unsigned kFull = 0xffffffffu;
#pragma unroll
  for (int i = 0; i < NJ; ++i) ext[R + i] = v[i];
#pragma unroll
  for (int k = 1; k <= R; ++k) {
    const int dl = (k + NJ - 1) / NJ;                 // lanes to the left holding position -k
    ext[R - k] = __shfl_up_sync(kFull, v[NJ * dl - k], dl);
    const int pos = NJ - 1 + k, dr = pos / NJ;        // lanes to the right holding position NJ-1+k
    ext[R + pos] = __shfl_down_sync(kFull, v[pos - NJ * dr], dr);
  }
}

// acc[o] += sum_k w[k] * ext[o + k]
template <int NJ, int K>
__device__ __forceinline__ void warp1d_conv(const float (&ext)[NJ + K - 1], const float* __restrict__ taps, float (&acc)[NJ]) {
  constexpr int NW = (K + 3) / 4;                      // 128-bit words that hold the K taps
  float w[4 * NW];
#pragma unroll
  for (int v = 0; v < NW; ++v) {
    const float4 q = reinterpret_cast<const float4*>(taps)[v];
    w[4 * v] = q.x; w[4 * v + 1] = q.y; w[4 * v + 2] = q.z; w[4 * v + 3] = q.w;
  }
#pragma unroll
  for (int k = 0; k < K; ++k)
#pragma unroll
    for (int o = 0; o < NJ; ++o) acc[o] = fmaf(w[k], ext[o + k], acc[o]);
}

// Levels J..L from the low band of level J-1 (`src`, 2*NJ values per thread); returns the
// reconstruction R_{J-1} in `rec` (2*NJ values): conv(lo) + R_J and conv(hi), then synthesis.
template <int K, int L, int J, int NJ>
struct Warp1dLevel {
  static __device__ __forceinline__ void run(const float (&src)[2 * NJ], const float* __restrict__ wch, float (&rec)[2 * NJ]) {
    constexpr int R = K / 2;
    constexpr int TS = (K + 1 + 3) / 4 * 4;            // floats per tap set (tapset_floats(K, 1))
    float lo[NJ], hi[NJ];
#pragma unroll
    for (int o = 0; o < NJ; ++o) { lo[o] = src[2 * o] + src[2 * o + 1]; hi[o] = src[2 * o] - src[2 * o + 1]; }
    float alo[NJ], ahi[NJ];
    if constexpr (J < L) {
      Warp1dLevel<K, L, J + 1, NJ / 2>::run(lo, wch, alo);     // R_J joins the low-pass result
    } else {
#pragma unroll
      for (int o = 0; o < NJ; ++o) alo[o] = 0.f;
    }
#pragma unroll
    for (int o = 0; o < NJ; ++o) ahi[o] = 0.f;
    float ext[NJ + 2 * R];
    warp1d_extend<NJ, R>(lo, ext);
    warp1d_conv<NJ, K>(ext, wch + TS * (1 + 2 * (J - 1)), alo);
    warp1d_extend<NJ, R>(hi, ext);
    warp1d_conv<NJ, K>(ext, wch + TS * (2 + 2 * (J - 1)), ahi);
#pragma unroll
    for (int o = 0; o < NJ; ++o) { rec[2 * o] = alo[o] + ahi[o]; rec[2 * o + 1] = alo[o] - ahi[o]; }
  }
};
#endif

template <typename T, int K, int L>
__global__ void __launch_bounds__(kWarp1dWarps * 32)
wt1d_warp_kernel(const __grid_constant__ Warp1dArgs a) {
#ifdef __CUDA_ARCH__
  static_assert(L >= 0 && L <= kWarp1dMaxLevels && K <= 7, "levels beyond 2^L = 16 samples per thread take the CTA-tile kernel");
  constexpr int SPT = kWarp1dSpt, R = K / 2;
  constexpr int HL = (R * (1 << L) + SPT - 1) / SPT;   // neighbour-only lanes per side
  constexpr int SEG = (32 - 2 * HL) * SPT;             // output samples per warp
  constexpr int VEC = 16 / (int)sizeof(T);             // samples per 128-bit access
  constexpr int NCH = SPT / VEC;                       // 128-bit accesses per thread
  typedef typename RawChunk<16>::type raw_t;
  constexpr int TS = (K + 1 + 3) / 4 * 4;              // floats per tap set
  constexpr int NW4 = (1 + 2 * L) * TS / 4;            // 128-bit words of a channel's tap sets (<= 18)
  __shared__ __align__(16) float stage[kWarp1dWarps][32 * kWarp1dPitch];
  __shared__ __align__(16) float taps[kWarp1dWarps][NW4 * 4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* st = stage[warp];
  // (row, segment) of this warp; the launcher keeps the warp count below 2^31
  const unsigned wid = blockIdx.x * (unsigned)kWarp1dWarps + warp;
  if (wid >= (unsigned)a.nwarps) return;               // whole warps leave together
  const unsigned row = wid / (unsigned)a.nseg;
  const int seg = (int)(wid - row * (unsigned)a.nseg);
  const unsigned n = row / (unsigned)a.C, c = row - n * (unsigned)a.C;
  const T* xr = static_cast<const T*>(a.x) + n * a.xs0 + c * a.xs1;
  T* yr = static_cast<T*>(a.y) + n * a.ys0 + c * a.ys1;
  // tap sets of the row's channel: requested first, stored after the samples have been requested
  float4 wq = make_float4(0.f, 0.f, 0.f, 0.f);
  if (lane < NW4) wq = __ldg(reinterpret_cast<const float4*>(a.packed + (size_t)c * a.wstride) + lane);
  const float* wch = taps[warp];
  const int tw = seg * SEG - HL * SPT;                 // first sample of the warp: a multiple of 16, negative in a row's first segment
  const int t0 = tw + lane * SPT;                      // first sample of this thread

  // ---- load: 16 samples, zeros outside the signal
  float xv[SPT];
  if ((reinterpret_cast<uintptr_t>(xr) & 15) == 0) {   // warp-uniform
#pragma unroll
    for (int v = 0; v < NCH; ++v) {
      const int t = t0 + v * VEC;
      if (t >= 0 && t + VEC <= a.N) {
        Chunk<T, 16> ch;
        ch.raw = __ldg(reinterpret_cast<const raw_t*>(xr + t));
#pragma unroll
        for (int i = 0; i < VEC; ++i) xv[v * VEC + i] = Elem<T>::to_f(ch.get(i));
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) xv[v * VEC + i] = (t + i >= 0 && t + i < a.N) ? Elem<T>::to_f(xr[t + i]) : 0.f;
      }
    }
  } else {
    // coalesced element-wise loads of the warp's 512 samples into the staging buffer, then each
    // thread's run of 16 (runs are 20 floats apart: 128-bit reads without bank conflicts)
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
      const int idx = lane + 32 * k;
      const int t = tw + idx;
      st[idx + (idx >> 4) * 4] = (t >= 0 && t < a.N) ? Elem<T>::to_f(xr[t]) : 0.f;
    }
    __syncwarp();
#pragma unroll
    for (int v = 0; v < SPT / 4; ++v) {
      const float4 q = *reinterpret_cast<const float4*>(st + lane * kWarp1dPitch + 4 * v);
      xv[4 * v] = q.x; xv[4 * v + 1] = q.y; xv[4 * v + 2] = q.z; xv[4 * v + 3] = q.w;
    }
    __syncwarp();
  }

  if (lane < NW4) reinterpret_cast<float4*>(taps[warp])[lane] = wq;
  __syncwarp();

  // ---- levels, deepest first (recursion), then the base convolution and the bias
  float out[SPT];
  if constexpr (L >= 1) {
    Warp1dLevel<K, L, 1, SPT / 2>::run(xv, wch, out);
  } else {
#pragma unroll
    for (int o = 0; o < SPT; ++o) out[o] = 0.f;
  }
  {
    const float bias = wch[K];
#pragma unroll
    for (int o = 0; o < SPT; ++o) out[o] += bias;
    float ext[SPT + 2 * R];
    warp1d_extend<SPT, R>(xv, ext);
    warp1d_conv<SPT, K>(ext, wch, out);
  }

  // ---- store (crop to the signal: wtconv1d.py:76); the neighbour-only lanes store nothing
  const bool owner = lane >= HL && lane < 32 - HL;
  if ((reinterpret_cast<uintptr_t>(yr) & 15) == 0) {
    if (owner) {
#pragma unroll
      for (int v = 0; v < NCH; ++v) {
        const int t = t0 + v * VEC;
        if (t + VEC <= a.N) {
          Chunk<T, 16> ch;
#pragma unroll
          for (int i = 0; i < VEC; ++i) ch.set(i, Elem<T>::from_f(out[v * VEC + i]));
          *reinterpret_cast<raw_t*>(yr + t) = ch.raw;
        } else {
#pragma unroll
          for (int i = 0; i < VEC; ++i)
            if (t + i < a.N) yr[t + i] = Elem<T>::from_f(out[v * VEC + i]);
        }
      }
    }
  } else {
#pragma unroll
    for (int v = 0; v < SPT / 4; ++v)
      *reinterpret_cast<float4*>(st + lane * kWarp1dPitch + 4 * v) = make_float4(out[4 * v], out[4 * v + 1], out[4 * v + 2], out[4 * v + 3]);
    __syncwarp();
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
      const int idx = lane + 32 * k;
      const int t = tw + idx;
      if (idx >= HL * SPT && idx < (32 - HL) * SPT && t < a.N) yr[t] = Elem<T>::from_f(st[idx + (idx >> 4) * 4]);
    }
  }
#endif
}

// x, y: (B, C, N) with unit time stride; dtype 0 fp32, 1 bf16, 2 fp16.  Returns cudaErrorNotSupported
// for combinations this kernel does not cover (the caller then takes the CTA-tile kernel).
cudaError_t launch_wt1d_warp(const Warp1dArgs& a, int K, int L, int dtype, cudaStream_t stream);
inline bool wt1d_warp_supported(int K, int L, int stride, long long x_tstride, long long y_tstride) {
  return stride == 1 && L >= 0 && L <= kWarp1dMaxLevels && (K == 1 || K == 3 || K == 5 || K == 7) &&
         x_tstride == 1 && y_tstride == 1;
}

}  // namespace wt
