// Shared host/device helpers of the WTConv kernels.
//
// The kernel bodies are written as sequences of "phases": inside a phase every
// thread of the CTA works independently, and a CTA-wide barrier separates two
// phases.  On the device WT_PHASE runs its body once for the calling thread and
// ends with __syncthreads(); compiled for the host (the test-only emulation
// library under tests/emu) the same macro becomes a loop over all thread ids,
// which executes the identical index arithmetic sequentially.  The product
// never uses the host form: the shared library built from this directory only
// launches the __global__ kernels.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define WT_HD __host__ __device__ __forceinline__
#else
#define WT_HD inline
#endif

#ifdef __CUDA_ARCH__
#define WT_PHASE(nthr) \
  for (int tid = threadIdx.x, wt_once_ = 1; wt_once_; wt_once_ = 0, __syncthreads())
#else
#define WT_PHASE(nthr) for (int tid = 0; tid < (nthr); ++tid)
#endif

namespace wt {

constexpr int kMaxFused = 8;    // wavelet levels one launch can fuse on chip
constexpr int kMaxLevels = 16;  // wt_levels accepted by the entry points
constexpr int kMaxK = 29;       // largest odd kernel size accepted (1, 3, 5, 7 are unrolled instances)

WT_HD int imin(int a, int b) { return a < b ? a : b; }
WT_HD int imax(int a, int b) { return a > b ? a : b; }
WT_HD int cdiv(int a, int b) { return (a + b - 1) / b; }
WT_HD int round_up(int a, int b) { return cdiv(a, b) * b; }
// log2 of the smallest power of two >= n, capped at 5 (one warp)
WT_HD int lane_shift(int n) {
  int s = 0;
  while (s < 5 && (1 << s) < n) ++s;
  return s;
}
// floor-mod for possibly negative a, positive b
WT_HD int pmod(int a, int b) { int m = a % b; return m < 0 ? m + b : m; }

// floats of one tap set in the packed parameter block: K^d taps + one slot
// (bias for the base set), rounded up to a 16-byte multiple.
WT_HD int tapset_floats(int K, int ndim) {
  int taps = (ndim == 2) ? K * K : K;
  return round_up(taps + 1, 4);
}
// floats per channel: base set, then `subbands` sets per level
WT_HD int packed_channel_floats(int K, int ndim, int L) {
  int sub = (ndim == 2) ? 4 : 2;
  return tapset_floats(K, ndim) * (1 + sub * L);
}

// 2-D packed blocks carry a second copy of every tap set for the channels-last kernels, laid out
// [channel group of 16][tap set][tap 0..K*K (last: bias slot)][16 channels] so that the sets one
// CTA needs are a single contiguous run.  It starts cl_param_offset() floats into the block.
WT_HD long long cl_param_offset(int C, int K, int L) {
  const long long n = (long long)C * packed_channel_floats(K, 2, L);
  return (n + 31) / 32 * 32;
}
WT_HD long long cl_param_floats(int C, int K, int L) {
  return (long long)cdiv(C, 16) * (1 + 4 * L) * (K * K + 1) * 16;
}

// 16-byte asynchronous copy global -> shared (cp.async, no register staging).  Both addresses
// must be 16-byte aligned.  async_wait_all() makes the calling thread's copies visible to it;
// the CTA barrier that ends the phase publishes them to the other threads.
WT_HD void async_copy16(void* smem_dst, const void* gmem_src) {
#ifdef __CUDA_ARCH__
  const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem_src) : "memory");
#else
  *static_cast<uint4*>(smem_dst) = *static_cast<const uint4*>(gmem_src);
#endif
}
// 4-byte asynchronous copy; when `valid` is false nothing is read and zero is written
WT_HD void async_copy4_zfill(void* smem_dst, const void* gmem_src, bool valid) {
#ifdef __CUDA_ARCH__
  const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  const int n = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(s), "l"(gmem_src), "r"(n) : "memory");
#else
  *static_cast<unsigned int*>(smem_dst) = valid ? *static_cast<const unsigned int*>(gmem_src) : 0u;
#endif
}
WT_HD void async_wait_all() {
#ifdef __CUDA_ARCH__
  asm volatile("cp.async.wait_all;" ::: "memory");
#endif
}

#if defined(__CUDACC__)
// Opt the kernel into the full dynamic shared memory of the SM once per device instead of on
// every launch (a driver call each time).  `done` is a per-kernel table owned by the caller.
constexpr int kMaxDevices = 64;
constexpr int kMaxDynamicSmem = 232448;   // 227 KB
template <typename Kern>
inline cudaError_t allow_full_smem(Kern kern, bool (&done)[kMaxDevices]) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  // the flag is read and written atomically: host threads may launch the same kernel concurrently
  // (setting the attribute twice is harmless)
  if (__atomic_load_n(&done[dev], __ATOMIC_ACQUIRE)) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem);
  if (e == cudaSuccess) __atomic_store_n(&done[dev], true, __ATOMIC_RELEASE);
  return e;
}
#endif

template <typename T> struct Elem;
template <> struct Elem<float> {
  static WT_HD float to_f(float v) { return v; }
  static WT_HD float from_f(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
  static WT_HD float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static WT_HD __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
  static WT_HD float to_f(__half v) { return __half2float(v); }
  static WT_HD __half from_f(float v) { return __float2half_rn(v); }
};

// CB-byte chunk (16, 8 or 4 bytes) of consecutive channels of one pixel
template <int CB> struct RawChunk;
template <> struct RawChunk<16> { typedef uint4 type; };
template <> struct RawChunk<8> { typedef uint2 type; };
template <> struct RawChunk<4> { typedef unsigned int type; };

template <typename T, int CB> struct Chunk {
  static constexpr int VEC = CB / (int)sizeof(T);
  union {                       // punning through a union: well defined for nvcc and gcc
    typename RawChunk<CB>::type raw;
    T e[VEC > 0 ? VEC : 1];
  };
  WT_HD Chunk() {}
  WT_HD T get(int i) const { return e[i]; }
  WT_HD void set(int i, T v) { e[i] = v; }
};

}  // namespace wt
