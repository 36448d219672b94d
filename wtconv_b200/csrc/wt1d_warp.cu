// Launcher of the register-resident 1-D kernel: every compiled (dtype, K, L) combination.
#include "wt1d_warp.cuh"

namespace wt {

namespace {

template <typename T, int K, int L>
cudaError_t launch_one(Warp1dArgs a, cudaStream_t stream) {
  constexpr int HL = ((K / 2) * (1 << L) + kWarp1dSpt - 1) / kWarp1dSpt;
  constexpr int SEG = (32 - 2 * HL) * kWarp1dSpt;
  a.nseg = cdiv(a.N, SEG);
  a.nwarps = (long long)a.B * a.C * a.nseg;
  if (a.nwarps >= (1LL << 31)) return cudaErrorNotSupported;     // 32-bit warp index in the kernel
  const long long blocks = (a.nwarps + kWarp1dWarps - 1) / kWarp1dWarps;
  wt1d_warp_kernel<T, K, L><<<(unsigned)blocks, kWarp1dWarps * 32, 0, stream>>>(a);
  return cudaGetLastError();
}

template <typename T, int K>
cudaError_t launch_levels(const Warp1dArgs& a, int L, cudaStream_t st) {
  switch (L) {
    case 0: return launch_one<T, K, 0>(a, st);
    case 1: return launch_one<T, K, 1>(a, st);
    case 2: return launch_one<T, K, 2>(a, st);
    case 3: return launch_one<T, K, 3>(a, st);
    case 4: return launch_one<T, K, 4>(a, st);
    default: return cudaErrorNotSupported;
  }
}

template <typename T>
cudaError_t launch_sizes(const Warp1dArgs& a, int K, int L, cudaStream_t st) {
  switch (K) {
    case 1: return launch_levels<T, 1>(a, L, st);
    case 3: return launch_levels<T, 3>(a, L, st);
    case 5: return launch_levels<T, 5>(a, L, st);
    case 7: return launch_levels<T, 7>(a, L, st);
    default: return cudaErrorNotSupported;
  }
}

}  // namespace

cudaError_t launch_wt1d_warp(const Warp1dArgs& a, int K, int L, int dtype, cudaStream_t stream) {
  switch (dtype) {
    case 0: return launch_sizes<float>(a, K, L, stream);
    case 1: return launch_sizes<__nv_bfloat16>(a, K, L, stream);
    default: return launch_sizes<__half>(a, K, L, stream);
  }
}

}  // namespace wt
