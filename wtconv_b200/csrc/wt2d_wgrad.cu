// __global__ wrappers and launchers of the parameter-gradient kernels (pyramid, correlation sums).
#include "wt2d_wgrad.cuh"
#include "wt_aux.h"

namespace wt {

template <typename T>
__global__ void __launch_bounds__(256)
wt2d_pyramid_kernel(const __grid_constant__ PyramidLevel a, const T* __restrict__ in, float* __restrict__ S) {
  const long long total = (long long)a.B * a.Hs * a.Ws * a.C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x)
    pyramid_item<T>(a, in, S, i);
}

template <typename T, int K>
__global__ void __launch_bounds__(kWgradThreads, 3)
wt2d_wgrad_kernel(const __grid_constant__ WGradSet a, const T* __restrict__ S, const T* __restrict__ G,
                  float* __restrict__ stat, long long sub_s, long long sub_g, long long sub_stat) {
  __shared__ float sm[kWgradWarps * (K * K + 1) * 32];
  // blockIdx.z: sub-band of the level (one set each)
  wgrad_cta<T, K>(a, S + blockIdx.z * sub_s, G + blockIdx.z * sub_g, stat + blockIdx.z * sub_stat, sm, blockIdx.x,
                  blockIdx.y);
}

cudaError_t launch_pyramid_level(const PyramidLevel& a, int dtype, const void* in, float* S, cudaStream_t stream) {
  const long long total = (long long)a.B * a.Hs * a.Ws * a.C;
  const int threads = 256;
  const long long want = (total + threads - 1) / threads;
  const int blocks = (int)(want > 148 * 32 ? 148 * 32 : (want < 1 ? 1 : want));
  switch (dtype) {
    case 0: wt2d_pyramid_kernel<float><<<blocks, threads, 0, stream>>>(a, static_cast<const float*>(in), S); break;
    case 1: wt2d_pyramid_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(a, static_cast<const __nv_bfloat16*>(in), S); break;
    default: wt2d_pyramid_kernel<__half><<<blocks, threads, 0, stream>>>(a, static_cast<const __half*>(in), S); break;
  }
  return cudaGetLastError();
}

namespace {

template <typename T, int K>
cudaError_t launch_wgrad_inst(const WGradSet& a, int nsub, const void* S, const void* G, float* stat, long long sub_s,
                              long long sub_g, long long sub_stat, cudaStream_t stream) {
  const dim3 blocks((unsigned)((a.C + 31) / 32), (unsigned)a.nsplit, (unsigned)nsub);
  wt2d_wgrad_kernel<T, K><<<blocks, kWgradThreads, 0, stream>>>(a, static_cast<const T*>(S), static_cast<const T*>(G),
                                                                stat, sub_s, sub_g, sub_stat);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_wgrad_t(const WGradSet& a, int K, int nsub, const void* S, const void* G, float* stat,
                           long long sub_s, long long sub_g, long long sub_stat, cudaStream_t stream) {
  switch (K) {
    case 1: return launch_wgrad_inst<T, 1>(a, nsub, S, G, stat, sub_s, sub_g, sub_stat, stream);
    case 3: return launch_wgrad_inst<T, 3>(a, nsub, S, G, stat, sub_s, sub_g, sub_stat, stream);
    case 5: return launch_wgrad_inst<T, 5>(a, nsub, S, G, stat, sub_s, sub_g, sub_stat, stream);
    case 7: return launch_wgrad_inst<T, 7>(a, nsub, S, G, stat, sub_s, sub_g, sub_stat, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

// `nsub` sets that share the geometry `a` (the four sub-bands of a level, or the base set alone);
// consecutive sets are sub_s / sub_g elements apart in S / G and sub_stat floats apart in stat.
cudaError_t launch_wgrad(const WGradSet& a, int K, int dtype, int nsub, const void* S, const void* G, float* stat,
                         long long sub_s, long long sub_g, long long sub_stat, cudaStream_t stream) {
  switch (dtype) {
    case 0: return launch_wgrad_t<float>(a, K, nsub, S, G, stat, sub_s, sub_g, sub_stat, stream);
    case 1: return launch_wgrad_t<__nv_bfloat16>(a, K, nsub, S, G, stat, sub_s, sub_g, sub_stat, stream);
    default: return launch_wgrad_t<__half>(a, K, nsub, S, G, stat, sub_s, sub_g, sub_stat, stream);
  }
}

}  // namespace wt
