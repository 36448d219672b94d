// __global__ wrapper and launcher of the fused 1-D kernel for one kernel size.
#pragma once

#include "wt1d_fused.cuh"

namespace wt {

template <typename T, int K>
__global__ void __launch_bounds__(256, 2)
wt1d_fused_kernel(const __grid_constant__ Plan1d p, const T* __restrict__ x, T* __restrict__ y,
                  const float* __restrict__ packed) {
  extern __shared__ __align__(16) float wt_smem[];
  wt1d_cta<T, K>(p, x, y, packed, wt_smem, blockIdx.x, blockIdx.y, blockIdx.z);
}

template <typename T, int K>
static cudaError_t launch_one_1d(const Plan1d& p, const void* x, void* y, const float* packed,
                                 size_t smem_bytes, cudaStream_t stream) {
  auto kern = wt1d_fused_kernel<T, K>;
  static bool done[kMaxDevices] = {false};
  cudaError_t e = allow_full_smem(kern, done);
  if (e != cudaSuccess) return e;
  const dim3 blocks((unsigned)p.ntile, (unsigned)p.ngroups, (unsigned)p.B);
  kern<<<blocks, p.nthreads, smem_bytes, stream>>>(p, static_cast<const T*>(x), static_cast<T*>(y), packed);
  return cudaGetLastError();
}

template <int K>
cudaError_t launch_wt1d_k(const Plan1d& p, int dtype, const void* x, void* y, const float* packed,
                          size_t smem_bytes, cudaStream_t stream) {
  switch (dtype) {
    case 0: return launch_one_1d<float, K>(p, x, y, packed, smem_bytes, stream);
    case 1: return launch_one_1d<__nv_bfloat16, K>(p, x, y, packed, smem_bytes, stream);
    default: return launch_one_1d<__half, K>(p, x, y, packed, smem_bytes, stream);
  }
}

}  // namespace wt
