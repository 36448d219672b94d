// __global__ wrapper and launcher of the fused 2-D kernel for one kernel size.
// Each wt2d_k<K>.cu includes this file with WT_INST_K defined, so the sizes
// compile in parallel.
#pragma once

#include "wt2d_fused.cuh"

namespace wt {

// Last stage of a layer: x -> y, base convolution included.
template <typename T, int K>
__global__ void __launch_bounds__(256, 2)
wt2d_final_kernel(const __grid_constant__ Plan2d p, const T* __restrict__ x, T* __restrict__ y,
                  const float* __restrict__ packed, const float* __restrict__ rin) {
  extern __shared__ __align__(16) float wt_smem[];
  wt2d_cta<T, K, true>(p, x, y, packed, rin, nullptr, wt_smem, blockIdx.x, blockIdx.y % p.ntile_x,
                       blockIdx.y / p.ntile_x, blockIdx.z);
}

// Deep stage: reconstruction of the levels below a cut, written as fp32 planes.
template <typename T, int K>
__global__ void __launch_bounds__(256, 2)
wt2d_deep_kernel(const __grid_constant__ Plan2d p, const T* __restrict__ x, const float* __restrict__ packed,
                 const float* __restrict__ rin, float* __restrict__ rout) {
  extern __shared__ __align__(16) float wt_smem[];
  wt2d_cta<T, K, false>(p, x, nullptr, packed, rin, rout, wt_smem, blockIdx.x, blockIdx.y % p.ntile_x,
                        blockIdx.y / p.ntile_x, blockIdx.z);
}

template <typename T, int K>
static cudaError_t launch_one(const Plan2d& p, const void* x, void* y, const float* packed, const float* rin,
                              float* rout, size_t smem_bytes, cudaStream_t stream) {
  // grid: x = channel group (fastest: CTAs sharing the sectors of a channels-last pixel are
  // scheduled together), y = tile, z = sample
  const dim3 blocks((unsigned)p.ngroups, (unsigned)(p.ntile_x * p.ntile_y), (unsigned)p.B);
  if (p.has_base) {
    auto kern = wt2d_final_kernel<T, K>;
    static bool done[kMaxDevices] = {false};
    cudaError_t e = allow_full_smem(kern, done);
    if (e != cudaSuccess) return e;
    kern<<<blocks, p.nthreads, smem_bytes, stream>>>(p, static_cast<const T*>(x), static_cast<T*>(y),
                                                               packed, rin);
  } else {
    auto kern = wt2d_deep_kernel<T, K>;
    static bool done[kMaxDevices] = {false};
    cudaError_t e = allow_full_smem(kern, done);
    if (e != cudaSuccess) return e;
    kern<<<blocks, p.nthreads, smem_bytes, stream>>>(p, static_cast<const T*>(x), packed, rin, rout);
  }
  return cudaGetLastError();
}

template <int K>
cudaError_t launch_wt2d_k(const Plan2d& p, int dtype, const void* x, void* y, const float* packed,
                          const float* rin, float* rout, size_t smem_bytes, cudaStream_t stream) {
  switch (dtype) {
    case 0: return launch_one<float, K>(p, x, y, packed, rin, rout, smem_bytes, stream);
    case 1: return launch_one<__nv_bfloat16, K>(p, x, y, packed, rin, rout, smem_bytes, stream);
    default: return launch_one<__half, K>(p, x, y, packed, rin, rout, smem_bytes, stream);
  }
}

}  // namespace wt
