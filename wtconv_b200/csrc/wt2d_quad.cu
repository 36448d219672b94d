// __global__ wrapper, instantiations and launcher of the four-warp 14 x 14 level kernel.
#include "wt2d_quad.cuh"
#include "wt_aux.h"

namespace wt {

template <typename T, int K, bool BASE>
__global__ void __launch_bounds__(kQuadThreads, 3)
wt2d_quad_kernel(const __grid_constant__ QuadPlane a, const T* __restrict__ x, T* __restrict__ y,
                 const float* __restrict__ rin, float* __restrict__ rout, const float* __restrict__ packed) {
  extern __shared__ __align__(16) float wt_smem[];
  quad_cta<T, K, BASE>(a, x, y, rin, rout, packed, wt_smem, blockIdx.x, blockIdx.y);
}

namespace {

template <typename T, bool BASE>
cudaError_t launch_inst(const QuadPlane& a, const void* x, void* y, const float* rin, float* rout,
                        const float* packed, size_t smem_bytes, cudaStream_t stream) {
  auto kern = wt2d_quad_kernel<T, 5, BASE>;
  static bool done[kMaxDevices] = {false};
  cudaError_t e = allow_full_smem(kern, done);
  if (e != cudaSuccess) return e;
  const dim3 blocks((unsigned)a.ngroups, (unsigned)a.nbatch);
  kern<<<blocks, kQuadThreads, smem_bytes, stream>>>(a, static_cast<const T*>(x), static_cast<T*>(y), rin, rout, packed);
  return cudaGetLastError();
}

}  // namespace

// `dtype` is the type of the plane read: the layer's with has_base, fp32 otherwise.
cudaError_t launch_quad(const QuadPlane& a, int dtype, const void* x, void* y, const float* rin, float* rout,
                        const float* packed, size_t smem_bytes, cudaStream_t stream) {
  if (a.K != 5) return cudaErrorInvalidValue;
  if (!a.has_base) {
    if (dtype != 0) return cudaErrorInvalidValue;
    return launch_inst<float, false>(a, x, nullptr, rin, rout, packed, smem_bytes, stream);
  }
  switch (dtype) {
    case 0: return launch_inst<float, true>(a, x, y, rin, rout, packed, smem_bytes, stream);
    case 1: return launch_inst<__nv_bfloat16, true>(a, x, y, rin, rout, packed, smem_bytes, stream);
    default: return launch_inst<__half, true>(a, x, y, rin, rout, packed, smem_bytes, stream);
  }
}

}  // namespace wt
