// __global__ wrapper, instantiations and launcher of the register-resident small-plane kernel.
#include "wt2d_regplane.cuh"
#include "wt_aux.h"

namespace wt {

template <typename T, int K, int PH, int PW, int NLEV, bool BASE>
__global__ void __launch_bounds__(kRegPlaneThreads, 3)
wt2d_regplane_kernel(const __grid_constant__ RegPlane a, const T* __restrict__ x, T* __restrict__ y,
                     float* __restrict__ rout, const float* __restrict__ packed) {
  extern __shared__ __align__(16) float wt_smem[];
  regplane_cta<T, K, PH, PW, NLEV, BASE>(a, x, y, rout, packed, wt_smem, blockIdx.x, blockIdx.y);
}

namespace {

template <typename T, int K, int PH, int PW, int NLEV, bool BASE>
cudaError_t launch_inst(const RegPlane& a, const void* x, void* y, float* rout, const float* packed,
                        size_t smem_bytes, cudaStream_t stream) {
  auto kern = wt2d_regplane_kernel<T, K, PH, PW, NLEV, BASE>;
  static bool done[kMaxDevices] = {false};
  cudaError_t e = allow_full_smem(kern, done);
  if (e != cudaSuccess) return e;
  const dim3 blocks((unsigned)a.ngroups, (unsigned)a.nbatch);
  kern<<<blocks, kRegPlaneThreads, smem_bytes, stream>>>(a, static_cast<const T*>(x), static_cast<T*>(y), rout, packed);
  return cudaGetLastError();
}

template <typename T, bool BASE>
cudaError_t launch_t(const RegPlane& a, const void* x, void* y, float* rout, const float* packed,
                     size_t smem_bytes, cudaStream_t stream) {
  switch (a.nlev) {
    case 1: return launch_inst<T, 5, 7, 7, 1, BASE>(a, x, y, rout, packed, smem_bytes, stream);
    case 2: return launch_inst<T, 5, 7, 7, 2, BASE>(a, x, y, rout, packed, smem_bytes, stream);
    case 3: return launch_inst<T, 5, 7, 7, 3, BASE>(a, x, y, rout, packed, smem_bytes, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

// `dtype` is the type of the tensor read: the layer's for a whole layer (has_base), fp32 planes
// otherwise.
cudaError_t launch_regplane(const RegPlane& a, int dtype, const void* x, void* y, float* rout,
                            const float* packed, size_t smem_bytes, cudaStream_t stream) {
  if (a.K != 5 || a.PH != 7 || a.PW != 7) return cudaErrorInvalidValue;
  if (!a.has_base) {
    if (dtype != 0) return cudaErrorInvalidValue;
    return launch_t<float, false>(a, x, y, rout, packed, smem_bytes, stream);
  }
  switch (dtype) {
    case 0: return launch_t<float, true>(a, x, y, rout, packed, smem_bytes, stream);
    case 1: return launch_t<__nv_bfloat16, true>(a, x, y, rout, packed, smem_bytes, stream);
    default: return launch_t<__half, true>(a, x, y, rout, packed, smem_bytes, stream);
  }
}

}  // namespace wt
