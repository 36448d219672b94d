// Small helper kernels of the WTConv library: parameter folding and the
// low-pass plane reduction used by the multi-stage path for large planes.
#include "wt_aux.h"

namespace wt {

template <typename P>
__global__ void pack_params_kernel(PackArgs a, float* __restrict__ packed) {
  const long long total = (long long)a.C * a.tapset * (1 + a.subbands * a.L);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x)
    packed[i] = pack_value<P>(a, i);
}

cudaError_t launch_pack(const PackArgs& a, int param_dtype, float* packed, cudaStream_t stream) {
  const long long total = (long long)a.C * a.tapset * (1 + a.subbands * a.L);
  const int threads = 256;
  const long long want = (total + threads - 1) / threads;
  const int blocks = (int)(want > 1184 ? 1184 : want);
  switch (param_dtype) {
    case 0: pack_params_kernel<float><<<blocks, threads, 0, stream>>>(a, packed); break;
    case 1: pack_params_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(a, packed); break;
    default: pack_params_kernel<__half><<<blocks, threads, 0, stream>>>(a, packed); break;
  }
  return cudaGetLastError();
}

template <typename T>
__global__ void reduce_planes_kernel(const T* __restrict__ in, float* __restrict__ out, int B, int C, int Hin,
                                     int Win, int Hout, int Wout, int shift, long long s0, long long s1,
                                     long long s2, long long s3) {
  const long long total = (long long)B * C * Hout * Wout;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = reduce_value<T>(in, i, C, Hin, Win, Hout, Wout, shift, s0, s1, s2, s3);
}

cudaError_t launch_reduce(int dtype, const void* in, float* out, int B, int C, int Hin, int Win, int Hout,
                          int Wout, int shift, const long long* s, cudaStream_t stream) {
  const long long total = (long long)B * C * Hout * Wout;
  const int threads = 256;
  const long long want = (total + threads - 1) / threads;
  const int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
  switch (dtype) {
    case 0:
      reduce_planes_kernel<float><<<blocks, threads, 0, stream>>>(static_cast<const float*>(in), out, B, C, Hin, Win,
                                                                   Hout, Wout, shift, s[0], s[1], s[2], s[3]);
      break;
    case 1:
      reduce_planes_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(in), out, B, C, Hin, Win, Hout, Wout, shift, s[0], s[1], s[2], s[3]);
      break;
    default:
      reduce_planes_kernel<__half><<<blocks, threads, 0, stream>>>(static_cast<const __half*>(in), out, B, C, Hin, Win,
                                                                    Hout, Wout, shift, s[0], s[1], s[2], s[3]);
      break;
  }
  return cudaGetLastError();
}

}  // namespace wt
