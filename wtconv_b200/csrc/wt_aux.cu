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
  if (a.cl_off > 0) {
    const long long ncl = (long long)cdiv(a.C, 16) * (1 + a.subbands * a.L) * (a.taps + 1) * 16;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < ncl;
         i += (long long)gridDim.x * blockDim.x)
      packed[a.cl_off + i] = pack_value_cl<P>(a, i);
  }
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

template <typename P>
__global__ void param_grads_kernel(GradArgs a) {
  const int nsub = (a.ndim == 2) ? 4 : 2;
  const long long total = (long long)(1 + nsub * a.L) * a.C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x)
    param_grad_item<P>(a, i);
}

cudaError_t launch_param_grads(const GradArgs& a, int param_dtype, cudaStream_t stream) {
  const int nsub = (a.ndim == 2) ? 4 : 2;
  const long long total = (long long)(1 + nsub * a.L) * a.C;
  const int threads = 128;
  const int blocks = (int)((total + threads - 1) / threads);
  switch (param_dtype) {
    case 0: param_grads_kernel<float><<<blocks, threads, 0, stream>>>(a); break;
    case 1: param_grads_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(a); break;
    default: param_grads_kernel<__half><<<blocks, threads, 0, stream>>>(a); break;
  }
  return cudaGetLastError();
}

template <typename T>
__global__ void reduce_planes_kernel(const T* __restrict__ in, float* __restrict__ out, int B, int C, int Hin,
                                     int Win, int Hout, int Wout, int shift, long long s0, long long s1,
                                     long long s2, long long s3, int out_cl) {
  const long long total = (long long)B * C * Hout * Wout;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x)
    out[out_cl ? reduce_cl_index(i, C, Hout, Wout) : i] =
        reduce_value<T>(in, i, C, Hin, Win, Hout, Wout, shift, s0, s1, s2, s3);
}

// Channels-last input: one thread sums the block for a 16-byte chunk of channels, so the
// loads of a warp cover whole pixels; same summation order as reduce_value.
template <typename T>
__global__ void reduce_planes_cl_kernel(const T* __restrict__ in, float* __restrict__ out, int B, int C, int Hin,
                                        int Win, int Hout, int Wout, int shift, long long s0, long long s2,
                                        long long s3, int out_cl) {
  constexpr int V = 16 / (int)sizeof(T);
  const int chunks = C / V;
  const int edge = 1 << shift;
  const long long total = (long long)B * Hout * Wout * chunks;
  const long long plane = (long long)Hout * Wout;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int ch = (int)(i % chunks);
    long long t = i / chunks;
    const int xo = (int)(t % Wout);
    t /= Wout;
    const int yo = (int)(t % Hout), n = (int)(t / Hout);
    const T* base = in + n * s0 + ch * V;
    const int ny = imin(edge, Hin - yo * edge), nx = imin(edge, Win - xo * edge);
    float acc[V];
#pragma unroll
    for (int e = 0; e < V; ++e) acc[e] = 0.f;
    for (int dy = 0; dy < ny; ++dy) {
      const T* row = base + (long long)(yo * edge + dy) * s2 + (long long)(xo * edge) * s3;
      float racc[V];
#pragma unroll
      for (int e = 0; e < V; ++e) racc[e] = 0.f;
#pragma unroll 4
      for (int dx = 0; dx < nx; ++dx) {
        Chunk<T, 16> c;
        c.raw = *reinterpret_cast<const uint4*>(row + dx * s3);
#pragma unroll
        for (int e = 0; e < V; ++e) racc[e] += Elem<T>::to_f(c.get(e));
      }
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] += racc[e];
    }
    if (out_cl) {       // V consecutive floats: 16-byte stores, coalesced over the chunks of a pixel
      float4* o = reinterpret_cast<float4*>(out + (((long long)n * Hout + yo) * Wout + xo) * C + ch * V);
#pragma unroll
      for (int e = 0; e < V; e += 4) o[e / 4] = make_float4(acc[e], acc[e + 1], acc[e + 2], acc[e + 3]);
    } else {
      float* o = out + ((long long)n * C + ch * V) * plane + (long long)yo * Wout + xo;
#pragma unroll
      for (int e = 0; e < V; ++e) o[e * plane] = acc[e];
    }
  }
}

template <typename T>
static bool reduce_cl_ok(const void* in, int C, const long long* s) {
  const int V = 16 / (int)sizeof(T);
  return s[1] == 1 && C % V == 0 && s[0] % V == 0 && s[2] % V == 0 && s[3] % V == 0 &&
         reinterpret_cast<uintptr_t>(in) % 16 == 0;
}

template <typename T>
static void launch_reduce_cl(const void* in, float* out, int B, int C, int Hin, int Win, int Hout, int Wout,
                             int shift, const long long* s, int out_cl, cudaStream_t stream) {
  const int V = 16 / (int)sizeof(T);
  const long long total = (long long)B * Hout * Wout * (C / V);
  const int threads = 256;
  const long long want = (total + threads - 1) / threads;
  const int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
  reduce_planes_cl_kernel<T><<<blocks, threads, 0, stream>>>(static_cast<const T*>(in), out, B, C, Hin, Win, Hout,
                                                              Wout, shift, s[0], s[2], s[3], out_cl);
}

cudaError_t launch_reduce(int dtype, const void* in, float* out, int B, int C, int Hin, int Win, int Hout,
                          int Wout, int shift, const long long* s, int out_cl, cudaStream_t stream) {
  if (dtype == 0 && reduce_cl_ok<float>(in, C, s)) {
    launch_reduce_cl<float>(in, out, B, C, Hin, Win, Hout, Wout, shift, s, out_cl, stream);
    return cudaGetLastError();
  }
  if (dtype == 1 && reduce_cl_ok<__nv_bfloat16>(in, C, s)) {
    launch_reduce_cl<__nv_bfloat16>(in, out, B, C, Hin, Win, Hout, Wout, shift, s, out_cl, stream);
    return cudaGetLastError();
  }
  if (dtype == 2 && reduce_cl_ok<__half>(in, C, s)) {
    launch_reduce_cl<__half>(in, out, B, C, Hin, Win, Hout, Wout, shift, s, out_cl, stream);
    return cudaGetLastError();
  }
  const long long total = (long long)B * C * Hout * Wout;
  const int threads = 256;
  const long long want = (total + threads - 1) / threads;
  const int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
  switch (dtype) {
    case 0:
      reduce_planes_kernel<float><<<blocks, threads, 0, stream>>>(static_cast<const float*>(in), out, B, C, Hin, Win,
                                                                   Hout, Wout, shift, s[0], s[1], s[2], s[3], out_cl);
      break;
    case 1:
      reduce_planes_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(in), out, B, C, Hin, Win, Hout, Wout, shift, s[0], s[1], s[2], s[3], out_cl);
      break;
    default:
      reduce_planes_kernel<__half><<<blocks, threads, 0, stream>>>(static_cast<const __half*>(in), out, B, C, Hin, Win,
                                                                    Hout, Wout, shift, s[0], s[1], s[2], s[3], out_cl);
      break;
  }
  return cudaGetLastError();
}

}  // namespace wt
