// Host side of the channels-last level stage: configuration table, tensor map, launch.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "wt2d_cl.cuh"
#include "wt2d_cl_host.h"

namespace wt {

namespace {

// Launch with or without the programmatic-dependent-launch attribute (the kernel then calls
// griddepcontrol.wait before it reads what the preceding kernel of the stream wrote)
template <typename Kern, typename... Args>
cudaError_t launch_maybe_dependent(Kern kern, dim3 grid, int threads, size_t smem, cudaStream_t stream, bool dependent,
                                   const Args&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point table (no link against libcuda)
EncodeTiledFn encode_tiled_fn() {
  static std::mutex mu;
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

template <typename T> struct TmaType;
template <> struct TmaType<float> { static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; };
template <> struct TmaType<__nv_bfloat16> { static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; };
template <> struct TmaType<__half> { static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; };

// Tensor map of a channels-last plane set (dimensions channel, column, row, sample) with the given box
template <typename T>
cudaError_t make_map(CUtensorMap& map, const void* x, int B, int C, int H, int W, const long long* xs, int box_w, int box_h) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return cudaErrorNotSupported;
  const cuuint64_t gdim[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)B};
  const cuuint64_t gstr[3] = {(cuuint64_t)xs[3] * sizeof(T), (cuuint64_t)xs[2] * sizeof(T), (cuuint64_t)xs[0] * sizeof(T)};
  const cuuint32_t box[4] = {(cuuint32_t)kClGroup, (cuuint32_t)box_w, (cuuint32_t)box_h, 1u};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(&map, TmaType<T>::v, 4, const_cast<void*>(x), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Tensor map of the second level's sub-bands, (B, h, w, 4, C): dimensions channel, sub-band, column,
// row, sample; one box covers the four sub-bands of a whole frame
template <typename T>
cudaError_t make_subband_map(CUtensorMap& map, const void* s2, int B, int C, int h, int w, int box_w, int box_h) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return cudaErrorNotSupported;
  const cuuint64_t gdim[5] = {(cuuint64_t)C, 4u, (cuuint64_t)w, (cuuint64_t)h, (cuuint64_t)B};
  const cuuint64_t gstr[4] = {(cuuint64_t)C * sizeof(T), (cuuint64_t)4 * C * sizeof(T), (cuuint64_t)w * 4 * C * sizeof(T),
                              (cuuint64_t)h * w * 4 * C * sizeof(T)};
  const cuuint32_t box[5] = {(cuuint32_t)kClGroup, 4u, (cuuint32_t)box_w, (cuuint32_t)box_h, 1u};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUresult r = enc(&map, TmaType<T>::v, 5, const_cast<void*>(s2), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

template <typename T, typename TO, int K, int NTY, int NTX, int NS, bool BASE, int MAXREG>
cudaError_t launch_cfg(const ClStage& s, const void* x, const float* rin, void* out, const float* packed, int* status,
                       cudaStream_t stream) {
  typedef ClGeo<T, K, NTY, NTX, NS> G;
  if constexpr (G::smem_bytes > (size_t)kMaxDynamicSmem) {
    return cudaErrorInvalidConfiguration;   // the planner never picks a configuration that does not fit
  } else {
  CUtensorMap map;
  cudaError_t me = make_map<T>(map, x, s.B, s.C, s.H, s.W, s.xs, G::XC, G::BOXR);
  if (me != cudaSuccess) return me;
  ClArgs a;
  a.B = s.B; a.C = s.C; a.H = s.H; a.W = s.W;
  a.Hh = (s.H + 1) / 2; a.Wh = (s.W + 1) / 2;
  a.nby = cdiv(a.Hh, NTY * kClRH);
  a.nbx = cdiv(a.Wh, NTX * kClCW);
  a.ngroups = cdiv(s.C, kClGroup);
  a.nslot_groups = cdiv(s.B, NS);
  a.packed = packed; a.cl_off = s.cl_off; a.nlevels = s.nlevels; a.level = s.level;
  a.rin = rin;
  a.out = out;
  for (int i = 0; i < 4; ++i) { a.rs[i] = s.rs[i]; a.os[i] = s.os[i]; }
  a.out_vec = s.out_vec; a.rin_vec = s.rin_vec; a.rin_scale = s.rin_scale;
  a.status = status;
  a.pdl = (s.pdl && rin) ? 1 : 0;

  auto kern = wt2d_cl_level_kernel<T, TO, K, NTY, NTX, NS, BASE, MAXREG>;
  constexpr size_t smem = G::smem_bytes;
  static bool done[kMaxDevices] = {false};
  cudaError_t e = allow_full_smem(kern, done);
  if (e != cudaSuccess) return e;
  if (a.nby * a.nbx > 65535) return cudaErrorInvalidConfiguration;   // grid.y carries the band (planes beyond about 3500 x 3500)
  const dim3 grid((unsigned)a.ngroups, (unsigned)(a.nby * a.nbx), (unsigned)a.nslot_groups);
  return launch_maybe_dependent(kern, grid, G::NT, smem, stream, a.pdl != 0, map, a);
  }
}

template <typename T, typename TO, int K, bool BASE>
cudaError_t launch_shape(const ClStage& s, const void* x, const float* rin, void* out, const float* packed,
                         int* status, cudaStream_t st) {
  switch (s.config) {
    case 0: return launch_cfg<T, TO, K, 4, 7, 1, BASE, 128>(s, x, rin, out, packed, status, st);
    case 1: return launch_cfg<T, TO, K, 7, 4, 1, BASE, 128>(s, x, rin, out, packed, status, st);
    case 2: return launch_cfg<T, TO, K, 4, 2, 2, BASE, 168>(s, x, rin, out, packed, status, st);
    default: return launch_cfg<T, TO, K, 2, 1, 4, BASE, 168>(s, x, rin, out, packed, status, st);
  }
}

template <typename T, int K>
cudaError_t launch_deep_t(const ClDeepArgs& a0, const void* s2, const float* packed, float* rout, int* status,
                          cudaStream_t stream) {
  CUtensorMap map;
  cudaError_t me = make_subband_map<T>(map, s2, a0.B, a0.C, a0.h[1], a0.w[1], a0.spitch[1], a0.srows[1]);
  if (me != cudaSuccess) return me;
  ClDeepArgs a = a0;
  a.packed = packed; a.rout = rout; a.status = status;
  auto kern = wt2d_cl_deep_kernel<T, K>;
  static bool done[kMaxDevices] = {false};
  cudaError_t e = allow_full_smem(kern, done);
  if (e != cudaSuccess) return e;
  const dim3 grid((unsigned)cdiv(a.C, kClGroup), (unsigned)cdiv(a.B, a.ns));
  return launch_maybe_dependent(kern, grid, kClDeepThreads, (size_t)a.smem_bytes, stream, a.pdl != 0, map, a);
}

template <typename T>
cudaError_t launch_pyramid_t(const void* x, const long long* xs, int x_vec, int B, int C, int H, int W, void* s2,
                             cudaStream_t stream) {
  ClPyramidArgs a;
  a.x = x;
  for (int i = 0; i < 4; ++i) a.xs[i] = xs[i];
  a.x_vec = x_vec;
  a.B = B; a.C = C; a.H = H; a.W = W;
  a.h2 = ((H + 1) / 2 + 1) / 2; a.w2 = ((W + 1) / 2 + 1) / 2;
  a.s2 = s2;
  // four channels per thread when the pixels allow 8- / 16-byte accesses (x_vec = 2), else pairs
  const bool quad = x_vec >= 2 && C % 4 == 0;
  a.total = (long long)B * a.h2 * a.w2 * (quad ? C / 4 : (C + 1) / 2);
  if (a.total >= (1LL << 31) - 148 * 64 * 256) return cudaErrorInvalidConfiguration;   // 32-bit item index in the kernel
  const long long want = (a.total + 255) / 256;
  const int blocks = (int)(want > 148 * 64 ? 148 * 64 : want);
  if (quad) wt2d_cl_pyramid4_kernel<T><<<blocks, 256, 0, stream>>>(a);
  else wt2d_cl_pyramid_kernel<T><<<blocks, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_lowpass_t(const void* x, const long long* xs, int x_vec, int B, int C, int H, int W, void* p1, void* p2,
                             cudaStream_t stream) {
  ClLowpassArgs a;
  a.x = x;
  for (int i = 0; i < 4; ++i) a.xs[i] = xs[i];
  a.x_vec = x_vec;
  a.B = B; a.C = C; a.H = H; a.W = W;
  a.h1 = (H + 1) / 2; a.w1 = (W + 1) / 2;
  a.h2 = (a.h1 + 1) / 2; a.w2 = (a.w1 + 1) / 2;
  a.p1 = p1; a.p2 = p2;
  const bool quad = x_vec >= 2 && C % 4 == 0;
  a.total = (long long)B * a.h2 * a.w2 * (quad ? C / 4 : (C + 1) / 2);
  if (a.total >= (1LL << 31) - 148 * 64 * 256) return cudaErrorInvalidConfiguration;   // 32-bit item index in the kernel
  const long long want = (a.total + 255) / 256;
  const int blocks = (int)(want > 148 * 64 ? 148 * 64 : want);
  if (quad) wt2d_cl_lowpass4_kernel<T><<<blocks, 256, 0, stream>>>(a);
  else wt2d_cl_lowpass_kernel<T><<<blocks, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_cl_lowpass(int dtype, const void* x, const long long* xs, int x_vec, int B, int C, int H, int W,
                              void* p1, void* p2, cudaStream_t st) {
  switch (dtype) {
    case 0: return launch_lowpass_t<float>(x, xs, x_vec, B, C, H, W, p1, p2, st);
    case 1: return launch_lowpass_t<__nv_bfloat16>(x, xs, x_vec, B, C, H, W, p1, p2, st);
    default: return launch_lowpass_t<__half>(x, xs, x_vec, B, C, H, W, p1, p2, st);
  }
}

cudaError_t launch_cl_pyramid(int dtype, const void* x, const long long* xs, int x_vec, int B, int C, int H, int W,
                              void* s2, cudaStream_t st) {
  switch (dtype) {
    case 0: return launch_pyramid_t<float>(x, xs, x_vec, B, C, H, W, s2, st);
    case 1: return launch_pyramid_t<__nv_bfloat16>(x, xs, x_vec, B, C, H, W, s2, st);
    default: return launch_pyramid_t<__half>(x, xs, x_vec, B, C, H, W, s2, st);
  }
}

cudaError_t launch_cl_deep(const ClDeepArgs& a, int K, int dtype, const void* s2, const float* packed, float* rout,
                           int* status, cudaStream_t st) {
  if (K != 5) return cudaErrorNotSupported;
  switch (dtype) {
    case 0: return launch_deep_t<float, 5>(a, s2, packed, rout, status, st);
    case 1: return launch_deep_t<__nv_bfloat16, 5>(a, s2, packed, rout, status, st);
    default: return launch_deep_t<__half, 5>(a, s2, packed, rout, status, st);
  }
}

cudaError_t launch_cl_level(const ClStage& s, int dtype, const void* x, const float* rin, void* out,
                            const float* packed, int* status, cudaStream_t st) {
  if (s.K != 5) return cudaErrorNotSupported;
  if (s.has_base) {
    switch (dtype) {
      case 0: return launch_shape<float, float, 5, true>(s, x, rin, out, packed, status, st);
      case 1: return launch_shape<__nv_bfloat16, __nv_bfloat16, 5, true>(s, x, rin, out, packed, status, st);
      default: return launch_shape<__half, __half, 5, true>(s, x, rin, out, packed, status, st);
    }
  }
  switch (dtype) {
    case 0: return launch_shape<float, float, 5, false>(s, x, rin, out, packed, status, st);
    case 1: return launch_shape<__nv_bfloat16, float, 5, false>(s, x, rin, out, packed, status, st);
    default: return launch_shape<__half, float, 5, false>(s, x, rin, out, packed, status, st);
  }
}

}  // namespace wt
