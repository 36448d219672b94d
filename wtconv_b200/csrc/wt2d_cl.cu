// Host side of the channels-last level stage: configuration table, tensor map, launch.
#include <cuda.h>

#include <mutex>

#include "wt2d_cl.cuh"
#include "wt2d_cl_host.h"

namespace wt {

namespace {

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

template <typename T, typename TO, int K, int NTY, int NTX, int NS, bool BASE, int MINB>
cudaError_t launch_cfg(const ClStage& s, const void* x, const float* rin, void* out, const float* packed, int* status,
                       cudaStream_t stream) {
  typedef ClGeo<T, K, NTY, NTX, NS> G;
  if constexpr (G::smem_bytes > (size_t)kMaxDynamicSmem) {
    return cudaErrorInvalidConfiguration;   // the planner never picks a configuration that does not fit
  } else {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return cudaErrorNotSupported;
  CUtensorMap map;
  const cuuint64_t gdim[4] = {(cuuint64_t)s.C, (cuuint64_t)s.W, (cuuint64_t)s.H, (cuuint64_t)s.B};
  const cuuint64_t gstr[3] = {(cuuint64_t)s.xs[3] * sizeof(T), (cuuint64_t)s.xs[2] * sizeof(T),
                              (cuuint64_t)s.xs[0] * sizeof(T)};
  const cuuint32_t box[4] = {(cuuint32_t)kClGroup, (cuuint32_t)G::XC, (cuuint32_t)2, (cuuint32_t)NS};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(&map, TmaType<T>::v, 4, const_cast<void*>(x), gdim, gstr, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;

  ClArgs a;
  a.B = s.B; a.C = s.C; a.H = s.H; a.W = s.W;
  a.Hh = (s.H + 1) / 2; a.Wh = (s.W + 1) / 2;
  a.nby = cdiv(a.Hh, NTY * kClRH);
  a.nbx = cdiv(a.Wh, NTX * kClCW);
  a.ngroups = cdiv(s.C, kClGroup);
  a.nslot_groups = cdiv(s.B, NS);
  a.packed = packed; a.wstride = s.wstride; a.tapset = s.tapset; a.level = s.level;
  a.rin = rin;
  a.out = out;
  for (int i = 0; i < 4; ++i) { a.rs[i] = s.rs[i]; a.os[i] = s.os[i]; }
  a.out_vec = s.out_vec; a.rin_vec = s.rin_vec;
  a.status = status;

  auto kern = wt2d_cl_level_kernel<T, TO, K, NTY, NTX, NS, BASE, MINB>;
  constexpr size_t smem = G::smem_bytes;
  static bool done[kMaxDevices] = {false};
  cudaError_t e = allow_full_smem(kern, done);
  if (e != cudaSuccess) return e;
  const dim3 grid((unsigned)(a.nby * a.nbx), (unsigned)a.ngroups, (unsigned)a.nslot_groups);
  kern<<<grid, G::NT, smem, stream>>>(map, a);
  return cudaGetLastError();
  }
}

template <typename T, typename TO, int K, bool BASE>
cudaError_t launch_shape(const ClStage& s, const void* x, const float* rin, void* out, const float* packed,
                         int* status, cudaStream_t st) {
  switch (s.config) {
    case 0: return launch_cfg<T, TO, K, 7, 7, 1, BASE, 1>(s, x, rin, out, packed, status, st);
    case 1: return launch_cfg<T, TO, K, 4, 7, 1, BASE, 2>(s, x, rin, out, packed, status, st);
    case 2: return launch_cfg<T, TO, K, 7, 4, 1, BASE, 2>(s, x, rin, out, packed, status, st);
    case 3: return launch_cfg<T, TO, K, 4, 2, 2, BASE, 2>(s, x, rin, out, packed, status, st);
    default: return launch_cfg<T, TO, K, 2, 1, 4, BASE, 2>(s, x, rin, out, packed, status, st);
  }
}

}  // namespace

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
  return cudaErrorNotSupported;
}

}  // namespace wt
