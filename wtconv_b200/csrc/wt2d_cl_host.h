// Launch description of the channels-last level stage (see wt2d_cl.cuh).
#pragma once

#include <cuda_runtime.h>

namespace wt {

struct ClStage {
  int B, C, H, W;        // input plane set of the level (channels-last)
  int K;
  int level;             // 0-based level inside the packed parameter block
  int has_base;          // 1: last stage of the layer (adds the base path, writes the layer output)
  int config;            // index into the compiled tile configurations
  int wstride, tapset;   // packed parameter layout: floats per channel / per tap set
  long long xs[4];       // input strides in elements: n, c (= 1), h, w
  long long rs[4];       // strides of the deeper reconstruction in floats: n, c, h, w
  long long os[4];       // output strides in elements: n, c (= 1), h, w
  int out_vec, rin_vec;  // channel pairs may be moved as one word
};

// dtype: 0 fp32, 1 bf16, 2 fp16 (type of the input plane set; the layer output has the same type)
cudaError_t launch_cl_level(const ClStage& s, int dtype, const void* x, const float* rin, void* out,
                            const float* packed, int* status, cudaStream_t stream);

}  // namespace wt
