// Fused 2-D WTConv forward, kernel size 7 (all activation dtypes).
#include "wt2d_inst.cuh"
namespace wt {
template cudaError_t launch_wt2d_k<0>(const Plan2d&, int, const void*, void*, const float*, const float*, float*,
                                      size_t, cudaStream_t);
}
