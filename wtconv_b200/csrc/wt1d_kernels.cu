// Fused 1-D WTConv forward, all compiled kernel sizes and activation dtypes.
#include "wt1d_inst.cuh"
namespace wt {
template cudaError_t launch_wt1d_k<1>(const Plan1d&, int, const void*, void*, const float*, size_t, cudaStream_t);
template cudaError_t launch_wt1d_k<3>(const Plan1d&, int, const void*, void*, const float*, size_t, cudaStream_t);
template cudaError_t launch_wt1d_k<5>(const Plan1d&, int, const void*, void*, const float*, size_t, cudaStream_t);
template cudaError_t launch_wt1d_k<7>(const Plan1d&, int, const void*, void*, const float*, size_t, cudaStream_t);
template cudaError_t launch_wt1d_k<0>(const Plan1d&, int, const void*, void*, const float*, size_t, cudaStream_t);   // run-time kernel size
}
