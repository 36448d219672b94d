// Launch descriptions of the channels-last kernels (see wt2d_cl.cuh): plain data and the
// host-side geometry, usable without any CUDA device code.
#pragma once

#include <cuda_runtime.h>

namespace wt {

constexpr int kClGroup = 16;          // channels per plane slot
constexpr int kClLanes = 8;           // lanes (channel pairs) per thread tile
constexpr int kClRH = 2, kClCW = 4;   // sub-band positions per thread tile
constexpr int kClDeepMaxLev = 8;      // levels the deep stage can hold on chip
constexpr int kClDeepThreads = 256;    // eight warps; two CTAs share an SM when their frames fit

struct ClStage {
  int B, C, H, W;        // input plane set of the level (channels-last)
  int K;
  int level;             // 0-based level inside the packed parameter block
  int has_base;          // 1: last stage of the layer (adds the base path, writes the layer output)
  int config;            // index into the compiled tile configurations
  int nlevels;           // wavelet levels of the layer
  long long cl_off;      // floats from the packed block to its channels-last copy
  long long xs[4];       // input strides in elements: n, c (= 1), h, w
  long long rs[4];       // strides of the deeper reconstruction in floats: n, c, h, w
  long long os[4];       // output strides in elements: n, c (= 1), h, w
  int out_vec, rin_vec, x_vec;  // channel pairs of the output / reconstruction / input may be moved as one word
  float rin_scale;       // factor applied to the deeper reconstruction (1/2: it is at the reference's scale)
  int pdl;               // 1: the kernel that writes the reconstruction is the preceding launch of the stream:
                         // launch as its programmatic dependent (starts while that kernel drains)
};

// dtype: 0 fp32, 1 bf16, 2 fp16 (type of the input plane set; the layer output has the same type)
// has_base = 0: the output is an fp32 reconstruction for the next shallower level
cudaError_t launch_cl_level(const ClStage& s, int dtype, const void* x, const float* rin, void* out,
                            const float* packed, int* status, cudaStream_t stream);

// Deep stage (every level below the top one, whole planes on chip); also the kernel argument.
struct ClDeepArgs {
  int B, C, H, W;                 // layer input
  int nlev;                       // levels on chip (layer levels 2 .. nlev+1)
  int nlevels;                    // wavelet levels of the layer
  int lvl0;                       // layer levels above the plane set this stage starts from (0: the layer input)
  int ns;                         // plane slots per CTA
  int h[kClDeepMaxLev + 1];       // h[0], w[0]: plane of LL_1; h[j] = ceil(h[j-1]/2)
  int w[kClDeepMaxLev + 1];
  int srows[kClDeepMaxLev + 1];   // frame rows of S_j
  int spitch[kClDeepMaxLev + 1];  // positions per frame row of S_j
  int soff[kClDeepMaxLev + 1];    // byte offset of S_j (slot 0); slots are sslot[j] elements apart,
                                  // a frame is [row][position][sub-band][16 channels]
  int sslot[kClDeepMaxLev + 1];
  int roff[kClDeepMaxLev + 2];    // byte offset of R_j (j >= 2), rslot[j] floats per slot
  int rslot[kClDeepMaxLev + 2];
  int woff, bar_off;              // byte offsets: staged tap sets, barriers
  int zero_off, zero_bytes;       // region to clear before use (S_2 and deeper)
  int smem_bytes;                 // dynamic shared memory of the launch
  const float* packed;
  long long cl_off;               // floats from `packed` to the channels-last parameter copy
  float* rout;                    // (B, h[0], w[0], C) fp32
  int* status;
  int pdl;                        // 1: launched as a programmatic dependent of the pyramid kernel
};

// Fills the geometry of the deep stage for `ns` slots per CTA; returns the shared memory it
// needs in bytes, or -1 when the plane set cannot be handled.
inline long long plan_cl_deep(ClDeepArgs& a, int B, int C, int H, int W, int K, int L, int elem_size, int ns) {
  const int HS = K / 2;
  a.B = B; a.C = C; a.H = H; a.W = W; a.ns = ns; a.nlevels = L; a.lvl0 = 0; a.pdl = 0;
  a.nlev = L - 1;
  if (a.nlev < 1 || a.nlev > kClDeepMaxLev || ns > 64) return -1;
  a.h[0] = (H + 1) / 2; a.w[0] = (W + 1) / 2;
  for (int j = 1; j <= a.nlev; ++j) { a.h[j] = (a.h[j - 1] + 1) / 2; a.w[j] = (a.w[j - 1] + 1) / 2; }
  long long off = 0;
  for (int j = 0; j <= kClDeepMaxLev; ++j) { a.srows[j] = a.spitch[j] = a.soff[j] = a.sslot[j] = 0; }
  for (int j = 1; j <= a.nlev; ++j) {
    a.srows[j] = (a.h[j] + 1) / 2 * 2 + 2 * HS;
    a.spitch[j] = (a.w[j] + 3) / 4 * 4 + 2 * HS;
    a.sslot[j] = a.srows[j] * a.spitch[j] * 4 * kClGroup;
    a.soff[j] = (int)off;
    off += (long long)ns * a.sslot[j] * elem_size;
    off = (off + 127) / 128 * 128;
    if (j == 1) a.zero_off = (int)off;
  }
  if (a.srows[1] > 256 || a.spitch[1] > 256) return -1;     // one TMA box per slot
  a.zero_bytes = (int)off - a.zero_off;
  for (int j = 0; j <= kClDeepMaxLev + 1; ++j) { a.roff[j] = 0; a.rslot[j] = 0; }
  for (int j = 2; j <= a.nlev; ++j) {
    a.rslot[j] = a.h[j - 1] * a.w[j - 1] * kClGroup;
    a.roff[j] = (int)off;
    off += (long long)ns * a.rslot[j] * 4;
  }
  off = (off + 127) / 128 * 128;
  a.woff = (int)off;
  off += (long long)2 * (((4 * ((K * K + 1) * kClGroup * 4 + 64)) + 127) / 128 * 128);   // two buffers of four padded tap sets
  off = (off + 127) / 128 * 128;
  a.bar_off = (int)off;
  off += 128;
  off += 128;   // alignment slack
  if (off > (1LL << 30)) return -1;
  a.smem_bytes = (int)off;
  return off;
}

// s2: the second level's sub-bands from launch_cl_pyramid, (B, h[1], w[1], 4, C) in the layer's type
cudaError_t launch_cl_deep(const ClDeepArgs& a, int K, int dtype, const void* s2, const float* packed, float* rout,
                           int* status, cudaStream_t stream);

// plane set (channels-last, strides xs in elements) -> low-pass planes one (p1) and two (p2, may be
// null) levels down, dense channels-last in the same type
cudaError_t launch_cl_lowpass(int dtype, const void* x, const long long* xs, int x_vec, int B, int C, int H, int W,
                              void* p1, void* p2, cudaStream_t stream);

// x (channels-last, strides xs in elements) -> s2
cudaError_t launch_cl_pyramid(int dtype, const void* x, const long long* xs, int x_vec, int B, int C, int H, int W,
                              void* s2, cudaStream_t stream);

}  // namespace wt
