// Channels-last level stage of the 2-D WTConv forward for sm_100a.
//
// One launch computes one wavelet level of wtconv/wtconv2d.py:46-78 on a channels-last
// plane set, optionally together with the base path of :81-82:
//
//   out = IWT( conv_s(WT(in)) * scale_s  +  [LL slot: reconstruction of the deeper levels] )
//         [+ base_scale * (base_conv(in) + bias)]
//
// Lanes are channels.  A CTA owns NS plane slots (sample, 16-channel group, band of
// NTY x NTX thread tiles); a thread owns one channel pair of one thread tile (2 x 4
// sub-band positions = 4 x 8 pixels), so every multiply-add is a packed fma.rn.f32x2
// over the pair, pixels of a tile are never exchanged between lanes, and the eight
// lanes of a tile read or write 32 (16-bit) or 64 (fp32) contiguous bytes of a
// pixel.
//
// Data flow of a CTA:
//   1. the input frame (band + halo of 2*(K/2) pixels, zero outside the plane: TMA
//      out-of-bounds fill reproduces both the odd-size padding of wtconv2d.py:49-51
//      and the 'same' padding of every convolution) arrives through a ring of
//      cp.async.bulk.tensor chunks of four pixel rows, each completing on an mbarrier;
//   2. every chunk is turned into one row of the four un-normalised Haar sub-bands
//      (wavelet.py:62-67 without the tap magnitude, which the packed parameters
//      carry) and, for the base path, copied pixel by pixel; both arrays are kept in
//      the tensor's own type (the reference rounds its sub-bands to that type as
//      well) in a rotated layout that keeps the shared-memory reads of the tiles of
//      one wavefront in different banks (cl_swizzle);
//   3. each thread runs the four K x K sub-band convolutions of its tile, adds the
//      deeper reconstruction to the low-pass result, applies the synthesis butterfly
//      (wavelet.py:70-75) in registers, accumulates the base convolution and bias
//      and stores its pixels.  All arithmetic is fp32.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "wt_common.h"

namespace wt {

constexpr int kClGroup = 16;          // channels per plane slot
constexpr int kClLanes = 8;           // lanes (channel pairs) per thread tile
constexpr int kClRH = 2, kClCW = 4;   // sub-band positions per thread tile
constexpr int kClStages = 3;          // TMA chunks in flight
constexpr unsigned kClWaitSpins = 1u << 22;   // bound of every mbarrier wait

struct ClArgs {
  int B, C, H, W;          // input plane set of this level
  int Hh, Wh;              // sub-band planes: ceil(H/2), ceil(W/2)
  int nby, nbx;            // bands per plane
  int ngroups;             // channel groups of 16
  int nslot_groups;        // ceil(B / NS)
  const float* packed;     // folded parameters (wtconv_pack_params layout)
  int wstride;             // floats per channel
  int tapset;              // floats per tap set
  int level;               // 0-based level of this stage inside the packed block
  const float* rin;        // deeper reconstruction (fp32), may be null
  long long rs[4];         // its strides in floats: n, c, h, w
  void* out;               // output tensor
  long long os[4];         // its strides in elements: n, c, h, w
  int out_vec;             // 1: channel pairs may be stored as one word
  int rin_vec;             // 1: channel pairs of rin may be loaded as one 8-byte word
  int* status;             // device word that receives a nonzero code when a wait gives up
};

// ---------------------------------------------------------------------------
// small device helpers
// ---------------------------------------------------------------------------
#ifdef __CUDA_ARCH__
__device__ __forceinline__ float2 cl_fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 cl_add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 cl_sub2(float2 a, float2 b) { return __ffma2_rn(b, make_float2(-1.f, -1.f), a); }

__device__ __forceinline__ unsigned cl_smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cl_mbar_init(void* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(cl_smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void cl_mbar_expect_tx(void* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(cl_smem_addr(bar)), "r"(bytes) : "memory");
}
// Bounded wait: returns false when the phase did not complete within the spin limit.
__device__ __forceinline__ bool cl_mbar_wait(void* bar, unsigned parity) {
  const unsigned addr = cl_smem_addr(bar);
  for (unsigned spin = 0; spin < kClWaitSpins; ++spin) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// 4-D tiled TMA load (channel, column, row, sample) -> shared memory, completing on `bar`
__device__ __forceinline__ void cl_tma_load4(void* dst, const CUtensorMap* map, void* bar, int c, int x, int y, int n) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(cl_smem_addr(dst)), "l"(map), "r"(cl_smem_addr(bar)), "r"(c), "r"(x), "r"(y), "r"(n)
      : "memory");
}

// channel pair of a staged pixel -> fp32 pair
template <typename T> struct ClPair;
template <> struct ClPair<float> {
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void store(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
};
template <> struct ClPair<__nv_bfloat16> {
  static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
    const unsigned u = *reinterpret_cast<const unsigned*>(p);
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float2 v) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __float22bfloat162_rn(v);
  }
};
template <> struct ClPair<__half> {
  static __device__ __forceinline__ float2 load(const __half* p) {
    return __half22float2(*reinterpret_cast<const __half2*>(p));
  }
  static __device__ __forceinline__ void store(__half* p, float2 v) {
    *reinterpret_cast<__half2*>(p) = __float22half2_rn(v);
  }
};
#endif

// Compile-time geometry of one kernel configuration (T: type of the planes kept in shared memory)
template <typename T, int K, int NTY, int NTX, int NS>
struct ClGeo {
  static constexpr int HS = K / 2;                          // halo of a K x K window
  static constexpr int SR = NTY * kClRH + 2 * HS;           // sub-band frame rows
  static constexpr int SC = ((NTX * kClCW + 2 * HS + 3) / 4) * 4;   // sub-band frame columns (whole rotation groups)
  static constexpr int XR = 2 * SR, XC = 2 * SC;            // pixel frame delivered by the TMA chunks
  static constexpr int XRA = XR - 2 * HS;                   // pixel rows kept for the base convolution (frame rows HS..)
  static constexpr int NCHUNK = SR;                         // one sub-band row (two pixel rows) per chunk
  static constexpr int NT = NTY * NTX * NS * kClLanes;      // threads per CTA
  static constexpr int TAPS = K * K + 1;                    // staged floats per tap set and channel (last: bias slot)
  static constexpr int PX = kClGroup;                       // elements of T per pixel
  static constexpr int SL = 128 / (kClGroup * (int)sizeof(T));   // pixels per 128-byte line
  static constexpr int SUB = SR * SC * PX;                  // elements per sub-band of a slot
  static constexpr int SLOT_S = 4 * SUB;
  static constexpr int SLOT_X = XRA * XC * PX;
  static constexpr size_t s_bytes = (size_t)NS * SLOT_S * sizeof(T);
  static constexpr size_t x_bytes = (size_t)NS * SLOT_X * sizeof(T);
  static constexpr size_t w_bytes = (size_t)5 * TAPS * kClLanes * sizeof(float2);
  static constexpr size_t chunk_elems = (size_t)NS * 2 * XC * kClGroup;
  static constexpr size_t stage_bytes = ((chunk_elems * sizeof(T) + 127) / 128) * 128;
  static constexpr size_t smem_bytes =
      128 /* alignment slack */ + s_bytes + x_bytes + w_bytes + kClStages * stage_bytes + 64 /* barriers */;
};

// Rotation swizzle.  A pixel (16 channels) takes 128/SL bytes; the SL thread tiles served by one
// 128-byte wavefront are consecutive tiles q = ty*NTX + tx of the CTA and all read the same window
// element.  Storing column f of row r at
//     (f & ~(SL-1)) + (((f & (SL-1)) + tile_column(f) + NTX * tile_row(r)) & (SL-1))
// rotates every line by the index of the tile it belongs to, so those SL reads fall into
// different bank groups; for a reader the rotation is (compile-time part + q) & (SL-1), i.e. one
// of SL per-thread base pointers plus a compile-time offset.
template <int SL, int NTX, int TWSH, int TRSH>
WT_HD int cl_swizzle(int r, int f) {
  const int rot = ((f >> TWSH) + NTX * (r >> TRSH)) & (SL - 1);
  return (f & ~(SL - 1)) + (((f & (SL - 1)) + rot) & (SL - 1));
}

#ifdef __CUDA_ARCH__
// acc[oy][ox] += sum_{dy,dx} w[dy][dx] * S(oy+dy, ox+dx) for one sub-band of the thread's window.
// p[v]: base pointers of the window (channel pair included) for rotation class v.
template <typename T, int K, int SC, int SL, int NTX>
__device__ __forceinline__ void cl_subband_conv(float2 (&acc)[kClRH][kClCW], const T* const (&p)[SL],
                                                const float2* __restrict__ w) {
  float2 wr[K * K];
#pragma unroll
  for (int t = 0; t < K * K; ++t) wr[t] = w[t * kClLanes];
#pragma unroll
  for (int iy = 0; iy < kClRH + K - 1; ++iy) {
    asm volatile("" ::: "memory");   // keeps the loads of one window row together (bounds register pressure)
    float2 in[kClCW + K - 1];
#pragma unroll
    for (int c = 0; c < kClCW + K - 1; ++c) {
      const int v = ((c & (SL - 1)) + (c >> 2) + NTX * (iy >> 1)) & (SL - 1);
      in[c] = ClPair<T>::load(p[v] + (iy * SC + (c & ~(SL - 1))) * kClGroup);
    }
#pragma unroll
    for (int dy = 0; dy < K; ++dy) {
      const int oy = iy - dy;
      if (oy >= 0 && oy < kClRH) {
#pragma unroll
        for (int dx = 0; dx < K; ++dx)
#pragma unroll
          for (int ox = 0; ox < kClCW; ++ox) acc[oy][ox] = cl_fma2(in[ox + dx], wr[dy * K + dx], acc[oy][ox]);
      }
    }
  }
}

// Base convolution of the 4 x 8 pixel tile from the pixel copy; the window starts HS pixels
// inside the frame, which the compile-time part of the rotation accounts for.
template <typename T, int K, int XC, int SL, int NTX>
__device__ __forceinline__ void cl_base_conv(float2 (&out)[2 * kClRH][2 * kClCW], const T* const (&p)[SL],
                                             const float2* __restrict__ w) {
  constexpr int HS = K / 2;
  float2 wr[K * K];
#pragma unroll
  for (int t = 0; t < K * K; ++t) wr[t] = w[t * kClLanes];
#pragma unroll
  for (int iy = 0; iy < 2 * kClRH + K - 1; ++iy) {
    asm volatile("" ::: "memory");
    float2 in[2 * kClCW + K - 1];
#pragma unroll
    for (int c = 0; c < 2 * kClCW + K - 1; ++c) {
      const int hc = HS + c, hd = HS + iy;
      const int v = ((hc & (SL - 1)) + (hc >> 3) + NTX * (hd >> 2)) & (SL - 1);
      in[c] = ClPair<T>::load(p[v] + (iy * XC + (hc & ~(SL - 1))) * kClGroup);
    }
#pragma unroll
    for (int dy = 0; dy < K; ++dy) {
      const int oy = iy - dy;
      if (oy >= 0 && oy < 2 * kClRH) {
#pragma unroll
        for (int dx = 0; dx < K; ++dx)
#pragma unroll
          for (int ox = 0; ox < 2 * kClCW; ++ox) out[oy][ox] = cl_fma2(in[ox + dx], wr[dy * K + dx], out[oy][ox]);
      }
    }
  }
}
#endif

// T: type of the input plane set (and of the copies in shared memory); TO: type of the output (T
// for the layer output, float for a reconstruction handed to the next shallower level); BASE: add
// the base path.
template <typename T, typename TO, int K, int NTY, int NTX, int NS, bool BASE, int MINB>
__global__ void __launch_bounds__(NTY* NTX* NS* kClLanes, MINB)
wt2d_cl_level_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ ClArgs a) {
#ifdef __CUDA_ARCH__
  typedef ClGeo<T, K, NTY, NTX, NS> G;
  constexpr int SC = G::SC, HS = G::HS, SL = G::SL, XC = G::XC;
  static_assert(kClRH == 2 && kClCW == 4, "the swizzle assumes 2 x 4 thread tiles");
  extern __shared__ unsigned char cl_smem_raw[];
  unsigned char* sm = cl_smem_raw + ((128u - (cl_smem_addr(cl_smem_raw) & 127u)) & 127u);
  T* S = reinterpret_cast<T*>(sm);
  T* XT = reinterpret_cast<T*>(sm + G::s_bytes);
  float2* Wsm = reinterpret_cast<float2*>(sm + G::s_bytes + G::x_bytes);
  unsigned char* stage0 = sm + G::s_bytes + G::x_bytes + G::w_bytes;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(stage0 + kClStages * G::stage_bytes);

  const int tid = threadIdx.x;
  // grid: x = band (column band fastest), y = channel group, z = slot group
  const int band = blockIdx.x;
  const int bx = band % a.nbx, by = band / a.nbx;
  const int c0 = blockIdx.y * kClGroup;
  const int n0 = blockIdx.z * NS;
  const int i0 = by * NTY * kClRH, j0 = bx * NTX * kClCW;    // first sub-band position of the band
  const int X0 = 2 * (j0 - HS), Y0 = 2 * (i0 - HS);          // pixel frame origin (may be negative)

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kClStages; ++s) cl_mbar_init(&bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  constexpr unsigned kChunkBytes = (unsigned)(G::chunk_elems * sizeof(T));
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kClStages; ++s) {
      if (s < G::NCHUNK) {
        cl_mbar_expect_tx(&bars[s], kChunkBytes);
        cl_tma_load4(stage0 + s * G::stage_bytes, &xmap, &bars[s], c0, X0, Y0 + 2 * s, n0);
      }
    }
  }
  // tap sets of this stage: [set][tap][channel] as fp32; set 0 = base (taps, bias), 1..4 = sub-bands
  {
    const int ts = a.tapset;
    for (int i = tid; i < 5 * G::TAPS * kClGroup; i += G::NT) {
      const int ch = i % kClGroup;
      const int t = (i / kClGroup) % G::TAPS;
      const int set = i / (kClGroup * G::TAPS);
      float v = 0.f;
      if (c0 + ch < a.C) {
        const float* pc = a.packed + (size_t)(c0 + ch) * a.wstride;
        if (set == 0) {
          if (BASE) v = pc[t];                 // taps 0..K*K-1, bias in slot K*K
        } else if (t < K * K) {
          v = pc[ts * (1 + 4 * a.level + (set - 1)) + t];
        }
      }
      reinterpret_cast<float*>(Wsm)[(set * G::TAPS + t) * kClGroup + ch] = v;
    }
  }

  // ---- pass 1: every chunk (two pixel rows) -> one row of the four sub-bands + the pixel copy
  bool ok = true;
#pragma unroll 1
  for (int k = 0; k < G::NCHUNK; ++k) {
    const int st = k % kClStages;
    ok = cl_mbar_wait(&bars[st], (unsigned)((k / kClStages) & 1)) && ok;
    const T* xs = reinterpret_cast<const T*>(stage0 + st * G::stage_bytes);
    constexpr int ITEMS = NS * SC * kClLanes;
    for (int it = tid; it < ITEMS; it += G::NT) {
      const int cp = it & (kClLanes - 1);
      const int blk = it >> 3;
      const int f = blk % SC;
      const int slot = blk / SC;
      // staged box: [slot][row 0..1][column][16 channels]
      const T* px = xs + (((size_t)slot * 2) * XC + 2 * f) * kClGroup + 2 * cp;
      const float2 va = ClPair<T>::load(px), vb = ClPair<T>::load(px + kClGroup);
      const float2 vc = ClPair<T>::load(px + XC * kClGroup), vd = ClPair<T>::load(px + XC * kClGroup + kClGroup);
      const float2 pp = cl_add2(va, vb), qq = cl_sub2(va, vb), uu = cl_add2(vc, vd), vv = cl_sub2(vc, vd);
      T* d = S + (size_t)slot * G::SLOT_S + ((size_t)k * SC + cl_swizzle<SL, NTX, 2, 1>(k, f)) * kClGroup + 2 * cp;
      ClPair<T>::store(d, cl_add2(pp, uu));               // LL = a+b+c+d
      ClPair<T>::store(d + G::SUB, cl_sub2(pp, uu));      // LH = a+b-c-d
      ClPair<T>::store(d + 2 * G::SUB, cl_add2(qq, vv));  // HL = a-b+c-d
      ClPair<T>::store(d + 3 * G::SUB, cl_sub2(qq, vv));  // HH = a-b-c+d
      if (BASE) {
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const int fr = 2 * k + rr;                       // frame row of this pixel row
          const int ra = fr - HS;                          // row of the pixel copy
          if (ra >= 0 && ra < G::XRA) {
            T* xr = XT + (size_t)slot * G::SLOT_X + (size_t)ra * XC * kClGroup + 2 * cp;
            ClPair<T>::store(xr + cl_swizzle<SL, NTX, 3, 2>(fr, 2 * f) * kClGroup, rr ? vc : va);
            ClPair<T>::store(xr + cl_swizzle<SL, NTX, 3, 2>(fr, 2 * f + 1) * kClGroup, rr ? vd : vb);
          }
        }
      }
    }
    __syncthreads();
    if (tid == 0 && k + kClStages < G::NCHUNK) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the chunk was read through the generic proxy
      cl_mbar_expect_tx(&bars[st], kChunkBytes);
      cl_tma_load4(stage0 + st * G::stage_bytes, &xmap, &bars[st], c0, X0, Y0 + 2 * (k + kClStages), n0);
    }
  }
  if (!ok && a.status) atomicExch(a.status, 1);

  // ---- pass 2: per-thread tile
  const int cp = tid & (kClLanes - 1);
  const int q = tid >> 3;
  const int slot = q / (NTY * NTX);
  const int rem = q - slot * (NTY * NTX);
  const int ty = rem / NTX, tx = rem - ty * NTX;
  const int n = n0 + slot;
  const int c = c0 + 2 * cp;
  const int gi = i0 + ty * kClRH, gj = j0 + tx * kClCW;      // first sub-band position of the tile
  const bool live = (n < a.B) && (c < a.C) && (gi < a.Hh) && (gj < a.Wh);
  const bool pair = (c + 1 < a.C);
  if (!live) return;

  float2 acc[4][kClRH][kClCW];
#pragma unroll
  for (int s = 0; s < 4; ++s)
#pragma unroll
    for (int i = 0; i < kClRH; ++i)
#pragma unroll
      for (int j = 0; j < kClCW; ++j) acc[s][i][j] = make_float2(0.f, 0.f);
  // deeper reconstruction -> low-pass accumulators (wtconv2d.py:71), requested before the convolutions
  if (a.rin) {
    const float* rb = a.rin + (size_t)n * a.rs[0] + (size_t)c * a.rs[1];
#pragma unroll
    for (int i = 0; i < kClRH; ++i)
#pragma unroll
      for (int j = 0; j < kClCW; ++j) {
        if (gi + i < a.Hh && gj + j < a.Wh) {
          const float* rp = rb + (size_t)(gi + i) * a.rs[2] + (size_t)(gj + j) * a.rs[3];
          if (a.rin_vec) acc[0][i][j] = __ldg(reinterpret_cast<const float2*>(rp));
          else {
            acc[0][i][j].x = __ldg(rp);
            if (pair) acc[0][i][j].y = __ldg(rp + a.rs[1]);
          }
        }
      }
  }
  const int rot = (tx + NTX * ty) & (SL - 1);
  {
    const T* sbase = S + (size_t)slot * G::SLOT_S + ((size_t)(ty * kClRH) * SC + tx * kClCW) * kClGroup + 2 * cp;
    const T* ps[SL];
#pragma unroll
    for (int v = 0; v < SL; ++v) ps[v] = sbase + ((v + rot) & (SL - 1)) * kClGroup;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const T* pss[SL];
#pragma unroll
      for (int v = 0; v < SL; ++v) pss[v] = ps[v] + s * G::SUB;
      cl_subband_conv<T, K, SC, SL, NTX>(acc[s], pss, Wsm + (1 + s) * G::TAPS * kClLanes + cp);
    }
  }

  // synthesis butterfly (un-normalised; the tap magnitudes are in the packed parameters)
  float2 out[2 * kClRH][2 * kClCW];
#pragma unroll
  for (int i = 0; i < kClRH; ++i)
#pragma unroll
    for (int j = 0; j < kClCW; ++j) {
      const float2 ll = acc[0][i][j], lh = acc[1][i][j], hl = acc[2][i][j], hh = acc[3][i][j];
      const float2 pp = cl_add2(ll, lh), qq = cl_sub2(ll, lh), uu = cl_add2(hl, hh), vv = cl_sub2(hl, hh);
      out[2 * i][2 * j] = cl_add2(pp, uu);
      out[2 * i][2 * j + 1] = cl_sub2(pp, uu);
      out[2 * i + 1][2 * j] = cl_add2(qq, vv);
      out[2 * i + 1][2 * j + 1] = cl_sub2(qq, vv);
    }
  if (BASE) {
    const float2 bias = Wsm[(K * K) * kClLanes + cp];
#pragma unroll
    for (int i = 0; i < 2 * kClRH; ++i)
#pragma unroll
      for (int j = 0; j < 2 * kClCW; ++j) out[i][j] = cl_add2(out[i][j], bias);
    // window of the tile in the pixel copy: copy row 4*ty (= frame row 4*ty + HS), frame column 8*tx + HS
    const T* xbase = XT + (size_t)slot * G::SLOT_X + ((size_t)(4 * ty) * XC + 8 * tx) * kClGroup + 2 * cp;
    const T* px[SL];
#pragma unroll
    for (int v = 0; v < SL; ++v) px[v] = xbase + ((v + rot) & (SL - 1)) * kClGroup;
    cl_base_conv<T, K, XC, SL, NTX>(out, px, Wsm + cp);
  }
  // store (cropped to the plane: wtconv2d.py:76)
  TO* ob = static_cast<TO*>(a.out) + (size_t)n * a.os[0] + c;
  const int y0 = 2 * gi, x0 = 2 * gj;
#pragma unroll
  for (int i = 0; i < 2 * kClRH; ++i) {
    if (y0 + i >= a.H) continue;
#pragma unroll
    for (int j = 0; j < 2 * kClCW; ++j) {
      if (x0 + j >= a.W) continue;
      TO* o = ob + (size_t)(y0 + i) * a.os[2] + (size_t)(x0 + j) * a.os[3];
      if (a.out_vec && pair) ClPair<TO>::store(o, out[i][j]);
      else {
        o[0] = Elem<TO>::from_f(out[i][j].x);
        if (pair) o[1] = Elem<TO>::from_f(out[i][j].y);
      }
    }
  }
#endif
}

}  // namespace wt
