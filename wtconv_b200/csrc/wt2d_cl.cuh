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
//   1. one elected thread requests the whole input frame (band + halo of 2*(K/2) pixels)
//      as four cp.async.bulk.tensor boxes per slot, each completing on its own mbarrier,
//      and the tap sets of the stage as one cp.async.bulk copy.  Pixels outside the plane
//      arrive as zeros: TMA out-of-bounds fill reproduces both the odd-size padding of
//      wtconv2d.py:49-51 and the 'same' padding of every convolution;
//   2. pass 1 turns pixel rows 2k, 2k+1 into row k of the four Haar sub-bands
//      (wavelet.py:62-67, at the reference's scale) as fp32 channel pairs.  The sub-bands
//      overlay the pixel frame in shared memory and are produced last rows first, a batch
//      at a time (load - barrier - store), so nothing is overwritten before it is read.
//      Columns are stored rotated by the index of the thread tile they belong to, which
//      keeps the reads of the tiles served by one 128-byte wavefront in different banks;
//   3. pass 2: each thread runs the four K x K sub-band convolutions of its tile, adds the
//      deeper reconstruction to the low-pass result, applies the synthesis butterfly
//      (wavelet.py:70-75) in registers and, for the base path, rebuilds the pixels of its
//      window from the sub-bands and accumulates the base convolution and bias, then
//      stores its 4 x 8 pixels.  All arithmetic is fp32.
//
// The file also holds the two kernels that feed the top level of a layer with more than one
// level: wt2d_cl_pyramid_kernel (input -> sub-bands of level 2) and wt2d_cl_deep_kernel
// (levels 2..L with whole planes on chip -> reconstruction handed to the top level).
//
// Every mbarrier wait is bounded (kClWaitSpins); a wait that gives up sets the device status
// word of ClArgs/ClDeepArgs and the CTA carries on to its end instead of spinning.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "wt_common.h"
#include "wt2d_cl_host.h"

namespace wt {

constexpr unsigned kClWaitSpins = 1u << 22;   // bound of every mbarrier wait

struct ClArgs {
  int B, C, H, W;          // input plane set of this level
  int Hh, Wh;              // sub-band planes: ceil(H/2), ceil(W/2)
  int nby, nbx;            // bands per plane
  int ngroups;             // channel groups of 16
  int nslot_groups;        // ceil(B / NS)
  const float* packed;     // folded parameters (wtconv_pack_params layout)
  long long cl_off;        // floats from `packed` to the channels-last parameter copy
  int nlevels;             // wavelet levels of the layer (tap sets per channel group = 1 + 4 * nlevels)
  int level;               // 0-based level of this stage inside the packed block
  const float* rin;        // deeper reconstruction (fp32), may be null
  long long rs[4];         // its strides in floats: n, c, h, w
  void* out;               // output tensor
  long long os[4];         // its strides in elements: n, c, h, w
  int out_vec;             // 1: channel pairs may be stored as one word
  int rin_vec;             // 1: channel pairs of rin may be loaded as one 8-byte word
  float rin_scale;         // factor applied to rin: 1/2 for a reconstruction at the reference's scale
  int* status;             // device word that receives a nonzero code when a wait gives up
  int pdl;                 // 1: launched as a programmatic dependent of the kernel that writes rin
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

// Programmatic dependent launch: the next kernel of the stream may be scheduled once every CTA of
// this grid has got here (it still waits for this grid's completion before it reads its results)
__device__ __forceinline__ void cl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// ... and the other side: blocks until the preceding grid of the stream has completed and its
// writes are visible (a no-op for a kernel that was launched without the attribute)
__device__ __forceinline__ void cl_wait_for_producer() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// 5-D tiled TMA load (channel, sub-band, column, row, sample) -> shared memory, completing on `bar`
__device__ __forceinline__ void cl_tma_load5(void* dst, const CUtensorMap* map, void* bar, int c, int sb, int x, int y, int n) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(cl_smem_addr(dst)), "l"(map), "r"(cl_smem_addr(bar)), "r"(c), "r"(sb), "r"(x), "r"(y), "r"(n)
      : "memory");
}

// One 2 x 2 Haar analysis step at the reference's scale (wavelet.py:27-30 with tap 1/2):
// sb = {LL, LH, HL, HH} = 1/2 {a+b+c+d, a+b-c-d, a-b+c-d, a-b-c+d}
__device__ __forceinline__ void cl_haar(float2 a, float2 b, float2 c, float2 d, float2 (&sb)[4]) {
  const float2 h = make_float2(0.5f, 0.5f), mh = make_float2(-0.5f, -0.5f);
  const float2 pp = cl_add2(a, b), qq = cl_sub2(a, b), uu = cl_add2(c, d), vv = cl_sub2(c, d);
  const float2 hu = __fmul2_rn(uu, h), hv = __fmul2_rn(vv, h);
  sb[0] = cl_fma2(pp, h, hu);
  sb[1] = cl_fma2(pp, h, __fmul2_rn(uu, mh));
  sb[2] = cl_fma2(qq, h, hv);
  sb[3] = cl_fma2(qq, h, __fmul2_rn(vv, mh));
}

// 8-byte shared-memory load that keeps its place among the other loads of this kind
__device__ __forceinline__ float2 cl_lds2_ordered(const float* p) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(cl_smem_addr(p)));
  return v;
}

// plain bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completing on `bar`
__device__ __forceinline__ void cl_bulk_load(void* dst, const void* src, unsigned bytes, void* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(cl_smem_addr(dst)), "l"(src), "r"(bytes), "r"(cl_smem_addr(bar))
               : "memory");
}

// channel pair of a staged pixel -> fp32 pair
template <typename T> struct ClPair;
template <> struct ClPair<float> {
  typedef float2 raw_t;
  static __device__ __forceinline__ raw_t load_raw(const float* p) { return *reinterpret_cast<const float2*>(p); }
  // two neighbouring pairs (four channels) with one 16-byte access
  static __device__ __forceinline__ void load_raw2(const float* p, raw_t& a, raw_t& b) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    a = make_float2(v.x, v.y); b = make_float2(v.z, v.w);
  }
  static __device__ __forceinline__ float2 widen(raw_t r) { return r; }
  static __device__ __forceinline__ void store_raw(float* p, raw_t r) { *reinterpret_cast<float2*>(p) = r; }
  // channel pair from global memory; `both`: the second channel exists
  static __device__ __forceinline__ raw_t load_global(const float* p, bool valid, bool vec, bool both) {
    raw_t r = make_float2(0.f, 0.f);
    if (valid) {
      if (vec) r = __ldg(reinterpret_cast<const float2*>(p));
      else { r.x = __ldg(p); if (both) r.y = __ldg(p + 1); }
    }
    return r;
  }
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void store(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
};
template <> struct ClPair<__nv_bfloat16> {
  typedef unsigned raw_t;
  static __device__ __forceinline__ raw_t load_raw(const __nv_bfloat16* p) { return *reinterpret_cast<const unsigned*>(p); }
  // two neighbouring pairs (four channels) with one 8-byte access
  static __device__ __forceinline__ void load_raw2(const __nv_bfloat16* p, raw_t& a, raw_t& b) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    a = v.x; b = v.y;
  }
  // bf16 -> fp32 is a move of the 16 bits into the upper half: two byte permutes (integer pipe).
  // Written as prmt so that the compiler does not turn shift/mask into conversion instructions,
  // which issue at a fraction of the integer rate.
  static __device__ __forceinline__ float2 widen(raw_t u) {
    unsigned lo, hi;
    asm("prmt.b32 %0, %1, 0, 0x1044;" : "=r"(lo) : "r"(u));
    asm("prmt.b32 %0, %1, 0, 0x3244;" : "=r"(hi) : "r"(u));
    return make_float2(__uint_as_float(lo), __uint_as_float(hi));
  }
  static __device__ __forceinline__ void store_raw(__nv_bfloat16* p, raw_t r) { *reinterpret_cast<unsigned*>(p) = r; }
  static __device__ __forceinline__ raw_t load_global(const __nv_bfloat16* p, bool valid, bool vec, bool both) {
    raw_t r = 0u;
    if (valid) {
      if (vec) r = __ldg(reinterpret_cast<const unsigned*>(p));
      else {
        r = (unsigned)__ldg(reinterpret_cast<const unsigned short*>(p));
        if (both) r |= ((unsigned)__ldg(reinterpret_cast<const unsigned short*>(p) + 1) << 16);
      }
    }
    return r;
  }
  static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) { return widen(load_raw(p)); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float2 v) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __float22bfloat162_rn(v);
  }
};
template <> struct ClPair<__half> {
  typedef unsigned raw_t;
  static __device__ __forceinline__ raw_t load_raw(const __half* p) { return *reinterpret_cast<const unsigned*>(p); }
  static __device__ __forceinline__ void load_raw2(const __half* p, raw_t& a, raw_t& b) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    a = v.x; b = v.y;
  }
  static __device__ __forceinline__ float2 widen(raw_t u) { return __half22float2(*reinterpret_cast<const __half2*>(&u)); }
  static __device__ __forceinline__ void store_raw(__half* p, raw_t r) { *reinterpret_cast<unsigned*>(p) = r; }
  static __device__ __forceinline__ raw_t load_global(const __half* p, bool valid, bool vec, bool both) {
    raw_t r = 0u;
    if (valid) {
      if (vec) r = __ldg(reinterpret_cast<const unsigned*>(p));
      else {
        r = (unsigned)__ldg(reinterpret_cast<const unsigned short*>(p));
        if (both) r |= ((unsigned)__ldg(reinterpret_cast<const unsigned short*>(p) + 1) << 16);
      }
    }
    return r;
  }
  static __device__ __forceinline__ float2 load(const __half* p) { return widen(load_raw(p)); }
  static __device__ __forceinline__ void store(__half* p, float2 v) {
    *reinterpret_cast<__half2*>(p) = __float22half2_rn(v);
  }
};

// Four consecutive channels of a pixel as one 8-byte (16-bit types) or 16-byte (fp32) access; the
// address must be aligned to the access.  The two channel pairs come back as ClPair raw values.
template <typename T> struct ClQuad;
template <> struct ClQuad<float> {
  static __device__ __forceinline__ void load(const float* p, bool valid, float2& a, float2& b) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (valid) v = __ldg(reinterpret_cast<const float4*>(p));
    a = make_float2(v.x, v.y); b = make_float2(v.z, v.w);
  }
  static __device__ __forceinline__ void store(float* p, float2 a, float2 b) {
    *reinterpret_cast<float4*>(p) = make_float4(a.x, a.y, b.x, b.y);
  }
};
template <> struct ClQuad<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, bool valid, unsigned& a, unsigned& b) {
    uint2 v = make_uint2(0u, 0u);
    if (valid) v = __ldg(reinterpret_cast<const uint2*>(p));
    a = v.x; b = v.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float2 a, float2 b) {
    const __nv_bfloat162 ha = __float22bfloat162_rn(a), hb = __float22bfloat162_rn(b);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const unsigned*>(&ha), *reinterpret_cast<const unsigned*>(&hb));
  }
};
template <> struct ClQuad<__half> {
  static __device__ __forceinline__ void load(const __half* p, bool valid, unsigned& a, unsigned& b) {
    uint2 v = make_uint2(0u, 0u);
    if (valid) v = __ldg(reinterpret_cast<const uint2*>(p));
    a = v.x; b = v.y;
  }
  static __device__ __forceinline__ void store(__half* p, float2 a, float2 b) {
    const __half2 ha = __float22half2_rn(a), hb = __float22half2_rn(b);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const unsigned*>(&ha), *reinterpret_cast<const unsigned*>(&hb));
  }
};
#endif

// Compile-time geometry of one kernel configuration (T: type of the input plane set).  The
// sub-bands are kept as fp32 channel pairs, [row][sub-band][column][16 channels]; the pixel frame
// (type T) lands at the start of the same region and is consumed, last rows first, just ahead of
// the sub-band rows that overwrite it (see pass 1 of the kernel).
template <typename T, int K, int NTY, int NTX, int NS>
struct ClGeo {
  static constexpr int HS = K / 2;                          // halo of a K x K window
  static constexpr int SR = NTY * kClRH + 2 * HS;           // sub-band frame rows
  static constexpr int SC = ((NTX * kClCW + 2 * HS + 3) / 4) * 4;   // sub-band frame columns (whole rotation groups)
  static constexpr int XR = 2 * SR, XC = 2 * SC;            // pixel frame delivered by the TMA boxes
  static constexpr int NBOX = 4;                            // TMA boxes per slot, stacked along the rows
  static constexpr int BOXR = XR / NBOX;                    // pixel rows per box
  static_assert(XR % NBOX == 0, "the pixel frame is a whole number of boxes");
  // batches of pass 1: the fewest (a divisor of SR) that keep a thread's share of a batch within
  // 64 registers of raw pixels (four pixels per block; one register per 16-bit pair, two per fp32 pair)
  static constexpr int pick_batches() {
    const int nt = (NTY * NTX * NS * kClLanes + 31) / 32 * 32;
    const int most = sizeof(T) == 2 ? 16 : 8;   // blocks per thread and batch
    for (int nb = 1; nb <= SR; ++nb) {
      if (SR % nb) continue;
      const int items = NS * (SR / nb) * SC * kClLanes;
      if ((items + nt - 1) / nt <= most) return nb;
    }
    return SR;
  }
  static constexpr int NB = pick_batches();
  static constexpr int NT = (NTY * NTX * NS * kClLanes + 31) / 32 * 32;   // threads per CTA (whole warps)
  static constexpr int TAPS = K * K + 1;                    // staged floats per tap set and channel (last: bias slot)
  static constexpr int SL = 128 / (kClGroup * (int)sizeof(float));   // sub-band positions per 128-byte line
  static constexpr int SUBS = SC * kClGroup;                // floats between the sub-bands of a row
  static constexpr int ROWS = 4 * SUBS;                     // floats between rows
  static constexpr int SLOT_S = SR * ROWS;                  // floats per slot
  static constexpr size_t s_bytes = (size_t)NS * SLOT_S * sizeof(float);
  static constexpr size_t frame_bytes = (size_t)XR * XC * kClGroup * sizeof(T);
  static_assert(frame_bytes <= (size_t)SLOT_S * sizeof(float), "the pixel frame fits under its sub-bands");
  static constexpr size_t box_bytes = (size_t)BOXR * XC * kClGroup * sizeof(T);
  static constexpr size_t w_bytes = (size_t)5 * TAPS * kClLanes * sizeof(float2);
  static constexpr size_t smem_bytes = 128 /* alignment slack */ + s_bytes + w_bytes + 64 /* barriers */;
};

// Rotation of the sub-band columns.  A position (16 channels, fp32) takes 128/SL bytes; the SL
// thread tiles served by one 128-byte wavefront are consecutive tiles q = ty*NTX + tx of the CTA
// and all read the same window element.  Column f of row r is stored at
//     (f & ~(SL-1)) + ((f + tile_column(f) + NTX * tile_row(r)) & (SL-1)),
// i.e. every line is rotated by the index of the tile it belongs to, so those SL reads fall into
// different bank groups; for a reader the rotation is (compile-time part + q) & (SL-1), one of SL
// per-thread base pointers plus a compile-time offset.

#ifdef __CUDA_ARCH__
// acc[oy][ox] += sum_{dy,dx} w[dy][dx] * S(oy+dy, ox+dx) for one sub-band of the thread's window.
// p[v]: base pointers of the window (channel pair and sub-band included) for rotation class v;
// RS: floats between rows.
template <int K, int RS, int SL, int NTX>
__device__ __forceinline__ void cl_subband_conv(float2 (&acc)[kClRH][kClCW], const float* const (&p)[SL],
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
      in[c] = *reinterpret_cast<const float2*>(p[v] + iy * RS + (c & ~(SL - 1)) * kClGroup);
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

// Base convolution of the 4 x 8 pixel tile.  The pixels are rebuilt from the four sub-bands, one
// 2 x 2 block at a time (the Haar step is its own inverse), and every rebuilt pixel is added at
// once to all the outputs it reaches, so no pixel rows are kept in registers.
template <int K, int RS, int SUBS, int SL, int NTX>
__device__ __forceinline__ void cl_base_conv(float2 (&out)[2 * kClRH][2 * kClCW], const float* const (&p)[SL],
                                             const float2* __restrict__ w) {
  constexpr int HS = K / 2, BH = (HS + 1) / 2;
  constexpr int OFF = 2 * BH - HS;                 // first rebuilt pixel row / column that is used
  constexpr int NBR = kClRH + 2 * BH, NBC = kClCW + 2 * BH;   // blocks rebuilt
  float2 wr[K * K];
#pragma unroll
  for (int t = 0; t < K * K; ++t) wr[t] = __fmul2_rn(w[t * kClLanes], make_float2(0.5f, 0.5f));   // 1/2 of the inverse step
#pragma unroll
  for (int br = 0; br < NBR; ++br) {
#pragma unroll
    for (int bc = 0; bc < NBC; ++bc) {
      const int fy = br + HS - BH, fx = bc + HS - BH;          // window position of this block
      const int v = ((fx & (SL - 1)) + (fx >> 2) + NTX * (fy >> 1)) & (SL - 1);
      const float* q = p[v] + fy * RS + (fx & ~(SL - 1)) * kClGroup;
      // ordered loads: left to itself the compiler requests all the blocks up front and runs out of registers
      const float2 ll = cl_lds2_ordered(q), lh = cl_lds2_ordered(q + SUBS);
      const float2 hl = cl_lds2_ordered(q + 2 * SUBS), hh = cl_lds2_ordered(q + 3 * SUBS);
      const float2 pp = cl_add2(ll, lh), qq = cl_sub2(ll, lh), uu = cl_add2(hl, hh), vv = cl_sub2(hl, hh);
      const float2 px[2][2] = {{cl_add2(pp, uu), cl_sub2(pp, uu)}, {cl_add2(qq, vv), cl_sub2(qq, vv)}};
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int iy = 2 * br + a - OFF, ix = 2 * bc + b - OFF;   // position in the tile's input window
          if (iy < 0 || iy >= 2 * kClRH + K - 1 || ix < 0 || ix >= 2 * kClCW + K - 1) continue;
#pragma unroll
          for (int dy = 0; dy < K; ++dy) {
            const int oy = iy - dy;
            if (oy < 0 || oy >= 2 * kClRH) continue;
#pragma unroll
            for (int dx = 0; dx < K; ++dx) {
              const int ox = ix - dx;
              if (ox < 0 || ox >= 2 * kClCW) continue;
              out[oy][ox] = cl_fma2(px[a][b], wr[dy * K + dx], out[oy][ox]);
            }
          }
        }
    }
  }
}
#endif

// T: type of the input plane set; TO: type of the output (T for the layer output, float for a
// reconstruction handed to the next shallower level); BASE: add the base path.
template <typename T, typename TO, int K, int NTY, int NTX, int NS, bool BASE, int MAXREG>
__global__ void __launch_bounds__((NTY * NTX * NS * kClLanes + 31) / 32 * 32) __maxnreg__(MAXREG)
wt2d_cl_level_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ ClArgs a) {
#ifdef __CUDA_ARCH__
  typedef ClGeo<T, K, NTY, NTX, NS> G;
  typedef typename ClPair<T>::raw_t raw_t;
  constexpr int SC = G::SC, SR = G::SR, HS = G::HS, SL = G::SL, XC = G::XC;
  static_assert(kClRH == 2 && kClCW == 4, "the swizzle assumes 2 x 4 thread tiles");
  extern __shared__ unsigned char cl_smem_raw[];
  unsigned char* sm = cl_smem_raw + ((128u - (cl_smem_addr(cl_smem_raw) & 127u)) & 127u);
  float* S = reinterpret_cast<float*>(sm);                          // sub-bands; the pixel frame lands on top of them
  float2* Wsm = reinterpret_cast<float2*>(sm + G::s_bytes);
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(sm + G::s_bytes + G::w_bytes);

  const int tid = threadIdx.x;
  cl_launch_dependents();
  // grid: x = channel group (fastest: the CTAs that share the 128-byte lines of a pixel run together),
  // y = band (column band fastest), z = slot group
  const int band = blockIdx.y;
  const int bx = band % a.nbx, by = band / a.nbx;
  const int c0 = blockIdx.x * kClGroup;
  const int n0 = blockIdx.z * NS;
  const int i0 = by * NTY * kClRH, j0 = bx * NTX * kClCW;    // first sub-band position of the band
  const int X0 = 2 * (j0 - HS), Y0 = 2 * (i0 - HS);          // pixel frame origin (may be negative)

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s <= G::NBOX; ++s) cl_mbar_init(&bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // The whole pixel frame is requested at once: NBOX boxes per slot, one barrier per row range.
    // Pixels outside the plane arrive as zeros (TMA out-of-bounds fill), which is both the odd-size
    // padding of wtconv2d.py:49-51 and the 'same' padding of the convolutions.
#pragma unroll
    for (int b = 0; b < G::NBOX; ++b) {
      cl_mbar_expect_tx(&bars[b], (unsigned)(NS * G::box_bytes));
#pragma unroll
      for (int sl = 0; sl < NS; ++sl)
        cl_tma_load4(sm + (size_t)sl * G::SLOT_S * sizeof(float) + (size_t)b * G::box_bytes, &xmap, &bars[b], c0, X0,
                     Y0 + b * G::BOXR, n0 + sl);
    }
    // tap sets of this stage, one bulk copy out of the channels-last parameter copy:
    // [set][tap][16 channels] fp32; set 0 = base (taps, bias), 1..4 = sub-bands of the level
    constexpr unsigned kSetBytes = (unsigned)(G::TAPS * kClGroup * sizeof(float));
    const int nset = 1 + 4 * a.nlevels;
    const float* src = a.packed + a.cl_off + ((size_t)blockIdx.x * nset + (BASE ? 0 : 1 + 4 * a.level)) * (G::TAPS * kClGroup);
    const unsigned bytes = (BASE ? 5u : 4u) * kSetBytes;
    cl_mbar_expect_tx(&bars[G::NBOX], bytes);
    cl_bulk_load(reinterpret_cast<unsigned char*>(Wsm) + (BASE ? 0u : kSetBytes), src, bytes, &bars[G::NBOX]);
  }
  __syncthreads();     // barrier words initialised before anyone waits on them

  // ---- pass 1: pixel rows 2k, 2k+1 of the frame -> row k of the four sub-bands (one Haar step at
  // the reference's scale).  The blocks (slot, row, column, channel pair) of a batch of rows are
  // dealt round-robin to the threads; a batch is read into registers, the CTA meets, and only then
  // are its sub-band rows written -- they cover frame rows of this and of later batches only (a
  // sub-band row takes at least the bytes of its two pixel rows and both arrays start at the same
  // address), and batches run last rows first.  16-bit frames fit the registers in one batch.
  // A block item is four channels (two pairs) of one position: 8- / 16-byte shared-memory accesses.
  constexpr int NB = G::NB, RB = SR / NB;
  constexpr int QL = kClLanes / 2;                     // items per position
  constexpr int BITEMS = NS * RB * SC * QL;
  constexpr int NIT = (BITEMS + G::NT - 1) / G::NT;
  bool ok = true;
#pragma unroll 1
  for (int bt = NB - 1; bt >= 0; --bt) {
    const int k0 = bt * RB;
    for (int b = (2 * k0) / G::BOXR; b <= (2 * (k0 + RB) - 1) / G::BOXR; ++b) ok = cl_mbar_wait(&bars[b], 0u) && ok;
    raw_t px[NIT][4][2];
#pragma unroll
    for (int j = 0; j < NIT; ++j) {
      const int it = tid + j * G::NT;
      if (it >= BITEMS) continue;
      const int cq = it & (QL - 1);
      const int blk = it / QL;
      const int f = blk % SC;
      const int t = blk / SC;
      const int k = k0 + t % RB;
      const int slot = t / RB;
      const T* p = reinterpret_cast<const T*>(S + (size_t)slot * G::SLOT_S) + ((size_t)(2 * k) * XC + 2 * f) * kClGroup + 4 * cq;
      ClPair<T>::load_raw2(p, px[j][0][0], px[j][0][1]);
      ClPair<T>::load_raw2(p + kClGroup, px[j][1][0], px[j][1][1]);
      ClPair<T>::load_raw2(p + XC * kClGroup, px[j][2][0], px[j][2][1]);
      ClPair<T>::load_raw2(p + XC * kClGroup + kClGroup, px[j][3][0], px[j][3][1]);
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < NIT; ++j) {
      const int it = tid + j * G::NT;
      if (it >= BITEMS) continue;
      const int cq = it & (QL - 1);
      const int blk = it / QL;
      const int f = blk % SC;
      const int t = blk / SC;
      const int k = k0 + t % RB;
      const int slot = t / RB;
      float2 sa[4], sb[4];
      cl_haar(ClPair<T>::widen(px[j][0][0]), ClPair<T>::widen(px[j][1][0]), ClPair<T>::widen(px[j][2][0]), ClPair<T>::widen(px[j][3][0]), sa);
      cl_haar(ClPair<T>::widen(px[j][0][1]), ClPair<T>::widen(px[j][1][1]), ClPair<T>::widen(px[j][2][1]), ClPair<T>::widen(px[j][3][1]), sb);
      const int rot = ((f >> 2) + NTX * (k >> 1)) & (SL - 1);
      const int fs = (f & ~(SL - 1)) + ((f + rot) & (SL - 1));
      float* d = S + (size_t)slot * G::SLOT_S + (size_t)k * G::ROWS + fs * kClGroup + 4 * cq;
#pragma unroll
      for (int sbi = 0; sbi < 4; ++sbi)
        *reinterpret_cast<float4*>(d + sbi * G::SUBS) = make_float4(sa[sbi].x, sa[sbi].y, sb[sbi].x, sb[sbi].y);
    }
  }
  ok = cl_mbar_wait(&bars[G::NBOX], 0u) && ok;        // tap sets
  if (!ok && a.status) atomicExch(a.status, 1);
  __syncthreads();

  // ---- pass 2: per-thread tile
  const int cp = tid & (kClLanes - 1);
  const int q = tid >> 3;
  const int slot = q / (NTY * NTX);
  const int rem = q - slot * (NTY * NTX);
  const int ty = rem / NTX, tx = rem - ty * NTX;
  const int n = n0 + slot;
  const int c = c0 + 2 * cp;
  const int gi = i0 + ty * kClRH, gj = j0 + tx * kClCW;      // first sub-band position of the tile
  const bool live = (q < NS * NTY * NTX) && (n < a.B) && (c < a.C) && (gi < a.Hh) && (gj < a.Wh);
  const bool pair = (c + 1 < a.C);
  if (!live) return;

  float2 acc[4][kClRH][kClCW];
#pragma unroll
  for (int s = 0; s < 4; ++s)
#pragma unroll
    for (int i = 0; i < kClRH; ++i)
#pragma unroll
      for (int j = 0; j < kClCW; ++j) acc[s][i][j] = make_float2(0.f, 0.f);
  // window of the tile: sub-band frame row 2*ty, column 4*tx; rotation classes relative to the tile's own
  const int rot = (tx + NTX * ty) & (SL - 1);
  const float* sbase = S + (size_t)slot * G::SLOT_S + (size_t)(ty * kClRH) * G::ROWS + (tx * kClCW) * kClGroup + 2 * cp;
  const float* ps[SL];
#pragma unroll
  for (int v = 0; v < SL; ++v) ps[v] = sbase + ((v + rot) & (SL - 1)) * kClGroup;
  // Deeper reconstruction (wtconv2d.py:71).  Its producer is the preceding kernel of the stream, which
  // may still be running when this one was launched early: the wait and the loads sit before the last
  // of the four sub-band convolutions, so a CTA that started early has three of them behind it when
  // it blocks, and the loads of the others are covered by the fourth.
  float2 rin[kClRH][kClCW];
#pragma unroll
  for (int i = 0; i < kClRH; ++i)
#pragma unroll
    for (int j = 0; j < kClCW; ++j) rin[i][j] = make_float2(0.f, 0.f);
  auto load_rin = [&]() {
    if (a.pdl) cl_wait_for_producer();
    if (a.rin) {
      const float* rb = a.rin + (size_t)n * a.rs[0] + (size_t)c * a.rs[1];
#pragma unroll
      for (int i = 0; i < kClRH; ++i)
#pragma unroll
        for (int j = 0; j < kClCW; ++j) {
          if (gi + i < a.Hh && gj + j < a.Wh) {
            const float* rp = rb + (size_t)(gi + i) * a.rs[2] + (size_t)(gj + j) * a.rs[3];
            if (a.rin_vec) rin[i][j] = __ldg(reinterpret_cast<const float2*>(rp));
            else {
              rin[i][j].x = __ldg(rp);
              if (pair) rin[i][j].y = __ldg(rp + a.rs[1]);
            }
          }
        }
    }
  };
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    if (s == 3) load_rin();
    const float* pss[SL];
#pragma unroll
    for (int v = 0; v < SL; ++v) pss[v] = ps[v] + s * G::SUBS;
    cl_subband_conv<K, G::ROWS, SL, NTX>(acc[s], pss, Wsm + (1 + s) * G::TAPS * kClLanes + cp);
  }

  // synthesis butterfly (its factor 1/2 is folded into the staged taps)
  float2 out[2 * kClRH][2 * kClCW];
  const float2 rsc = make_float2(a.rin_scale, a.rin_scale);
#pragma unroll
  for (int i = 0; i < kClRH; ++i)
#pragma unroll
    for (int j = 0; j < kClCW; ++j) {
      const float2 ll = cl_fma2(rin[i][j], rsc, acc[0][i][j]), lh = acc[1][i][j], hl = acc[2][i][j], hh = acc[3][i][j];
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
    cl_base_conv<K, G::ROWS, G::SUBS, SL, NTX>(out, ps, Wsm + cp);
  }
  // store (cropped to the plane: wtconv2d.py:76)
  const int y0 = 2 * gi, x0 = 2 * gj;
  TO* ob = static_cast<TO*>(a.out) + (size_t)n * a.os[0] + (size_t)y0 * a.os[2] + (size_t)x0 * a.os[3] + c;
  if (a.out_vec && pair && y0 + 2 * kClRH <= a.H && x0 + 2 * kClCW <= a.W) {
#pragma unroll
    for (int i = 0; i < 2 * kClRH; ++i)
#pragma unroll
      for (int j = 0; j < 2 * kClCW; ++j) ClPair<TO>::store(ob + (size_t)i * a.os[2] + (size_t)j * a.os[3], out[i][j]);
  } else {
#pragma unroll
    for (int i = 0; i < 2 * kClRH; ++i) {
      if (y0 + i >= a.H) continue;
#pragma unroll
      for (int j = 0; j < 2 * kClCW; ++j) {
        if (x0 + j >= a.W) continue;
        TO* o = ob + (size_t)i * a.os[2] + (size_t)j * a.os[3];
        if (a.out_vec && pair) ClPair<TO>::store(o, out[i][j]);
        else {
          o[0] = Elem<TO>::from_f(out[i][j].x);
          if (pair) o[1] = Elem<TO>::from_f(out[i][j].y);
        }
      }
    }
  }
#endif
}

// ---------------------------------------------------------------------------
// Sub-band pyramid kernel: the layer input -> the four sub-bands of the second level.
//
// One thread owns one channel pair of one 4 x 4 pixel block: the four 2 x 2 blocks give four
// values of the first level's low-pass plane LL_1 (never stored) and their Haar step gives one
// position of S_2 = {LL_2, LH_2, HL_2, HH_2}, written as (B, h, w, 4, C) in the input's type at
// the reference's scale (the four sub-bands of a position are neighbours in memory).  Channel pairs are the fastest thread index, so a warp reads
// and writes 128 contiguous bytes per pixel.  Pixels outside the plane count as zeros
// (wtconv2d.py:49-51).
// ---------------------------------------------------------------------------
struct ClPyramidArgs {
  const void* x;
  long long xs[4];      // strides in elements: n, c (= 1), h, w
  int x_vec;            // 1: channel pairs may be loaded as one word; 2: four channels as one 8- / 16-byte access
  int B, C, H, W;
  int h2, w2;           // size of the second level's sub-bands: ceil(ceil(H/2)/2), ...
  void* s2;             // (B, h2, w2, 4, C)
  long long total;      // B * h2 * w2 * ceil(C/2)
};

template <typename T>
__global__ void __launch_bounds__(256) wt2d_cl_pyramid_kernel(const __grid_constant__ ClPyramidArgs a) {
#ifdef __CUDA_ARCH__
  cl_launch_dependents();
  const int P = (a.C + 1) / 2;
  const bool cpair = a.x_vec != 0;
  // 32-bit index arithmetic (the launcher keeps the item count below 2^31)
  for (unsigned id = blockIdx.x * blockDim.x + threadIdx.x; id < (unsigned)a.total; id += gridDim.x * blockDim.x) {
    const int p = (int)(id % (unsigned)P);
    unsigned t = id / (unsigned)P;
    const int f = (int)(t % (unsigned)a.w2);
    t /= (unsigned)a.w2;
    const int k = (int)(t % (unsigned)a.h2);
    const int n = (int)(t / (unsigned)a.h2);
    const int c = 2 * p;
    const T* p0 = static_cast<const T*>(a.x) + (long long)n * a.xs[0] + (long long)(4 * k) * a.xs[2] + (long long)(4 * f) * a.xs[3] + c;
    const bool both = (c + 1 < a.C);
    typename ClPair<T>::raw_t r[4][4];
#pragma unroll
    for (int yy = 0; yy < 4; ++yy)
#pragma unroll
      for (int xx = 0; xx < 4; ++xx)
        r[yy][xx] = ClPair<T>::load_global(p0 + yy * a.xs[2] + xx * a.xs[3], 4 * k + yy < a.H && 4 * f + xx < a.W, cpair && both, both);
    float2 l[2][2];
#pragma unroll
    for (int by = 0; by < 2; ++by)
#pragma unroll
      for (int bx = 0; bx < 2; ++bx) {
        const float2 va = ClPair<T>::widen(r[2 * by][2 * bx]), vb = ClPair<T>::widen(r[2 * by][2 * bx + 1]);
        const float2 vc = ClPair<T>::widen(r[2 * by + 1][2 * bx]), vd = ClPair<T>::widen(r[2 * by + 1][2 * bx + 1]);
        l[by][bx] = __fmul2_rn(cl_add2(cl_add2(va, vb), cl_add2(vc, vd)), make_float2(0.5f, 0.5f));
      }
    float2 sb[4];
    cl_haar(l[0][0], l[0][1], l[1][0], l[1][1], sb);
    T* d = static_cast<T*>(a.s2) + (((size_t)n * a.h2 + k) * a.w2 + f) * 4 * a.C + c;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      if (both && (a.C & 1) == 0) ClPair<T>::store(d + (size_t)s * a.C, sb[s]);
      else { d[(size_t)s * a.C] = Elem<T>::from_f(sb[s].x); if (both) d[(size_t)s * a.C + 1] = Elem<T>::from_f(sb[s].y); }
    }
  }
#endif
}

// The same with four channels per thread (channel counts that are multiples of four on tensors
// whose pixels start on 16-byte boundaries -- every tensor the channels-last chains accept): half
// the index arithmetic and half the memory instructions per byte.
template <typename T>
__global__ void __launch_bounds__(256) wt2d_cl_pyramid4_kernel(const __grid_constant__ ClPyramidArgs a) {
#ifdef __CUDA_ARCH__
  typedef typename ClPair<T>::raw_t raw_t;
  cl_launch_dependents();
  const unsigned Q = (unsigned)a.C / 4u;
  for (unsigned id = blockIdx.x * blockDim.x + threadIdx.x; id < (unsigned)a.total; id += gridDim.x * blockDim.x) {
    const int c = 4 * (int)(id % Q);
    unsigned t = id / Q;
    const int f = (int)(t % (unsigned)a.w2);
    t /= (unsigned)a.w2;
    const int k = (int)(t % (unsigned)a.h2);
    const int n = (int)(t / (unsigned)a.h2);
    const T* p0 = static_cast<const T*>(a.x) + (long long)n * a.xs[0] + (long long)(4 * k) * a.xs[2] + (long long)(4 * f) * a.xs[3] + c;
    float2 l[2][2][2];                          // [pair][block row][block column]
#pragma unroll
    for (int by = 0; by < 2; ++by)
#pragma unroll
      for (int bx = 0; bx < 2; ++bx) {
        raw_t r[2][2][2];                       // [pair][row][column] of the 2 x 2 pixel block
#pragma unroll
        for (int yy = 0; yy < 2; ++yy)
#pragma unroll
          for (int xx = 0; xx < 2; ++xx) {
            const int py = 2 * by + yy, px = 2 * bx + xx;
            ClQuad<T>::load(p0 + (long long)py * a.xs[2] + (long long)px * a.xs[3], 4 * k + py < a.H && 4 * f + px < a.W,
                            r[0][yy][xx], r[1][yy][xx]);
          }
#pragma unroll
        for (int h = 0; h < 2; ++h)
          l[h][by][bx] = __fmul2_rn(cl_add2(cl_add2(ClPair<T>::widen(r[h][0][0]), ClPair<T>::widen(r[h][0][1])),
                                            cl_add2(ClPair<T>::widen(r[h][1][0]), ClPair<T>::widen(r[h][1][1]))),
                                    make_float2(0.5f, 0.5f));
      }
    float2 sa[4], sb[4];
    cl_haar(l[0][0][0], l[0][0][1], l[0][1][0], l[0][1][1], sa);
    cl_haar(l[1][0][0], l[1][0][1], l[1][1][0], l[1][1][1], sb);
    T* d = static_cast<T*>(a.s2) + (((size_t)n * a.h2 + k) * a.w2 + f) * 4 * a.C + c;
#pragma unroll
    for (int s4 = 0; s4 < 4; ++s4) ClQuad<T>::store(d + (size_t)s4 * a.C, sa[s4], sb[s4]);
  }
#endif
}

// ---------------------------------------------------------------------------
// Low-pass planes for the level stages below the top one (large planes only): a plane set
// (the layer input, or a low-pass plane set written by an earlier launch of this kernel) ->
// the low-pass planes one and, optionally, two levels down, dense channels-last in the input's
// type and at the reference's scale (the reference also keeps its low-pass planes in that type,
// wtconv2d.py:55).  One thread owns one channel pair of one 4 x 4 pixel block.
// ---------------------------------------------------------------------------
struct ClLowpassArgs {
  const void* x;
  long long xs[4];      // strides in elements: n, c (= 1), h, w
  int x_vec;            // 1: channel pairs may be loaded as one word; 2: four channels as one 8- / 16-byte access
  int B, C, H, W;
  int h1, w1, h2, w2;   // sizes one and two levels down
  void* p1;             // (B, h1, w1, C)
  void* p2;             // (B, h2, w2, C) or null
  long long total;      // B * h2 * w2 * ceil(C/2)
};

template <typename T>
__global__ void __launch_bounds__(256) wt2d_cl_lowpass_kernel(const __grid_constant__ ClLowpassArgs a) {
#ifdef __CUDA_ARCH__
  const int P = (a.C + 1) / 2;
  const bool cpair = a.x_vec != 0;
  const bool even_c = (a.C & 1) == 0;
  // 32-bit index arithmetic (the launcher keeps the item count below 2^31)
  for (unsigned id = blockIdx.x * blockDim.x + threadIdx.x; id < (unsigned)a.total; id += gridDim.x * blockDim.x) {
    const int p = (int)(id % (unsigned)P);
    unsigned t = id / (unsigned)P;
    const int f = (int)(t % (unsigned)a.w2);
    t /= (unsigned)a.w2;
    const int k = (int)(t % (unsigned)a.h2);
    const int n = (int)(t / (unsigned)a.h2);
    const int c = 2 * p;
    const T* p0 = static_cast<const T*>(a.x) + (long long)n * a.xs[0] + (long long)(4 * k) * a.xs[2] + (long long)(4 * f) * a.xs[3] + c;
    const bool both = (c + 1 < a.C);
    typename ClPair<T>::raw_t r[4][4];
#pragma unroll
    for (int yy = 0; yy < 4; ++yy)
#pragma unroll
      for (int xx = 0; xx < 4; ++xx)
        r[yy][xx] = ClPair<T>::load_global(p0 + yy * a.xs[2] + xx * a.xs[3], 4 * k + yy < a.H && 4 * f + xx < a.W, cpair && both, both);
    float2 l[2][2];
#pragma unroll
    for (int by = 0; by < 2; ++by)
#pragma unroll
      for (int bx = 0; bx < 2; ++bx) {
        const float2 va = ClPair<T>::widen(r[2 * by][2 * bx]), vb = ClPair<T>::widen(r[2 * by][2 * bx + 1]);
        const float2 vc = ClPair<T>::widen(r[2 * by + 1][2 * bx]), vd = ClPair<T>::widen(r[2 * by + 1][2 * bx + 1]);
        l[by][bx] = __fmul2_rn(cl_add2(cl_add2(va, vb), cl_add2(vc, vd)), make_float2(0.5f, 0.5f));
        const int y1 = 2 * k + by, x1 = 2 * f + bx;
        if (y1 < a.h1 && x1 < a.w1) {
          T* d = static_cast<T*>(a.p1) + (((size_t)n * a.h1 + y1) * a.w1 + x1) * a.C + c;
          if (both && even_c) ClPair<T>::store(d, l[by][bx]);
          else { d[0] = Elem<T>::from_f(l[by][bx].x); if (both) d[1] = Elem<T>::from_f(l[by][bx].y); }
        }
      }
    if (a.p2) {
      const float2 ll = __fmul2_rn(cl_add2(cl_add2(l[0][0], l[0][1]), cl_add2(l[1][0], l[1][1])), make_float2(0.5f, 0.5f));
      T* d = static_cast<T*>(a.p2) + (((size_t)n * a.h2 + k) * a.w2 + f) * a.C + c;
      if (both && even_c) ClPair<T>::store(d, ll);
      else { d[0] = Elem<T>::from_f(ll.x); if (both) d[1] = Elem<T>::from_f(ll.y); }
    }
  }
#endif
}

// Four channels per thread (see wt2d_cl_pyramid4_kernel)
template <typename T>
__global__ void __launch_bounds__(256) wt2d_cl_lowpass4_kernel(const __grid_constant__ ClLowpassArgs a) {
#ifdef __CUDA_ARCH__
  typedef typename ClPair<T>::raw_t raw_t;
  const unsigned Q = (unsigned)a.C / 4u;
  for (unsigned id = blockIdx.x * blockDim.x + threadIdx.x; id < (unsigned)a.total; id += gridDim.x * blockDim.x) {
    const int c = 4 * (int)(id % Q);
    unsigned t = id / Q;
    const int f = (int)(t % (unsigned)a.w2);
    t /= (unsigned)a.w2;
    const int k = (int)(t % (unsigned)a.h2);
    const int n = (int)(t / (unsigned)a.h2);
    const T* p0 = static_cast<const T*>(a.x) + (long long)n * a.xs[0] + (long long)(4 * k) * a.xs[2] + (long long)(4 * f) * a.xs[3] + c;
    float2 l[2][2][2];
#pragma unroll
    for (int by = 0; by < 2; ++by)
#pragma unroll
      for (int bx = 0; bx < 2; ++bx) {
        raw_t r[2][2][2];
#pragma unroll
        for (int yy = 0; yy < 2; ++yy)
#pragma unroll
          for (int xx = 0; xx < 2; ++xx) {
            const int py = 2 * by + yy, px = 2 * bx + xx;
            ClQuad<T>::load(p0 + (long long)py * a.xs[2] + (long long)px * a.xs[3], 4 * k + py < a.H && 4 * f + px < a.W,
                            r[0][yy][xx], r[1][yy][xx]);
          }
#pragma unroll
        for (int h = 0; h < 2; ++h)
          l[h][by][bx] = __fmul2_rn(cl_add2(cl_add2(ClPair<T>::widen(r[h][0][0]), ClPair<T>::widen(r[h][0][1])),
                                            cl_add2(ClPair<T>::widen(r[h][1][0]), ClPair<T>::widen(r[h][1][1]))),
                                    make_float2(0.5f, 0.5f));
        const int y1 = 2 * k + by, x1 = 2 * f + bx;
        if (y1 < a.h1 && x1 < a.w1)
          ClQuad<T>::store(static_cast<T*>(a.p1) + (((size_t)n * a.h1 + y1) * a.w1 + x1) * a.C + c, l[0][by][bx], l[1][by][bx]);
      }
    if (a.p2) {
      const float2 h2 = make_float2(0.5f, 0.5f);
      const float2 la = __fmul2_rn(cl_add2(cl_add2(l[0][0][0], l[0][0][1]), cl_add2(l[0][1][0], l[0][1][1])), h2);
      const float2 lb = __fmul2_rn(cl_add2(cl_add2(l[1][0][0], l[1][0][1]), cl_add2(l[1][1][0], l[1][1][1])), h2);
      ClQuad<T>::store(static_cast<T*>(a.p2) + (((size_t)n * a.h2 + k) * a.w2 + f) * a.C + c, la, lb);
    }
  }
#endif
}

// ---------------------------------------------------------------------------
// Deep stage: every level from the second one down, whole planes on chip.
//
// A CTA owns NS plane slots (sample, 16-channel group).  The sub-bands of the second level
// (from the pyramid kernel) arrive as one 5-D TMA box per slot, with the zero border the
// convolutions need supplied by the out-of-bounds fill.  The analyses of the deeper levels,
// the sub-band convolutions and the synthesis of every level then run out of shared memory,
// deepest level first, and the reconstruction that the top level adds to its low-pass result
// (wtconv2d.py:64-76) leaves as fp32 channels-last planes.
//
// On-chip level j = 1..nlev is layer level lvl0+j+1 (lvl0 = 0 when the stage starts from the layer
// input's second level).  S_j: frame of (h_j + 2*HS) x (w_j + 2*HS)
// positions (rounded up to whole thread tiles) with a zero border, stored
// [row][column][sub-band][16 channels] in the input's type at the reference's scale;
// R_j: fp32 reconstruction of level j, h_{j-1} x w_{j-1} positions of 16 channels.
//
// A warp owns one tile of RT x CT positions: lane = (sub-band, channel pair), so the four
// sub-band convolutions of a tile run side by side, a warp reads one contiguous 128-byte
// (16-bit) or 256-byte (fp32) line per position, and the synthesis butterfly
// (wavelet.py:70-75) is two xor-shuffles across the sub-band bits of the lane index.
// ---------------------------------------------------------------------------
constexpr int kClDeepSetPitch = (5 * 5 + 1) * kClGroup * 4 + 64;   // bytes between the staged tap sets of a level (K = 5):
                                                                  // 64 past a multiple of 128, so the two sets read by a half warp (64 bytes each) fall into different banks
constexpr int kClDeepLevelBytes = (4 * kClDeepSetPitch + 127) / 128 * 128;

#ifdef __CUDA_ARCH__
// Sub-band convolutions + synthesis of level j for every tile of the CTA's slots.
template <typename T, int K, int RT, int CT>
__device__ __forceinline__ void cl_deep_level(const ClDeepArgs& a, int j, unsigned char* sm, const unsigned char* wlev,
                                              int c0, int n0, int tid, int nthr) {
  constexpr unsigned kFull = 0xffffffffu;
  constexpr int POS = 4 * kClGroup;                 // elements per frame position
  const int lane = tid & 31, sbi = lane >> 3, cp = lane & (kClLanes - 1);
  const int warp = tid >> 5, nwarp = nthr >> 5;
  const int hj = a.h[j], wj = a.w[j], hp = a.h[j - 1], wp = a.w[j - 1];
  const int tyn = cdiv(hj, RT), txn = cdiv(wj, CT);
  const int ntile = a.ns * tyn * txn;
  const int pitch = a.spitch[j];
  const T* Sj = reinterpret_cast<const T*>(sm + a.soff[j]);
  const float* Rin = (j < a.nlev) ? reinterpret_cast<const float*>(sm + a.roff[j + 1]) : nullptr;
  float* Rout = (j > 1) ? reinterpret_cast<float*>(sm + a.roff[j]) : nullptr;
  // taps of this lane's sub-band and channel pair: once per level
  float2 wr[K * K];
  {
    const float2* w = reinterpret_cast<const float2*>(wlev + sbi * kClDeepSetPitch) + cp;
#pragma unroll
    for (int t = 0; t < K * K; ++t) wr[t] = w[t * kClLanes];
  }
  // signs of the two butterfly stages for this lane: v' = partner + sign * v
  const float2 sg0 = (sbi & 1) ? make_float2(-1.f, -1.f) : make_float2(1.f, 1.f);
  const float2 sg1 = (sbi & 2) ? make_float2(-1.f, -1.f) : make_float2(1.f, 1.f);
  const int dy = sbi & 1, dx = sbi >> 1;                       // pixel of the 2 x 2 block this lane ends up with
  const bool chan_ok = c0 + 2 * cp < a.C, chan_pair = c0 + 2 * cp + 1 < a.C && (a.C & 1) == 0;
  // tile coordinates advance with the tile index (no division in the loop)
  const int per_slot = tyn * txn;
  int slot = warp / per_slot, rem = warp - slot * per_slot;
  int ty = rem / txn, tx = rem - ty * txn;
  const int dslot = nwarp / per_slot, drem = nwarp - dslot * per_slot, dty = drem / txn, dtx = drem - dty * txn;
  for (int q = warp; q < ntile; q += nwarp) {      // warp-uniform bound: every lane takes part in the shuffles
    const int gi = ty * RT, gj = tx * CT;
    float2 y[RT][CT];
#pragma unroll
    for (int i = 0; i < RT; ++i)
#pragma unroll
      for (int jj = 0; jj < CT; ++jj) y[i][jj] = make_float2(0.f, 0.f);
    if (Rin && sbi == 0) {                         // the deeper reconstruction joins the low-pass result
      const float* rb = Rin + (size_t)slot * a.rslot[j + 1] + (gi * wj + gj) * kClGroup + 2 * cp;
#pragma unroll
      for (int i = 0; i < RT; ++i)
#pragma unroll
        for (int jj = 0; jj < CT; ++jj)
          if (gi + i < hj && gj + jj < wj)
            y[i][jj] = __fmul2_rn(*reinterpret_cast<const float2*>(rb + (i * wj + jj) * kClGroup), make_float2(0.5f, 0.5f));
    }
    const T* win = Sj + (size_t)slot * a.sslot[j] + ((size_t)gi * pitch + gj) * POS + sbi * kClGroup + 2 * cp;
#pragma unroll
    for (int iy = 0; iy < RT + K - 1; ++iy) {
      float2 in[CT + K - 1];
#pragma unroll
      for (int c = 0; c < CT + K - 1; ++c) in[c] = ClPair<T>::load(win + (iy * pitch + c) * POS);
#pragma unroll
      for (int ddy = 0; ddy < K; ++ddy) {
        const int oy = iy - ddy;
        if (oy >= 0 && oy < RT) {
#pragma unroll
          for (int ddx = 0; ddx < K; ++ddx)
#pragma unroll
            for (int ox = 0; ox < CT; ++ox) y[oy][ox] = cl_fma2(in[ox + ddx], wr[ddy * K + ddx], y[oy][ox]);
        }
      }
    }
    // synthesis: out(2i+dy, 2j+dx) = LL + (-1)^dy LH + (-1)^dx HL + (-1)^(dy+dx) HH.  Two butterfly
    // stages over the sub-band bits of the lane; afterwards the lane of "sub-band" k holds the
    // pixel with dy = k & 1, dx = k >> 1.
    const int y0 = 2 * gi + dy, x0 = 2 * gj + dx;              // this lane's pixel of position (0, 0) of the tile
    float* obase;
    int rowstep, colstep;                                      // floats between the pixels of neighbouring positions
    bool writes;
    if (Rout) {
      obase = Rout + (size_t)slot * a.rslot[j] + (y0 * wp + x0) * kClGroup + 2 * cp;
      rowstep = 2 * wp * kClGroup; colstep = 2 * kClGroup;
      writes = true;
    } else {
      const int n = n0 + slot;
      obase = a.rout + (((size_t)n * hp + y0) * wp + x0) * a.C + c0 + 2 * cp;
      rowstep = 2 * wp * a.C; colstep = 2 * a.C;
      writes = n < a.B && chan_ok;
    }
    const bool vec = Rout || chan_pair;
#pragma unroll
    for (int i = 0; i < RT; ++i)
#pragma unroll
      for (int jj = 0; jj < CT; ++jj) {
        float2 v = y[i][jj], o;
        o.x = __shfl_xor_sync(kFull, v.x, 8);
        o.y = __shfl_xor_sync(kFull, v.y, 8);
        v = cl_fma2(v, sg0, o);
        o.x = __shfl_xor_sync(kFull, v.x, 16);
        o.y = __shfl_xor_sync(kFull, v.y, 16);
        v = cl_fma2(v, sg1, o);
        if (writes && y0 + 2 * i < hp && x0 + 2 * jj < wp) {
          float* g = obase + i * rowstep + jj * colstep;
          if (vec) *reinterpret_cast<float2*>(g) = v;
          else { g[0] = v.x; if (c0 + 2 * cp + 1 < a.C) g[1] = v.y; }
        }
      }
    // next tile of this warp
    slot += dslot; ty += dty; tx += dtx;
    if (tx >= txn) { tx -= txn; ++ty; }
    if (ty >= tyn) { ty -= tyn; ++slot; }
  }
}
#endif

template <typename T, int K>
__global__ void __launch_bounds__(kClDeepThreads, 2)
wt2d_cl_deep_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ ClDeepArgs a) {
#ifdef __CUDA_ARCH__
  static_assert(K == 5, "the staged tap sets are laid out for K = 5");
  constexpr int HS = K / 2;
  constexpr int TAPS = K * K + 1;
  constexpr int POS = 4 * kClGroup;
  constexpr unsigned kSetBytes = (unsigned)(TAPS * kClGroup * sizeof(float));
  extern __shared__ unsigned char cl_smem_raw[];
  unsigned char* sm = cl_smem_raw + ((128u - (cl_smem_addr(cl_smem_raw) & 127u)) & 127u);
  unsigned char* wbuf = sm + a.woff;                 // two buffers of the four tap sets of a level
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(sm + a.bar_off);   // two tap-set barriers, one for S_1
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int c0 = blockIdx.x * kClGroup;
  const int n0 = blockIdx.y * a.ns;
  const int nset = 1 + 4 * a.nlevels;
  const float* wsrc = a.packed + a.cl_off + (size_t)blockIdx.x * nset * (TAPS * kClGroup);

  // the four tap sets of on-chip level j (layer level index j, 0-based) -> buffer `buf`
  auto load_taps = [&](int j, int buf) {
    cl_mbar_expect_tx(&bars[buf], 4u * kSetBytes);
    for (int sb = 0; sb < 4; ++sb)
      cl_bulk_load(wbuf + (size_t)buf * kClDeepLevelBytes + (size_t)sb * kClDeepSetPitch,
                   wsrc + (size_t)(1 + 4 * (a.lvl0 + j) + sb) * (TAPS * kClGroup), kSetBytes, &bars[buf]);
  };

  cl_launch_dependents();
  if (tid == 0) {
    for (int s = 0; s < 3; ++s) cl_mbar_init(&bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    load_taps(a.nlev, 0);                            // deepest level first
    // the sub-bands come from the preceding kernel of the stream (this one may have been launched early)
    if (a.pdl) cl_wait_for_producer();
    // S_1 of every slot: one box over the four sub-bands, starting HS positions outside the plane
    cl_mbar_expect_tx(&bars[2], (unsigned)(a.ns * a.sslot[1] * (int)sizeof(T)));
    for (int sl = 0; sl < a.ns; ++sl)
      cl_tma_load5(sm + a.soff[1] + (size_t)sl * a.sslot[1] * sizeof(T), &xmap, &bars[2], c0, 0, -HS, -HS, n0 + sl);
  }
  // zero borders (and overhang) of the deeper frames (S_1 is filled whole by the TMA boxes)
  for (int i = tid; i < a.zero_bytes / 16; i += nthr)
    reinterpret_cast<uint4*>(sm + a.zero_off)[i] = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();
  bool ok = cl_mbar_wait(&bars[2], 0u);

  // ---- pass 2: analyses of the deeper levels, low-pass band of S_{j-1} -> S_j; a thread forms the
  // four sub-bands of one channel pair at one position
  for (int j = 2; j <= a.nlev; ++j) {
    const T* Sp = reinterpret_cast<const T*>(sm + a.soff[j - 1]);
    T* Sj = reinterpret_cast<T*>(sm + a.soff[j]);
    const unsigned hj = a.h[j], wj = a.w[j];
    const int pp_ = a.spitch[j - 1], pj = a.spitch[j];
    const unsigned items = a.ns * hj * wj * kClLanes;
    for (unsigned it = tid; it < items; it += nthr) {
      const int cp = it & (kClLanes - 1);
      const unsigned blk = it >> 3;
      const int f = (int)(blk % wj);
      const unsigned rs = blk / wj;
      const int r = (int)(rs % hj);
      const int slot = (int)(rs / hj);
      // positions (2r, 2f) .. (2r+1, 2f+1) of the low-pass band; beyond the plane the frame holds zeros
      const T* p = Sp + (size_t)slot * a.sslot[j - 1] + ((size_t)(2 * r + HS) * pp_ + 2 * f + HS) * POS + 2 * cp;
      const float2 va = ClPair<T>::load(p), vb = ClPair<T>::load(p + POS);
      const float2 vc = ClPair<T>::load(p + (size_t)pp_ * POS), vd = ClPair<T>::load(p + (size_t)pp_ * POS + POS);
      float2 sb[4];
      cl_haar(va, vb, vc, vd, sb);
      T* d = Sj + (size_t)slot * a.sslot[j] + ((size_t)(r + HS) * pj + f + HS) * POS + 2 * cp;
#pragma unroll
      for (int s4 = 0; s4 < 4; ++s4) ClPair<T>::store(d + s4 * kClGroup, sb[s4]);
    }
    __syncthreads();
  }

  // ---- pass 3: convolutions + synthesis, deepest level first; the tap sets of the next level are
  // copied while this one is computed
  int cur = 0;
  unsigned wphase[2] = {0u, 0u};
  for (int j = a.nlev; j >= 1; --j) {
    if (tid == 0 && j > 1) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the other buffer was read two levels ago
      load_taps(j - 1, 1 - cur);
    }
    ok = cl_mbar_wait(&bars[cur], wphase[cur]) && ok;
    wphase[cur] ^= 1u;
    const unsigned char* wlev = wbuf + (size_t)cur * kClDeepLevelBytes;
    if (a.h[j] * a.w[j] >= 32) cl_deep_level<T, K, kClRH, kClCW>(a, j, sm, wlev, c0, n0, tid, nthr);
    else cl_deep_level<T, K, 1, 2>(a, j, sm, wlev, c0, n0, tid, nthr);
    __syncthreads();
    cur ^= 1;
  }
  if (!ok && a.status) atomicExch(a.status, 1);
#endif
}

}  // namespace wt
