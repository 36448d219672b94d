// Stand-alone microbenchmark (not part of the library): sustained issue rates of scalar FFMA,
// packed fma.rn.f32x2, HFMA2 (bf16 / fp16) and FFMA mixed with 128-bit shared-memory loads on
// sm_100a.  These set the FP32-issue ceiling the depthwise WTConv kernels are designed against.
// Build: make -C wtconv_b200/csrc fma_issue      Run: wtconv_b200/csrc/build/fma_issue
#include <cstdio>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#define CK(x) do{cudaError_t e=(x); if(e!=cudaSuccess){printf("ERR %s line %d\n", cudaGetErrorString(e), __LINE__); return 1;}}while(0)

constexpr int ITER = 4096;
constexpr int NACC = 16;

__global__ void k_ffma(float* out, float a, float b, long long* cyc) {
  float acc[NACC];
  #pragma unroll
  for (int i=0;i<NACC;i++) acc[i] = threadIdx.x*0.001f + i;
  long long t0 = clock64();
  for (int it=0; it<ITER; ++it) {
    #pragma unroll
    for (int i=0;i<NACC;i++) acc[i] = fmaf(acc[i], a, b);
  }
  long long t1 = clock64();
  float s=0; 
  #pragma unroll
  for (int i=0;i<NACC;i++) s+=acc[i];
  out[blockIdx.x*blockDim.x+threadIdx.x]=s;
  if (threadIdx.x==0) cyc[blockIdx.x]=t1-t0;
}

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  unsigned long long ra = *reinterpret_cast<unsigned long long*>(&a);
  unsigned long long rb = *reinterpret_cast<unsigned long long*>(&b);
  unsigned long long rc = *reinterpret_cast<unsigned long long*>(&c);
  unsigned long long rd;
  asm volatile("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  return *reinterpret_cast<float2*>(&rd);
}

__global__ void k_ffma2(float* out, float a, float b, long long* cyc) {
  float2 acc[NACC];
  #pragma unroll
  for (int i=0;i<NACC;i++) acc[i] = make_float2(threadIdx.x*0.001f + i, i*0.5f);
  float2 aa = make_float2(a, a*0.99f), bb = make_float2(b, b*1.01f);
  long long t0 = clock64();
  for (int it=0; it<ITER; ++it) {
    #pragma unroll
    for (int i=0;i<NACC;i++) acc[i] = ffma2(acc[i], aa, bb);
  }
  long long t1 = clock64();
  float s=0; 
  #pragma unroll
  for (int i=0;i<NACC;i++) s+=acc[i].x+acc[i].y;
  out[blockIdx.x*blockDim.x+threadIdx.x]=s;
  if (threadIdx.x==0) cyc[blockIdx.x]=t1-t0;
}

__global__ void k_hfma2_bf16(float* out, float a, float b, long long* cyc) {
  __nv_bfloat162 acc[NACC];
  #pragma unroll
  for (int i=0;i<NACC;i++) acc[i] = __floats2bfloat162_rn(threadIdx.x*0.001f + i, i*0.5f);
  __nv_bfloat162 aa = __floats2bfloat162_rn(a, a*0.99f), bb = __floats2bfloat162_rn(b, b*1.01f);
  long long t0 = clock64();
  for (int it=0; it<ITER; ++it) {
    #pragma unroll
    for (int i=0;i<NACC;i++) acc[i] = __hfma2(acc[i], aa, bb);
  }
  long long t1 = clock64();
  float s=0; 
  #pragma unroll
  for (int i=0;i<NACC;i++) s+=__low2float(acc[i])+__high2float(acc[i]);
  out[blockIdx.x*blockDim.x+threadIdx.x]=s;
  if (threadIdx.x==0) cyc[blockIdx.x]=t1-t0;
}

__global__ void k_hfma2_f16(float* out, float a, float b, long long* cyc) {
  __half2 acc[NACC];
  #pragma unroll
  for (int i=0;i<NACC;i++) acc[i] = __floats2half2_rn(threadIdx.x*0.001f + i, i*0.5f);
  __half2 aa = __floats2half2_rn(a, a*0.99f), bb = __floats2half2_rn(b, b*1.01f);
  long long t0 = clock64();
  for (int it=0; it<ITER; ++it) {
    #pragma unroll
    for (int i=0;i<NACC;i++) acc[i] = __hfma2(acc[i], aa, bb);
  }
  long long t1 = clock64();
  float s=0; 
  #pragma unroll
  for (int i=0;i<NACC;i++) s+=__low2float(acc[i])+__high2float(acc[i]);
  out[blockIdx.x*blockDim.x+threadIdx.x]=s;
  if (threadIdx.x==0) cyc[blockIdx.x]=t1-t0;
}

// FFMA mixed with LDS.128: R ffma per LDS.128 (4 floats)
template<int FPL, bool PACKED>
__global__ void k_mix(float* out, float a, long long* cyc) {
  __shared__ float4 sm[2048];
  for (int i=threadIdx.x;i<2048;i+=blockDim.x) sm[i]=make_float4(i*1e-3f,1.f,2.f,3.f);
  __syncthreads();
  float acc[16];
  #pragma unroll
  for (int i=0;i<16;i++) acc[i]=i;
  int idx = threadIdx.x;
  long long t0 = clock64();
  for (int it=0; it<ITER/4; ++it) {
    #pragma unroll
    for (int u=0;u<4;u++){
      float4 v = sm[(idx + u*256 + it) & 2047];
      float vv[4] = {v.x,v.y,v.z,v.w};
      if (!PACKED) {
        #pragma unroll
        for (int f=0; f<FPL; ++f) acc[f%16] = fmaf(vv[f%4], a, acc[f%16]);
      } else {
        #pragma unroll
        for (int f=0; f<FPL/2; ++f) {
          float2 c = make_float2(acc[(2*f)%16], acc[(2*f+1)%16]);
          float2 x = make_float2(vv[(2*f)%4], vv[(2*f+1)%4]);
          float2 r = ffma2(x, make_float2(a,a), c);
          acc[(2*f)%16]=r.x; acc[(2*f+1)%16]=r.y;
        }
      }
    }
  }
  long long t1 = clock64();
  float s=0;
  #pragma unroll
  for (int i=0;i<16;i++) s+=acc[i];
  out[blockIdx.x*blockDim.x+threadIdx.x]=s;
  if (threadIdx.x==0) cyc[blockIdx.x]=t1-t0;
}

template<typename F> int run(const char* name, F launch, double fma_per_thread, int blocks, int threads, float* out, long long* cyc) {
  launch(); CK(cudaDeviceSynchronize());
  cudaEvent_t e0,e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  cudaEventRecord(e0); launch(); cudaEventRecord(e1); CK(cudaEventSynchronize(e1));
  float ms; cudaEventElapsedTime(&ms,e0,e1);
  long long hc[4096]; CK(cudaMemcpy(hc,cyc,sizeof(long long)*blocks,cudaMemcpyDeviceToHost));
  double avg=0; for(int i=0;i<blocks;i++) avg+=hc[i]; avg/=blocks;
  int sms=148; double blocks_per_sm = (double)blocks/sms;
  double fma_per_sm = fma_per_thread*threads*blocks_per_sm;
  printf("%-28s ms=%.3f cyc/block=%.0f  FMA/clk/SM=%.1f  TFMA/s(total)=%.2f\n", name, ms, avg, fma_per_sm/avg, fma_per_thread*threads*blocks/(ms*1e-3)/1e12);
  return 0;
}

int main(){
  int blocks=148*4, threads=256;   // 1024 threads/SM
  float* out; long long* cyc; CK(cudaMalloc(&out, sizeof(float)*blocks*threads)); CK(cudaMalloc(&cyc,sizeof(long long)*4096));
  cudaDeviceProp p; cudaGetDeviceProperties(&p,0); printf("%s SMs=%d clock=%d kHz smemPerSM=%zu\n", p.name,p.multiProcessorCount,p.clockRate,p.sharedMemPerMultiprocessor);
  for (int rep=0; rep<2; ++rep) {
  run("ffma scalar", [&]{k_ffma<<<blocks,threads>>>(out,1.0001f,0.5f,cyc);}, (double)ITER*NACC, blocks,threads,out,cyc);
  run("ffma2 packed", [&]{k_ffma2<<<blocks,threads>>>(out,1.0001f,0.5f,cyc);}, (double)ITER*NACC*2, blocks,threads,out,cyc);
  run("hfma2 bf16", [&]{k_hfma2_bf16<<<blocks,threads>>>(out,1.0001f,0.5f,cyc);}, (double)ITER*NACC*2, blocks,threads,out,cyc);
  run("hfma2 f16", [&]{k_hfma2_f16<<<blocks,threads>>>(out,1.0001f,0.5f,cyc);}, (double)ITER*NACC*2, blocks,threads,out,cyc);
  run("mix scalar 4 fma/LDS128", [&]{k_mix<4,false><<<blocks,threads>>>(out,1.0001f,cyc);}, (double)ITER*4, blocks,threads,out,cyc);
  run("mix scalar 8 fma/LDS128", [&]{k_mix<8,false><<<blocks,threads>>>(out,1.0001f,cyc);}, (double)ITER*8, blocks,threads,out,cyc);
  run("mix scalar 16 fma/LDS128", [&]{k_mix<16,false><<<blocks,threads>>>(out,1.0001f,cyc);}, (double)ITER*16, blocks,threads,out,cyc);
  run("mix scalar 32 fma/LDS128", [&]{k_mix<32,false><<<blocks,threads>>>(out,1.0001f,cyc);}, (double)ITER*32, blocks,threads,out,cyc);
  run("mix packed 8 fma/LDS128", [&]{k_mix<8,true><<<blocks,threads>>>(out,1.0001f,cyc);}, (double)ITER*8, blocks,threads,out,cyc);
  run("mix packed 16 fma/LDS128", [&]{k_mix<16,true><<<blocks,threads>>>(out,1.0001f,cyc);}, (double)ITER*16, blocks,threads,out,cyc);
  run("mix packed 32 fma/LDS128", [&]{k_mix<32,true><<<blocks,threads>>>(out,1.0001f,cyc);}, (double)ITER*32, blocks,threads,out,cyc);
  }
  // 512 threads/SM occupancy variant
  blocks=148*2;
  run("ffma scalar 512thr/SM", [&]{k_ffma<<<blocks,threads>>>(out,1.0001f,0.5f,cyc);}, (double)ITER*NACC, blocks,threads,out,cyc);
  run("ffma2 packed 512thr/SM", [&]{k_ffma2<<<blocks,threads>>>(out,1.0001f,0.5f,cyc);}, (double)ITER*NACC*2, blocks,threads,out,cyc);
  printf("done\n");
  return 0;
}
