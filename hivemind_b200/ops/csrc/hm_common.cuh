// Shared device helpers for the sm_100a kernels of hivemind_b200.
//
// Conventions used by every kernel in this directory:
//  * every launcher is an `extern "C"` function that takes raw device pointers and a
//    `cudaStream_t` (passed from Python as an integer) and returns a `cudaError_t` as int;
//  * no launcher allocates device memory: callers own inputs, outputs and scratch;
//  * every wait on a flag, a peer or an mbarrier is bounded; a wait that runs out records
//    a status word that the host reads, and the kernel carries on or returns.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#define HM_API extern "C" __attribute__((visibility("default")))

enum HmDtype : int { HM_F32 = 0, HM_BF16 = 1, HM_F16 = 2 };

__device__ __forceinline__ float hm_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float hm_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `red` is shared scratch of at least 32 floats. All threads get the result.
__device__ __forceinline__ float hm_block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = hm_warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
    r = hm_warp_sum(r);
    if (lane == 0) red[0] = r;
  }
  __syncthreads();
  return red[0];
}
__device__ __forceinline__ float hm_block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = hm_warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nw) ? red[threadIdx.x] : -INFINITY;
  if (warp == 0) {
    r = hm_warp_max(r);
    if (lane == 0) red[0] = r;
  }
  __syncthreads();
  return red[0];
}

__device__ __forceinline__ float hm_load_as_float(const void* p, long long i, int dtype) {
  if (dtype == HM_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == HM_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ void hm_store_from_float(void* p, long long i, int dtype, float v) {
  if (dtype == HM_F32) reinterpret_cast<float*>(p)[i] = v;
  else if (dtype == HM_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(v);
  else reinterpret_cast<__half*>(p)[i] = __float2half(v);
}

__device__ __forceinline__ unsigned long long hm_globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// System-scope acquire load / release store for flags that another GPU writes or reads.
__device__ __forceinline__ unsigned int hm_ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void hm_st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ float hm_gelu_tanh(float x) {
  // 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}
__device__ __forceinline__ float hm_gelu_tanh_grad(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float x2 = x * x;
  float u = k0 * (x + k1 * x * x2);
  float t = tanhf(u);
  float du = k0 * (1.f + 3.f * k1 * x2);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}
