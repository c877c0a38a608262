// Stand-alone bandwidth check: how fast can the SMs of GPU 0 read GPU 1's memory (and their own, for comparison)
// with plain 8- and 16-byte loads at several depths per thread, and with bulk asynchronous copies into shared
// memory (cp.async.bulk completing on an mbarrier; every wait is bounded to 0.2 s and reported through a flag).
// One process, two GPUs with peer access; no kernel waits on another kernel. The device butterfly's data path is
// sized against these numbers.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o peer_read_bandwidth benchmarks/peer_read_bandwidth.cu
//   ./peer_read_bandwidth
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>
#include <cstdint>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1);} } while (0)

template <typename V, int U>
__global__ void __launch_bounds__(256) ld_kernel(const V* __restrict__ src, size_t n, float* sink) {
  float acc = 0.f;
  const size_t stride = (size_t)gridDim.x * 256 * U;
  for (size_t base = (size_t)blockIdx.x * 256 * U + threadIdx.x; base + (U - 1) * 256 < n; base += stride) {
    V v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = src[base + u * 256];
#pragma unroll
    for (int u = 0; u < U; ++u) acc += (float)(reinterpret_cast<const unsigned int*>(&v[u])[0] & 1);
  }
  if (acc == -1.f) *sink = acc;
}

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// each CTA: STAGES buffers of PIECE bytes; thread 0 keeps them full with cp.async.bulk; all threads "consume" by reading smem
template <int PIECE, int STAGES>
__global__ void __launch_bounds__(256) bulk_kernel(const unsigned char* __restrict__ src, size_t nbytes, float* sink, int* err) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long full[STAGES];
  const size_t n_pieces = nbytes / PIECE;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&full[s])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  float acc = 0.f;
  size_t issued = blockIdx.x, consumed = blockIdx.x;
  int is = 0;
  // prologue
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES && issued < n_pieces; ++s, issued += gridDim.x) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(&full[s])), "r"(PIECE) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   :: "r"(smem_u32(smem + (size_t)s * PIECE)), "l"(src + issued * PIECE), "r"(PIECE), "r"(smem_u32(&full[s])) : "memory");
    }
  }
  int phase_bits = 0;
  for (; consumed < n_pieces; consumed += gridDim.x) {
    const int s = is;
    const unsigned parity = (phase_bits >> s) & 1;
    unsigned ok = 0;
    unsigned long long t0; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    while (true) {
      asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                   : "=r"(ok) : "r"(smem_u32(&full[s])), "r"(parity) : "memory");
      if (ok) break;
      unsigned long long t1; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > 200000000ull) { *err = 1; return; }  // 0.2 s: give up
    }
    const uint4* p = reinterpret_cast<const uint4*>(smem + (size_t)s * PIECE);
#pragma unroll 4
    for (int q = threadIdx.x; q < PIECE / 16; q += 256) acc += (float)(p[q].x & 1);
    __syncthreads();
    phase_bits ^= 1 << s;
    if (threadIdx.x == 0 && issued < n_pieces) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(&full[s])), "r"(PIECE) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   :: "r"(smem_u32(smem + (size_t)s * PIECE)), "l"(src + issued * PIECE), "r"(PIECE), "r"(smem_u32(&full[s])) : "memory");
      issued += gridDim.x;
    }
    is = (is + 1) % STAGES;
  }
  if (acc == -1.f) *sink = acc;
}

template <typename F>
float time_ms(F f) {
  cudaEvent_t a, b; CK(cudaEventCreate(&a)); CK(cudaEventCreate(&b));
  for (int i = 0; i < 2; ++i) f();
  CK(cudaDeviceSynchronize());
  CK(cudaEventRecord(a));
  for (int i = 0; i < 5; ++i) f();
  CK(cudaEventRecord(b)); CK(cudaEventSynchronize(b));
  float ms; CK(cudaEventElapsedTime(&ms, a, b));
  CK(cudaGetLastError());
  return ms / 5;
}

int main() {
  int ndev = 0; CK(cudaGetDeviceCount(&ndev));
  const size_t bytes = 256ull << 20;
  unsigned char *local, *remote = nullptr; float* sink; int* err;
  CK(cudaSetDevice(0));
  CK(cudaMalloc(&local, bytes)); CK(cudaMemset(local, 1, bytes)); CK(cudaMalloc(&sink, 4)); CK(cudaMalloc(&err, 4)); CK(cudaMemset(err, 0, 4));
  if (ndev > 1) {
    int can = 0; CK(cudaDeviceCanAccessPeer(&can, 0, 1));
    if (can) { CK(cudaSetDevice(1)); CK(cudaMalloc(&remote, bytes)); CK(cudaMemset(remote, 1, bytes)); CK(cudaDeviceSynchronize()); CK(cudaSetDevice(0)); CK(cudaDeviceEnablePeerAccess(1, 0)); }
  }
  cudaDeviceProp prop; CK(cudaGetDeviceProperties(&prop, 0));
  const int sms = prop.multiProcessorCount;
  for (int where = 0; where < 2; ++where) {
    const unsigned char* src = where ? remote : local;
    if (!src) continue;
    const char* name = where ? "remote" : "local";
    for (int per_sm : {2, 4, 8}) {
      const int grid = sms * per_sm;
      float ms;
      ms = time_ms([&] { ld_kernel<uint4, 4><<<grid, 256>>>((const uint4*)src, bytes / 16, sink); });
      printf("%s ld16 U=4  ctas/sm=%d: %.1f GB/s\n", name, per_sm, bytes / ms / 1e6);
      ms = time_ms([&] { ld_kernel<uint4, 8><<<grid, 256>>>((const uint4*)src, bytes / 16, sink); });
      printf("%s ld16 U=8  ctas/sm=%d: %.1f GB/s\n", name, per_sm, bytes / ms / 1e6);
      ms = time_ms([&] { ld_kernel<uint4, 16><<<grid, 256>>>((const uint4*)src, bytes / 16, sink); });
      printf("%s ld16 U=16 ctas/sm=%d: %.1f GB/s\n", name, per_sm, bytes / ms / 1e6);
      ms = time_ms([&] { ld_kernel<uint2, 4><<<grid, 256>>>((const uint2*)src, bytes / 8, sink); });
      printf("%s ld8  U=4  ctas/sm=%d: %.1f GB/s\n", name, per_sm, bytes / ms / 1e6);
      ms = time_ms([&] { ld_kernel<uint2, 8><<<grid, 256>>>((const uint2*)src, bytes / 8, sink); });
      printf("%s ld8  U=8  ctas/sm=%d: %.1f GB/s\n", name, per_sm, bytes / ms / 1e6);
    }
    {
      CK(cudaFuncSetAttribute(bulk_kernel<16384, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 * 4));
      CK(cudaFuncSetAttribute(bulk_kernel<32768, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * 3));
      CK(cudaFuncSetAttribute(bulk_kernel<8192, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8192 * 4));
      for (int per_sm : {1, 2, 3}) {
        const int grid = sms * per_sm;
        float ms = time_ms([&] { bulk_kernel<16384, 4><<<grid, 256, 16384 * 4>>>(src, bytes, sink, err); });
        printf("%s bulk 16K x4 ctas/sm=%d: %.1f GB/s\n", name, per_sm, bytes / ms / 1e6);
        ms = time_ms([&] { bulk_kernel<32768, 3><<<grid, 256, 32768 * 3>>>(src, bytes, sink, err); });
        printf("%s bulk 32K x3 ctas/sm=%d: %.1f GB/s\n", name, per_sm, bytes / ms / 1e6);
        ms = time_ms([&] { bulk_kernel<8192, 4><<<grid, 256, 8192 * 4>>>(src, bytes, sink, err); });
        printf("%s bulk  8K x4 ctas/sm=%d: %.1f GB/s\n", name, per_sm, bytes / ms / 1e6);
      }
    }
    int herr = 0; CK(cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost));
    printf("%s wait-timeout flag: %d\n", name, herr);
    // copy engine for reference
    float ms = time_ms([&] { CK(cudaMemcpyAsync(local, src, bytes, cudaMemcpyDefault, 0)); });
    if (where) printf("remote cudaMemcpy: %.1f GB/s\n", bytes / ms / 1e6);
  }
  return 0;
}
