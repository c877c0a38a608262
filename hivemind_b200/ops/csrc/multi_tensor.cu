// Multi-tensor elementwise kernels: gradient accumulation, scaling, zeroing, finite check,
// per-tensor norms, and the optimizer updates (SGD, Adam/AdamW, LAMB).
//
// One launch covers any number of tensors. The host uploads two tables once per parameter set:
//   tensors: int64[T][8] = {ptr0, ptr1, ptr2, ptr3, ptr4, ptr5, numel, dtypes}
//            (dtypes packs one HmDtype per pointer slot, 4 bits each, slot 0 in the low bits)
//   chunks : int32[C][2] = {tensor index, chunk index inside that tensor}
// and each CTA processes one chunk of HM_MT_CHUNK elements. The meaning of the pointer slots is
// given beside each kernel.
//
// These replace the ATen call sites of the reference's optimizer path:
//   hivemind/optim/grad_averager.py:130-148,204-219 (accumulate, scale, zero),
//   hivemind/optim/grad_scaler.py:59-74,118-127 (unscale + finite check),
//   hivemind/optim/state_averager.py:515-523 (optimizer.step; LAMB per examples/albert/run_trainer.py:240-248),
//   hivemind/moe/server/layers/optim.py:53-57 (global-norm clipping).
#include "hm_common.cuh"

#define HM_MT_CHUNK 16384
#define HM_MT_THREADS 256

struct MtRef {
  void* p[6];
  long long n;
  int dt[6];
};

__device__ __forceinline__ bool mt_setup(const long long* tensors, const int* chunks, MtRef& r, long long& lo,
                                         long long& hi) {
  const int t = chunks[2 * blockIdx.x], c = chunks[2 * blockIdx.x + 1];
  const long long* row = tensors + 8LL * t;
#pragma unroll
  for (int s = 0; s < 6; ++s) {
    r.p[s] = reinterpret_cast<void*>(row[s]);
    r.dt[s] = int((row[7] >> (4 * s)) & 15);
  }
  r.n = row[6];
  lo = (long long)c * HM_MT_CHUNK;
  hi = lo + HM_MT_CHUNK < r.n ? lo + HM_MT_CHUNK : r.n;
  return lo < hi;
}

__device__ __forceinline__ int mt_tensor_index(const int* chunks) { return chunks[2 * blockIdx.x]; }

// 4-wide access helpers. `vec` says that the slot's address at element `i` is suitably aligned.
__device__ __forceinline__ void mt_load4(const void* p, long long i, int dt, bool vec, long long hi, float v[4]) {
  if (vec && i + 4 <= hi) {
    if (dt == HM_F32) {
      float4 x = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
      v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    } else if (dt == HM_BF16) {
      uint2 x = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
      __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&x.x), b = *reinterpret_cast<__nv_bfloat162*>(&x.y);
      v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    } else {
      uint2 x = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(p) + i);
      __half2 a = *reinterpret_cast<__half2*>(&x.x), b = *reinterpret_cast<__half2*>(&x.y);
      v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = (i + k < hi) ? hm_load_as_float(p, i + k, dt) : 0.f;
  }
}
__device__ __forceinline__ void mt_store4(void* p, long long i, int dt, bool vec, long long hi, const float v[4]) {
  if (vec && i + 4 <= hi) {
    if (dt == HM_F32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = make_float4(v[0], v[1], v[2], v[3]);
    } else if (dt == HM_BF16) {
      __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
      uint2 x;
      x.x = *reinterpret_cast<unsigned int*>(&a);
      x.y = *reinterpret_cast<unsigned int*>(&b);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = x;
    } else {
      __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
      uint2 x;
      x.x = *reinterpret_cast<unsigned int*>(&a);
      x.y = *reinterpret_cast<unsigned int*>(&b);
      *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p) + i) = x;
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (i + k < hi) hm_store_from_float(p, i + k, dt, v[k]);
  }
}
__device__ __forceinline__ bool mt_aligned(const void* p, int dt) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  return p != nullptr && (a % (dt == HM_F32 ? 16 : 8)) == 0;
}

// ------------------------------------------------------------------------------------------------
// op codes for the simple elementwise kernel
enum MtOp : int {
  MT_AXPY = 0,        // p0 += alpha * p1
  MT_SCALE_COPY = 1,  // p0 = alpha * p1
  MT_ZERO = 2,        // p0 = 0
  MT_SCALE_CHECK = 3, // p0 *= alpha ; flag |= any non-finite in p0 (before scaling)
  MT_DELTA = 4,       // p0 += alpha * (p1 - p2)         (delta rule: local += new - old)
  MT_COPY2 = 5        // p0 = p2 = p1                    (two destinations, e.g. fp32 master + bf16 copy)
};

__global__ void __launch_bounds__(HM_MT_THREADS)
mt_elementwise_kernel(const long long* __restrict__ tensors, const int* __restrict__ chunks, int op, float alpha,
                      int* __restrict__ flag) {
  MtRef r;
  long long lo, hi;
  if (!mt_setup(tensors, chunks, r, lo, hi)) return;
  const bool v0 = mt_aligned(r.p[0], r.dt[0]);
  const bool v1 = mt_aligned(r.p[1], r.dt[1]);
  const bool v2 = mt_aligned(r.p[2], r.dt[2]);
  bool bad = false;
  for (long long i = lo + 4LL * threadIdx.x; i < hi; i += 4LL * HM_MT_THREADS) {
    float a[4], b[4], c[4];
    switch (op) {
      case MT_AXPY:
        mt_load4(r.p[0], i, r.dt[0], v0, hi, a);
        mt_load4(r.p[1], i, r.dt[1], v1, hi, b);
#pragma unroll
        for (int k = 0; k < 4; ++k) a[k] = fmaf(alpha, b[k], a[k]);
        mt_store4(r.p[0], i, r.dt[0], v0, hi, a);
        break;
      case MT_SCALE_COPY:
        mt_load4(r.p[1], i, r.dt[1], v1, hi, b);
#pragma unroll
        for (int k = 0; k < 4; ++k) a[k] = alpha * b[k];
        mt_store4(r.p[0], i, r.dt[0], v0, hi, a);
        break;
      case MT_ZERO:
#pragma unroll
        for (int k = 0; k < 4; ++k) a[k] = 0.f;
        mt_store4(r.p[0], i, r.dt[0], v0, hi, a);
        break;
      case MT_SCALE_CHECK:
        mt_load4(r.p[0], i, r.dt[0], v0, hi, a);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          bad |= !isfinite(a[k]);
          a[k] *= alpha;
        }
        if (alpha != 1.f) mt_store4(r.p[0], i, r.dt[0], v0, hi, a);
        break;
      case MT_DELTA:
        mt_load4(r.p[0], i, r.dt[0], v0, hi, a);
        mt_load4(r.p[1], i, r.dt[1], v1, hi, b);
        mt_load4(r.p[2], i, r.dt[2], v2, hi, c);
#pragma unroll
        for (int k = 0; k < 4; ++k) a[k] += alpha * (b[k] - c[k]);
        mt_store4(r.p[0], i, r.dt[0], v0, hi, a);
        break;
      case MT_COPY2:
        mt_load4(r.p[1], i, r.dt[1], v1, hi, b);
        mt_store4(r.p[0], i, r.dt[0], v0, hi, b);
        if (r.p[2]) mt_store4(r.p[2], i, r.dt[2], v2, hi, b);
        break;
    }
  }
  if (op == MT_SCALE_CHECK && __syncthreads_or(bad) && threadIdx.x == 0) atomicOr(flag, 1);
}

// Per-tensor sum of squares of slot `slot` into out[tensor] (float atomics; `out` zeroed by the caller),
// and the grand total into out[num_tensors].
__global__ void __launch_bounds__(HM_MT_THREADS)
mt_sumsq_kernel(const long long* __restrict__ tensors, const int* __restrict__ chunks, int slot, int num_tensors,
                float* __restrict__ out) {
  __shared__ float red[32];
  MtRef r;
  long long lo, hi;
  if (!mt_setup(tensors, chunks, r, lo, hi)) return;
  const bool v = mt_aligned(r.p[slot], r.dt[slot]);
  float acc = 0.f;
  for (long long i = lo + 4LL * threadIdx.x; i < hi; i += 4LL * HM_MT_THREADS) {
    float a[4];
    mt_load4(r.p[slot], i, r.dt[slot], v, hi, a);
#pragma unroll
    for (int k = 0; k < 4; ++k) acc = fmaf(a[k], a[k], acc);
  }
  acc = hm_block_sum(acc, red);
  if (threadIdx.x == 0) {
    atomicAdd(out + mt_tensor_index(chunks), acc);
    atomicAdd(out + num_tensors, acc);
  }
}

// p0 *= min(1, max_norm / (sqrt(total[num_tensors]) + 1e-6))   (torch.nn.utils.clip_grad_norm_ semantics)
__global__ void __launch_bounds__(HM_MT_THREADS)
mt_clip_kernel(const long long* __restrict__ tensors, const int* __restrict__ chunks, const float* __restrict__ sumsq,
               int num_tensors, float max_norm) {
  MtRef r;
  long long lo, hi;
  if (!mt_setup(tensors, chunks, r, lo, hi)) return;
  const float coef = max_norm / (sqrtf(sumsq[num_tensors]) + 1e-6f);
  if (coef >= 1.f) return;
  const bool v0 = mt_aligned(r.p[0], r.dt[0]);
  for (long long i = lo + 4LL * threadIdx.x; i < hi; i += 4LL * HM_MT_THREADS) {
    float a[4];
    mt_load4(r.p[0], i, r.dt[0], v0, hi, a);
#pragma unroll
    for (int k = 0; k < 4; ++k) a[k] *= coef;
    mt_store4(r.p[0], i, r.dt[0], v0, hi, a);
  }
}

// ------------------------------------------------------------------------------------------------
// Optimizer updates. Slots: p0 = param (fp32 master), p1 = grad (any dtype), p2 = exp_avg, p3 = exp_avg_sq,
// p4 = optional low-precision model copy written back with the new value, p5 = LAMB update scratch (fp32).
struct HmOptArgs {
  float lr, beta1, beta2, eps, weight_decay;
  float bias1, bias2;   // 1 - beta1^t, 1 - beta2^t
  float grad_scale;     // gradients are multiplied by this before use (1/loss_scale, 1/accumulations, clip)
  float momentum, dampening, clamp_value;
  int decoupled_wd;     // AdamW (1) vs Adam with L2 (0)
  int nesterov, first_step, debias;
};

__global__ void __launch_bounds__(HM_MT_THREADS)
mt_adam_kernel(const long long* __restrict__ tensors, const int* __restrict__ chunks, HmOptArgs h) {
  MtRef r;
  long long lo, hi;
  if (!mt_setup(tensors, chunks, r, lo, hi)) return;
  bool v[5];
#pragma unroll
  for (int s = 0; s < 5; ++s) v[s] = mt_aligned(r.p[s], r.dt[s]);
  const float step_size = h.lr / h.bias1;
  const float inv_sqrt_b2 = rsqrtf(h.bias2);
  for (long long i = lo + 4LL * threadIdx.x; i < hi; i += 4LL * HM_MT_THREADS) {
    float p[4], g[4], m[4], q[4];
    mt_load4(r.p[0], i, r.dt[0], v[0], hi, p);
    mt_load4(r.p[1], i, r.dt[1], v[1], hi, g);
    mt_load4(r.p[2], i, r.dt[2], v[2], hi, m);
    mt_load4(r.p[3], i, r.dt[3], v[3], hi, q);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float gk = g[k] * h.grad_scale;
      if (h.decoupled_wd) p[k] *= (1.f - h.lr * h.weight_decay);
      else gk = fmaf(h.weight_decay, p[k], gk);
      m[k] = fmaf(h.beta1, m[k], (1.f - h.beta1) * gk);
      q[k] = fmaf(h.beta2, q[k], (1.f - h.beta2) * gk * gk);
      const float denom = sqrtf(q[k]) * inv_sqrt_b2 + h.eps;
      p[k] -= step_size * m[k] / denom;
    }
    mt_store4(r.p[0], i, r.dt[0], v[0], hi, p);
    mt_store4(r.p[2], i, r.dt[2], v[2], hi, m);
    mt_store4(r.p[3], i, r.dt[3], v[3], hi, q);
    if (r.p[4]) mt_store4(r.p[4], i, r.dt[4], v[4], hi, p);
  }
}

__global__ void __launch_bounds__(HM_MT_THREADS)
mt_sgd_kernel(const long long* __restrict__ tensors, const int* __restrict__ chunks, HmOptArgs h) {
  MtRef r;
  long long lo, hi;
  if (!mt_setup(tensors, chunks, r, lo, hi)) return;
  bool v[5];
#pragma unroll
  for (int s = 0; s < 5; ++s) v[s] = mt_aligned(r.p[s], r.dt[s]);
  const bool has_mom = h.momentum != 0.f && r.p[2] != nullptr;
  for (long long i = lo + 4LL * threadIdx.x; i < hi; i += 4LL * HM_MT_THREADS) {
    float p[4], g[4], m[4];
    mt_load4(r.p[0], i, r.dt[0], v[0], hi, p);
    mt_load4(r.p[1], i, r.dt[1], v[1], hi, g);
    if (has_mom) mt_load4(r.p[2], i, r.dt[2], v[2], hi, m);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float gk = fmaf(h.weight_decay, p[k], g[k] * h.grad_scale);
      if (has_mom) {
        m[k] = h.first_step ? gk : fmaf(h.momentum, m[k], (1.f - h.dampening) * gk);
        gk = h.nesterov ? fmaf(h.momentum, m[k], gk) : m[k];
      }
      p[k] -= h.lr * gk;
    }
    mt_store4(r.p[0], i, r.dt[0], v[0], hi, p);
    if (has_mom) mt_store4(r.p[2], i, r.dt[2], v[2], hi, m);
    if (r.p[4]) mt_store4(r.p[4], i, r.dt[4], v[4], hi, p);
  }
}

// LAMB stage 1: moments, adam step u = m / (sqrt(v) + eps) + wd * p into scratch slot 5, and the per-tensor
// squared norms of p and u into norms[2*t], norms[2*t+1] (zeroed by the caller).
__global__ void __launch_bounds__(HM_MT_THREADS)
mt_lamb_stage1_kernel(const long long* __restrict__ tensors, const int* __restrict__ chunks, HmOptArgs h,
                      float* __restrict__ norms) {
  __shared__ float red[32];
  MtRef r;
  long long lo, hi;
  if (!mt_setup(tensors, chunks, r, lo, hi)) return;
  bool v[6];
#pragma unroll
  for (int s = 0; s < 6; ++s) v[s] = mt_aligned(r.p[s], r.dt[s]);
  float pn = 0.f, un = 0.f;
  for (long long i = lo + 4LL * threadIdx.x; i < hi; i += 4LL * HM_MT_THREADS) {
    float p[4], g[4], m[4], q[4], u[4];
    mt_load4(r.p[0], i, r.dt[0], v[0], hi, p);
    mt_load4(r.p[1], i, r.dt[1], v[1], hi, g);
    mt_load4(r.p[2], i, r.dt[2], v[2], hi, m);
    mt_load4(r.p[3], i, r.dt[3], v[3], hi, q);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = g[k] * h.grad_scale;
      m[k] = fmaf(h.beta1, m[k], (1.f - h.beta1) * gk);
      q[k] = fmaf(h.beta2, q[k], (1.f - h.beta2) * gk * gk);
      u[k] = m[k] / (sqrtf(q[k]) + h.eps) + h.weight_decay * p[k];
      if (i + k < hi) {
        pn = fmaf(p[k], p[k], pn);
        un = fmaf(u[k], u[k], un);
      }
    }
    mt_store4(r.p[2], i, r.dt[2], v[2], hi, m);
    mt_store4(r.p[3], i, r.dt[3], v[3], hi, q);
    mt_store4(r.p[5], i, r.dt[5], v[5], hi, u);
  }
  pn = hm_block_sum(pn, red);
  un = hm_block_sum(un, red);
  if (threadIdx.x == 0) {
    const int t = mt_tensor_index(chunks);
    atomicAdd(norms + 2 * t, pn);
    atomicAdd(norms + 2 * t + 1, un);
  }
}

// LAMB stage 2: p -= lr * bias_correction * trust_ratio(t) * u, with
// trust = clamp(|p|, 0, clamp_value) / |u| (1 when either norm is zero).
__global__ void __launch_bounds__(HM_MT_THREADS)
mt_lamb_stage2_kernel(const long long* __restrict__ tensors, const int* __restrict__ chunks, HmOptArgs h,
                      const float* __restrict__ norms) {
  MtRef r;
  long long lo, hi;
  if (!mt_setup(tensors, chunks, r, lo, hi)) return;
  const int t = mt_tensor_index(chunks);
  const float wn = fminf(sqrtf(norms[2 * t]), h.clamp_value), un = sqrtf(norms[2 * t + 1]);
  const float trust = (wn == 0.f || un == 0.f) ? 1.f : wn / un;
  const float bc = h.debias ? sqrtf(h.bias2) / h.bias1 : 1.f;
  const float step = h.lr * bc * trust;
  const bool v0 = mt_aligned(r.p[0], r.dt[0]), v4 = mt_aligned(r.p[4], r.dt[4]), v5 = mt_aligned(r.p[5], r.dt[5]);
  for (long long i = lo + 4LL * threadIdx.x; i < hi; i += 4LL * HM_MT_THREADS) {
    float p[4], u[4];
    mt_load4(r.p[0], i, r.dt[0], v0, hi, p);
    mt_load4(r.p[5], i, r.dt[5], v5, hi, u);
#pragma unroll
    for (int k = 0; k < 4; ++k) p[k] = fmaf(-step, u[k], p[k]);
    mt_store4(r.p[0], i, r.dt[0], v0, hi, p);
    if (r.p[4]) mt_store4(r.p[4], i, r.dt[4], v4, hi, p);
  }
}

// ------------------------------------------------------------------------------------------------
HM_API int hm_mt_chunk_size() { return HM_MT_CHUNK; }

HM_API int hm_mt_elementwise(const void* tensors, const void* chunks, int num_chunks, int op, float alpha, void* flag,
                             cudaStream_t stream) {
  if (num_chunks <= 0) return 0;
  mt_elementwise_kernel<<<num_chunks, HM_MT_THREADS, 0, stream>>>((const long long*)tensors, (const int*)chunks, op,
                                                                  alpha, (int*)flag);
  return (int)cudaGetLastError();
}

HM_API int hm_mt_sumsq(const void* tensors, const void* chunks, int num_chunks, int slot, int num_tensors, void* out,
                       cudaStream_t stream) {
  if (num_chunks <= 0) return 0;
  mt_sumsq_kernel<<<num_chunks, HM_MT_THREADS, 0, stream>>>((const long long*)tensors, (const int*)chunks, slot,
                                                            num_tensors, (float*)out);
  return (int)cudaGetLastError();
}

HM_API int hm_mt_clip(const void* tensors, const void* chunks, int num_chunks, const void* sumsq, int num_tensors,
                      float max_norm, cudaStream_t stream) {
  if (num_chunks <= 0) return 0;
  mt_clip_kernel<<<num_chunks, HM_MT_THREADS, 0, stream>>>((const long long*)tensors, (const int*)chunks,
                                                           (const float*)sumsq, num_tensors, max_norm);
  return (int)cudaGetLastError();
}

HM_API int hm_mt_adam(const void* tensors, const void* chunks, int num_chunks, const HmOptArgs* h,
                      cudaStream_t stream) {
  if (num_chunks <= 0) return 0;
  mt_adam_kernel<<<num_chunks, HM_MT_THREADS, 0, stream>>>((const long long*)tensors, (const int*)chunks, *h);
  return (int)cudaGetLastError();
}

HM_API int hm_mt_sgd(const void* tensors, const void* chunks, int num_chunks, const HmOptArgs* h,
                     cudaStream_t stream) {
  if (num_chunks <= 0) return 0;
  mt_sgd_kernel<<<num_chunks, HM_MT_THREADS, 0, stream>>>((const long long*)tensors, (const int*)chunks, *h);
  return (int)cudaGetLastError();
}

// LAMB in two launches; `norms` is fp32[2 * num_tensors] scratch owned by the caller (zeroed here).
HM_API int hm_mt_lamb(const void* tensors, const void* chunks, int num_chunks, int num_tensors, const HmOptArgs* h,
                      void* norms, cudaStream_t stream) {
  if (num_chunks <= 0) return 0;
  cudaError_t e = cudaMemsetAsync(norms, 0, sizeof(float) * 2 * num_tensors, stream);
  if (e != cudaSuccess) return (int)e;
  mt_lamb_stage1_kernel<<<num_chunks, HM_MT_THREADS, 0, stream>>>((const long long*)tensors, (const int*)chunks, *h,
                                                                  (float*)norms);
  mt_lamb_stage2_kernel<<<num_chunks, HM_MT_THREADS, 0, stream>>>((const long long*)tensors, (const int*)chunks, *h,
                                                                  (const float*)norms);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Allocation-free gradient clipping (declared in hm_noalloc.h). Scratch lives in this file-scope device array.
#include <mutex>
#include <cstdio>
#include "hm_noalloc.h"

static __device__ __align__(256) float hm_noalloc_sumsq[HM_NOALLOC_MAX_TENSORS + 1];

__global__ void mt_write_norm_kernel(const float* __restrict__ sumsq, int num_tensors, float* __restrict__ out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) out[0] = sqrtf(sumsq[num_tensors]);
}

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_scratch[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device. In host code the array's name is only a handle for
// the runtime, never an address a kernel may use; the real address differs per device and is looked up once.
int noalloc_scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return -21;
  std::lock_guard<std::mutex> guard(g_noalloc_mutex);
  if (g_noalloc_scratch[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, hm_noalloc_sumsq);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_scratch[dev] = ptr;
  }
  *out = g_noalloc_scratch[dev];
  return 0;
}
}  // namespace

HM_API int hm_mt_clip_grad_norm_noalloc(const void* tensors, const void* chunks, int num_chunks, int num_tensors,
                                        float max_norm, float* total_norm_out, cudaStream_t stream) {
  if (num_tensors < 0 || num_chunks < 0) return -22;
  if (num_tensors > HM_NOALLOC_MAX_TENSORS) {
    fprintf(stderr, "hm_mt_clip_grad_norm_noalloc: %d tensors exceed the built-in scratch (at most %d per call); "
                    "split the call or use hm_mt_sumsq + hm_mt_clip with a caller-owned buffer\n",
            num_tensors, HM_NOALLOC_MAX_TENSORS);
    return -20;
  }
  float* scratch = nullptr;
  int rc = noalloc_scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  // the array still holds the previous call's sums: everything this call accumulates into starts from zero
  cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(float) * (size_t)(num_tensors + 1), stream);
  if (e != cudaSuccess) return (int)e;
  if (num_chunks > 0) {
    mt_sumsq_kernel<<<num_chunks, HM_MT_THREADS, 0, stream>>>((const long long*)tensors, (const int*)chunks, 0,
                                                              num_tensors, scratch);
    mt_clip_kernel<<<num_chunks, HM_MT_THREADS, 0, stream>>>((const long long*)tensors, (const int*)chunks, scratch,
                                                             num_tensors, max_norm);
  }
  if (total_norm_out != nullptr) mt_write_norm_kernel<<<1, 32, 0, stream>>>(scratch, num_tensors, total_norm_out);
  return (int)cudaGetLastError();
}
