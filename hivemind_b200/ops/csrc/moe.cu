// Mixture-of-experts routing kernels for sm_100a: gate top-k over a grid of live experts, dispatch (sort token rows
// by expert into a packed buffer), combine (masked softmax over the chosen experts and weighted sum of their
// outputs, optional residual) and the backward passes of dispatch and combine.
//
// The math follows the client layers of the reference: an expert's logit is the sum of its per-dimension grid
// scores and the mixture weights are a softmax over the experts that answered (hivemind/moe/client/moe.py:95-137);
// the Switch variant multiplies per-dimension softmax probabilities instead (hivemind/moe/client/switch_moe.py:78-145).
// The expert FFN itself runs on the tcgen05 GEMM of tc_gemm.cu over the packed rows of each expert.
#include "hm_common.cuh"

#define MOE_MAX_K 8
#define MOE_MAX_DIMS 3
#define MOE_MAX_GRID 512  // sum of grid sizes held in shared memory per warp

struct HmMoeGrid {
  int ndim;
  int dims[MOE_MAX_DIMS];
  int num_experts;  // product of dims
};

// ---------------------------------------------------------------------------------------------------------------
// Gate: for every token choose the k best live experts.
//   scores  fp32 [T, ld]  per-dimension scores, concatenated (dimension d starts at sum(dims[:d]))
//   alive   uint8 [E]     1 where an expert exists (row-major over the grid); nullptr = all alive
//   mode 0: value = sum of scores            (expert logits)
//   mode 1: value = product of per-dim softmax probabilities (scores may hold -inf for dropped coordinates)
// Output: idx int32 [T, k] (expert id, -1 if fewer than k live experts), val fp32 [T, k] (-inf / 0 where idx < 0).
// One warp per token; each lane scans experts lane, lane+32, ... keeping a sorted private top-k, then k rounds of
// warp arg-max merge the 32 private lists. Ties go to the smaller expert id, so the result is deterministic.
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) moe_gate_topk_kernel(const float* __restrict__ scores, int T, int ld,
                                                            HmMoeGrid grid, const unsigned char* __restrict__ alive,
                                                            int k, int mode, int* __restrict__ out_idx,
                                                            float* __restrict__ out_val) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  int total = 0;
  for (int d = 0; d < grid.ndim; ++d) total += grid.dims[d];
  float* s = smem + warp * total;
  if (t >= T) return;
  for (int i = lane; i < total; i += 32) s[i] = scores[(long long)t * ld + i];
  __syncwarp();
  if (mode == 1) {
    int base = 0;
    for (int d = 0; d < grid.ndim; ++d) {
      const int n = grid.dims[d];
      float m = -INFINITY;
      for (int i = lane; i < n; i += 32) m = fmaxf(m, s[base + i]);
      m = hm_warp_max(m);
      float z = 0.f;
      for (int i = lane; i < n; i += 32) z += (m == -INFINITY) ? 0.f : __expf(s[base + i] - m);
      z = hm_warp_sum(z);
      __syncwarp();
      for (int i = lane; i < n; i += 32) s[base + i] = (z > 0.f) ? __expf(s[base + i] - m) / z : 0.f;
      base += n;
    }
    __syncwarp();
  }
  const float worst = (mode == 1) ? -1.f : -INFINITY;  // below every admissible value
  float best_v[MOE_MAX_K];
  int best_i[MOE_MAX_K];
#pragma unroll
  for (int j = 0; j < MOE_MAX_K; ++j) { best_v[j] = worst; best_i[j] = -1; }
  for (int e0 = lane; e0 < grid.num_experts; e0 += 32) {
    if (alive != nullptr && !alive[e0]) continue;
    int rem = e0, base = total;
    float v = (mode == 1) ? 1.f : 0.f;
    for (int d = grid.ndim - 1; d >= 0; --d) {
      base -= grid.dims[d];
      const int c = rem % grid.dims[d];
      rem /= grid.dims[d];
      const float sd = s[base + c];
      v = (mode == 1) ? v * sd : v + sd;
    }
    if (mode == 0 && v == -INFINITY) continue;
    if (mode == 1 && !(v > 0.f)) continue;
    int ci = e0;  // sorted insertion (descending); ids arrive in increasing order, so ">" keeps the smaller id on ties
    bool carrying = false;  // once an entry is displaced, everything below it shifts down by one
#pragma unroll
    for (int j = 0; j < MOE_MAX_K; ++j) {
      if (j < k && (carrying || v > best_v[j])) {
        const float tv = best_v[j]; const int ti = best_i[j];
        best_v[j] = v; best_i[j] = ci;
        v = tv; ci = ti;
        carrying = true;
      }
    }
  }
  // merge: k rounds of warp arg-max over the heads of the private lists
  int head = 0;
  for (int j = 0; j < k; ++j) {
    float v = worst; int id = 0x7fffffff;
#pragma unroll
    for (int q = 0; q < MOE_MAX_K; ++q)
      if (q == head) { v = best_v[q]; id = (best_i[q] >= 0) ? best_i[q] : 0x7fffffff; }
    if (head >= k) { v = worst; id = 0x7fffffff; }
    float bv = v; int bi = id;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi != 0x7fffffff && bi == id) ++head;  // the winning lane pops its head
    if (lane == 0) {
      const bool found = (bi != 0x7fffffff);
      out_idx[(long long)t * k + j] = found ? bi : -1;
      out_val[(long long)t * k + j] = found ? bv : ((mode == 1) ? 0.f : -INFINITY);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Dispatch: counting sort of the (token, slot) pairs by expert.
//   count:   counts[e] += 1 for every routed pair; rank[t, j] = arrival order within the expert
//   scan:    offsets[e] = sum(counts[:e]), offsets[E] = total  (one block)
//   permute: pos[t, j] = offsets[e] + rank[t, j]; packed[pos] = x[t]; src[pos] = t * k + j
// Rows of one expert are contiguous in `packed`; their order inside an expert is the arrival order of the atomics
// (rows are independent, so only the summation order of weight gradients depends on it).
// ---------------------------------------------------------------------------------------------------------------
__global__ void moe_count_kernel(const int* __restrict__ idx, long long n, int num_experts, int* __restrict__ counts,
                                 int* __restrict__ rank) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = idx[i];
  rank[i] = (e >= 0 && e < num_experts) ? atomicAdd(&counts[e], 1) : -1;
}

// `align` > 1 pads every expert's row range to a multiple of `align` rows (128 for the grouped GEMM, whose M tiles
// must not straddle experts); tile_group[m] then names the expert that owns rows 128*m .. 128*m+127 (-1: none).
__global__ void __launch_bounds__(1024) moe_scan_kernel(const int* __restrict__ counts, int num_experts,
                                                        int* __restrict__ offsets, int align,
                                                        int* __restrict__ tile_group, int max_tiles) {
  __shared__ int warp_tot[32];
  __shared__ int carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < num_experts; base += blockDim.x) {
    const int e = base + threadIdx.x;
    const int c = (e < num_experts) ? ((counts[e] + align - 1) / align) * align : 0;
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = (lane < (blockDim.x >> 5)) ? warp_tot[lane] : 0;
      int wi = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, wi, o);
        if (lane >= o) wi += up;
      }
      warp_tot[lane] = wi - w;  // exclusive prefix of the warp totals
    }
    __syncthreads();
    const int excl = carry + warp_tot[warp] + incl - c;
    if (e < num_experts) offsets[e] = excl;
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry = excl + c;
    __syncthreads();
  }
  if (threadIdx.x == 0) offsets[num_experts] = carry;
  if (tile_group == nullptr) return;
  __syncthreads();  // the offsets written above by this block are read back below
  const int total = carry;
  for (int m = threadIdx.x; m < max_tiles; m += blockDim.x) {
    const int row = m << 7;
    int g = -1;
    if (row < total) {
      int lo = 0, hi = num_experts;  // last e with offsets[e] <= row (the non-empty one among equal offsets)
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (offsets[mid] <= row) lo = mid; else hi = mid;
      }
      g = lo;
    }
    tile_group[m] = g;
  }
}

// One block per token: the row is read once and written to each of its (up to k) packed positions.
template <typename T>
__global__ void __launch_bounds__(128) moe_permute_kernel(const T* __restrict__ x, long long ldx, int H,
                                                          const int* __restrict__ idx, const int* __restrict__ rank,
                                                          const int* __restrict__ offsets, int k, int num_experts,
                                                          T* __restrict__ packed, int* __restrict__ pos,
                                                          int* __restrict__ src) {
  const long long t = blockIdx.x;
  __shared__ int p[MOE_MAX_K];
  if (threadIdx.x < k) {
    const int e = idx[t * k + threadIdx.x];
    const int r = rank[t * k + threadIdx.x];
    const int q = (e >= 0 && e < num_experts && r >= 0) ? offsets[e] + r : -1;
    p[threadIdx.x] = q;
    pos[t * k + threadIdx.x] = q;
    if (q >= 0) src[q] = (int)(t * k + threadIdx.x);
  }
  __syncthreads();
  constexpr int V = 16 / sizeof(T);
  const int nv = H / V;
  const uint4* xr = reinterpret_cast<const uint4*>(x + t * ldx);
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const uint4 v = xr[i];
    for (int j = 0; j < k; ++j)
      if (p[j] >= 0) reinterpret_cast<uint4*>(packed + (long long)p[j] * H)[i] = v;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Combine: out[t] = residual[t] + sum_j w[t, j] * y[pos[t, j]]
//   mode 0: w = softmax of gate[t, :] over the slots with pos >= 0 (and keep[t, j] != 0 when `keep` is given)
//   mode 1: w = gate[t, j] on those slots (probabilities; the Switch variant)
//   mode 2: w = 1 on those slots (plain gather-sum: the backward of dispatch)
// The weights are also written to w_out (fp32 [T, k]) for the backward pass. One block of 128 threads per token.
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void moe_unpack8(const uint4& v, float* f);
template <>
__device__ __forceinline__ void moe_unpack8<__nv_bfloat16>(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 a = __bfloat1622float2(h[i]); f[2 * i] = a.x; f[2 * i + 1] = a.y; }
}
template <>
__device__ __forceinline__ void moe_unpack8<float>(const uint4& v, float* f) {
  const float* h = reinterpret_cast<const float*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) f[i] = h[i];
}
template <typename T>
__device__ __forceinline__ uint4 moe_pack8(const float* f);
template <>
__device__ __forceinline__ uint4 moe_pack8<__nv_bfloat16>(const float* f) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}
template <>
__device__ __forceinline__ uint4 moe_pack8<float>(const float* f) {
  uint4 v;
  float* h = reinterpret_cast<float*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = f[i];
  return v;
}

__device__ __forceinline__ void moe_slot_weights(const float* gate, const int* pos, const unsigned char* keep,
                                                 long long t, int k, int mode, float* w /* smem [k] */) {
  if (threadIdx.x == 0) {
    float m = -INFINITY;
    for (int j = 0; j < k; ++j) {
      const bool on = pos[t * k + j] >= 0 && (keep == nullptr || keep[t * k + j]);
      const float g = (mode == 2) ? 1.f : gate[t * k + j];
      w[j] = on ? g : ((mode == 0) ? -INFINITY : 0.f);
      if (mode == 0 && on) m = fmaxf(m, g);
    }
    if (mode == 0) {
      float z = 0.f;
      for (int j = 0; j < k; ++j) { w[j] = (w[j] == -INFINITY) ? 0.f : __expf(w[j] - m); z += w[j]; }
      const float inv = (z > 0.f) ? 1.f / z : 0.f;
      for (int j = 0; j < k; ++j) w[j] *= inv;
    }
  }
  __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(128) moe_combine_fwd_kernel(const T* __restrict__ y, int H,
                                                              const int* __restrict__ pos,
                                                              const float* __restrict__ gate,
                                                              const unsigned char* __restrict__ keep,
                                                              const T* __restrict__ residual, int k, int mode,
                                                              T* __restrict__ out, float* __restrict__ w_out) {
  const long long t = blockIdx.x;
  __shared__ float w[MOE_MAX_K];
  __shared__ int p[MOE_MAX_K];
  moe_slot_weights(gate, pos, keep, t, k, mode, w);
  if (threadIdx.x < k) {
    p[threadIdx.x] = (w[threadIdx.x] != 0.f || mode != 0) ? pos[t * k + threadIdx.x] : -1;
    if (keep != nullptr && !keep[t * k + threadIdx.x]) p[threadIdx.x] = -1;
    if (w_out != nullptr) w_out[t * k + threadIdx.x] = w[threadIdx.x];
  }
  __syncthreads();
  constexpr int V = 16 / sizeof(T);
  const int nv = H / V;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float acc[V], f[V];
    if (residual != nullptr) {
      moe_unpack8<T>(reinterpret_cast<const uint4*>(residual + t * H)[i], acc);
    } else {
#pragma unroll
      for (int q = 0; q < V; ++q) acc[q] = 0.f;
    }
    for (int j = 0; j < k; ++j) {
      if (p[j] < 0) continue;
      moe_unpack8<T>(reinterpret_cast<const uint4*>(y + (long long)p[j] * H)[i], f);
      const float wj = w[j];
#pragma unroll
      for (int q = 0; q < V; ++q) acc[q] = fmaf(wj, f[q], acc[q]);
    }
    reinterpret_cast<uint4*>(out + t * H)[i] = moe_pack8<T>(acc);
  }
}

// Backward of combine. For every routed slot: dy[pos] = w * dout[t] and dw = <dout[t], y[pos]>; then
//   mode 0: dgate[j] = w[j] * (dw[j] - sum_i w[i] * dw[i]);  mode 1: dgate[j] = dw[j];  mode 2: no gate.
// Slots that were masked out by `keep` get dy = 0 (their packed row still exists) and dgate = 0.
template <typename T>
__global__ void __launch_bounds__(128) moe_combine_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ y,
                                                              int H, const int* __restrict__ pos,
                                                              const float* __restrict__ w_saved,
                                                              const unsigned char* __restrict__ keep, int k, int mode,
                                                              T* __restrict__ dy, float* __restrict__ dgate) {
  const long long t = blockIdx.x;
  __shared__ float w[MOE_MAX_K];
  __shared__ int p[MOE_MAX_K];
  __shared__ float dots[MOE_MAX_K];
  __shared__ float red[32];
  if (threadIdx.x < k) {
    const bool on = keep == nullptr || keep[t * k + threadIdx.x];
    p[threadIdx.x] = pos[t * k + threadIdx.x];
    w[threadIdx.x] = on ? w_saved[t * k + threadIdx.x] : 0.f;
  }
  __syncthreads();
  constexpr int V = 16 / sizeof(T);
  const int nv = H / V;
  float dot[MOE_MAX_K];
#pragma unroll
  for (int j = 0; j < MOE_MAX_K; ++j) dot[j] = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float g[V], f[V], o[V];
    moe_unpack8<T>(reinterpret_cast<const uint4*>(dout + t * H)[i], g);
#pragma unroll
    for (int j = 0; j < MOE_MAX_K; ++j) {
      if (j >= k || p[j] < 0) continue;
      if (y != nullptr && mode != 2) {
        moe_unpack8<T>(reinterpret_cast<const uint4*>(y + (long long)p[j] * H)[i], f);
#pragma unroll
        for (int q = 0; q < V; ++q) dot[j] = fmaf(g[q], f[q], dot[j]);
      }
      const float wj = w[j];
#pragma unroll
      for (int q = 0; q < V; ++q) o[q] = wj * g[q];
      reinterpret_cast<uint4*>(dy + (long long)p[j] * H)[i] = moe_pack8<T>(o);
    }
  }
  if (mode == 2 || dgate == nullptr) return;
#pragma unroll
  for (int j = 0; j < MOE_MAX_K; ++j) {
    if (j < k) {  // uniform branch: k is a kernel argument
      const float s = hm_block_sum(dot[j], red);
      if (threadIdx.x == 0) dots[j] = s;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float mix = 0.f;
    for (int j = 0; j < k; ++j) mix += w[j] * dots[j];
    for (int j = 0; j < k; ++j) {
      const bool on = p[j] >= 0 && (keep == nullptr || keep[t * k + j]);
      dgate[t * k + j] = !on ? 0.f : ((mode == 0) ? w[j] * (dots[j] - mix) : dots[j]);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Launchers
// ---------------------------------------------------------------------------------------------------------------
HM_API int hm_moe_gate_topk(const float* scores, int T, int ld, int ndim, const int* dims_host,
                            const unsigned char* alive, int k, int mode, int* out_idx, float* out_val,
                            cudaStream_t stream) {
  if (ndim < 1 || ndim > MOE_MAX_DIMS || k < 1 || k > MOE_MAX_K) return -10;
  HmMoeGrid grid;
  grid.ndim = ndim;
  grid.num_experts = 1;
  int total = 0;
  for (int d = 0; d < MOE_MAX_DIMS; ++d) {
    grid.dims[d] = d < ndim ? dims_host[d] : 1;
    if (d < ndim) { grid.num_experts *= dims_host[d]; total += dims_host[d]; }
  }
  if (total > MOE_MAX_GRID || total > ld || grid.num_experts > (1 << 20)) return -11;
  if (T == 0) return 0;
  const int warps = 4;
  moe_gate_topk_kernel<<<(T + warps - 1) / warps, warps * 32, warps * total * sizeof(float), stream>>>(
      scores, T, ld, grid, alive, k, mode, out_idx, out_val);
  return (int)cudaGetLastError();
}

// rank/pos are int32 [T*k]; src is int32 [packed_rows] (-1 for rows that hold no token); offsets int32 [E+1].
// align = 1: experts' rows are dense. align = 128: every expert's range is padded to whole 128-row tiles, the pad
// rows of `packed` are zero, and tile_group (int32 [max_tiles], max_tiles = packed_rows / 128) is filled.
HM_API int hm_moe_dispatch(const void* x, long long ldx, int H, int dtype, const int* idx, int T, int k,
                           int num_experts, int* counts, int* offsets, int* rank, void* packed, long long packed_rows,
                           int* pos, int* src, int align, int* tile_group, int max_tiles, cudaStream_t stream) {
  if (k < 1 || k > MOE_MAX_K) return -10;
  if (align != 1 && align != 128) return -12;
  if (align == 128 && (tile_group == nullptr || (long long)max_tiles * 128 > packed_rows ||
                       packed_rows < (long long)T * k + (long long)num_experts * 127))
    return -12;
  const int esize = (dtype == HM_F32) ? 4 : 2;
  if (dtype == HM_F16 || (H * esize) % 16 != 0 || (ldx * esize) % 16 != 0) return -11;
  cudaError_t err = cudaMemsetAsync(counts, 0, sizeof(int) * num_experts, stream);
  if (err != cudaSuccess) return (int)err;
  err = cudaMemsetAsync(src, 0xff, sizeof(int) * packed_rows, stream);
  if (err != cudaSuccess) return (int)err;
  if (align > 1) {
    err = cudaMemsetAsync(packed, 0, (size_t)packed_rows * H * esize, stream);
    if (err != cudaSuccess) return (int)err;
  }
  const long long n = (long long)T * k;
  if (n > 0) moe_count_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(idx, n, num_experts, counts, rank);
  moe_scan_kernel<<<1, 1024, 0, stream>>>(counts, num_experts, offsets, align, align > 1 ? tile_group : nullptr,
                                          max_tiles);
  if (T > 0) {
    if (dtype == HM_BF16)
      moe_permute_kernel<__nv_bfloat16><<<T, 128, 0, stream>>>((const __nv_bfloat16*)x, ldx, H, idx, rank, offsets, k,
                                                               num_experts, (__nv_bfloat16*)packed, pos, src);
    else
      moe_permute_kernel<float><<<T, 128, 0, stream>>>((const float*)x, ldx, H, idx, rank, offsets, k, num_experts,
                                                       (float*)packed, pos, src);
  }
  return (int)cudaGetLastError();
}

HM_API int hm_moe_combine_fwd(const void* y, int H, int dtype, const int* pos, const float* gate,
                              const unsigned char* keep, const void* residual, int T, int k, int mode, void* out,
                              float* w_out, cudaStream_t stream) {
  if (k < 1 || k > MOE_MAX_K || mode < 0 || mode > 2) return -10;
  const int esize = (dtype == HM_F32) ? 4 : 2;
  if (dtype == HM_F16 || (H * esize) % 16 != 0) return -11;
  if (T == 0) return 0;
  if (dtype == HM_BF16)
    moe_combine_fwd_kernel<__nv_bfloat16><<<T, 128, 0, stream>>>((const __nv_bfloat16*)y, H, pos, gate, keep,
                                                                 (const __nv_bfloat16*)residual, k, mode,
                                                                 (__nv_bfloat16*)out, w_out);
  else
    moe_combine_fwd_kernel<float><<<T, 128, 0, stream>>>((const float*)y, H, pos, gate, keep, (const float*)residual,
                                                         k, mode, (float*)out, w_out);
  return (int)cudaGetLastError();
}

HM_API int hm_moe_combine_bwd(const void* dout, const void* y, int H, int dtype, const int* pos, const float* w_saved,
                              const unsigned char* keep, int T, int k, int mode, void* dy, float* dgate,
                              cudaStream_t stream) {
  if (k < 1 || k > MOE_MAX_K || mode < 0 || mode > 2) return -10;
  const int esize = (dtype == HM_F32) ? 4 : 2;
  if (dtype == HM_F16 || (H * esize) % 16 != 0) return -11;
  if (T == 0) return 0;
  if (dtype == HM_BF16)
    moe_combine_bwd_kernel<__nv_bfloat16><<<T, 128, 0, stream>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)y,
                                                                 H, pos, w_saved, keep, k, mode, (__nv_bfloat16*)dy,
                                                                 dgate);
  else
    moe_combine_bwd_kernel<float><<<T, 128, 0, stream>>>((const float*)dout, (const float*)y, H, pos, w_saved, keep, k,
                                                         mode, (float*)dy, dgate);
  return (int)cudaGetLastError();
}
