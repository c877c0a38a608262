// Whole-tensor codec kernels: fp16, mean/std-scaled fp16, uniform / quantile / block-wise 8-bit encoders that produce
// the reference's wire layouts (one statistics record per tensor or per row: hivemind/compression/floating.py:18-64,
// hivemind/compression/quantization.py:60-153) for CUDA tensors, so that only compressed bytes cross PCIe when a
// tensor is serialised (state downloads, expert RPC payloads).
//
// A tensor (or each of its rows) is a "part" of a one-rank group whose outbox is the caller's output buffer; parts
// are processed in chunks of 16384 elements by separate launches:  [stats] -> [borders] -> encode -> publish (header).
// The averaging rounds between GPUs do not use these kernels: they run the fused per-chunk codecs of
// butterfly_round.cu.
#include "hb_codec.cuh"

#define HB_MAX_PEERS 16
#define HB_CHUNK 16384
#define HB_THREADS 256
#define HB_SAMPLE 8192         // samples per part for quantile borders (32 per bin)


struct HbPeer {
  float* data;                 // the peer's flat vector
  unsigned char* outbox;       // encoded parts; record of part p starts at outbox + part.enc_off
  unsigned char* deltabox;     // as reducer: region of sender s starts at deltabox + s * delta_stride
  unsigned int* ready;         // [n_parts] == epoch once the outbox record of part p is complete
  unsigned int* delta_ready;   // [HB_MAX_PEERS][max_local_parts]: epoch (| HB_FAIL_BIT) once the delta is complete
  float* avg;                  // as reducer: averages of its own span (read by senders of uncompressed parts)
};

struct HbPart {
  long long start;             // first element in the flat vector
  long long enc_off;           // byte offset of the encoded record in every peer's outbox
  long long span_off;          // byte offset of the record inside a per-sender region of the owner's delta box
  long long avg_off;           // element offset inside the owner's avg buffer
  int len, owner, local_idx, codec;
};

struct HbGroup {
  int n_peers, n_parts, me, max_local_parts;
  unsigned int epoch;
  float alpha;
  unsigned long long sender_timeout_ns, reducer_timeout_ns, delta_stride;
  float weight[HB_MAX_PEERS];
  int sends[HB_MAX_PEERS];     // 1 if the peer contributes data (mode != AUX)
  HbPeer peer[HB_MAX_PEERS];
  const HbPart* parts;         // [n_parts], local copy
  // per-round local scratch (zeroed by the host at round start)
  double* part_stats;          // [n_parts][2] sum, sum of squares (forward encode)
  double* dstats;              // [HB_MAX_PEERS][max_local_parts][2] (delta encode)
  float* bins;                 // [n_parts][256] per-bin sums; int counts follow in bin_cnt
  int* bin_cnt;                // [n_parts][256]
  float* dbins;                // [HB_MAX_PEERS][max_local_parts][256]
  int* dbin_cnt;
  float* borders;              // [n_parts][256] quantile borders (255 used)
  float* dborders;             // [HB_MAX_PEERS][max_local_parts][256]
  int* include;                // [max_local_parts][HB_MAX_PEERS] 0 undecided, 1 in, 2 out
  int* apply_decision;         // [n_parts] 0 undecided, 1 apply, 2 skip
  int* ban;                    // [HB_MAX_PEERS]
  unsigned long long* t_start; // [2] start time of the reduce / apply phase on this GPU
  unsigned long long* status;  // [0] banned sender mask [1] failed reducer mask [2] elements left unaveraged
  float* avg;                  // local averages of my span
};

__constant__ float hb_code[256];      // block-wise dynamic code (sorted)
__constant__ float hb_code_mid[256];  // midpoints between consecutive code entries (255 used)

HM_API int hm_bf_set_blockwise_code(const float* host_code256) {
  float mid[256];
  for (int i = 0; i < 255; ++i) mid[i] = 0.5f * (host_code256[i] + host_code256[i + 1]);
  mid[255] = INFINITY;
  cudaError_t e = cudaMemcpyToSymbol(hb_code, host_code256, sizeof(float) * 256);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemcpyToSymbol(hb_code_mid, mid, sizeof(float) * 256);
}

// ---------------------------------------------------------------------------------------------------------------
// record geometry (the host uses the same formulas through hm_bf_record_bytes)
__host__ __device__ inline long long hb_header_bytes(int codec, int len) {
  switch (codec) {
    case HB_MEANSTD16: return 16;
    case HB_QUANTILE8:
    case HB_UNIFORM8: return 1024;
    case HB_BLOCKWISE8: return (((long long)(len + HB_BLOCK - 1) / HB_BLOCK) * 4 + 15) / 16 * 16;
    default: return 0;
  }
}
__host__ __device__ inline long long hb_record_bytes(int codec, int len) {
  return hb_header_bytes(codec, len) + ((long long)len * hb_elem_bytes(codec) + 15) / 16 * 16;
}
HM_API long long hm_bf_record_bytes(int codec, int len) { return hb_record_bytes(codec, len); }
HM_API int hm_bf_sizeof_group() { return (int)sizeof(HbGroup); }
HM_API int hm_bf_sizeof_part() { return (int)sizeof(HbPart); }
HM_API int hm_bf_chunk() { return HB_CHUNK; }

// Per-part decoding context, loaded once per CTA.
struct HbDecode {
  int codec;
  float mean, std;            // MEANSTD16
  const float* absmax;        // BLOCKWISE8 (global, possibly remote)
  const unsigned char* payload;
};

__device__ __forceinline__ void hb_decode_setup(HbDecode& d, int codec, const unsigned char* rec, int len,
                                                float* codebook_smem) {
  d.codec = codec;
  d.payload = rec + hb_header_bytes(codec, len);
  d.mean = 0.f;
  d.std = 1.f;
  d.absmax = reinterpret_cast<const float*>(rec);
  if (codec == HB_MEANSTD16) {
    d.mean = reinterpret_cast<const float*>(rec)[0];
    d.std = reinterpret_cast<const float*>(rec)[1];
  } else if (codec == HB_UNIFORM8 || codec == HB_QUANTILE8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) codebook_smem[i] = reinterpret_cast<const float*>(rec)[i];
  } else if (codec == HB_BLOCKWISE8) {
    // constant memory serialises lanes that index it differently: look the code up in shared memory instead
    for (int i = threadIdx.x; i < 256; i += blockDim.x) codebook_smem[i] = hb_code[i];
  }
}

// Decode 4 consecutive elements starting at element i (multiple of 4) of a record; elements >= len read as 0.
__device__ __forceinline__ void hb_decode4(const HbDecode& d, const float* codebook_smem, int i, int len, float v[4]) {
  if (i + 4 <= len) {
    switch (d.codec) {
      case HB_NONE: {
        float4 x = *reinterpret_cast<const float4*>(d.payload + (size_t)i * 4);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
        return;
      }
      case HB_FLOAT16:
      case HB_MEANSTD16: {
        uint2 x = *reinterpret_cast<const uint2*>(d.payload + (size_t)i * 2);
        __half2 a = *reinterpret_cast<__half2*>(&x.x), b = *reinterpret_cast<__half2*>(&x.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
        if (d.codec == HB_MEANSTD16) {
#pragma unroll
          for (int k = 0; k < 4; ++k) v[k] = fmaf(v[k], d.std, d.mean);
        }
        return;
      }
      case HB_UNIFORM8:
      case HB_QUANTILE8: {
        uchar4 q = *reinterpret_cast<const uchar4*>(d.payload + i);
        v[0] = codebook_smem[q.x]; v[1] = codebook_smem[q.y]; v[2] = codebook_smem[q.z]; v[3] = codebook_smem[q.w];
        return;
      }
      default: {  // HB_BLOCKWISE8
        uchar4 q = *reinterpret_cast<const uchar4*>(d.payload + i);
        const float a = d.absmax[i / HB_BLOCK];
        v[0] = codebook_smem[q.x] * a; v[1] = codebook_smem[q.y] * a;
        v[2] = codebook_smem[q.z] * a; v[3] = codebook_smem[q.w] * a;
        return;
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int e = i + k;
    if (e >= len) { v[k] = 0.f; continue; }
    switch (d.codec) {
      case HB_NONE: v[k] = reinterpret_cast<const float*>(d.payload)[e]; break;
      case HB_FLOAT16: v[k] = __half2float(reinterpret_cast<const __half*>(d.payload)[e]); break;
      case HB_MEANSTD16: v[k] = fmaf(__half2float(reinterpret_cast<const __half*>(d.payload)[e]), d.std, d.mean); break;
      case HB_UNIFORM8:
      case HB_QUANTILE8: v[k] = codebook_smem[d.payload[e]]; break;
      default: v[k] = codebook_smem[d.payload[e]] * d.absmax[e / HB_BLOCK]; break;
    }
  }
}


// ---------------------------------------------------------------------------------------------------------------
// What is being encoded: mode 0 = my own data (for the outbox), mode 1 = avg - decode(copy of sender's record)
// (the delta for that sender, written over the copy).
struct HbSource {
  int mode;
  const float* values;   // mode 0: part start in data; mode 1: part start in avg
  HbDecode dec;          // mode 1
};

__device__ __forceinline__ void hb_src4(const HbSource& s, const float* codebook_smem, int i, int len, float v[4]) {
  if (i + 4 <= len) {
    const float4 x = *reinterpret_cast<const float4*>(s.values + i);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = (i + k < len) ? s.values[i + k] : 0.f;
  }
  if (s.mode == 1) {
    float o[4];
    hb_decode4(s.dec, codebook_smem, i, len, o);
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] -= o[k];
  }
}

struct HbItemCtx {
  const HbPart* part;
  unsigned char* rec;      // record being written (outbox or delta box)
  double* stats;           // [2]
  float* bins;             // [256]
  int* cnt;                // [256]
  float* borders;          // [256]
};

__device__ __forceinline__ HbItemCtx hb_item_ctx(const HbGroup& g, int p, int s, int mode) {
  HbItemCtx c;
  c.part = g.parts + p;
  if (mode == 0) {
    c.rec = g.peer[g.me].outbox + c.part->enc_off;
    c.stats = g.part_stats + 2 * (size_t)p;
    c.bins = g.bins + 256 * (size_t)p;
    c.cnt = g.bin_cnt + 256 * (size_t)p;
    c.borders = g.borders + 256 * (size_t)p;
  } else {
    const size_t slot = (size_t)s * g.max_local_parts + c.part->local_idx;
    c.rec = g.peer[g.me].deltabox + (size_t)s * g.delta_stride + c.part->span_off;
    c.stats = g.dstats + 2 * slot;
    c.bins = g.dbins + 256 * slot;
    c.cnt = g.dbin_cnt + 256 * slot;
    c.borders = g.dborders + 256 * slot;
  }
  return c;
}

__device__ __forceinline__ void hb_source_setup(HbSource& src, const HbGroup& g, const HbItemCtx& c, int mode,
                                                float* codebook_smem) {
  src.mode = mode;
  if (mode == 0) {
    src.values = g.peer[g.me].data + c.part->start;
  } else {
    src.values = g.avg + c.part->avg_off;
    hb_decode_setup(src.dec, c.part->codec, c.rec, c.part->len, codebook_smem);
  }
}

// sum and sum of squares per part (needed by MEANSTD16 and UNIFORM8 before they can quantise)
__global__ void __launch_bounds__(HB_THREADS)
hb_stats_kernel(const HbGroup* __restrict__ gp, const int4* __restrict__ items) {
  __shared__ float red[32];
  __shared__ float cb[256];
  const HbGroup& g = *gp;
  const int4 it = items[blockIdx.x];
  const HbItemCtx c = hb_item_ctx(g, it.x, it.z, 0);
  HbSource src;
  hb_source_setup(src, g, c, 0, cb);
  const int len = c.part->len, lo = it.y * HB_CHUNK, hi = min(lo + HB_CHUNK, len);
  float s1 = 0.f, s2 = 0.f;
  for (int i = lo + 4 * threadIdx.x; i < hi; i += 4 * HB_THREADS) {
    float v[4];
    hb_src4(src, cb, i, len, v);
#pragma unroll
    for (int k = 0; k < 4; ++k) { s1 += v[k]; s2 = fmaf(v[k], v[k], s2); }
  }
  s1 = hm_block_sum(s1, red);
  s2 = hm_block_sum(s2, red);
  if (threadIdx.x == 0) {
    atomicAdd(c.stats, (double)s1);
    atomicAdd(c.stats + 1, (double)s2);
  }
}

// Quantile borders from an evenly strided sample of the part, sorted in shared memory (bitonic, 1024 threads).
__global__ void __launch_bounds__(1024)
hb_borders_kernel(const HbGroup* __restrict__ gp, const int4* __restrict__ items, int mode) {
  __shared__ float smp[HB_SAMPLE];
  __shared__ float cb[256];
  const HbGroup& g = *gp;
  const int4 it = items[blockIdx.x];
  const HbItemCtx c = hb_item_ctx(g, it.x, it.z, mode);
  HbSource src;
  hb_source_setup(src, g, c, mode, cb);
  __syncthreads();
  const int len = c.part->len;
  const int S = len < HB_SAMPLE ? len : HB_SAMPLE;
  for (int k = threadIdx.x; k < HB_SAMPLE; k += blockDim.x) {
    float val = INFINITY;
    if (k < S) {
      const int e = (int)(((long long)k * len) / S);
      float v[4];
      hb_src4(src, cb, e & ~3, len, v);
      val = v[e & 3];
    }
    smp[k] = val;
  }
  __syncthreads();
  for (int size = 2; size <= HB_SAMPLE; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < HB_SAMPLE / 2; t += blockDim.x) {
        const int i = 2 * t - (t & (stride - 1));
        const int j = i + stride;
        const bool up = (i & size) == 0;
        const float a = smp[i], b = smp[j];
        if ((a > b) == up) { smp[i] = b; smp[j] = a; }
      }
      __syncthreads();
    }
  }
  for (int k = threadIdx.x; k < 256; k += blockDim.x) {
    float b = INFINITY;
    if (k < 255 && S > 0) {
      int r = (int)(((long long)(k + 1) * S) / 256);
      r = r >= S ? S - 1 : r;
      b = smp[r];
    }
    c.borders[k] = b;
  }
}

__global__ void __launch_bounds__(HB_THREADS)
hb_encode_kernel(const HbGroup* __restrict__ gp, const int4* __restrict__ items, int mode) {
  __shared__ float red[32];
  __shared__ float cb[256];          // codebook of the record being replaced (mode 1)
  __shared__ float table[256];       // quantile borders
  // per-warp bin sums and counts: a skewed distribution (most values in a few bins) would otherwise serialise the
  // whole CTA on a handful of shared-memory addresses
  __shared__ float hsum[HB_THREADS / 32][256];
  __shared__ int hcnt[HB_THREADS / 32][256];
  const int warp = threadIdx.x >> 5;
  const HbGroup& g = *gp;
  const int4 it = items[blockIdx.x];
  const HbItemCtx c = hb_item_ctx(g, it.x, it.z, mode);
  const int codec = c.part->codec, len = c.part->len;
  HbSource src;
  hb_source_setup(src, g, c, mode, cb);
  const bool binned = codec == HB_UNIFORM8 || codec == HB_QUANTILE8;
  if (binned) {
    for (int i = threadIdx.x; i < 256 * (HB_THREADS / 32); i += HB_THREADS) { (&hsum[0][0])[i] = 0.f; (&hcnt[0][0])[i] = 0; }
    if (codec == HB_QUANTILE8)
      for (int i = threadIdx.x; i < 256; i += HB_THREADS) table[i] = c.borders[i];
  }
  if (codec == HB_BLOCKWISE8)
    for (int i = threadIdx.x; i < 256; i += HB_THREADS) table[i] = hb_code_mid[i];
  float mean = 0.f, inv_scale = 1.f;
  if (codec == HB_MEANSTD16 || codec == HB_UNIFORM8) {
    const double n = (double)len, s1 = c.stats[0], s2 = c.stats[1];
    const double m = s1 / n;
    const double centered = fmax(s2 - n * m * m, 0.0);
    mean = (float)m;
    if (codec == HB_MEANSTD16) {
      const float sd = fmaxf((float)sqrt(centered / n), 1.1920929e-07f);
      inv_scale = 1.f / sd;
    } else {
      const float scale = 6.f * (float)sqrt(centered / fmax(n - 1.0, 1.0)) / 256.f;
      inv_scale = (scale > 0.f && isfinite(scale)) ? 1.f / scale : 1.f;
    }
  }
  __syncthreads();
  unsigned char* payload = c.rec + hb_header_bytes(codec, len);
  float* absmax_out = reinterpret_cast<float*>(c.rec);
  const int lo = it.y * HB_CHUNK;
  for (int b0 = lo; b0 < min(lo + HB_CHUNK, len); b0 += HB_BLOCK) {
    // one block of up to 4096 elements: 16 per thread, held in registers so that in-place re-encoding is safe
    float v[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r) hb_src4(src, cb, b0 + (r * HB_THREADS + threadIdx.x) * 4, len, v[r]);
    float inv_absmax = 1.f;
    if (codec == HB_BLOCKWISE8) {
      float m = 0.f;
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int k = 0; k < 4; ++k) m = fmaxf(m, fabsf(v[r][k]));
      m = hm_block_max(m, red);
      inv_absmax = 1.f / fmaxf(m, 1.17549435e-38f);
      if (threadIdx.x == 0) absmax_out[b0 / HB_BLOCK] = m;
    } else {
      __syncthreads();  // every thread has read its inputs of this block before anybody overwrites the record
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = b0 + (r * HB_THREADS + threadIdx.x) * 4;
      if (i >= len) continue;
      const int valid = min(4, len - i);
      if (codec == HB_NONE) {
        if (valid == 4) *reinterpret_cast<float4*>(payload + (size_t)i * 4) = make_float4(v[r][0], v[r][1], v[r][2], v[r][3]);
        else for (int k = 0; k < valid; ++k) reinterpret_cast<float*>(payload)[i + k] = v[r][k];
      } else if (codec == HB_FLOAT16 || codec == HB_MEANSTD16) {
        float h[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) h[k] = hb_clamp_half((v[r][k] - mean) * inv_scale);
        if (valid == 4) {
          __half2 a = __floats2half2_rn(h[0], h[1]), b = __floats2half2_rn(h[2], h[3]);
          uint2 o;
          o.x = *reinterpret_cast<unsigned int*>(&a);
          o.y = *reinterpret_cast<unsigned int*>(&b);
          *reinterpret_cast<uint2*>(payload + (size_t)i * 2) = o;
        } else {
          for (int k = 0; k < valid; ++k) reinterpret_cast<__half*>(payload)[i + k] = __float2half_rn(h[k]);
        }
      } else {
        unsigned char q[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          int b;
          if (codec == HB_UNIFORM8) b = (int)rintf((v[r][k] - mean) * inv_scale) + 128;
          else if (codec == HB_QUANTILE8) b = hb_bucketize(table, v[r][k]);
          else b = hb_bucketize(table, v[r][k] * inv_absmax);
          b = b < 0 ? 0 : (b > 255 ? 255 : b);
          q[k] = (unsigned char)b;
          if (binned && k < valid) {
            atomicAdd(&hsum[warp][b], v[r][k]);
            atomicAdd(&hcnt[warp][b], 1);
          }
        }
        if (valid == 4) *reinterpret_cast<uchar4*>(payload + i) = make_uchar4(q[0], q[1], q[2], q[3]);
        else for (int k = 0; k < valid; ++k) payload[i + k] = q[k];
      }
    }
  }
  if (binned) {
    __syncthreads();
    for (int i = threadIdx.x; i < 256; i += HB_THREADS) {
      float total = 0.f;
      int count = 0;
#pragma unroll
      for (int w = 0; w < HB_THREADS / 32; ++w) { total += hsum[w][i]; count += hcnt[w][i]; }
      if (count) {
        atomicAdd(c.bins + i, total);
        atomicAdd(c.cnt + i, count);
      }
    }
  }
}

// Writes the record header (codebook or mean/std) and then publishes the record: one CTA per item.
__global__ void __launch_bounds__(256)
hb_publish_kernel(const HbGroup* __restrict__ gp, const int4* __restrict__ items, int mode) {
  const HbGroup& g = *gp;
  const int4 it = items[blockIdx.x];
  const HbItemCtx c = hb_item_ctx(g, it.x, it.z, mode);
  const int codec = c.part->codec, len = c.part->len;
  bool failed = false;
  if (mode == 1) failed = g.include[(size_t)c.part->local_idx * HB_MAX_PEERS + it.z] != 1;
  if (!failed) {
    if (codec == HB_UNIFORM8 || codec == HB_QUANTILE8) {
      const int n = c.cnt[threadIdx.x];
      reinterpret_cast<float*>(c.rec)[threadIdx.x] = c.bins[threadIdx.x] / (float)(n > 0 ? n : 1);
    } else if (codec == HB_MEANSTD16 && threadIdx.x == 0) {
      const double n = (double)len, m = c.stats[0] / n;
      const double centered = fmax(c.stats[1] - n * m * m, 0.0);
      reinterpret_cast<float*>(c.rec)[0] = (float)m;
      reinterpret_cast<float*>(c.rec)[1] = fmaxf((float)sqrt(centered / n), 1.1920929e-07f);
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int value = failed ? (g.epoch | HB_FAIL_BIT) : g.epoch;
    unsigned int* flag = mode == 0 ? g.peer[g.me].ready + it.x
                                   : g.peer[g.me].delta_ready + (size_t)it.z * g.max_local_parts + c.part->local_idx;
    hm_st_release_sys(flag, value);
  }
}

// ---------------------------------------------------------------------------------------------------------------
enum HbPhase : int { HB_PH_STATS = 0, HB_PH_BORDERS = 1, HB_PH_ENCODE = 2, HB_PH_PUBLISH = 3 };

// Launch one phase for one rank. `group` and `items` are device pointers; `mode` 0 = forward records, 1 = deltas.
HM_API int hm_bf_launch(int phase, const void* group, const void* items, int n_items, int mode, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  const HbGroup* g = (const HbGroup*)group;
  const int4* it = (const int4*)items;
  switch (phase) {
    case HB_PH_STATS: hb_stats_kernel<<<n_items, HB_THREADS, 0, stream>>>(g, it); break;
    case HB_PH_BORDERS: hb_borders_kernel<<<n_items, 1024, 0, stream>>>(g, it, mode); break;
    case HB_PH_ENCODE: hb_encode_kernel<<<n_items, HB_THREADS, 0, stream>>>(g, it, mode); break;
    case HB_PH_PUBLISH: hb_publish_kernel<<<n_items, 256, 0, stream>>>(g, it, mode); break;
    default: return -1;
  }
  return (int)cudaGetLastError();
}
