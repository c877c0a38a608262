// Device butterfly all-reduce: weighted averaging of a flat fp32 vector across up to 16 GPUs of one NVLink box,
// with the tensor codecs fused into the reduce-scatter and all-gather halves and sender / reducer timeouts
// honoured through device-visible flags.
//
// Semantics are those of the reference's RPC butterfly (hivemind/averaging/allreduce.py:151-359,
// hivemind/averaging/partition.py:179-277): the vector is cut into parts, part p is reduced by peer owner(p);
//   avg_p = sum_{s alive} w_s * x~_{s,p} / sum_{s alive} w_s,   x~ = decode(encode(x)) for remote senders, x for
//   the reducer's own data;   sender s then applies x_s += alpha * decode(encode_codec(avg_p - x~_{s,p})).
// A sender whose part is not published within `sender_timeout` is banned for that and all later parts (the
// denominator shrinks); a reducer whose delta is not published within `reducer_timeout` leaves the sender's
// values unchanged (zero delta).
//
// Data movement is pull-only: every peer writes only its own memory (encoded parts into its outbox, encoded
// deltas into its delta box, flags into its flag page) and reads peers' memory with plain loads through
// peer-mapped pointers (cudaIpc / peer access), CTA by CTA. Nothing here uses TMA or cluster-wide loads.
//
// Uncompressed parts (codec NONE) are lossless, so they skip both staging copies: the reducer reads the senders'
// vectors in place (a sender modifies a part only after the part's owner has published the result for it) and the
// senders read the owner's average instead of a per-sender delta record; x += alpha * (avg - x) is the same number.
// Every reducer applies the average to its own span inside the reduce kernel.
//
// Phases (separate launches on one stream per GPU; a phase that consumes remote data first waits, bounded, on the
// producer's flag):  [stats] -> [borders] -> encode -> publish   |   reduce -> [delta borders] -> encode deltas ->
// publish deltas   |   apply.  One launch can cover one rank (normal operation, one process per GPU) or, for
// testing on fewer GPUs than ranks, each phase is launched for every emulated rank before the next phase starts,
// so no launch ever waits for a later launch.
#include "hm_common.cuh"

#define HB_MAX_PEERS 16
#define HB_CHUNK 16384
#define HB_THREADS 256
#define HB_BLOCK 4096          // block-wise quantization block
#define HB_SAMPLE 2048         // samples per part for quantile borders
#define HB_FAIL_BIT 0x80000000u

enum HbCodec : int { HB_NONE = 0, HB_MEANSTD16 = 1, HB_FLOAT16 = 2, HB_QUANTILE8 = 3, HB_UNIFORM8 = 4, HB_BLOCKWISE8 = 5 };

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
__host__ __device__ inline int hb_elem_bytes(int codec) {
  return codec == HB_NONE ? 4 : ((codec == HB_FLOAT16 || codec == HB_MEANSTD16) ? 2 : 1);
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

__device__ __forceinline__ float hb_clamp_half(float x) { return fminf(fmaxf(x, -65504.f), 65504.f); }

// number of entries of a sorted table (255 used) that are < x  ==  torch.bucketize(x, table)
__device__ __forceinline__ int hb_bucketize(const float* table, float x) {
  int lo = 0, hi = 255;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (table[mid] < x) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// Bounded wait on a flag that another GPU (or an earlier launch) publishes. Thread 0 of the CTA polls; the
// outcome is stored in `decision` with a compare-and-swap so that every CTA working on the same part agrees.
// Returns 1 (ready) or 2 (gave up). `deadline_ns` is absolute on this GPU's globaltimer.
__device__ int hb_wait_decide(const unsigned int* flag, unsigned int want, int* decision, const int* ban_flag,
                              unsigned long long deadline_ns, int* shared_out) {
  if (threadIdx.x == 0) {
    int d = *reinterpret_cast<volatile int*>(decision);
    while (d == 0) {
      const unsigned int v = hm_ld_acquire_sys(flag);
      if (v == want) {
        atomicCAS(decision, 0, 1);
      } else if (v == (want | HB_FAIL_BIT) || (ban_flag && *reinterpret_cast<const volatile int*>(ban_flag)) ||
                 hm_globaltimer_ns() > deadline_ns) {
        atomicCAS(decision, 0, 2);
      } else {
        __nanosleep(256);
      }
      d = *reinterpret_cast<volatile int*>(decision);
    }
    *shared_out = d;
  }
  __syncthreads();
  const int out = *shared_out;
  __syncthreads();
  return out;
}

__device__ __forceinline__ unsigned long long hb_phase_start(unsigned long long* slot) {
  // first CTA of the phase records the start time; everybody measures timeouts from it
  unsigned long long t = *reinterpret_cast<volatile unsigned long long*>(slot);
  if (t == 0) {
    const unsigned long long now = hm_globaltimer_ns();
    const unsigned long long prev = atomicCAS(slot, 0ull, now);
    t = prev == 0 ? now : prev;
  }
  return t;
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
// Reduce (the reduce-scatter half): for one chunk of one of my parts, wait (bounded) for every sender's record,
// pull the chunk over NVLink once into the local delta box, average, store the average and accumulate the
// statistics that the per-sender delta encoders will need.
__global__ void __launch_bounds__(HB_THREADS, 4)
hb_reduce_kernel(const HbGroup* __restrict__ gp, const int4* __restrict__ items) {
  __shared__ float cbs[HB_MAX_PEERS][256];
  __shared__ float red[32];
  __shared__ int inc[HB_MAX_PEERS];
  __shared__ int wait_out;
  const HbGroup& g = *gp;
  const int4 it = items[blockIdx.x];
  const HbPart part = g.parts[it.x];
  const int codec = part.codec, len = part.len, j = part.local_idx, me = g.me;
  const int lo = it.y * HB_CHUNK, hi = min(lo + HB_CHUNK, len);
  const unsigned long long deadline = hb_phase_start(g.t_start) + g.sender_timeout_ns;
  const long long hdr = hb_header_bytes(codec, len);
  const int eb = hb_elem_bytes(codec);

  for (int s = 0; s < g.n_peers; ++s) {
    if (s == me || !g.sends[s]) {
      if (threadIdx.x == 0) inc[s] = 0;
      continue;
    }
    const int d = hb_wait_decide(g.peer[s].ready + it.x, g.epoch, g.include + (size_t)j * HB_MAX_PEERS + s, g.ban + s,
                                 deadline, &wait_out);
    if (threadIdx.x == 0) {
      inc[s] = d == 1;
      if (d != 1) {
        atomicExch(g.ban + s, 1);  // a sender that missed one part is left out of the later ones too
        atomicOr(g.status, 1ull << s);
      }
    }
  }
  __syncthreads();

  const bool direct = codec == HB_NONE;  // lossless part: accumulate straight from the senders' vectors
  // every reducer walks the senders in its own rotation (and every chunk starts one further), so that at any moment
  // the reducers of a group read from different GPUs instead of all draining the same sender's links
  const int rot = (me + 1 + (int)(blockIdx.x % (unsigned)g.n_peers)) % g.n_peers;
  // pull: remote record chunk -> local copy (each byte crosses NVLink once), headers as far as this CTA needs them
  for (int t = 0; t < g.n_peers; ++t) {
    const int s = rot + t < g.n_peers ? rot + t : rot + t - g.n_peers;
    if (!inc[s] || direct) continue;
    const unsigned char* remote = g.peer[s].outbox + part.enc_off;
    unsigned char* local = g.peer[me].deltabox + (size_t)s * g.delta_stride + part.span_off;
    const size_t b0 = (size_t)lo * eb, b1 = ((size_t)hi * eb + 15) / 16 * 16;
    {
      // four independent 16-byte loads per thread before the first store: NVLink latency is paid once per batch
      const uint4* __restrict__ rsrc = reinterpret_cast<const uint4*>(remote + hdr + b0);
      uint4* __restrict__ ldst = reinterpret_cast<uint4*>(local + hdr + b0);
      const int n16 = (int)((b1 - b0) / 16);
      int q = threadIdx.x;
      for (; q + 3 * HB_THREADS < n16; q += 4 * HB_THREADS) {
        const uint4 a0 = rsrc[q], a1 = rsrc[q + HB_THREADS], a2 = rsrc[q + 2 * HB_THREADS], a3 = rsrc[q + 3 * HB_THREADS];
        ldst[q] = a0; ldst[q + HB_THREADS] = a1; ldst[q + 2 * HB_THREADS] = a2; ldst[q + 3 * HB_THREADS] = a3;
      }
      for (; q < n16; q += HB_THREADS) ldst[q] = rsrc[q];
    }
    if (codec == HB_UNIFORM8 || codec == HB_QUANTILE8) {
      const float cv = reinterpret_cast<const float*>(remote)[threadIdx.x];
      cbs[s][threadIdx.x] = cv;
      if (it.y == 0) reinterpret_cast<float*>(local)[threadIdx.x] = cv;
    } else if (codec == HB_MEANSTD16) {
      if (it.y == 0 && threadIdx.x < 2) reinterpret_cast<float*>(local)[threadIdx.x] = reinterpret_cast<const float*>(remote)[threadIdx.x];
    } else if (codec == HB_BLOCKWISE8) {
      cbs[s][threadIdx.x] = hb_code[threadIdx.x];  // shared-memory copy of the code (see hb_decode_setup)
      const int blk0 = lo / HB_BLOCK, blk1 = (hi + HB_BLOCK - 1) / HB_BLOCK;
      if (threadIdx.x < blk1 - blk0)
        reinterpret_cast<float*>(local)[blk0 + threadIdx.x] = reinterpret_cast<const float*>(remote)[blk0 + threadIdx.x];
    }
  }
  __syncthreads();

  const bool i_send = g.sends[me] != 0;
  float den = i_send ? g.weight[me] : 0.f;
  for (int s = 0; s < g.n_peers; ++s) if (inc[s]) den += g.weight[s];
  const float inv_den = den > 0.f ? 1.f / den : 0.f;
  float* x_local = g.peer[me].data + part.start;
  float* avg_out = g.avg + part.avg_off;
  const float alpha = g.alpha;
  const bool need_stats = codec == HB_MEANSTD16 || codec == HB_UNIFORM8;

  for (int b0 = lo; b0 < hi; b0 += HB_BLOCK) {
    float acc[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = b0 + (r * HB_THREADS + threadIdx.x) * 4;
      if (i_send && i + 4 <= len) {
        const float4 own = *reinterpret_cast<const float4*>(x_local + i);  // part starts are 16-byte aligned
        const float wm = g.weight[me];
        acc[r][0] = wm * own.x; acc[r][1] = wm * own.y; acc[r][2] = wm * own.z; acc[r][3] = wm * own.w;
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[r][k] = (i_send && i + k < len) ? g.weight[me] * x_local[i + k] : 0.f;
      }
    }
    for (int t = 0; t < g.n_peers; ++t) {
      const int s = rot + t < g.n_peers ? rot + t : rot + t - g.n_peers;
      if (!inc[s]) continue;
      const float w = g.weight[s];
      if (direct) {
        // four independent 16-byte loads from the sender's memory per thread, issued before the first use
        const float* __restrict__ rx = g.peer[s].data + part.start;
        float4 rv[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int i = b0 + (r * HB_THREADS + threadIdx.x) * 4;
          if (i + 4 <= len) {
            rv[r] = *reinterpret_cast<const float4*>(rx + i);
          } else {
            rv[r].x = i < len ? rx[i] : 0.f;
            rv[r].y = i + 1 < len ? rx[i + 1] : 0.f;
            rv[r].z = i + 2 < len ? rx[i + 2] : 0.f;
            rv[r].w = 0.f;
          }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          acc[r][0] = fmaf(w, rv[r].x, acc[r][0]); acc[r][1] = fmaf(w, rv[r].y, acc[r][1]);
          acc[r][2] = fmaf(w, rv[r].z, acc[r][2]); acc[r][3] = fmaf(w, rv[r].w, acc[r][3]);
        }
        continue;
      }
      const unsigned char* rec = g.peer[me].deltabox + (size_t)s * g.delta_stride + part.span_off;
      HbDecode dec;
      dec.codec = codec;
      dec.payload = rec + hdr;
      dec.absmax = reinterpret_cast<const float*>(rec);
      dec.mean = 0.f; dec.std = 1.f;
      if (codec == HB_MEANSTD16) {
        const float* rh = reinterpret_cast<const float*>(g.peer[s].outbox + part.enc_off);
        dec.mean = rh[0]; dec.std = rh[1];
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        float v[4];
        hb_decode4(dec, cbs[s], b0 + (r * HB_THREADS + threadIdx.x) * 4, len, v);
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[r][k] = fmaf(w, v[k], acc[r][k]);
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = b0 + (r * HB_THREADS + threadIdx.x) * 4;
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[r][k] *= inv_den;
      // store the average (senders' deltas are computed from it) and apply it to this reducer's own values
      if (i + 4 <= len) {
        *reinterpret_cast<float4*>(avg_out + i) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
        if (i_send) {
          float4 own = *reinterpret_cast<const float4*>(x_local + i);
          own.x = fmaf(alpha, acc[r][0] - own.x, own.x); own.y = fmaf(alpha, acc[r][1] - own.y, own.y);
          own.z = fmaf(alpha, acc[r][2] - own.z, own.z); own.w = fmaf(alpha, acc[r][3] - own.w, own.w);
          *reinterpret_cast<float4*>(x_local + i) = own;
        }
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (i + k < len) {
            avg_out[i + k] = acc[r][k];
            if (i_send) x_local[i + k] = fmaf(alpha, acc[r][k] - x_local[i + k], x_local[i + k]);
          }
        }
      }
    }
    if (need_stats) {
      for (int s = 0; s < g.n_peers; ++s) {
        if (!inc[s]) continue;
        const unsigned char* rec = g.peer[me].deltabox + (size_t)s * g.delta_stride + part.span_off;
        HbDecode dec;
        dec.codec = codec;
        dec.payload = rec + hdr;
        dec.absmax = reinterpret_cast<const float*>(rec);
        dec.mean = 0.f; dec.std = 1.f;
        if (codec == HB_MEANSTD16) {
          const float* rh = reinterpret_cast<const float*>(g.peer[s].outbox + part.enc_off);
          dec.mean = rh[0]; dec.std = rh[1];
        }
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int i = b0 + (r * HB_THREADS + threadIdx.x) * 4;
          float v[4];
          hb_decode4(dec, cbs[s], i, len, v);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (i + k < len) {
              const float d = acc[r][k] - v[k];
              s1 += d;
              s2 = fmaf(d, d, s2);
            }
          }
        }
        s1 = hm_block_sum(s1, red);
        s2 = hm_block_sum(s2, red);
        if (threadIdx.x == 0) {
          double* st = g.dstats + 2 * ((size_t)s * g.max_local_parts + j);
          atomicAdd(st, (double)s1);
          atomicAdd(st + 1, (double)s2);
        }
      }
    }
  }
}

// Apply (the all-gather half) for the parts that other peers reduced: x += alpha * decode(delta), or
// x += alpha * (avg - x) with the owner's average for uncompressed parts.
__global__ void __launch_bounds__(HB_THREADS)
hb_apply_kernel(const HbGroup* __restrict__ gp, const int4* __restrict__ items) {
  __shared__ float cb[256];
  __shared__ int wait_out;
  const HbGroup& g = *gp;
  const int4 it = items[blockIdx.x];
  const HbPart part = g.parts[it.x];
  const int len = part.len, me = g.me, owner = part.owner;
  const int lo = it.y * HB_CHUNK, hi = min(lo + HB_CHUNK, len);
  if (!g.sends[me]) return;
  float* x = g.peer[me].data + part.start;
  const float alpha = g.alpha;
  if (owner == me) return;  // the reduce kernel has already applied the average to this GPU's own span
  const unsigned long long deadline = hb_phase_start(g.t_start + 1) + g.reducer_timeout_ns;
  const unsigned int* flag = g.peer[owner].delta_ready + (size_t)me * g.max_local_parts + part.local_idx;
  const int d = hb_wait_decide(flag, g.epoch, g.apply_decision + it.x, nullptr, deadline, &wait_out);
  if (d != 1) {
    if (threadIdx.x == 0) {
      atomicOr(g.status + 1, 1ull << owner);
      atomicAdd(g.status + 2, (unsigned long long)(hi - lo));
    }
    return;  // zero delta: keep local values
  }
  if (part.codec == HB_NONE) {
    // uncompressed part: pull the owner's average itself; chunk starts are multiples of 16 elements
    const float* __restrict__ avg = g.peer[owner].avg + part.avg_off;
    const int n4 = (hi - lo) / 4;
    float4* x4 = reinterpret_cast<float4*>(x + lo);
    const float4* a4 = reinterpret_cast<const float4*>(avg + lo);
    int q = threadIdx.x;
    for (; q + 3 * HB_THREADS < n4; q += 4 * HB_THREADS) {
      float4 xv[4], av[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) { av[u] = a4[q + u * HB_THREADS]; xv[u] = x4[q + u * HB_THREADS]; }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        xv[u].x = fmaf(alpha, av[u].x - xv[u].x, xv[u].x); xv[u].y = fmaf(alpha, av[u].y - xv[u].y, xv[u].y);
        xv[u].z = fmaf(alpha, av[u].z - xv[u].z, xv[u].z); xv[u].w = fmaf(alpha, av[u].w - xv[u].w, xv[u].w);
        x4[q + u * HB_THREADS] = xv[u];
      }
    }
    for (; q < n4; q += HB_THREADS) {
      float4 xv = x4[q];
      const float4 av = a4[q];
      xv.x = fmaf(alpha, av.x - xv.x, xv.x); xv.y = fmaf(alpha, av.y - xv.y, xv.y);
      xv.z = fmaf(alpha, av.z - xv.z, xv.z); xv.w = fmaf(alpha, av.w - xv.w, xv.w);
      x4[q] = xv;
    }
    for (int i = lo + n4 * 4 + threadIdx.x; i < hi; i += HB_THREADS) x[i] = fmaf(alpha, avg[i] - x[i], x[i]);
    return;
  }
  const unsigned char* rec = g.peer[owner].deltabox + (size_t)me * g.delta_stride + part.span_off;
  HbDecode dec;
  hb_decode_setup(dec, part.codec, rec, len, cb);
  __syncthreads();
  int i = lo + 4 * threadIdx.x;
  for (; i + 12 * HB_THREADS + 4 <= hi; i += 16 * HB_THREADS) {
    // four groups of 4 elements per thread: all delta and x loads are issued before the first store
    float v[4][4];
    float4 xv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      hb_decode4(dec, cb, i + u * 4 * HB_THREADS, len, v[u]);
      xv[u] = *reinterpret_cast<const float4*>(x + i + u * 4 * HB_THREADS);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      xv[u].x = fmaf(alpha, v[u][0], xv[u].x); xv[u].y = fmaf(alpha, v[u][1], xv[u].y);
      xv[u].z = fmaf(alpha, v[u][2], xv[u].z); xv[u].w = fmaf(alpha, v[u][3], xv[u].w);
      *reinterpret_cast<float4*>(x + i + u * 4 * HB_THREADS) = xv[u];
    }
  }
  for (; i < hi; i += 4 * HB_THREADS) {
    float v[4];
    hb_decode4(dec, cb, i, len, v);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (i + k < hi) x[i + k] = fmaf(alpha, v[k], x[i + k]);
  }
}

// ---------------------------------------------------------------------------------------------------------------
enum HbPhase : int { HB_PH_STATS = 0, HB_PH_BORDERS = 1, HB_PH_ENCODE = 2, HB_PH_PUBLISH = 3, HB_PH_REDUCE = 4, HB_PH_APPLY = 5 };

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
    case HB_PH_REDUCE: hb_reduce_kernel<<<n_items, HB_THREADS, 0, stream>>>(g, it); break;
    case HB_PH_APPLY: hb_apply_kernel<<<n_items, HB_THREADS, 0, stream>>>(g, it); break;
    default: return -1;
  }
  return (int)cudaGetLastError();
}

// Stand-alone codec kernels for whole tensors (state downloads, expert RPCs, the compression module): they reuse
// the part machinery with a one-rank group whose "outbox" is the caller's output buffer.
