// Fused butterfly all-reduce round: weighted averaging of a flat fp32 vector across up to 16 GPUs of one NVLink
// box in ONE persistent kernel per GPU (plus a one-CTA gate kernel in front of it), with the tensor codecs fused into
// the reduce-scatter and all-gather halves.
//
// Semantics are those of the reference's RPC butterfly (hivemind/averaging/allreduce.py:151-359,
// hivemind/averaging/partition.py:179-277): the vector is cut into parts, part p is reduced by peer owner(p);
//   avg_p = sum_{s alive} w_s x~_{s,p} / sum_{s alive} w_s,   x~ = decode(encode(x)) for remote senders, x for the
//   reducer's own data;   sender s then applies x_s += alpha * decode(encode(avg_p - x~_{s,p})).
// A sender whose part is not published within `sender_timeout` is banned for that and all later parts (the
// denominator shrinks); a reducer whose delta is not published within `reducer_timeout` leaves the sender's values
// unchanged (allreduce.py:192-199,317-321 have the same two timeouts).
//
// Data movement is pull-only: a GPU writes only its own arena and reads its groupmates' arenas with plain loads
// through peer-mapped pointers. Nothing here uses TMA, cluster-wide loads or multimem.
//
// One round on one GPU:
//   gate kernel (1 CTA)  : waits (bounded) until the groupmates that read this arena two rounds ago have
//                          acknowledged that they are done, announces this GPU's round and waits (bounded) for every
//                          groupmate's announcement, so that the big kernel does not occupy the SMs while a peer is
//                          still busy elsewhere.
//   round kernel         : a persistent grid (two 256-thread CTAs per SM) that takes work items from a queue in a
//                          fixed order: send items, then reduce items, then apply items. A CTA that waits for a
//                          remote flag therefore never delays work that another GPU needs from this one.
//     send   (part of a groupmate, chunk)  : 8192 values are read ONCE into registers; statistics, quantisation,
//                          per-bin sums and the record header are computed in the same CTA; the CTA that completes
//                          a part publishes its flag together with this GPU's weight (64-bit store, release.sys).
//     reduce (own part, chunk)             : waits (bounded) for the senders' flags; pulls each sender's chunk record
//                          over NVLink once (keeping a local copy), accumulates in registers, applies the average to
//                          its own values, and for every sender encodes  avg - decode(copy)  in place: no separate
//                          statistics / encode / publish passes. Uncompressed parts are read straight from the
//                          senders' vectors and publish the average itself.
//     apply  (part of a groupmate, chunk)  : waits (bounded) for the owner's flag, x += alpha * decode(delta).
//
// Codecs work on chunks: every chunk of 8192 elements carries its own header (mean/std, codebook or block maxima),
// which is what lets a CTA finish a chunk without a second launch. Records never leave this box.
//
// Buffers that other GPUs read (outbox, delta box, averages, flags) exist twice and alternate with the parity of
// the owner's round counter; a reader finds the parity by looking for the round's epoch in both flag sets. Together
// with the acknowledgement ring (every GPU records the epochs of the rounds whose remote reads it has finished) a
// GPU never overwrites staging memory that a slower groupmate of an earlier round may still be reading.
#include "hb_codec.cuh"

#define HR_MAX_PEERS 16
#define HR_CHUNK 8192
#define HR_THREADS 512
#define HR_ROWS 4              // float4 groups per thread and chunk: 4 * 4 * 512 = 8192
#define HR_BLOCKS (HR_CHUNK / HB_BLOCK)   // block-wise quantization blocks per chunk
#define HR_SAMPLE 2048         // sample size for quantile borders
#define HR_RING 8              // acknowledgement ring entries

struct HrPart {
  long long start;             // first element in the flat vector
  long long enc_off;           // byte offset of the part's chunk records in every peer's outbox
  long long span_off;          // byte offset of the part's chunk records inside a per-sender region of the delta box
  long long avg_off;           // element offset inside the owner's average buffer
  int len, owner, local_idx, codec;
};

struct HrLayout {              // byte offsets inside every arena of a group (all members use the same layout)
  unsigned long long data, avg[2], outbox[2], deltabox[2], ready[2], dready[2], hello, done_ring;
};

struct HrRound {
  int n_peers, n_parts, me, max_local_parts;
  unsigned int epoch;
  int parity;                  // which copy of this GPU's staging buffers the round uses
  float alpha, my_weight;
  unsigned long long sender_timeout_ns, reducer_timeout_ns, delta_stride;
  int sends[HR_MAX_PEERS];     // 1 if the peer contributes data (mode != AUX)
  unsigned char* base[HR_MAX_PEERS];
  HrLayout lay;
  const HrPart* parts;
  const int4* items;           // {part, first chunk, chunks, -}; part == -1: publish pub_list[y .. y + z)
  const int* pub_list;         // uncompressed parts this GPU sends: only their flags are published
  int n_send, n_reduce, n_apply;
  int item_begin, item_end, queue_slot, final_stage;
  // per-round local scratch, all zero between rounds (the last CTA of a round clears it)
  // decisions: low word 0 undecided, 1 / 3 included (flag set 0 / 1), 2 left out; high word: the sender's weight
  unsigned long long* include;         // [max_local_parts][HR_MAX_PEERS]
  unsigned long long* apply_decision;  // [n_parts]
  int* ban;                    // [HR_MAX_PEERS]
  unsigned long long* t_start; // [2] start of the reduce / apply phase on this GPU
  unsigned long long* status;  // [0] banned sender mask [1] failed reducer mask [2] elements left unaveraged
  unsigned long long* status_out;
  int* part_done;              // [n_parts] chunks of a sent part that are complete
  int* dpart_done;             // [HR_MAX_PEERS][max_local_parts] chunks of a delta that are complete
  int* queue;                  // [4]: [3] counts the CTAs that have finished
  const float* code;           // [512] block-wise code and midpoints between consecutive entries
  unsigned int done_slot;
};

struct HrGate {
  int n_peers, me, parity, n_prev;
  unsigned int epoch, prev_epoch;
  unsigned long long ack_timeout_ns, hello_timeout_ns;
  unsigned char* base[HR_MAX_PEERS];
  unsigned char* prev_base[HR_MAX_PEERS];
  HrLayout lay;
  unsigned long long* gate_status;   // [0] peers without acknowledgement, [1] peers without announcement (masks)
};

HM_API int hm_br_sizeof_round() { return (int)sizeof(HrRound); }
HM_API int hm_br_sizeof_gate() { return (int)sizeof(HrGate); }
HM_API int hm_br_sizeof_part() { return (int)sizeof(HrPart); }
HM_API int hm_br_chunk() { return HR_CHUNK; }

__host__ __device__ inline int hr_header_bytes(int codec) {
  switch (codec) {
    case HB_MEANSTD16: return 16;
    case HB_QUANTILE8:
    case HB_UNIFORM8: return 1024;
    case HB_BLOCKWISE8: return 16;   // block maxima (HR_BLOCKS floats, padded to 16 bytes)
    default: return 0;
  }
}
__host__ __device__ inline long long hr_chunk_stride(int codec) {
  return hr_header_bytes(codec) + (long long)HR_CHUNK * hb_elem_bytes(codec);
}
// bytes of all chunk records of a part (every chunk takes a full stride, which keeps chunk records 16-byte aligned)
HM_API long long hm_br_record_bytes(int codec, int len) {
  if (codec == HB_NONE) return 0;
  return hr_chunk_stride(codec) * ((len + HR_CHUNK - 1) / HR_CHUNK);
}

__device__ __forceinline__ unsigned long long hr_ld_acquire_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void hr_st_release_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

struct HrShared {
  float red[4][HR_THREADS / 32];        // up to four simultaneous block reductions
  float cb[256];                        // codebook of the record being decoded
  float table[256];                     // borders (quantile) or code midpoints (block-wise) for bucketize
  float hsum[HR_THREADS / 64][256];     // per warp-pair bin sums and counts: a skewed distribution would otherwise
  int hcnt[HR_THREADS / 64][256];       //   serialise the whole CTA on a handful of addresses
  float smp[HR_SAMPLE];
  float w[HR_MAX_PEERS];
  int inc[HR_MAX_PEERS];
  int par[HR_MAX_PEERS];
  int item;
  int bcast;
  unsigned long long bcast64;
};

// element index inside the chunk handled by (row r, thread, k)
__device__ __forceinline__ int hr_elem(int r) { return (r * HR_THREADS + (int)threadIdx.x) * 4; }

// up to four block-wide sums / maxima at once; every thread gets the results
template <int N, bool MAX>
__device__ __forceinline__ void hr_block_reduce(float (&v)[N], HrShared& sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = MAX ? hm_warp_max(v[i]) : hm_warp_sum(v[i]);
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) sh.red[i][warp] = v[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < N; ++i) {
    float r = lane < HR_THREADS / 32 ? sh.red[i][lane] : 0.f;   // maxima here are of absolute values
    v[i] = MAX ? hm_warp_max(r) : hm_warp_sum(r);
  }
}

// Decode this thread's 32 elements of a chunk record (header already consumed by the caller: `cb` holds the
// codebook for the 8-bit codecs, mean / std / block maxima are passed in).
__device__ __forceinline__ void hr_decode_row(int codec, const unsigned char* payload, int i, float mean, float sd,
                                              const float* cb, const float* absmax, float out[4]) {
  switch (codec) {
    case HB_FLOAT16:
    case HB_MEANSTD16: {
      const uint2 x = *reinterpret_cast<const uint2*>(payload + (size_t)i * 2);
      const __half2 a = *reinterpret_cast<const __half2*>(&x.x), b = *reinterpret_cast<const __half2*>(&x.y);
      out[0] = __low2float(a); out[1] = __high2float(a); out[2] = __low2float(b); out[3] = __high2float(b);
      if (codec == HB_MEANSTD16) {
#pragma unroll
        for (int k = 0; k < 4; ++k) out[k] = fmaf(out[k], sd, mean);
      }
      return;
    }
    case HB_UNIFORM8:
    case HB_QUANTILE8: {
      const uchar4 q = *reinterpret_cast<const uchar4*>(payload + i);
      out[0] = cb[q.x]; out[1] = cb[q.y]; out[2] = cb[q.z]; out[3] = cb[q.w];
      return;
    }
    default: {  // HB_BLOCKWISE8
      const uchar4 q = *reinterpret_cast<const uchar4*>(payload + i);
      const float a = absmax[i / HB_BLOCK];
      out[0] = cb[q.x] * a; out[1] = cb[q.y] * a; out[2] = cb[q.z] * a; out[3] = cb[q.w] * a;
      return;
    }
  }
}

// Encode the chunk held in registers (v[r][k] = element hr_elem(r) + k, elements >= n are zero) into `rec`
// (header + payload). Every thread of the CTA calls this. Elements >= n still get payload bytes (of value zero or
// whatever zero maps to); they are never decoded.
__device__ void hr_encode_chunk(const float (&v)[HR_ROWS][4], int n, int codec, unsigned char* rec, HrShared& sh,
                                const float* code_tables) {
  unsigned char* payload = rec + hr_header_bytes(codec);
  if (codec == HB_FLOAT16) {
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
      const __half2 a = __floats2half2_rn(hb_clamp_half(v[r][0]), hb_clamp_half(v[r][1]));
      const __half2 b = __floats2half2_rn(hb_clamp_half(v[r][2]), hb_clamp_half(v[r][3]));
      uint2 o;
      o.x = *reinterpret_cast<const unsigned int*>(&a);
      o.y = *reinterpret_cast<const unsigned int*>(&b);
      *reinterpret_cast<uint2*>(payload + (size_t)i * 2) = o;
    }
    return;
  }
  if (codec == HB_MEANSTD16 || codec == HB_UNIFORM8) {
    float s1[1] = {0.f}, s2[1] = {0.f};
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r)
#pragma unroll
      for (int k = 0; k < 4; ++k) s1[0] += v[r][k];   // padding elements are zero
    hr_block_reduce<1, false>(s1, sh);
    const float mean = s1[0] / (float)n;
    // centred second pass over the registers: no cancellation
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float d = (i + k < n) ? v[r][k] - mean : 0.f;
        s2[0] = fmaf(d, d, s2[0]);
      }
    }
    hr_block_reduce<1, false>(s2, sh);
    if (codec == HB_MEANSTD16) {
      const float sd = fmaxf(sqrtf(s2[0] / (float)n), 1.1920929e-07f);
      const float inv = 1.f / sd;
      if (threadIdx.x == 0) {
        reinterpret_cast<float*>(rec)[0] = mean;
        reinterpret_cast<float*>(rec)[1] = sd;
      }
#pragma unroll
      for (int r = 0; r < HR_ROWS; ++r) {
        const int i = hr_elem(r);
        const __half2 a = __floats2half2_rn(hb_clamp_half((v[r][0] - mean) * inv), hb_clamp_half((v[r][1] - mean) * inv));
        const __half2 b = __floats2half2_rn(hb_clamp_half((v[r][2] - mean) * inv), hb_clamp_half((v[r][3] - mean) * inv));
        uint2 o;
        o.x = *reinterpret_cast<const unsigned int*>(&a);
        o.y = *reinterpret_cast<const unsigned int*>(&b);
        *reinterpret_cast<uint2*>(payload + (size_t)i * 2) = o;
      }
      return;
    }
    // HB_UNIFORM8: 256 levels of width 6 sigma / 256 around the mean; the codebook holds the mean of every level
    const float scale = 6.f * sqrtf(s2[0] / fmaxf((float)n - 1.f, 1.f)) / 256.f;
    const float inv = (scale > 0.f && isfinite(scale)) ? 1.f / scale : 1.f;
    for (int i = threadIdx.x; i < (HR_THREADS / 64) * 256; i += HR_THREADS) { (&sh.hsum[0][0])[i] = 0.f; (&sh.hcnt[0][0])[i] = 0; }
    __syncthreads();
    const int hw = threadIdx.x >> 6;
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
      unsigned char q[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        int b = (int)rintf((v[r][k] - mean) * inv) + 128;
        b = b < 0 ? 0 : (b > 255 ? 255 : b);
        q[k] = (unsigned char)b;
        if (i + k < n) {
          atomicAdd(&sh.hsum[hw][b], v[r][k]);
          atomicAdd(&sh.hcnt[hw][b], 1);
        }
      }
      *reinterpret_cast<uchar4*>(payload + i) = make_uchar4(q[0], q[1], q[2], q[3]);
    }
    __syncthreads();
    if (threadIdx.x < 256) {
      float total = 0.f;
      int count = 0;
#pragma unroll
      for (int w = 0; w < HR_THREADS / 64; ++w) { total += sh.hsum[w][threadIdx.x]; count += sh.hcnt[w][threadIdx.x]; }
      reinterpret_cast<float*>(rec)[threadIdx.x] = total / (float)(count > 0 ? count : 1);
    }
    return;
  }
  if (codec == HB_QUANTILE8) {
    // borders from a regular sample of at most 2048 values (every value when the chunk has no more than that)
    int stride = 1;
    while (stride * HR_SAMPLE < n) stride <<= 1;
    const int S = (n + stride - 1) / stride;
    for (int i = threadIdx.x; i < HR_SAMPLE; i += HR_THREADS) sh.smp[i] = INFINITY;
    for (int i = threadIdx.x; i < (HR_THREADS / 64) * 256; i += HR_THREADS) { (&sh.hsum[0][0])[i] = 0.f; (&sh.hcnt[0][0])[i] = 0; }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (i + k < n && ((i + k) & (stride - 1)) == 0) sh.smp[(i + k) / stride] = v[r][k];
    }
    __syncthreads();
    for (int size = 2; size <= HR_SAMPLE; size <<= 1) {
      for (int st = size >> 1; st > 0; st >>= 1) {
        for (int t = threadIdx.x; t < HR_SAMPLE / 2; t += HR_THREADS) {
          const int i = 2 * t - (t & (st - 1));
          const int j = i + st;
          const bool up = (i & size) == 0;
          const float a = sh.smp[i], b = sh.smp[j];
          if ((a > b) == up) { sh.smp[i] = b; sh.smp[j] = a; }
        }
        __syncthreads();
      }
    }
    if (threadIdx.x < 256) {
      float b = INFINITY;
      if (threadIdx.x < 255 && S > 0) {
        int rk = (int)(((long long)(threadIdx.x + 1) * S) / 256);
        rk = rk >= S ? S - 1 : rk;
        b = sh.smp[rk];
      }
      sh.table[threadIdx.x] = b;
    }
    __syncthreads();
    const int hw = threadIdx.x >> 6;
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
      unsigned char q[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int b = hb_bucketize(sh.table, v[r][k]);
        q[k] = (unsigned char)b;
        if (i + k < n) {
          atomicAdd(&sh.hsum[hw][b], v[r][k]);
          atomicAdd(&sh.hcnt[hw][b], 1);
        }
      }
      *reinterpret_cast<uchar4*>(payload + i) = make_uchar4(q[0], q[1], q[2], q[3]);
    }
    __syncthreads();
    if (threadIdx.x < 256) {
      float total = 0.f;
      int count = 0;
#pragma unroll
      for (int w = 0; w < HR_THREADS / 64; ++w) { total += sh.hsum[w][threadIdx.x]; count += sh.hcnt[w][threadIdx.x]; }
      reinterpret_cast<float*>(rec)[threadIdx.x] = total / (float)(count > 0 ? count : 1);
    }
    return;
  }
  // HB_BLOCKWISE8: rows [b * RPB, (b + 1) * RPB) of every thread belong to block b (4096 elements)
  {
    constexpr int RPB = HR_ROWS / HR_BLOCKS;
    float m[HR_BLOCKS];
#pragma unroll
    for (int b = 0; b < HR_BLOCKS; ++b) {
      m[b] = 0.f;
#pragma unroll
      for (int rr = 0; rr < RPB; ++rr)
#pragma unroll
        for (int k = 0; k < 4; ++k) m[b] = fmaxf(m[b], fabsf(v[RPB * b + rr][k]));
    }
    if (threadIdx.x < 256) sh.table[threadIdx.x] = code_tables[256 + threadIdx.x];
    hr_block_reduce<HR_BLOCKS, true>(m, sh);   // also orders the table writes before the reads below
    if (threadIdx.x < HR_BLOCKS) reinterpret_cast<float*>(rec)[threadIdx.x] = m[threadIdx.x];
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
      const float inv = 1.f / fmaxf(m[r / RPB], 1.17549435e-38f);
      unsigned char q[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) q[k] = (unsigned char)hb_bucketize(sh.table, v[r][k] * inv);
      *reinterpret_cast<uchar4*>(payload + i) = make_uchar4(q[0], q[1], q[2], q[3]);
    }
  }
}

// Load what decoding a chunk record needs besides the payload: the codebook into shared memory, scalars into
// registers. Every thread calls this; it ends with a barrier.
__device__ __forceinline__ void hr_decode_setup(int codec, const unsigned char* rec, HrShared& sh, const float* code_tables,
                                                float& mean, float& sd, float absmax[HR_BLOCKS]) {
  mean = 0.f;
  sd = 1.f;
  __syncthreads();   // the previous user of sh.cb is done
  if (codec == HB_MEANSTD16) {
    mean = reinterpret_cast<const float*>(rec)[0];
    sd = reinterpret_cast<const float*>(rec)[1];
  } else if (codec == HB_UNIFORM8 || codec == HB_QUANTILE8) {
    if (threadIdx.x < 256) sh.cb[threadIdx.x] = reinterpret_cast<const float*>(rec)[threadIdx.x];
  } else if (codec == HB_BLOCKWISE8) {
    if (threadIdx.x < 256) sh.cb[threadIdx.x] = code_tables[threadIdx.x];
#pragma unroll
    for (int b = 0; b < HR_BLOCKS; ++b) absmax[b] = reinterpret_cast<const float*>(rec)[b];
  }
  __syncthreads();
}

__device__ __forceinline__ unsigned long long hr_ld_acquire_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long hr_cas_release_gpu_u64(unsigned long long* p, unsigned long long expected,
                                                                    unsigned long long desired) {
  unsigned long long old;
  asm volatile("atom.release.gpu.global.cas.b64 %0, [%1], %2, %3;" : "=l"(old) : "l"(p), "l"(expected), "l"(desired) : "memory");
  return old;
}

__device__ __forceinline__ unsigned long long hr_phase_start(unsigned long long* slot) {
  unsigned long long t = *reinterpret_cast<volatile unsigned long long*>(slot);
  if (t == 0) {
    const unsigned long long now = hm_globaltimer_ns();
    const unsigned long long prev = atomicCAS(slot, 0ull, now);
    t = prev == 0 ? now : prev;
  }
  return t;
}

// Bounded wait of ONE thread for a flag that a groupmate publishes in one of its two flag sets. The outcome goes
// into `decision` by compare-and-swap, so that all CTAs that work on the same part agree; its low word says 1 / 3 =
// published (in flag set 0 / 1) or 2 = gave up, its high word carries the weight that came with the flag. Only the
// first CTA to get here talks to the groupmate: it reads the flag with acquire.sys and publishes the decision with
// release.gpu; every later CTA finds the decision with ONE acquire.gpu load, which orders its reads of the
// groupmate's data after the groupmate's writes just the same (release / acquire chains are cumulative). The clock
// is only looked at while the flag is missing: the time limit runs from the moment this GPU first had to wait in
// the phase (`t_start`).
__device__ unsigned long long hr_decide(const unsigned long long* flag0, const unsigned long long* flag1, bool wide,
                                        unsigned int want, unsigned long long* decision, const int* ban_flag,
                                        unsigned long long* t_start, unsigned long long timeout_ns) {
  auto load = [&](const unsigned long long* f) -> unsigned long long {
    return wide ? hr_ld_acquire_sys_u64(f) : (unsigned long long)hm_ld_acquire_sys(reinterpret_cast<const unsigned int*>(f));
  };
  unsigned long long d = hr_ld_acquire_gpu_u64(decision);
  unsigned long long deadline = 0;
  while ((unsigned int)d == 0) {
    const unsigned long long v0 = load(flag0), v1 = load(flag1);
    unsigned long long verdict = 0;
    if ((unsigned int)v0 == want) {
      verdict = 1ull | (v0 & 0xffffffff00000000ull);
    } else if ((unsigned int)v1 == want) {
      verdict = 3ull | (v1 & 0xffffffff00000000ull);
    } else {
      if (deadline == 0) deadline = hr_phase_start(t_start) + timeout_ns;
      if ((unsigned int)v0 == (want | HB_FAIL_BIT) || (unsigned int)v1 == (want | HB_FAIL_BIT) ||
          (ban_flag && *reinterpret_cast<const volatile int*>(ban_flag)) || hm_globaltimer_ns() > deadline)
        verdict = 2ull;
    }
    if (verdict == 0) __nanosleep(200);
    else hr_cas_release_gpu_u64(decision, 0ull, verdict);
    d = hr_ld_acquire_gpu_u64(decision);
  }
  return d;
}

// Chunks [.., .. + add) of a part are complete; true for the thread whose increment completes the part. The caller
// has passed a CTA barrier after the chunks' writes; the fence (cumulative) makes them visible system-wide before the
// count moves, and the thread that completes the part fences again before it publishes the part's flag.
__device__ __forceinline__ bool hr_chunks_done(int* counter, int add, int n_chunks) {
  __threadfence_system();
  const bool last = atomicAdd(counter, add) == n_chunks - add;
  if (last) __threadfence_system();
  return last;
}

// ---------------------------------------------------------------------------------------------------------------
__device__ void hr_send_item(const HrRound& g, int p, int c0, int z, HrShared& sh) {
  unsigned char* my = g.base[g.me];
  unsigned long long* ready = reinterpret_cast<unsigned long long*>(my + g.lay.ready[g.parity]);
  const unsigned long long flag = (unsigned long long)g.epoch | ((unsigned long long)__float_as_uint(g.my_weight) << 32);
  if (p < 0) {
    // uncompressed parts: readers take the values from the vector itself, only the flags are published
    for (int i = threadIdx.x; i < z; i += HR_THREADS) hr_st_release_sys_u64(ready + g.pub_list[c0 + i], flag);
    return;
  }
  const HrPart part = g.parts[p];
  const long long stride = hr_chunk_stride(part.codec);
  for (int c = c0; c < c0 + z; ++c) {
    const int lo = c * HR_CHUNK, n = min(HR_CHUNK, part.len - lo);
    const float* x = reinterpret_cast<const float*>(my + g.lay.data) + part.start + lo;
    float v[HR_ROWS][4];
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
      if (i + 4 <= n) {
        const float4 t = *reinterpret_cast<const float4*>(x + i);
        v[r][0] = t.x; v[r][1] = t.y; v[r][2] = t.z; v[r][3] = t.w;
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) v[r][k] = (i + k < n) ? x[i + k] : 0.f;
      }
    }
    if (c != c0) __syncthreads();   // the previous chunk's encoder is done with the shared tables
    hr_encode_chunk(v, n, part.codec, my + g.lay.outbox[g.parity] + part.enc_off + (long long)c * stride, sh, g.code);
  }
  const int n_chunks = (part.len + HR_CHUNK - 1) / HR_CHUNK;
  __syncthreads();
  if (threadIdx.x == 0 && hr_chunks_done(g.part_done + p, z, n_chunks)) hr_st_release_sys_u64(ready + p, flag);
}

__device__ __forceinline__ void hr_load_rows(const float* __restrict__ src, int n, float4 (&rv)[HR_ROWS]) {
#pragma unroll
  for (int r = 0; r < HR_ROWS; ++r) {
    const int i = hr_elem(r);
    if (i + 4 <= n) {
      rv[r] = *reinterpret_cast<const float4*>(src + i);
    } else {
      rv[r].x = i < n ? src[i] : 0.f;
      rv[r].y = i + 1 < n ? src[i + 1] : 0.f;
      rv[r].z = i + 2 < n ? src[i + 2] : 0.f;
      rv[r].w = 0.f;
    }
  }
}

__device__ void hr_reduce_item(const HrRound& g, int p, int c0, int z, HrShared& sh) {
  const HrPart part = g.parts[p];
  const int codec = part.codec, j = part.local_idx, me = g.me;
  const int n_chunks = (part.len + HR_CHUNK - 1) / HR_CHUNK;
  unsigned char* my = g.base[me];

  // one lane per sender waits for (or looks up the decision about) that sender's flag
  if (threadIdx.x < HR_MAX_PEERS) {
    const int s = threadIdx.x;
    int inc = 0, par = 0;
    float w = 0.f;
    if (s < g.n_peers && s != me && g.sends[s]) {
      const unsigned long long* f0 = reinterpret_cast<const unsigned long long*>(g.base[s] + g.lay.ready[0]) + p;
      const unsigned long long* f1 = reinterpret_cast<const unsigned long long*>(g.base[s] + g.lay.ready[1]) + p;
      const unsigned long long d = hr_decide(f0, f1, true, g.epoch, g.include + (size_t)j * HR_MAX_PEERS + s, g.ban + s,
                                             g.t_start, g.sender_timeout_ns);
      const unsigned int v = (unsigned int)d;
      inc = v == 1u || v == 3u;
      par = (int)(v >> 1);
      w = __uint_as_float((unsigned int)(d >> 32));
      if (v == 2u) {
        atomicExch(g.ban + s, 1);   // a sender that missed one part is left out of the later ones too
        atomicOr(g.status, 1ull << s);
      }
    }
    sh.inc[s] = inc;
    sh.par[s] = par;
    sh.w[s] = w;
  }
  __syncthreads();

  const bool i_send = g.sends[me] != 0;
  float den = i_send ? g.my_weight : 0.f;
  for (int s = 0; s < g.n_peers; ++s) if (sh.inc[s]) den += sh.w[s];
  // a total weight of zero (every member tagging along) averages nothing: values stay, deltas are reported as failed
  const bool dead = !(den > 0.f);
  const float inv_den = dead ? 0.f : 1.f / den;
  const float alpha_own = dead ? 0.f : g.alpha;
  const long long stride = hr_chunk_stride(codec);
  const int hdr = hr_header_bytes(codec);
  // every reducer walks the senders in its own rotation, so that at any moment the reducers of a group read from
  // different GPUs instead of all draining the same sender's links
  const int rot = (me + 1) % g.n_peers;
  // uncompressed parts: the first sender's rows of the NEXT chunk are requested before this chunk's results are
  // written, which keeps remote reads in flight while the CTA is busy with local memory
  int first = -1;
  if (codec == HB_NONE) {
    for (int t = 0; t < g.n_peers && first < 0; ++t) {
      const int s = rot + t < g.n_peers ? rot + t : rot + t - g.n_peers;
      if (sh.inc[s]) first = s;
    }
  }
  float4 ahead[HR_ROWS];
  if (first >= 0)
    hr_load_rows(reinterpret_cast<const float*>(g.base[first] + g.lay.data) + part.start + c0 * HR_CHUNK,
                 min(HR_CHUNK, part.len - c0 * HR_CHUNK), ahead);

  for (int c = c0; c < c0 + z; ++c) {
    const int lo = c * HR_CHUNK, n = min(HR_CHUNK, part.len - lo);
    float* x_local = reinterpret_cast<float*>(my + g.lay.data) + part.start + lo;
    float acc[HR_ROWS][4];
    {
      float4 own[HR_ROWS];
      if (i_send) hr_load_rows(x_local, n, own);
#pragma unroll
      for (int r = 0; r < HR_ROWS; ++r) {
        acc[r][0] = i_send ? g.my_weight * own[r].x : 0.f; acc[r][1] = i_send ? g.my_weight * own[r].y : 0.f;
        acc[r][2] = i_send ? g.my_weight * own[r].z : 0.f; acc[r][3] = i_send ? g.my_weight * own[r].w : 0.f;
      }
    }
    for (int t = 0; t < g.n_peers; ++t) {
      const int s = rot + t < g.n_peers ? rot + t : rot + t - g.n_peers;
      if (!sh.inc[s]) continue;
      const float w = sh.w[s];
      if (codec == HB_NONE) {
        float4 rv[HR_ROWS];
        if (s == first) {
#pragma unroll
          for (int r = 0; r < HR_ROWS; ++r) rv[r] = ahead[r];
          if (c + 1 < c0 + z)
            hr_load_rows(reinterpret_cast<const float*>(g.base[s] + g.lay.data) + part.start + lo + HR_CHUNK,
                         min(HR_CHUNK, part.len - lo - HR_CHUNK), ahead);
        } else {
          hr_load_rows(reinterpret_cast<const float*>(g.base[s] + g.lay.data) + part.start + lo, n, rv);
        }
#pragma unroll
        for (int r = 0; r < HR_ROWS; ++r) {
          acc[r][0] = fmaf(w, rv[r].x, acc[r][0]); acc[r][1] = fmaf(w, rv[r].y, acc[r][1]);
          acc[r][2] = fmaf(w, rv[r].z, acc[r][2]); acc[r][3] = fmaf(w, rv[r].w, acc[r][3]);
        }
        continue;
      }
      // compressed: pull the sender's chunk record once, keep a copy where its delta will be written
      const unsigned char* remote = g.base[s] + g.lay.outbox[sh.par[s]] + part.enc_off + (long long)c * stride;
      unsigned char* local = my + g.lay.deltabox[g.parity] + (size_t)s * g.delta_stride + part.span_off + (long long)c * stride;
      float mean, sd, absmax[HR_BLOCKS] = {};
      hr_decode_setup(codec, remote, sh, g.code, mean, sd, absmax);
      if (hdr == 1024) {
        if (threadIdx.x < 256) reinterpret_cast<float*>(local)[threadIdx.x] = sh.cb[threadIdx.x];
      } else if (hdr == 16 && threadIdx.x < 4) {   // mean / std or block maxima: one 16-byte header
        reinterpret_cast<float*>(local)[threadIdx.x] = reinterpret_cast<const float*>(remote)[threadIdx.x];
      }
      if (hb_elem_bytes(codec) == 2) {
        uint2 raw[HR_ROWS];
#pragma unroll
        for (int r = 0; r < HR_ROWS; ++r) raw[r] = *reinterpret_cast<const uint2*>(remote + hdr + (size_t)hr_elem(r) * 2);
#pragma unroll
        for (int r = 0; r < HR_ROWS; ++r) {
          *reinterpret_cast<uint2*>(local + hdr + (size_t)hr_elem(r) * 2) = raw[r];
          const __half2 a = *reinterpret_cast<const __half2*>(&raw[r].x), b = *reinterpret_cast<const __half2*>(&raw[r].y);
          float o[4] = {__low2float(a), __high2float(a), __low2float(b), __high2float(b)};
#pragma unroll
          for (int k = 0; k < 4; ++k) acc[r][k] = fmaf(w, fmaf(o[k], sd, mean), acc[r][k]);
        }
      } else {
        uchar4 raw[HR_ROWS];
#pragma unroll
        for (int r = 0; r < HR_ROWS; ++r) raw[r] = *reinterpret_cast<const uchar4*>(remote + hdr + hr_elem(r));
#pragma unroll
        for (int r = 0; r < HR_ROWS; ++r) {
          *reinterpret_cast<uchar4*>(local + hdr + hr_elem(r)) = raw[r];
          const float a = codec == HB_BLOCKWISE8 ? absmax[r / (HR_ROWS / HR_BLOCKS)] : 1.f;
          acc[r][0] = fmaf(w, sh.cb[raw[r].x] * a, acc[r][0]); acc[r][1] = fmaf(w, sh.cb[raw[r].y] * a, acc[r][1]);
          acc[r][2] = fmaf(w, sh.cb[raw[r].z] * a, acc[r][2]); acc[r][3] = fmaf(w, sh.cb[raw[r].w] * a, acc[r][3]);
        }
      }
    }
    // the average; applied to this reducer's own values right here
    float* avg_out = reinterpret_cast<float*>(my + g.lay.avg[g.parity]) + part.avg_off + lo;
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[r][k] *= inv_den;
      if (i + 4 <= n) {
        if (codec == HB_NONE) *reinterpret_cast<float4*>(avg_out + i) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
        if (i_send) {
          float4 own = *reinterpret_cast<const float4*>(x_local + i);
          own.x = fmaf(alpha_own, acc[r][0] - own.x, own.x); own.y = fmaf(alpha_own, acc[r][1] - own.y, own.y);
          own.z = fmaf(alpha_own, acc[r][2] - own.z, own.z); own.w = fmaf(alpha_own, acc[r][3] - own.w, own.w);
          *reinterpret_cast<float4*>(x_local + i) = own;
        }
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (i + k < n) {
            if (codec == HB_NONE) avg_out[i + k] = acc[r][k];
            if (i_send) x_local[i + k] = fmaf(alpha_own, acc[r][k] - x_local[i + k], x_local[i + k]);
          } else {
            acc[r][k] = 0.f;
          }
        }
      }
    }
    // deltas: avg - decode(copy of the sender's record), encoded over the copy, one sender after the other
    if (codec != HB_NONE && !dead) {
      for (int s = 0; s < g.n_peers; ++s) {
        if (!sh.inc[s]) continue;
        unsigned char* local = my + g.lay.deltabox[g.parity] + (size_t)s * g.delta_stride + part.span_off + (long long)c * stride;
        float mean, sd, absmax[HR_BLOCKS] = {};
        hr_decode_setup(codec, local, sh, g.code, mean, sd, absmax);
        float d[HR_ROWS][4];
#pragma unroll
        for (int r = 0; r < HR_ROWS; ++r) {
          const int i = hr_elem(r);
          float o[4];
          hr_decode_row(codec, local + hdr, i, mean, sd, sh.cb, absmax, o);
#pragma unroll
          for (int k = 0; k < 4; ++k) d[r][k] = (i + k < n) ? acc[r][k] - o[k] : 0.f;
        }
        __syncthreads();   // every thread has decoded with the old header before anybody writes the new one
        hr_encode_chunk(d, n, codec, local, sh, g.code);
      }
    }
  }
  // one lane per sender counts the chunks of its delta; the lane that completes a part publishes its flag
  __syncthreads();
  if (threadIdx.x < g.n_peers) {
    const int s = threadIdx.x;
    if (s != me && g.sends[s] && hr_chunks_done(g.dpart_done + (size_t)s * g.max_local_parts + j, z, n_chunks)) {
      unsigned int* flag = reinterpret_cast<unsigned int*>(my + g.lay.dready[g.parity]) + (size_t)s * g.max_local_parts + j;
      hm_st_release_sys(flag, (sh.inc[s] && !dead) ? g.epoch : (g.epoch | HB_FAIL_BIT));
    }
  }
}

__device__ void hr_apply_item(const HrRound& g, int p, int c0, int z, HrShared& sh) {
  if (!g.sends[g.me]) return;
  const HrPart part = g.parts[p];
  const int me = g.me, owner = part.owner, codec = part.codec;
  if (owner == me) return;   // the reduce item has already applied the average to this GPU's own span
  if (threadIdx.x == 0) {
    const size_t fidx = (size_t)me * g.max_local_parts + part.local_idx;
    const unsigned int* f0 = reinterpret_cast<const unsigned int*>(g.base[owner] + g.lay.dready[0]) + fidx;
    const unsigned int* f1 = reinterpret_cast<const unsigned int*>(g.base[owner] + g.lay.dready[1]) + fidx;
    sh.bcast = (int)(unsigned int)hr_decide(reinterpret_cast<const unsigned long long*>(f0), reinterpret_cast<const unsigned long long*>(f1),
                                            false, g.epoch, g.apply_decision + p, nullptr, g.t_start + 1, g.reducer_timeout_ns);
  }
  __syncthreads();
  const int d = sh.bcast;
  if (d == 2) {
    if (threadIdx.x == 0) {
      atomicOr(g.status + 1, 1ull << owner);
      atomicAdd(g.status + 2, (unsigned long long)(min((c0 + z) * HR_CHUNK, part.len) - c0 * HR_CHUNK));
    }
    return;   // zero delta: keep the local values
  }
  const int opar = d >> 1;
  const float alpha = g.alpha;
  const long long stride = hr_chunk_stride(codec);
  const int hdr = hr_header_bytes(codec);
  for (int c = c0; c < c0 + z; ++c) {
    const int lo = c * HR_CHUNK, n = min(HR_CHUNK, part.len - lo);
    float* x = reinterpret_cast<float*>(g.base[me] + g.lay.data) + part.start + lo;
    float dv[HR_ROWS][4];
    if (codec == HB_NONE) {
      float4 av[HR_ROWS];
      hr_load_rows(reinterpret_cast<const float*>(g.base[owner] + g.lay.avg[opar]) + part.avg_off + lo, n, av);
#pragma unroll
      for (int r = 0; r < HR_ROWS; ++r) { dv[r][0] = av[r].x; dv[r][1] = av[r].y; dv[r][2] = av[r].z; dv[r][3] = av[r].w; }
    } else {
      const unsigned char* rec = g.base[owner] + g.lay.deltabox[opar] + (size_t)me * g.delta_stride + part.span_off + (long long)c * stride;
      float mean, sd, absmax[HR_BLOCKS] = {};
      hr_decode_setup(codec, rec, sh, g.code, mean, sd, absmax);
#pragma unroll
      for (int r = 0; r < HR_ROWS; ++r) hr_decode_row(codec, rec + hdr, hr_elem(r), mean, sd, sh.cb, absmax, dv[r]);
    }
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
      if (i + 4 <= n) {
        float4 xv = *reinterpret_cast<const float4*>(x + i);
        if (codec == HB_NONE) {
          xv.x = fmaf(alpha, dv[r][0] - xv.x, xv.x); xv.y = fmaf(alpha, dv[r][1] - xv.y, xv.y);
          xv.z = fmaf(alpha, dv[r][2] - xv.z, xv.z); xv.w = fmaf(alpha, dv[r][3] - xv.w, xv.w);
        } else {
          xv.x = fmaf(alpha, dv[r][0], xv.x); xv.y = fmaf(alpha, dv[r][1], xv.y);
          xv.z = fmaf(alpha, dv[r][2], xv.z); xv.w = fmaf(alpha, dv[r][3], xv.w);
        }
        *reinterpret_cast<float4*>(x + i) = xv;
      } else {
        for (int k = 0; k < 4; ++k)
          if (i + k < n) x[i + k] = codec == HB_NONE ? fmaf(alpha, dv[r][k] - x[i + k], x[i + k]) : fmaf(alpha, dv[r][k], x[i + k]);
      }
    }
  }
}

__global__ void __launch_bounds__(HR_THREADS, 2) hr_round_kernel(const __grid_constant__ HrRound g) {
  __shared__ HrShared sh;
  // Items are dealt round-robin. The list is ordered send, reduce, apply, so every CTA finishes its send items
  // before it may wait for a groupmate, and nothing that a groupmate needs from this GPU queues up behind a wait.
  for (int idx = g.item_begin + (int)blockIdx.x; idx < g.item_end; idx += (int)gridDim.x) {
    __syncthreads();
    const int4 it = g.items[idx];
    if (idx < g.n_send) hr_send_item(g, it.x, it.y, it.z, sh);
    else if (idx < g.n_send + g.n_reduce) hr_reduce_item(g, it.x, it.y, it.z, sh);
    else hr_apply_item(g, it.x, it.y, it.z, sh);
  }
  // the last CTA to leave closes the round: acknowledges that this GPU has finished reading its groupmates'
  // arenas, hands the status words to the host and clears the scratch for the next round
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    sh.bcast = atomicAdd(g.queue + 3, 1) == (int)gridDim.x - 1;
  }
  __syncthreads();
  if (!sh.bcast) return;
  if (threadIdx.x == 0) g.queue[3] = 0;
  if (!g.final_stage) return;
  __threadfence();
  if (threadIdx.x < 4) g.status_out[threadIdx.x] = *reinterpret_cast<volatile unsigned long long*>(g.status + threadIdx.x);
  __syncthreads();
  for (int i = threadIdx.x; i < g.max_local_parts * HR_MAX_PEERS; i += HR_THREADS) { g.include[i] = 0ull; g.dpart_done[i] = 0; }
  for (int i = threadIdx.x; i < g.n_parts; i += HR_THREADS) { g.apply_decision[i] = 0ull; g.part_done[i] = 0; }
  if (threadIdx.x < HR_MAX_PEERS) g.ban[threadIdx.x] = 0;
  if (threadIdx.x < 2) g.t_start[threadIdx.x] = 0;
  if (threadIdx.x < 4) g.status[threadIdx.x] = 0;
  if (threadIdx.x == 0) {
    unsigned int* ring = reinterpret_cast<unsigned int*>(g.base[g.me] + g.lay.done_ring);
    hm_st_release_sys(ring + (g.done_slot % HR_RING), g.epoch);
  }
}

// One CTA in front of the round kernel (see the file comment). Lane t looks after groupmate t.
__global__ void __launch_bounds__(32) hr_gate_kernel(const __grid_constant__ HrGate g) {
  const int t = threadIdx.x;
  const unsigned long long t0 = hm_globaltimer_ns();
  // 1. groupmates of the round that last used this parity of the staging buffers must have finished reading them
  bool acked = true;
  if (t < g.n_prev && g.prev_base[t] != nullptr) {
    const unsigned int* ring = reinterpret_cast<const unsigned int*>(g.prev_base[t] + g.lay.done_ring);
    acked = false;
    for (;;) {
      // the whole ring in two 16-byte loads; the acknowledgement only has to precede this GPU's later writes, which
      // the fence after the loop takes care of
      uint4 lo, hi;
      asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w) : "l"(ring));
      asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w) : "l"(ring + 4));
      const unsigned int e = g.prev_epoch;
      acked = lo.x == e || lo.y == e || lo.z == e || lo.w == e || hi.x == e || hi.y == e || hi.z == e || hi.w == e;
      if (acked || hm_globaltimer_ns() - t0 > g.ack_timeout_ns) break;
      __nanosleep(500);
    }
    __threadfence_system();
  }
  const unsigned int missing_ack = __ballot_sync(0xffffffffu, !acked);
  // 2. announce this GPU's round, then wait for everybody else's announcement
  if (t == 0) {
    unsigned int* hello = reinterpret_cast<unsigned int*>(g.base[g.me] + g.lay.hello) + g.parity;
    hm_st_release_sys(hello, g.epoch);
  }
  bool present = true;
  if (t < g.n_peers && t != g.me) {
    const unsigned int* hello = reinterpret_cast<const unsigned int*>(g.base[t] + g.lay.hello);
    present = false;
    const unsigned long long t1 = hm_globaltimer_ns();
    for (;;) {
      uint2 both;   // the flags of both parities at once
      asm volatile("ld.acquire.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(both.x), "=r"(both.y) : "l"(hello) : "memory");
      present = both.x == g.epoch || both.y == g.epoch;
      if (present || hm_globaltimer_ns() - t1 > g.hello_timeout_ns) break;
      __nanosleep(500);
    }
  }
  const unsigned int missing_hello = __ballot_sync(0xffffffffu, !present);
  if (t == 0 && g.gate_status != nullptr) {
    g.gate_status[0] = missing_ack;
    g.gate_status[1] = missing_hello;
  }
}

// Launch the gate kernel (one small CTA) on `stream`. `gate` is a host pointer to an HrGate.
HM_API int hm_br_gate(const void* gate, cudaStream_t stream) {
  const HrGate* g = (const HrGate*)gate;
  hr_gate_kernel<<<1, 32, 0, stream>>>(*g);
  return (int)cudaGetLastError();
}

// Launch the round kernel with `ctas` persistent CTAs on `stream`. `round` is a host pointer to an HrRound whose
// [item_begin, item_end) range selects the work (the whole list in normal operation; one stage at a time when several
// ranks are emulated on one GPU, so that no launch waits for a later one).
HM_API int hm_br_round(const void* round, int ctas, cudaStream_t stream) {
  const HrRound* g = (const HrRound*)round;
  const int items = g->item_end - g->item_begin;
  if (items <= 0 && !g->final_stage) return 0;   // a final stage without items still closes the round (one CTA)
  if (ctas > items) ctas = items;
  if (ctas < 1) ctas = 1;
  hr_round_kernel<<<ctas, HR_THREADS, 0, stream>>>(*g);
  return (int)cudaGetLastError();
}
