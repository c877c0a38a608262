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
//   round kernel         : a persistent grid (two 512-thread CTAs per SM). Work items are runs of consecutive chunks
//                          of one part (by default the whole part), listed send, reduce, apply and dealt round-robin:
//                          a CTA finishes its send items before it may wait for a groupmate, so a wait for a
//                          remote flag never delays work that another GPU needs from this one.
//     send   (part of a groupmate)         : every chunk of 8192 values is read ONCE into registers; statistics,
//                          quantisation, per-bin sums and the record header are computed by the same CTA; the CTA
//                          that completes a part publishes its flag together with this GPU's weight (64-bit store,
//                          release.sys).
//     reduce (own part)                    : one lane per sender waits (bounded) for that sender's flag; the CTA then
//                          pulls each sender's chunk record over NVLink once, one chunk ahead of its use (keeping a
//                          local copy), accumulates in registers, applies the average to its own values, and for
//                          every sender encodes  avg - decode(copy)  in place: no separate statistics / encode /
//                          publish passes. Uncompressed parts are read straight from the senders' vectors and
//                          publish the average itself.
//     apply  (part of a groupmate)         : waits (bounded) for the owner's flag, x += alpha * decode(delta), the
//                          records again requested one chunk ahead.
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
  const float* code;           // block-wise code [256], midpoints between consecutive entries [256], search table [16384 B]
  unsigned int done_slot;
  int uses_blockwise;          // some part uses the block-wise codec: CTAs load the search table
  unsigned long long* trace;   // optional [gridDim.x][12] globaltimer stamps per CTA (see hr_round_kernel); null = off
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

// Flag stores that follow an explicit system-scope fence of the same thread (fence + strong write = release pattern)
__device__ __forceinline__ void hr_st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void hr_st_relaxed_sys_u32(unsigned int* p, unsigned int v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct HrShared {
  double redd[2][2][HR_THREADS / 32];   // two alternating scratch copies for block-wide sums (one barrier per reduction)
  float redf[2][2][HR_THREADS / 32];    //   and maxima
  float cb[2][256];                     // codebook of the record being decoded (two alternating copies)
  float table[256];                     // quantile borders for bucketize
  // Per warp-pair bin sums and counts (a skewed distribution would otherwise serialise the whole CTA on a handful of
  // addresses), zero between uses. Sums are integers: fixed-point offsets from a reference value of the bin, because
  // shared memory adds integers natively, whereas a float add there is a compare-and-swap loop. The two outermost
  // bins (open-ended, rarely hit) keep float sums.
  int hfix[HR_THREADS / 64][256];
  int hcnt[HR_THREADS / 64][256];
  float hedge[HR_THREADS / 64][2];
  float smp[HR_SAMPLE];
  float code[256];                      // block-wise code and the midpoints between its entries: loaded once per CTA
  float mid[256];
  unsigned char lut[1 << 14];           // where the search for a value's code starts (see hr_code_index)
  float w[HR_MAX_PEERS];
  int inc[HR_MAX_PEERS];
  int par[HR_MAX_PEERS];
  int order[HR_MAX_PEERS];              // included senders in this reducer's rotation order
  int n_inc;
  int bcast;
};

// Per-thread bookkeeping with the same value in every thread of the CTA: which scratch copy comes next.
struct HrThread {
  int red = 0, cb = 0;
  unsigned long long* stamps = nullptr;   // this CTA's row of the optional trace (thread 0 writes)
};

// element index inside the chunk handled by (row r, thread, k)
__device__ __forceinline__ int hr_elem(int r) { return (r * HR_THREADS + (int)threadIdx.x) * 4; }

// Block-wide sums of two doubles (or maxima of two floats); every thread gets the results. One barrier: consecutive
// reductions alternate between two scratch copies, and a thread can only get to the reduction after next once all
// threads have passed the barrier of the next one, i.e. have finished reading this one's copy.
__device__ __forceinline__ void hr_block_sum2(double& a, double& b, HrShared& sh, HrThread& th) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
  double(*buf)[HR_THREADS / 32] = sh.redd[th.red++ & 1];
  if (lane == 0) {
    buf[0][warp] = a;
    buf[1][warp] = b;
  }
  __syncthreads();
  a = lane < HR_THREADS / 32 ? buf[0][lane] : 0.0;
  b = lane < HR_THREADS / 32 ? buf[1][lane] : 0.0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
}
__device__ __forceinline__ void hr_block_max2(float& a, float& b, HrShared& sh, HrThread& th) {   // of absolute values
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  a = hm_warp_max(a);
  b = hm_warp_max(b);
  float(*buf)[HR_THREADS / 32] = sh.redf[th.red++ & 1];
  if (lane == 0) {
    buf[0][warp] = a;
    buf[1][warp] = b;
  }
  __syncthreads();
  a = hm_warp_max(lane < HR_THREADS / 32 ? buf[0][lane] : 0.f);
  b = hm_warp_max(lane < HR_THREADS / 32 ? buf[1][lane] : 0.f);
}

// Index of the block-wise code entry nearest to x in [-1, 1] = number of midpoints below x. The top 14 bits of the
// value's order-preserving key (float bits with the sign handled) pick a starting count from a table; at most a
// few midpoints lie inside one such slice of the number line, and they are stepped over one by one.
__device__ __forceinline__ int hr_code_index(const HrShared& sh, float x) {
  unsigned int u = __float_as_uint(x);
  u ^= (u >> 31) ? 0xffffffffu : 0x80000000u;
  int b = sh.lut[u >> 18];
  while (b < 255 && sh.mid[b] < x) ++b;
  return b;
}

// Quantise with the bin index `bin(x)`, note every value in its bin, then (after a barrier) write the bins' means as
// the record's codebook and leave the histogram zeroed for its next user. A value enters its bin's sum as the integer
// (x - ref(bin)) * to_fixed, where the caller guarantees |.| <= 2^17 for the inner bins (8192 of them cannot overflow);
// the outermost bins add x itself to a float.
template <typename BinFn, typename RefFn>
__device__ __forceinline__ void hr_quantise_with_bin_means(const float (&v)[HR_ROWS][4], int n, unsigned char* rec,
                                                           unsigned char* payload, HrShared& sh, float to_fixed,
                                                           BinFn bin, RefFn ref) {
  const int hw = threadIdx.x >> 6;
#pragma unroll
  for (int r = 0; r < HR_ROWS; ++r) {
    const int i = hr_elem(r);
    uint32_t packed = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float x = v[r][k];
      const int b = bin(x);
      packed |= (uint32_t)b << (8 * k);
      if (i + k < n) {
        atomicAdd(&sh.hcnt[hw][b], 1);
        if (b == 0 || b == 255) atomicAdd(&sh.hedge[hw][b & 1], x);
        else atomicAdd(&sh.hfix[hw][b], __float2int_rn((x - ref(b)) * to_fixed));
      }
    }
    *reinterpret_cast<uint32_t*>(payload + i) = packed;
  }
  __syncthreads();
  if (threadIdx.x < 256) {
    const int b = threadIdx.x;
    long long fixed = 0;
    int count = 0;
    float edge = 0.f;
#pragma unroll
    for (int w = 0; w < HR_THREADS / 64; ++w) {
      fixed += sh.hfix[w][b];
      count += sh.hcnt[w][b];
      sh.hfix[w][b] = 0;
      sh.hcnt[w][b] = 0;
      if (b == 0 || b == 255) {
        edge += sh.hedge[w][b & 1];
        sh.hedge[w][b & 1] = 0.f;
      }
    }
    const float members = (float)(count > 0 ? count : 1);
    float mean;
    if (b == 0 || b == 255) mean = edge / members;
    else mean = count > 0 ? ref(b) + (to_fixed > 0.f ? (float)fixed / (to_fixed * members) : 0.f) : 0.f;
    reinterpret_cast<float*>(rec)[b] = mean;
  }
}

// Encode the chunk held in registers (v[r][k] = element hr_elem(r) + k, elements >= n are zero) into `rec`
// (header + payload). Every thread of the CTA calls this. Elements >= n still get payload bytes (of value zero or
// whatever zero maps to); they are never decoded. The bin histogram in shared memory is zero on entry and on return;
// a caller may start the next encode (or hr_open) without a barrier in between.
__device__ void hr_encode_chunk(const float (&v)[HR_ROWS][4], int n, int codec, unsigned char* rec, HrShared& sh, HrThread& th) {
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
    // sum and sum of squares in double precision (padding elements are zero): one reduction, no cancellation to
    // speak of even when the mean dwarfs the spread
    double s1 = 0.0, s2 = 0.0;
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r)
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const double x = (double)v[r][k];
        s1 += x;
        s2 = fma(x, x, s2);
      }
    hr_block_sum2(s1, s2, sh, th);
    const double mean_d = s1 / (double)n;
    const double m2 = fmax(s2 - s1 * mean_d, 0.0);   // centred sum of squares
    const float mean = (float)mean_d;
    if (codec == HB_MEANSTD16) {
      const float sd = fmaxf((float)sqrt(m2 / (double)n), 1.1920929e-07f);
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
    const float scale = 6.f * (float)sqrt(m2 / fmax((double)n - 1.0, 1.0)) / 256.f;
    const float inv = (scale > 0.f && isfinite(scale)) ? 1.f / scale : 1.f;
    // inner levels hold values within half a level of their centre: offsets of at most 2^15 units of scale / 2^16
    hr_quantise_with_bin_means(
        v, n, rec, payload, sh, 65536.f * inv,
        [&](float x) {
          const int b = __float2int_rn((x - mean) * inv) + 128;
          return b < 0 ? 0 : (b > 255 ? 255 : b);
        },
        [&](int b) { return fmaf((float)(b - 128), scale > 0.f && isfinite(scale) ? scale : 1.f, mean); });
    return;
  }
  if (codec == HB_QUANTILE8) {
    // borders from a regular sample of at most 2048 values (every value when the chunk has no more than that)
    int stride = 1;
    while (stride * HR_SAMPLE < n) stride <<= 1;
    const int S = (n + stride - 1) / stride;
    for (int i = S + threadIdx.x; i < HR_SAMPLE; i += HR_THREADS) sh.smp[i] = INFINITY;
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (i + k < n && ((i + k) & (stride - 1)) == 0) sh.smp[(i + k) / stride] = v[r][k];
    }
    __syncthreads();
    for (int size = 2; size <= HR_SAMPLE; size <<= 1) {   // bitonic sort
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
    // inner bin b holds values in (table[b - 1], table[b]]: offsets from the lower border, in units of the whole
    // range of borders / 2^17
    const float range = sh.table[254] - sh.table[0];
    const float to_fixed = (range > 0.f && isfinite(range)) ? 131072.f / range : 0.f;
    hr_quantise_with_bin_means(
        v, n, rec, payload, sh, to_fixed, [&](float x) { return hb_bucketize(sh.table, x); },
        [&](int b) { return sh.table[b - 1]; });
    return;
  }
  // HB_BLOCKWISE8: rows [b * RPB, (b + 1) * RPB) of every thread belong to block b (4096 elements)
  {
    constexpr int RPB = HR_ROWS / HR_BLOCKS;
    static_assert(HR_BLOCKS == 2, "two block maxima travel in one reduction");
    float m[HR_BLOCKS];
#pragma unroll
    for (int b = 0; b < HR_BLOCKS; ++b) {
      m[b] = 0.f;
#pragma unroll
      for (int rr = 0; rr < RPB; ++rr)
#pragma unroll
        for (int k = 0; k < 4; ++k) m[b] = fmaxf(m[b], fabsf(v[RPB * b + rr][k]));
    }
    hr_block_max2(m[0], m[1], sh, th);
    if (threadIdx.x < HR_BLOCKS) reinterpret_cast<float*>(rec)[threadIdx.x] = m[threadIdx.x];
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
      const float inv = 1.f / fmaxf(m[r / RPB], 1.17549435e-38f);
      uint32_t packed = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) packed |= (uint32_t)hr_code_index(sh, v[r][k] * inv) << (8 * k);
      *reinterpret_cast<uint32_t*>(payload + i) = packed;
    }
  }
}

// What a thread holds of a chunk that it has requested ahead of time: its rows of the payload (or of the fp32 vector
// for uncompressed parts) and its share of the header. Remote reads are issued one chunk before they are used, so
// that NVLink latency is spent while the CTA works on the previous chunk.
struct HrAhead {
  uint32_t w[HR_ROWS * 4];   // uncompressed: HR_ROWS float4; 16-bit codecs: HR_ROWS uint2; 8-bit codecs: HR_ROWS words
  float4 hdr;                // 16-byte headers whole (every thread); 1 KB codebooks: entry threadIdx.x in hdr.x
};

__device__ __forceinline__ void hr_fetch(int codec, const unsigned char* src, int n, HrAhead& a) {
  if (codec == HB_NONE) {
    const float* x = reinterpret_cast<const float*>(src);
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
      float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i + 4 <= n) {
        t = *reinterpret_cast<const float4*>(x + i);
      } else {
        if (i < n) t.x = x[i];
        if (i + 1 < n) t.y = x[i + 1];
        if (i + 2 < n) t.z = x[i + 2];
      }
      a.w[4 * r] = __float_as_uint(t.x); a.w[4 * r + 1] = __float_as_uint(t.y);
      a.w[4 * r + 2] = __float_as_uint(t.z); a.w[4 * r + 3] = __float_as_uint(t.w);
    }
    return;
  }
  const int hdr = hr_header_bytes(codec);
  if (hdr == 1024) {
    if (threadIdx.x < 256) a.hdr.x = reinterpret_cast<const float*>(src)[threadIdx.x];
  } else if (hdr == 16) {
    a.hdr = *reinterpret_cast<const float4*>(src);
  }
  if (hb_elem_bytes(codec) == 2) {
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const uint2 t = *reinterpret_cast<const uint2*>(src + hdr + (size_t)hr_elem(r) * 2);
      a.w[2 * r] = t.x; a.w[2 * r + 1] = t.y;
    }
  } else {
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) a.w[r] = *reinterpret_cast<const uint32_t*>(src + hdr + hr_elem(r));
  }
}

// Make a fetched record decodable: the codebook of an 8-bit record goes to shared memory (one barrier; consecutive
// records alternate between two copies), the scalars of the other headers are handed back in registers. `copy`
// (optional) receives the header as well. Returns the codebook to decode with.
__device__ __forceinline__ const float* hr_open(int codec, const HrAhead& a, HrShared& sh, HrThread& th, unsigned char* copy,
                                                float& mean, float& sd, float absmax[HR_BLOCKS]) {
  mean = 0.f;
  sd = 1.f;
  if (codec == HB_UNIFORM8 || codec == HB_QUANTILE8) {
    float* cb = sh.cb[th.cb++ & 1];
    if (threadIdx.x < 256) {
      cb[threadIdx.x] = a.hdr.x;
      if (copy) reinterpret_cast<float*>(copy)[threadIdx.x] = a.hdr.x;
    }
    __syncthreads();
    return cb;
  }
  if (codec == HB_MEANSTD16) {
    mean = a.hdr.x;
    sd = a.hdr.y;
  } else if (codec == HB_BLOCKWISE8) {
    absmax[0] = a.hdr.x;
    if (HR_BLOCKS > 1) absmax[HR_BLOCKS - 1] = a.hdr.y;
  }
  if (copy && threadIdx.x == 0 && hr_header_bytes(codec) == 16) *reinterpret_cast<float4*>(copy) = a.hdr;
  return sh.code;
}

// Decode row r of a fetched record.
__device__ __forceinline__ void hr_decode_ahead(int codec, const HrAhead& a, int r, float mean, float sd, const float* cb,
                                                const float* absmax, float out[4]) {
  if (codec == HB_NONE) {
    out[0] = __uint_as_float(a.w[4 * r]); out[1] = __uint_as_float(a.w[4 * r + 1]);
    out[2] = __uint_as_float(a.w[4 * r + 2]); out[3] = __uint_as_float(a.w[4 * r + 3]);
  } else if (hb_elem_bytes(codec) == 2) {
    const __half2 lo = *reinterpret_cast<const __half2*>(&a.w[2 * r]), hi = *reinterpret_cast<const __half2*>(&a.w[2 * r + 1]);
    out[0] = __low2float(lo); out[1] = __high2float(lo); out[2] = __low2float(hi); out[3] = __high2float(hi);
    if (codec == HB_MEANSTD16) {
#pragma unroll
      for (int k = 0; k < 4; ++k) out[k] = fmaf(out[k], sd, mean);
    }
  } else {
    const uint32_t q = a.w[r];
    const float m = codec == HB_BLOCKWISE8 ? absmax[r / (HR_ROWS / HR_BLOCKS)] : 1.f;
    out[0] = cb[q & 255u] * m; out[1] = cb[(q >> 8) & 255u] * m;
    out[2] = cb[(q >> 16) & 255u] * m; out[3] = cb[q >> 24] * m;
  }
}

__device__ __forceinline__ unsigned long long hr_ld_acquire_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long hr_cas_relaxed_gpu_u64(unsigned long long* p, unsigned long long expected,
                                                                    unsigned long long desired) {
  unsigned long long old;
  asm volatile("atom.relaxed.gpu.global.cas.b64 %0, [%1], %2, %3;" : "=l"(old) : "l"(p), "l"(expected), "l"(desired) : "memory");
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
// first CTA to get here talks to the groupmate: it polls the flag, fences and publishes the decision; every later
// CTA finds the decision with ONE acquire.gpu load, which orders its reads of the
// groupmate's data after the groupmate's writes just the same (release / acquire chains are cumulative). The clock
// is only looked at while the flag is missing: the time limit runs from the moment this GPU first had to wait in
// the phase (`t_start`).
__device__ unsigned long long hr_decide(const unsigned long long* flag0, const unsigned long long* flag1, bool wide,
                                        unsigned int want, unsigned long long* decision, const int* ban_flag,
                                        unsigned long long* t_start, unsigned long long timeout_ns) {
  // both flag sets are polled with relaxed loads (independent of each other: one round trip instead of two); the
  // fence behind a hit turns the load that saw the flag into an acquire
  auto load = [&](const unsigned long long* f) -> unsigned long long {
    unsigned long long v;
    if (wide) {
      asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(f) : "memory");
    } else {
      unsigned int w;
      asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(w) : "l"(f) : "memory");
      v = w;
    }
    return v;
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
    if (verdict == 0) {
      __nanosleep(200);
    } else {
      // the fence makes the poll that saw the flag an acquire, and is the release half for the CTAs that will read
      // the decision (fence + strong write); a give-up verdict has no data behind it
      if (verdict != 2ull) __threadfence_system();
      hr_cas_relaxed_gpu_u64(decision, 0ull, verdict);
    }
    d = hr_ld_acquire_gpu_u64(decision);
  }
  return d;
}

// Chunks [.., .. + add) of a part are complete; true for the thread whose increment completes the part. The caller
// has passed a CTA barrier after the chunks' writes. The count lives on this GPU, so the fence in front of it only
// has to order the CTA's writes for this GPU's other CTAs (gpu scope); the thread that completes the part then
// fences at system scope before it publishes the part's flag, and that release carries everything that
// happened before it, the other CTAs' chunks included, to the groupmate that acquires the flag.
__device__ __forceinline__ bool hr_chunks_done(int* counter, int add, int n_chunks) {
  __threadfence();
  const bool last = atomicAdd(counter, add) == n_chunks - add;
  if (last) __threadfence_system();
  return last;
}

// ---------------------------------------------------------------------------------------------------------------
__device__ void hr_send_item(const HrRound& g, int p, int c0, int z, HrShared& sh, HrThread& th) {
  unsigned char* my = g.base[g.me];
  unsigned long long* ready = reinterpret_cast<unsigned long long*>(my + g.lay.ready[g.parity]);
  const unsigned long long flag = (unsigned long long)g.epoch | ((unsigned long long)__float_as_uint(g.my_weight) << 32);
  if (p < 0) {
    // uncompressed parts: readers take the values from the vector itself (written before this kernel began), only
    // the flags are published: one fence per thread, then plain flag stores
    if ((int)threadIdx.x < z) __threadfence_system();
    for (int i = threadIdx.x; i < z; i += HR_THREADS) hr_st_relaxed_sys_u64(ready + g.pub_list[c0 + i], flag);
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
    hr_encode_chunk(v, n, part.codec, my + g.lay.outbox[g.parity] + part.enc_off + (long long)c * stride, sh, th);
  }
  const int n_chunks = (part.len + HR_CHUNK - 1) / HR_CHUNK;
  __syncthreads();
  if (threadIdx.x == 0 && hr_chunks_done(g.part_done + p, z, n_chunks)) hr_st_relaxed_sys_u64(ready + p, flag);
}

__device__ void hr_reduce_item(const HrRound& g, int p, int c0, int z, HrShared& sh, HrThread& th) {
  const HrPart part = g.parts[p];
  const int codec = part.codec, j = part.local_idx, me = g.me;
  const int n_chunks = (part.len + HR_CHUNK - 1) / HR_CHUNK;
  unsigned char* my = g.base[me];
  // every reducer walks the senders in its own rotation, so that at any moment the reducers of a group read from
  // different GPUs instead of all draining the same sender's links
  const int rot = (me + 1) % g.n_peers;

  // one lane per sender waits for (or looks up the decision about) that sender's flag
  if (threadIdx.x < 32) {
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
    if (s < HR_MAX_PEERS) {
      sh.inc[s] = inc;
      sh.par[s] = par;
      sh.w[s] = w;
    }
    const unsigned int mask = __ballot_sync(0xffffffffu, inc != 0);
    if (s == 0) {
      int k = 0;
      for (int t = 0; t < g.n_peers; ++t) {
        const int q = rot + t < g.n_peers ? rot + t : rot + t - g.n_peers;
        if (mask >> q & 1u) sh.order[k++] = q;
      }
      sh.n_inc = k;
    }
  }
  __syncthreads();
  if (th.stamps != nullptr && threadIdx.x == 0 && th.stamps[8] == 0) th.stamps[8] = hm_globaltimer_ns();

  const bool i_send = g.sends[me] != 0;
  const int n_inc = sh.n_inc;
  float den = i_send ? g.my_weight : 0.f;
  for (int k = 0; k < n_inc; ++k) den += sh.w[sh.order[k]];
  // a total weight of zero (every member tagging along) averages nothing: values stay, deltas are reported as failed
  const bool dead = !(den > 0.f);
  const float inv_den = dead ? 0.f : 1.f / den;
  const float alpha_own = dead ? 0.f : g.alpha;
  const long long stride = hr_chunk_stride(codec);
  const int hdr = hr_header_bytes(codec);

  // where sender s keeps chunk c of this part
  auto source = [&](int s, int c) -> const unsigned char* {
    if (codec == HB_NONE) return g.base[s] + g.lay.data + (size_t)(part.start + (long long)c * HR_CHUNK) * 4;
    return g.base[s] + g.lay.outbox[sh.par[s]] + part.enc_off + (long long)c * stride;
  };
  auto chunk_len = [&](int c) { return min(HR_CHUNK, part.len - c * HR_CHUNK); };
  const int total = z * n_inc;
  // One remote sender (a group of two, or everybody else left out): its record stays in registers until the delta
  // has been encoded, so no copy is written and read back
  const bool single = n_inc == 1 && codec != HB_NONE && !dead;
  HrAhead ahead;
  if (total > 0) hr_fetch(codec, source(sh.order[0], c0), chunk_len(c0), ahead);

  for (int c = c0; c < c0 + z; ++c) {
    const int lo = c * HR_CHUNK, n = chunk_len(c);
    float* x_local = reinterpret_cast<float*>(my + g.lay.data) + part.start + lo;
    if (single) {
      // row by row: average, own values updated, delta taken, while the record is in registers
      const int s = sh.order[0];
      const float w = sh.w[s];
      const HrAhead cur = ahead;
      if (c + 1 < c0 + z) hr_fetch(codec, source(s, c + 1), chunk_len(c + 1), ahead);
      float mean, sd, absmax[HR_BLOCKS] = {};
      const float* cb = hr_open(codec, cur, sh, th, nullptr, mean, sd, absmax);
      float d1[HR_ROWS][4];
#pragma unroll
      for (int r = 0; r < HR_ROWS; ++r) {
        const int i = hr_elem(r);
        const bool inside = i + 4 <= n;   // parts are whole multiples of four elements
        float4 own = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i_send && inside) own = *reinterpret_cast<const float4*>(x_local + i);
        float o[4];
        hr_decode_ahead(codec, cur, r, mean, sd, cb, absmax, o);
        const float mine4[4] = {own.x, own.y, own.z, own.w};
        float a[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          a[q] = fmaf(w, o[q], g.my_weight * mine4[q]) * inv_den;
          d1[r][q] = inside ? a[q] - o[q] : 0.f;
        }
        if (i_send && inside)
          *reinterpret_cast<float4*>(x_local + i) =
              make_float4(fmaf(alpha_own, a[0] - own.x, own.x), fmaf(alpha_own, a[1] - own.y, own.y),
                          fmaf(alpha_own, a[2] - own.z, own.z), fmaf(alpha_own, a[3] - own.w, own.w));
      }
      hr_encode_chunk(d1, n, codec,
                      my + g.lay.deltabox[g.parity] + (size_t)s * g.delta_stride + part.span_off + (long long)c * stride, sh, th);
      continue;
    }
    float acc[HR_ROWS][4];
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
      float4 own = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i_send && i + 4 <= n) own = *reinterpret_cast<const float4*>(x_local + i);
      acc[r][0] = g.my_weight * own.x; acc[r][1] = g.my_weight * own.y;
      acc[r][2] = g.my_weight * own.z; acc[r][3] = g.my_weight * own.w;
    }
    for (int k = 0; k < n_inc; ++k) {
      const int s = sh.order[k];
      const float w = sh.w[s];
      const HrAhead cur = ahead;
      {   // request the next (chunk, sender) before working on this one
        const int k2 = k + 1 < n_inc ? k + 1 : 0, c2 = k + 1 < n_inc ? c : c + 1;
        if (c2 < c0 + z) hr_fetch(codec, source(sh.order[k2], c2), chunk_len(c2), ahead);
      }
      unsigned char* local = my + g.lay.deltabox[g.parity] + (size_t)s * g.delta_stride + part.span_off + (long long)c * stride;
      const bool keep_copy = codec != HB_NONE;
      float mean, sd, absmax[HR_BLOCKS] = {};
      const float* cb = hr_open(codec, cur, sh, th, keep_copy ? local : nullptr, mean, sd, absmax);
#pragma unroll
      for (int r = 0; r < HR_ROWS; ++r) {
        // several senders: keep a copy of each record where that sender's delta will be written
        if (keep_copy && hb_elem_bytes(codec) == 2)
          *reinterpret_cast<uint2*>(local + hdr + (size_t)hr_elem(r) * 2) = make_uint2(cur.w[2 * r], cur.w[2 * r + 1]);
        else if (keep_copy && hb_elem_bytes(codec) == 1)
          *reinterpret_cast<uint32_t*>(local + hdr + hr_elem(r)) = cur.w[r];
        float o[4];
        hr_decode_ahead(codec, cur, r, mean, sd, cb, absmax, o);
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[r][q] = fmaf(w, o[q], acc[r][q]);
      }
    }
    // the average; applied to this reducer's own values right here
    float* avg_out = reinterpret_cast<float*>(my + g.lay.avg[g.parity]) + part.avg_off + lo;
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[r][q] = (i + q < n) ? acc[r][q] * inv_den : 0.f;
      if (i + 4 <= n) {   // parts are whole multiples of four elements
        if (codec == HB_NONE) *reinterpret_cast<float4*>(avg_out + i) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
        if (i_send && alpha_own == 1.f) {   // the usual case: the average replaces the values, no second read
          *reinterpret_cast<float4*>(x_local + i) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
        } else if (i_send && alpha_own != 0.f) {
          float4 own = *reinterpret_cast<const float4*>(x_local + i);
          own.x = fmaf(alpha_own, acc[r][0] - own.x, own.x); own.y = fmaf(alpha_own, acc[r][1] - own.y, own.y);
          own.z = fmaf(alpha_own, acc[r][2] - own.z, own.z); own.w = fmaf(alpha_own, acc[r][3] - own.w, own.w);
          *reinterpret_cast<float4*>(x_local + i) = own;
        }
      }
    }
    // deltas: avg - decode(copy of the sender's record), encoded over the copy, one sender after the other
    if (codec != HB_NONE && !dead) {
      if (hdr == 16) __syncthreads();   // the copies' 16-byte headers were written by thread 0
      for (int k = 0; k < n_inc; ++k) {
        const int s = sh.order[k];
        unsigned char* local = my + g.lay.deltabox[g.parity] + (size_t)s * g.delta_stride + part.span_off + (long long)c * stride;
        HrAhead mine;
        hr_fetch(codec, local, n, mine);
        float mean, sd, absmax[HR_BLOCKS] = {};
        const float* cb = hr_open(codec, mine, sh, th, nullptr, mean, sd, absmax);
        float d[HR_ROWS][4];
#pragma unroll
        for (int r = 0; r < HR_ROWS; ++r) {
          const int i = hr_elem(r);
          float o[4];
          hr_decode_ahead(codec, mine, r, mean, sd, cb, absmax, o);
#pragma unroll
          for (int q = 0; q < 4; ++q) d[r][q] = (i + q < n) ? acc[r][q] - o[q] : 0.f;
        }
        hr_encode_chunk(d, n, codec, local, sh, th);
      }
    }
  }
  // one lane per sender counts the chunks of its delta; the lane that completes a part publishes its flag
  __syncthreads();
  if (threadIdx.x < g.n_peers) {
    const int s = threadIdx.x;
    if (s != me && g.sends[s] && hr_chunks_done(g.dpart_done + (size_t)s * g.max_local_parts + j, z, n_chunks)) {
      unsigned int* flag = reinterpret_cast<unsigned int*>(my + g.lay.dready[g.parity]) + (size_t)s * g.max_local_parts + j;
      hr_st_relaxed_sys_u32(flag, (sh.inc[s] && !dead) ? g.epoch : (g.epoch | HB_FAIL_BIT));
    }
  }
}

__device__ void hr_apply_item(const HrRound& g, int p, int c0, int z, HrShared& sh, HrThread& th) {
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
  if (th.stamps != nullptr && threadIdx.x == 0 && th.stamps[9] == 0) th.stamps[9] = hm_globaltimer_ns();
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
  auto source = [&](int c) -> const unsigned char* {
    if (codec == HB_NONE) return g.base[owner] + g.lay.avg[opar] + (size_t)(part.avg_off + (long long)c * HR_CHUNK) * 4;
    return g.base[owner] + g.lay.deltabox[opar] + (size_t)me * g.delta_stride + part.span_off + (long long)c * stride;
  };
  auto chunk_len = [&](int c) { return min(HR_CHUNK, part.len - c * HR_CHUNK); };
  HrAhead ahead;
  hr_fetch(codec, source(c0), chunk_len(c0), ahead);
  for (int c = c0; c < c0 + z; ++c) {
    const int lo = c * HR_CHUNK, n = chunk_len(c);
    float* x = reinterpret_cast<float*>(g.base[me] + g.lay.data) + part.start + lo;
    const HrAhead cur = ahead;
    if (c + 1 < c0 + z) hr_fetch(codec, source(c + 1), chunk_len(c + 1), ahead);
    float mean, sd, absmax[HR_BLOCKS] = {};
    const float* cb = hr_open(codec, cur, sh, th, nullptr, mean, sd, absmax);
#pragma unroll
    for (int r = 0; r < HR_ROWS; ++r) {
      const int i = hr_elem(r);
      if (i + 4 > n) continue;   // parts are whole multiples of four elements
      float dv[4];
      hr_decode_ahead(codec, cur, r, mean, sd, cb, absmax, dv);
      if (codec == HB_NONE && alpha == 1.f) {   // the average replaces the values: nothing to read
        *reinterpret_cast<float4*>(x + i) = make_float4(dv[0], dv[1], dv[2], dv[3]);
        continue;
      }
      float4 xv = *reinterpret_cast<const float4*>(x + i);
      if (codec == HB_NONE) {   // the record is the average itself
        xv.x = fmaf(alpha, dv[0] - xv.x, xv.x); xv.y = fmaf(alpha, dv[1] - xv.y, xv.y);
        xv.z = fmaf(alpha, dv[2] - xv.z, xv.z); xv.w = fmaf(alpha, dv[3] - xv.w, xv.w);
      } else {
        xv.x = fmaf(alpha, dv[0], xv.x); xv.y = fmaf(alpha, dv[1], xv.y);
        xv.z = fmaf(alpha, dv[2], xv.z); xv.w = fmaf(alpha, dv[3], xv.w);
      }
      *reinterpret_cast<float4*>(x + i) = xv;
    }
  }
}

__global__ void __launch_bounds__(HR_THREADS, 2) hr_round_kernel(const __grid_constant__ HrRound g) {
  __shared__ HrShared sh;
  HrThread th;
  if (threadIdx.x < 256) {
    sh.code[threadIdx.x] = g.code[threadIdx.x];
    sh.mid[threadIdx.x] = g.code[256 + threadIdx.x];
  }
  for (int i = threadIdx.x; i < (HR_THREADS / 64) * 256; i += HR_THREADS) { (&sh.hfix[0][0])[i] = 0; (&sh.hcnt[0][0])[i] = 0; }
  if (threadIdx.x < (HR_THREADS / 64) * 2) (&sh.hedge[0][0])[threadIdx.x] = 0.f;
  if (g.uses_blockwise) {
    const uint4* src = reinterpret_cast<const uint4*>(g.code + 512);
    for (int i = threadIdx.x; i < (1 << 14) / 16; i += HR_THREADS) reinterpret_cast<uint4*>(sh.lut)[i] = src[i];
  }
  // Items are dealt round-robin. The list is ordered send, reduce, apply, so every CTA finishes its send items
  // before it may wait for a groupmate, and nothing that a groupmate needs from this GPU queues up behind a wait.
  // With g.trace set, thread 0 stamps: [0] start, [1] / [2] first reduce item entered / left, [3] last reduce item
  // left, [4] / [5] first apply item entered / left, [6] last item left, [7] items done by this CTA, [8] / [9] the
  // moment the first reduce / apply item knew about its flags (the waits end there).
  unsigned long long* stamps = g.trace != nullptr ? g.trace + 12 * (size_t)blockIdx.x : nullptr;
  th.stamps = stamps;
  if (stamps != nullptr && threadIdx.x == 0) stamps[0] = hm_globaltimer_ns();
  int seen_reduce = 0, seen_apply = 0, n_items = 0;
  for (int idx = g.item_begin + (int)blockIdx.x; idx < g.item_end; idx += (int)gridDim.x) {
    __syncthreads();
    const int4 it = g.items[idx];
    const int kind = idx < g.n_send ? 0 : (idx < g.n_send + g.n_reduce ? 1 : 2);
    if (stamps != nullptr && threadIdx.x == 0) {
      if (kind == 1 && !seen_reduce) stamps[1] = hm_globaltimer_ns();
      if (kind == 2 && !seen_apply) stamps[4] = hm_globaltimer_ns();
    }
    if (kind == 0) hr_send_item(g, it.x, it.y, it.z, sh, th);
    else if (kind == 1) hr_reduce_item(g, it.x, it.y, it.z, sh, th);
    else hr_apply_item(g, it.x, it.y, it.z, sh, th);
    if (stamps != nullptr && threadIdx.x == 0) {
      const unsigned long long now = hm_globaltimer_ns();
      if (kind == 1) { if (!seen_reduce) stamps[2] = now; stamps[3] = now; }
      if (kind == 2 && !seen_apply) stamps[5] = now;
      stamps[6] = now;
      stamps[7] = (unsigned long long)(++n_items);
    }
    seen_reduce |= kind == 1;
    seen_apply |= kind == 2;
  }
  // the last CTA to leave closes the round: acknowledges that this GPU has finished reading its groupmates'
  // arenas, hands the status words to the host and clears the scratch for the next round
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();   // gpu scope: the last CTA's system-scope release below carries it further
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
