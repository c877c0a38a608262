// Fused multi-head attention for sm_100a: forward and backward on tcgen05 tensor cores, head dimension 64.
//
// Serves the self-attention of the ALBERT-shaped and GPT-2-shaped models and of the `transformer` expert
// (hivemind/moe/server/layers/common.py:33-62 uses nn.MultiheadAttention for the same computation).
//
// Data layout. The kernels read q, k and v straight out of the packed projection output
//     qkv [B][S][3][H][64]   (bf16; what y = x W_qkv^T + b looks like without any transpose)
// and write the context as  out [B][S][H][64] = [B][S][hidden], the layout the output projection consumes.
// The backward pass reads d(out) in that layout and writes d(qkv) packed like qkv. All tiles move with unicast TMA
// through 3-D tensor maps (column, position, batch), so positions beyond S are zero-filled on load and clipped
// on store; nothing is transposed or copied outside these kernels.
//
// Forward (one CTA per (batch, head, 128 queries); two CTAs fit one SM and overlap each other):
//   warp 0     : TMA producer: Q once, then K_0 V_0 K_1 V_1 ... through a 3-deep ring of 16 KB tiles
//   warp 1     : one lane issues  S = Q K_j^T  (128x128x64, accumulator in TMEM)  and  O_j = P_j V_j  (128x64x128)
//   warps 2..5 : one thread per query row: tcgen05.ld of S, running maximum and sum (online softmax, base 2),
//                P_j written as bf16 into 128-byte-swizzled shared memory (operand A of the second product),
//                O accumulated in registers: O = (O + O_{j-1}) * 2^(m_{j-1} - m_j); final O / l by TMA store,
//                log-sum-exp (base 2, scale included) saved for the backward pass.
//   S_{j+1} is issued as soon as the softmax threads have read S_j, so the tensor pipe works on the next block's
//   scores (and on P_j V_j) while the exponentials of block j / j+1 are computed.
//
// Backward (one CTA per (batch, head, 128 keys), loops over the query tiles; 320 threads):
//   recomputes S = Q_i K_j^T and dP = dO_i V_j^T (TMEM), then per element P = 2^(S c - lse), dS = P (dP - D) scale,
//   with D = rowsum(dO * O) from a small pre-pass; P and dS go to swizzled shared memory as bf16 and feed
//       dV += P^T dO_i     dK += dS^T Q_i     (A operands read MN-major from the same bytes)
//       dQ_i = dS K_j      (fp32 tile added into a global accumulator by TMA reduce-add; double-buffered in TMEM)
//   dK and dV stay in TMEM across the query loop and are stored once. Two warpgroups share the element-wise work
//   (each takes 64 of the 128 key columns of every row).
//
// Every mbarrier wait is bounded (tc_ptx.cuh); when one runs out the CTA records an error word, skips its
// stores, lets copies in flight land, frees its tensor memory and returns.
#include <cstdio>
#include "tc_ptx.cuh"

namespace {

constexpr int HD = 64;                    // head dimension
constexpr int TILE = 128;                 // queries per tile, keys per block
constexpr int TILE_BYTES = TILE * 128;    // 128 rows x 64 bf16
constexpr int FWD_THREADS = 192;
constexpr int BWD_THREADS = 320;
constexpr int BWD_COMPUTE = 256;

struct AttnParams {
  int B, S, H;
  int causal;
  float scale;        // softmax scale (1/sqrt(64) unless overridden)
  float scale_log2;   // scale * log2(e)
  float* lse;         // [B][H][S], base-2 log-sum-exp of the scaled scores
  float* delta;       // [B][H][S], rowsum(dO * O) (backward only)
  int* err;
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map), "r"(src),
               "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map),
               "r"(src), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <int COUNT>
__device__ __forceinline__ void named_bar_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(COUNT) : "memory");
}
// A warp-uniform bounded wait: every lane polls; if any lane gave up, the CTA-wide abort flag is raised.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const bool ok = __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
  if (!ok) *abort_flag = 1;
  return ok;
}

// ---------------------------------------------------------------------------------------------
// forward
struct FwdSmem {
  static constexpr int Q_OFF = 0;
  static constexpr int RING_OFF = TILE_BYTES;
  static constexpr int RING = 3;
  static constexpr int P_OFF = RING_OFF + RING * TILE_BYTES;     // two 16 KB slabs (keys 0..63, 64..127)
  static constexpr int BAR_OFF = P_OFF + 2 * TILE_BYTES;
  static constexpr int NUM_BARS = 1 + 2 * RING + 5;
  static constexpr int TOTAL = BAR_OFF + NUM_BARS * 8 + 16;
};

__global__ void __launch_bounds__(FWD_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_out,
                const AttnParams p) {
  using L = FwdSmem;
  constexpr uint32_t TMEM_COLS = 256;
  constexpr uint32_t IDESC_QK = make_idesc(1, false, false, TILE, TILE);
  constexpr uint32_t IDESC_PV = make_idesc(1, false, true, TILE, HD);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::BAR_OFF;
  const uint32_t q_full = bar_base;
  auto kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (1 + L::RING + s); };
  const uint32_t s_full = bar_base + 8u * (1 + 2 * L::RING);
  const uint32_t s_empty = s_full + 8, p_full = s_full + 16, o_full = s_full + 24, o_empty = s_full + 32;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::BAR_OFF + L::NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::BAR_OFF + L::NUM_BARS * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_q_tiles = (p.S + TILE - 1) / TILE;
  const int q_tile = num_q_tiles - 1 - (int)blockIdx.x;   // longest (causal) tiles first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int q0 = q_tile * TILE;
  const int n_blocks = p.causal ? q_tile + 1 : num_q_tiles;
  const int hidden = p.H * HD;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < L::RING; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 128);
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
    mbar_init(o_empty, 128);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tc_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
    tc_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

  bool failed = false;
  int where = 0;   // source line of the wait in progress: reported if it runs out

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, TILE_BYTES);
      tma_load_3d(smem_base + L::Q_OFF, &map_qkv, q_full, head * HD, q0, batch);
      for (int t = 0; t < 2 * n_blocks; ++t) {
        const int stage = t % L::RING, use = t / L::RING;
        if (!(where = __LINE__, mbar_wait(kv_empty(stage), (use & 1) ^ 1, abort_flag))) { failed = true; break; }
        mbar_expect_tx(kv_full(stage), TILE_BYTES);
        const int col = ((t & 1) ? 2 * hidden : hidden) + head * HD;
        tma_load_3d(smem_base + L::RING_OFF + stage * TILE_BYTES, &map_qkv, kv_full(stage), col, (t >> 1) * TILE, batch);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      auto issue_pv = [&](int j) -> bool {
        const int t = 2 * j + 1, stage = t % L::RING, use = t / L::RING;
        if (!(where = __LINE__, mbar_wait(kv_full(stage), use & 1, abort_flag))) return false;
        if (!(where = __LINE__, mbar_wait(p_full, j & 1, abort_flag))) return false;
        if (j > 0 && !(where = __LINE__, mbar_wait(o_empty, (j - 1) & 1, abort_flag))) return false;
        tc_fence_after();
        const uint32_t v_addr = smem_base + L::RING_OFF + stage * TILE_BYTES;
        const uint32_t p_addr = smem_base + L::P_OFF;
#pragma unroll
        for (int kk = 0; kk < TILE / 16; ++kk) {
          const uint64_t a_desc = make_smem_desc(p_addr + (kk >> 2) * TILE_BYTES + (kk & 3) * 32, 16, 1024);
          const uint64_t b_desc = make_smem_desc(v_addr + kk * 16 * 128, TILE_BYTES, 1024, 2);
          tc_mma<false>(tmem_o, a_desc, b_desc, IDESC_PV, kk > 0 ? 1u : 0u);
        }
        tc_commit(kv_empty(stage));
        tc_commit(o_full);
        return true;
      };
      if (!(where = __LINE__, mbar_wait(q_full, 0, abort_flag))) failed = true;
      for (int j = 0; j < n_blocks && !failed; ++j) {
        const int t = 2 * j, stage = t % L::RING, use = t / L::RING;
        if (!(where = __LINE__, mbar_wait(kv_full(stage), use & 1, abort_flag))) { failed = true; break; }
        if (j > 0 && !(where = __LINE__, mbar_wait(s_empty, (j - 1) & 1, abort_flag))) { failed = true; break; }
        tc_fence_after();
        const uint32_t k_addr = smem_base + L::RING_OFF + stage * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t a_desc = make_smem_desc(smem_base + L::Q_OFF + k * 32, 16, 1024);
          const uint64_t b_desc = make_smem_desc(k_addr + k * 32, 16, 1024);
          tc_mma<false>(tmem_s, a_desc, b_desc, IDESC_QK, k > 0 ? 1u : 0u);
        }
        tc_commit(kv_empty(stage));
        tc_commit(s_full);
        if (j > 0 && !issue_pv(j - 1)) { failed = true; break; }
      }
      if (!failed && !issue_pv(n_blocks - 1)) failed = true;
    }
  } else {
    // ------------------------------------------------------------------ softmax + output (warps 2..5)
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int q_idx = q0 + row;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    uint8_t* p_smem = smem + L::P_OFF;
    float o_acc[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY;   // running maximum of the raw (unscaled) scores
    float l_run = 0.f;
    const float c = p.scale_log2;

    for (int j = 0; j < n_blocks; ++j) {
      if (!(where = __LINE__, warp_wait(s_full, j & 1, abort_flag))) { failed = true; break; }
      tc_fence_after();
      const int key0 = j * TILE;
      const bool need_mask = (key0 + TILE > p.S) || (p.causal && j == q_tile);
      const int key_limit = p.causal ? min(p.S, q_idx + 1) : p.S;   // keys below this index are visible
      // pass 1: row maximum
      float mx = m_run;
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t r[32];
        tc_ld32(tmem_s + lane_base + (uint32_t)(ch * 32), r);
        tc_wait_ld();
        // four independent chains; measured neutral against one chain of 32 (the pass waits on TMEM loads, not on these)
        float m4[4] = {mx, -INFINITY, -INFINITY, -INFINITY};
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (key0 + ch * 32 + i < key_limit) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(r[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              m4[q] = fmaxf(m4[q], fmaxf(__uint_as_float(r[i + 2 * q]), __uint_as_float(r[i + 2 * q + 1])));
          }
        }
        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      }
      const float m_use = (mx == -INFINITY) ? 0.f : mx;
      const float alpha = fast_exp2((m_run - m_use) * c);   // 0 on the first block
      m_run = mx;
      // fold in the previous block's P V (also tells us that the P buffer may be overwritten)
      if (j > 0) {
        if (!(where = __LINE__, warp_wait(o_full, (j - 1) & 1, abort_flag))) { failed = true; break; }
        tc_fence_after();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tc_ld32(tmem_o + lane_base + (uint32_t)(half * 32), r);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[half * 32 + i] = (o_acc[half * 32 + i] + __uint_as_float(r[i])) * alpha;
        }
        tc_fence_before();
        mbar_arrive(o_empty);
      }
      // pass 2: exponentials, row sum, P as bf16 into the swizzled operand buffer
      const float neg_mc = -m_use * c;
      float sum = 0.f;
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t r[32];
        tc_ld32(tmem_s + lane_base + (uint32_t)(ch * 32), r);
        tc_wait_ld();
        float e[32];
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            e[i] = (key0 + ch * 32 + i < key_limit) ? fast_exp2(fmaf(__uint_as_float(r[i]), c, neg_mc)) : 0.f;
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) e[i] = fast_exp2(fmaf(__uint_as_float(r[i]), c, neg_mc));
        }
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 32; ++i) s4[i & 3] += e[i];
        sum += (s4[0] + s4[1]) + (s4[2] + s4[3]);
        uint8_t* slab = p_smem + (ch >> 1) * TILE_BYTES + row * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 o;
          o.x = pack_bf16(e[8 * q], e[8 * q + 1]);
          o.y = pack_bf16(e[8 * q + 2], e[8 * q + 3]);
          o.z = pack_bf16(e[8 * q + 4], e[8 * q + 5]);
          o.w = pack_bf16(e[8 * q + 6], e[8 * q + 7]);
          const int chunk = (ch & 1) * 4 + q;
          *reinterpret_cast<uint4*>(slab + ((chunk ^ (row & 7)) << 4)) = o;
        }
      }
      l_run = l_run * alpha + sum;
      tc_fence_before();
      mbar_arrive(s_empty);        // this thread's reads of S_j are complete
      fence_proxy_async_smem();
      mbar_arrive(p_full);
    }
    if (!failed) {
      if (!(where = __LINE__, warp_wait(o_full, (n_blocks - 1) & 1, abort_flag))) failed = true;
    }
    if (!failed) {
      tc_fence_after();
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      uint8_t* stage_row = p_smem + row * 128;   // the last P V has completed: its operand buffer is free
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r[32];
        tc_ld32(tmem_o + lane_base + (uint32_t)(half * 32), r);
        tc_wait_ld();
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = (o_acc[half * 32 + i] + __uint_as_float(r[i])) * inv_l;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 o;
          o.x = pack_bf16(v[8 * q], v[8 * q + 1]);
          o.y = pack_bf16(v[8 * q + 2], v[8 * q + 3]);
          o.z = pack_bf16(v[8 * q + 4], v[8 * q + 5]);
          o.w = pack_bf16(v[8 * q + 6], v[8 * q + 7]);
          const int chunk = half * 4 + q;
          *reinterpret_cast<uint4*>(stage_row + ((chunk ^ (row & 7)) << 4)) = o;
        }
      }
      if (q_idx < p.S && p.lse != nullptr)
        p.lse[((long long)batch * p.H + head) * p.S + q_idx] = (l_run > 0.f) ? m_run * c + log2f(l_run) : -INFINITY;
      fence_proxy_async_smem();
    }
    // every softmax thread reaches this barrier, whether or not its waits succeeded
    named_bar_sync<128>();
    if (threadIdx.x == 64 && !*abort_flag) {
      tma_store_3d(&map_out, smem_base + L::P_OFF, head * HD, q0, batch);
      tma_commit();
      tma_wait_all<0>();
    }
  }

  if (failed) {
    *abort_flag = 1;
    if (p.err) atomicCAS(p.err, 0, 1000000 + warp * 10000 + where);   // the first failure is kept
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tc_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// backward pre-pass: delta[b][h][s] = sum_d dO * O, and the fp32 dQ accumulator is cleared
__global__ void attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ delta, float* __restrict__ dq_acc, int B, int S, int H) {
  // eight threads per (token, head): 8 elements each
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)B * S * H * 8;
  const bool active = gid < total;
  float acc = 0.f;
  if (active) {
    const uint4 a = *reinterpret_cast<const uint4*>(out + gid * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(dout + gid * 8);
    const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(ah[i]), y = __bfloat1622float2(gh[i]);
      acc += x.x * y.x + x.y * y.y;
    }
    float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    float4* dq = reinterpret_cast<float4*>(dq_acc + gid * 8);
    dq[0] = z;
    dq[1] = z;
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  acc += __shfl_xor_sync(0xffffffffu, acc, 4);
  if (active && (threadIdx.x & 7) == 0) {
    const long long th = gid >> 3;            // (b * S + s) * H + h
    const int h = (int)(th % H);
    const long long bs = th / H;
    const int s = (int)(bs % S);
    const long long b = bs / S;
    delta[(b * H + h) * S + s] = acc;
  }
}

// backward post-pass: the fp32 dQ accumulator [B*S][hidden] becomes the q third of d(qkv) [B*S][3*hidden] (bf16)
__global__ void attn_bwd_dq_convert_kernel(const float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv,
                                           long long rows, int hidden) {
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // 8 elements each
  const int per_row = hidden / 8;
  if (gid >= rows * per_row) return;
  const long long r = gid / per_row;
  const int c8 = (int)(gid % per_row);
  const float4 a = *reinterpret_cast<const float4*>(dq_acc + r * hidden + c8 * 8);
  const float4 b = *reinterpret_cast<const float4*>(dq_acc + r * hidden + c8 * 8 + 4);
  uint4 o;
  o.x = pack_bf16(a.x, a.y);
  o.y = pack_bf16(a.z, a.w);
  o.z = pack_bf16(b.x, b.y);
  o.w = pack_bf16(b.z, b.w);
  *reinterpret_cast<uint4*>(dqkv + r * 3 * hidden + c8 * 8) = o;
}

// ---------------------------------------------------------------------------------------------
// backward main kernel
struct BwdSmem {
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = TILE_BYTES;
  static constexpr int RING_OFF = 2 * TILE_BYTES;                 // 2 stages x (Q 16 KB + dO 16 KB)
  static constexpr int RING = 2;
  static constexpr int P_OFF = RING_OFF + RING * 2 * TILE_BYTES;  // P  : two slabs by key half
  static constexpr int DS_OFF = P_OFF + 2 * TILE_BYTES;           // dS : two slabs by key half
  static constexpr int DQ_OFF = DS_OFF + 2 * TILE_BYTES;          // fp32 staging: two boxes of 128 rows x 32 columns
  static constexpr int BAR_OFF = DQ_OFF + 2 * TILE_BYTES;
  static constexpr int NUM_BARS = 1 + 2 * RING + 7;
  static constexpr int TOTAL = BAR_OFF + NUM_BARS * 8 + 16;
};

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_dout,
                const __grid_constant__ CUtensorMap map_dqkv, const __grid_constant__ CUtensorMap map_dq,
                const AttnParams p) {
  using L = BwdSmem;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t IDESC_S = make_idesc(1, false, false, TILE, TILE);   // S = Q K^T, dP = dO V^T
  constexpr uint32_t IDESC_KV = make_idesc(1, true, true, TILE, HD);      // dV = P^T dO, dK = dS^T Q
  constexpr uint32_t IDESC_DQ = make_idesc(1, false, true, TILE, HD);     // dQ = dS K

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::BAR_OFF;
  const uint32_t kv_full = bar_base;
  auto qdo_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto qdo_empty = [&](int s) { return bar_base + 8u * (1 + L::RING + s); };
  const uint32_t s_full = bar_base + 8u * (1 + 2 * L::RING);
  const uint32_t s_empty = s_full + 8, pds_full = s_full + 16, grads_done = s_full + 24, all_done = s_full + 32;
  // one barrier per dQ buffer in TMEM: a barrier shared by both buffers could complete two phases between two looks
  // of the MMA thread, which a parity wait cannot tell from none
  auto dq_empty = [&](int it) { return s_full + 40u + 8u * (uint32_t)(it & 1); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::BAR_OFF + L::NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::BAR_OFF + L::NUM_BARS * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = (p.S + TILE - 1) / TILE;
  const int kv_tile = blockIdx.x;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int key0 = kv_tile * TILE;
  const int i0 = p.causal ? kv_tile : 0;          // first query tile that sees these keys
  const int n_iter = num_tiles - i0;
  const int hidden = p.H * HD;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < L::RING; ++s) {
      mbar_init(qdo_full(s), 1);
      mbar_init(qdo_empty(s), 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, BWD_COMPUTE);
    mbar_init(pds_full, BWD_COMPUTE);
    mbar_init(grads_done, 1);
    mbar_init(dq_empty(0), BWD_COMPUTE);
    mbar_init(dq_empty(1), BWD_COMPUTE);
    mbar_init(all_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tc_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
    tc_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_dp = tmem_base + 128, tmem_dv = tmem_base + 256, tmem_dk = tmem_base + 320;
  auto tmem_dq = [&](int it) { return tmem_base + 384u + 64u * (uint32_t)(it & 1); };

  bool failed = false;
  int where = 0;   // source line of the wait in progress: reported if it runs out

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * TILE_BYTES);
      tma_load_3d(smem_base + L::K_OFF, &map_qkv, kv_full, hidden + head * HD, key0, batch);
      tma_load_3d(smem_base + L::V_OFF, &map_qkv, kv_full, 2 * hidden + head * HD, key0, batch);
      for (int it = 0; it < n_iter; ++it) {
        const int stage = it % L::RING, use = it / L::RING;
        if (!(where = __LINE__, mbar_wait(qdo_empty(stage), (use & 1) ^ 1, abort_flag))) { failed = true; break; }
        mbar_expect_tx(qdo_full(stage), 2 * TILE_BYTES);
        const uint32_t dst = smem_base + L::RING_OFF + stage * 2 * TILE_BYTES;
        tma_load_3d(dst, &map_qkv, qdo_full(stage), head * HD, (i0 + it) * TILE, batch);
        tma_load_3d(dst + TILE_BYTES, &map_dout, qdo_full(stage), head * HD, (i0 + it) * TILE, batch);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t k_addr = smem_base + L::K_OFF, v_addr = smem_base + L::V_OFF;
      const uint32_t p_addr = smem_base + L::P_OFF, ds_addr = smem_base + L::DS_OFF;
      auto issue_grads = [&](int it) -> bool {
        const int stage = it % L::RING;
        if (!(where = __LINE__, mbar_wait(pds_full, it & 1, abort_flag))) return false;
        if (it >= 2 && !(where = __LINE__, mbar_wait(dq_empty(it), ((it >> 1) - 1) & 1, abort_flag))) return false;   // drain of iteration it - 2
        tc_fence_after();
        const uint32_t q_addr = smem_base + L::RING_OFF + stage * 2 * TILE_BYTES, do_addr = q_addr + TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < TILE / 16; ++kk) {   // dV += P^T dO : contraction over the 128 queries
          const uint64_t a_desc = make_smem_desc(p_addr + kk * 16 * 128, TILE_BYTES, 1024, 2);
          const uint64_t b_desc = make_smem_desc(do_addr + kk * 16 * 128, TILE_BYTES, 1024, 2);
          tc_mma<false>(tmem_dv, a_desc, b_desc, IDESC_KV, (it > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < TILE / 16; ++kk) {   // dK += dS^T Q
          const uint64_t a_desc = make_smem_desc(ds_addr + kk * 16 * 128, TILE_BYTES, 1024, 2);
          const uint64_t b_desc = make_smem_desc(q_addr + kk * 16 * 128, TILE_BYTES, 1024, 2);
          tc_mma<false>(tmem_dk, a_desc, b_desc, IDESC_KV, (it > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < TILE / 16; ++kk) {   // dQ = dS K : contraction over the 128 keys
          const uint64_t a_desc = make_smem_desc(ds_addr + (kk >> 2) * TILE_BYTES + (kk & 3) * 32, 16, 1024);
          const uint64_t b_desc = make_smem_desc(k_addr + kk * 16 * 128, TILE_BYTES, 1024, 2);
          tc_mma<false>(tmem_dq(it), a_desc, b_desc, IDESC_DQ, kk > 0 ? 1u : 0u);
        }
        tc_commit(qdo_empty(stage));
        tc_commit(grads_done);
        return true;
      };
      if (!(where = __LINE__, mbar_wait(kv_full, 0, abort_flag))) failed = true;
      for (int it = 0; it < n_iter && !failed; ++it) {
        const int stage = it % L::RING, use = it / L::RING;
        if (!(where = __LINE__, mbar_wait(qdo_full(stage), use & 1, abort_flag))) { failed = true; break; }
        if (it > 0 && !(where = __LINE__, mbar_wait(s_empty, (it - 1) & 1, abort_flag))) { failed = true; break; }
        tc_fence_after();
        const uint32_t q_addr = smem_base + L::RING_OFF + stage * 2 * TILE_BYTES, do_addr = q_addr + TILE_BYTES;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t a_desc = make_smem_desc(q_addr + k * 32, 16, 1024);
          const uint64_t b_desc = make_smem_desc(k_addr + k * 32, 16, 1024);
          tc_mma<false>(tmem_s, a_desc, b_desc, IDESC_S, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t a_desc = make_smem_desc(do_addr + k * 32, 16, 1024);
          const uint64_t b_desc = make_smem_desc(v_addr + k * 32, 16, 1024);
          tc_mma<false>(tmem_dp, a_desc, b_desc, IDESC_S, k > 0 ? 1u : 0u);
        }
        tc_commit(s_full);
        if (it > 0 && !issue_grads(it - 1)) { failed = true; break; }
      }
      if (!failed && !issue_grads(n_iter - 1)) failed = true;
      if (!failed) tc_commit(all_done);
    }
  } else {
    // ------------------------------------------------------------------ element-wise work (warps 2..9)
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;            // which 64 key columns of the tile this thread handles
    const int row = quad * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const float c = p.scale_log2;
    const long long stat_base = ((long long)batch * p.H + head) * p.S;
    uint8_t* dq_stage = smem + L::DQ_OFF + half * TILE_BYTES + row * 128;

    // Control flow of these 256 threads is kept identical whether or not a wait ran out: `ok` only gates the work,
    // every named barrier below is reached by all of them in every iteration. After a failure the abort flag is
    // up, so the remaining waits return at once.
    bool ok = true;

    // moves the finished dQ tile of iteration `it` (64 fp32 columns, 32 per warpgroup) into the global accumulator
    auto drain_dq = [&](int it, bool need_wait) {
      if (ok && need_wait) ok = (where = __LINE__, warp_wait(grads_done, it & 1, abort_flag));
      uint32_t r[32];
      if (ok) {
        tc_fence_after();
        tc_ld32(tmem_dq(it) + lane_base + (uint32_t)(half * 32), r);
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(dq_empty(it));
      }
      if (threadIdx.x == 64) tma_wait_read<0>();   // the staging buffer has been read by the previous reduce-add
      named_bar_sync<BWD_COMPUTE>();
      if (ok) {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<uint4*>(dq_stage + ((q ^ (row & 7)) << 4)) = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
        fence_proxy_async_smem();
      }
      named_bar_sync<BWD_COMPUTE>();
      if (threadIdx.x == 64 && !*abort_flag) {
        const int qrow0 = (i0 + it) * TILE;
        tma_reduce_add_3d(&map_dq, smem_base + L::DQ_OFF, head * HD, qrow0, batch);
        tma_reduce_add_3d(&map_dq, smem_base + L::DQ_OFF + TILE_BYTES, head * HD + 32, qrow0, batch);
        tma_commit();
      }
    };

    for (int it = 0; it < n_iter; ++it) {
      const int q_idx = (i0 + it) * TILE + row;
      const bool row_ok = q_idx < p.S;
      const float lse = row_ok ? __ldg(p.lse + stat_base + q_idx) : 0.f;
      const float dlt = row_ok ? __ldg(p.delta + stat_base + q_idx) * p.scale : 0.f;
      uint32_t pk[32], dk[32];   // this thread's 64 P and 64 dS values as packed bf16 pairs
      if (ok) ok = (where = __LINE__, warp_wait(s_full, it & 1, abort_flag));
      if (ok) {
        tc_fence_after();
        const bool need_mask = (key0 + TILE > p.S) || (p.causal && (i0 + it) == kv_tile) || ((i0 + it) * TILE + TILE > p.S);
        const int key_limit = row_ok ? (p.causal ? min(p.S, q_idx + 1) : p.S) : 0;
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t rs[32], rd[32];
          const uint32_t col = (uint32_t)(half * 64 + ch * 32);
          tc_ld32(tmem_s + lane_base + col, rs);
          tc_ld32(tmem_dp + lane_base + col, rd);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = fast_exp2(fmaf(__uint_as_float(rs[i]), c, -lse));
            float p1 = fast_exp2(fmaf(__uint_as_float(rs[i + 1]), c, -lse));
            if (need_mask) {
              const int key = key0 + (int)col + i;
              if (key >= key_limit) p0 = 0.f;
              if (key + 1 >= key_limit) p1 = 0.f;
            }
            const float d0 = p0 * fmaf(__uint_as_float(rd[i]), p.scale, -dlt);
            const float d1 = p1 * fmaf(__uint_as_float(rd[i + 1]), p.scale, -dlt);
            pk[ch * 16 + (i >> 1)] = pack_bf16(p0, p1);
            dk[ch * 16 + (i >> 1)] = pack_bf16(d0, d1);
          }
        }
        tc_fence_before();
        mbar_arrive(s_empty);
        // the operand buffers are free once the gradient products of the previous iteration have completed
        if (it > 0) ok = (where = __LINE__, warp_wait(grads_done, (it - 1) & 1, abort_flag));
      }
      if (ok) {
        uint8_t* p_row = smem + L::P_OFF + half * TILE_BYTES + row * 128;
        uint8_t* ds_row = smem + L::DS_OFF + half * TILE_BYTES + row * 128;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int off = (q ^ (row & 7)) << 4;
          *reinterpret_cast<uint4*>(p_row + off) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
          *reinterpret_cast<uint4*>(ds_row + off) = make_uint4(dk[4 * q], dk[4 * q + 1], dk[4 * q + 2], dk[4 * q + 3]);
        }
        fence_proxy_async_smem();
        mbar_arrive(pds_full);
      }
      if (it > 0) drain_dq(it - 1, false);   // grads_done of it - 1 was observed above
    }
    drain_dq(n_iter - 1, true);
    // dK (first warpgroup) and dV (second warpgroup): 128 keys x 64 columns each, staged over the P / dS buffers
    if (ok) ok = (where = __LINE__, warp_wait(all_done, 0, abort_flag));
    if (ok) {
      tc_fence_after();
      uint8_t* stage_row = smem + (half == 0 ? L::P_OFF : L::DS_OFF) + row * 128;
      const uint32_t src = (half == 0 ? tmem_dk : tmem_dv) + lane_base;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t r[32];
        tc_ld32(src + (uint32_t)(hh * 32), r);
        tc_wait_ld();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 o;
          o.x = pack_bf16(__uint_as_float(r[8 * q]), __uint_as_float(r[8 * q + 1]));
          o.y = pack_bf16(__uint_as_float(r[8 * q + 2]), __uint_as_float(r[8 * q + 3]));
          o.z = pack_bf16(__uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5]));
          o.w = pack_bf16(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7]));
          const int chunk = hh * 4 + q;
          *reinterpret_cast<uint4*>(stage_row + ((chunk ^ (row & 7)) << 4)) = o;
        }
      }
      fence_proxy_async_smem();
    }
    named_bar_sync<BWD_COMPUTE>();
    if (threadIdx.x == 64) {
      if (!*abort_flag) {
        tma_store_3d(&map_dqkv, smem_base + L::P_OFF, hidden + head * HD, key0, batch);
        tma_store_3d(&map_dqkv, smem_base + L::DS_OFF, 2 * hidden + head * HD, key0, batch);
        tma_commit();
      }
      tma_wait_all<0>();
    }
    if (!ok) failed = true;
  }

  if (failed) {
    *abort_flag = 1;
    if (p.err) atomicCAS(p.err, 0, 2000000 + warp * 10000 + where);   // the first failure is kept
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tc_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn attn_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(ptr);
  return fn;
}

// 3-D map over [B][S][cols] (cols contiguous): box = box_cols x 128 positions x 1 batch, 128-byte swizzle.
int make_map_3d(CUtensorMap* map, const void* base, bool is_f32, int B, int S, long long cols, int box_cols) {
  EncodeTiledFn fn = attn_encode_fn();
  if (!fn) return -10;
  ensure_context_on_this_thread();
  const int elem = is_f32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (cols * elem) % 16 != 0) return -11;
  cuuint64_t gdim[3] = {(cuuint64_t)cols, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t gstride[2] = {(cuuint64_t)(cols * elem), (cuuint64_t)((long long)S * cols * elem)};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)TILE, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, is_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                  const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "attention: cuTensorMapEncodeTiled failed (%d): base %p f32 %d dims (%lld, %d, %d) box %d\n", (int)r, base,
            (int)is_f32, cols, S, B, box_cols);
    return -12;
  }
  return 0;
}

}  // namespace

// out[B][S][H*64] = softmax(q k^T * scale (+ causal mask)) v for the packed bf16 qkv [B][S][3][H][64].
// lse (fp32 [B][H][S]) receives the base-2 log-sum-exp of the scaled scores, which hm_attn_bwd needs.
// err: device int set non-zero if a bounded wait ran out. Returns 0, a CUDA error (> 0) or an argument error (< 0).
HM_API int hm_attn_fwd(const void* qkv, void* out, float* lse, int B, int S, int H, int head_dim, int causal,
                       float scale, int* err, cudaStream_t stream) {
  if (B <= 0 || S <= 0 || H <= 0) return 0;
  if (head_dim != HD) return -30;
  CUtensorMap mq, mo;
  int rc = make_map_3d(&mq, qkv, false, B, S, 3LL * H * HD, HD);
  if (rc) return rc;
  rc = make_map_3d(&mo, out, false, B, S, (long long)H * HD, HD);
  if (rc) return rc;
  AttnParams p;
  p.B = B; p.S = S; p.H = H; p.causal = causal; p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse; p.delta = nullptr; p.err = err;
  const int smem = FwdSmem::TOTAL + 1024;
  cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid((S + TILE - 1) / TILE, H, B);
  attn_fwd_kernel<<<grid, FWD_THREADS, smem, stream>>>(mq, mo, p);
  return (int)cudaGetLastError();
}

// d(qkv) [B][S][3][H][64] (bf16, every element written) from d(out) [B][S][H*64], the forward inputs and outputs.
// Scratch supplied by the caller: delta fp32 [B][H][S], dq_acc fp32 [B][S][H*64]. Three launches: pre-pass
// (delta, clear dq_acc), main kernel (dK, dV stored; dQ tiles added into dq_acc), conversion of dq_acc to bf16.
HM_API int hm_attn_bwd(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv, float* delta,
                       float* dq_acc, int B, int S, int H, int head_dim, int causal, float scale, int* err,
                       cudaStream_t stream) {
  if (B <= 0 || S <= 0 || H <= 0) return 0;
  if (head_dim != HD) return -30;
  const long long hidden = (long long)H * HD;
  CUtensorMap mq, mdo, mdqkv, mdq;
  int rc = make_map_3d(&mq, qkv, false, B, S, 3 * hidden, HD);
  if (rc) return rc;
  rc = make_map_3d(&mdo, dout, false, B, S, hidden, HD);
  if (rc) return rc;
  rc = make_map_3d(&mdqkv, dqkv, false, B, S, 3 * hidden, HD);
  if (rc) return rc;
  rc = make_map_3d(&mdq, dq_acc, true, B, S, hidden, 32);
  if (rc) return rc;
  AttnParams p;
  p.B = B; p.S = S; p.H = H; p.causal = causal; p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = const_cast<float*>(lse); p.delta = delta; p.err = err;
  {
    const long long threads = (long long)B * S * H * 8;
    const int block = 256;
    attn_bwd_prep_kernel<<<(unsigned)((threads + block - 1) / block), block, 0, stream>>>(
        (const __nv_bfloat16*)out, (const __nv_bfloat16*)dout, delta, dq_acc, B, S, H);
  }
  const int smem = BwdSmem::TOTAL + 1024;
  cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid((S + TILE - 1) / TILE, H, B);
  attn_bwd_kernel<<<grid, BWD_THREADS, smem, stream>>>(mq, mdo, mdqkv, mdq, p);
  {
    const long long threads = (long long)B * S * hidden / 8;
    const int block = 256;
    attn_bwd_dq_convert_kernel<<<(unsigned)((threads + block - 1) / block), block, 0, stream>>>(
        dq_acc, (__nv_bfloat16*)dqkv, (long long)B * S, (int)hidden);
  }
  return (int)cudaGetLastError();
}
