// Persistent, warp-specialised tcgen05 GEMM for sm_100a with fused epilogues.
//
//   D[M,N] (row-major) = epilogue( sum_k A(m,k) * B(n,k) )
//
// Operands are bf16 (kind::f16) or fp32 fed as tf32 (kind::tf32); accumulation is fp32 in TMEM.
// Each operand is either K-major (stored [rows][K], K contiguous) or MN-major (stored [K][rows], rows
// contiguous), so that y = x W^T, dx = dy W and dW = dy^T x all run without a transposed copy:
//     forward   y [T,out] : A = x  [T,in]  K-major,  B = W  [out,in] K-major
//     grad in   dx[T,in]  : A = dy [T,out] K-major,  B = W  [out,in] MN-major (contraction over `out`)
//     grad w    dW[out,in]: A = dy [T,out] MN-major, B = x  [T,in]   MN-major (contraction over T)
//
// Structure (one CTA per SM, 192 threads, tiles 128 x BLOCK_N x 128 bytes of K):
//   warp 0      : TMA producer — unicast cp.async.bulk.tensor loads into a STAGES-deep smem ring
//   warp 1      : allocates TMEM, issues tcgen05.mma from one elected lane, commits to mbarriers
//   warps 2..5  : epilogue — tcgen05.ld the accumulator (double-buffered in TMEM so that the next tile's
//                 MMAs overlap), apply bias / tanh-GELU, stage in 128B-swizzled smem, TMA store
//                 (or TMA reduce-add into an fp32 destination: split-K and gradient accumulation for free).
// Every mbarrier wait is bounded by a wall-clock budget; on expiry the CTA records an error word, lets
// in-flight copies land, frees its TMEM and returns.
//
// Call sites served: the expert FFN of hivemind/moe/server/layers/common.py:17-30, the transformer
// blocks of the ALBERT / GPT-2 shaped models, and PowerSGD's P = M Q, Q = M^T P
// (hivemind/optim/power_sgd_averager.py:158-170).
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "tc_ptx.cuh"

namespace {

constexpr int BLOCK_M = 128;
constexpr int ROW_BYTES = 128;           // one swizzle-128B row
constexpr int NUM_THREADS = 192;

enum Epi : int { EPI_NONE = 0, EPI_BIAS = 1, EPI_BIAS_GELU = 2 };

struct GemmParams {
  int M, N, K;
  int num_m_tiles, num_n_tiles, num_splits, kblocks_per_split, total_kblocks;
  int epi, out_f32, reduce_add, has_aux;
  const float* bias;
  const __nv_bfloat16* add;   // optional bf16 [M][N] (row stride ld_add) combined with the result before it is stored:
  long long ld_add;           //   add_mode 0: result + add;  1: result * gelu_tanh'(add)
  int add_mode;
  float alpha;
  int* err;
  // Grouped problems (many experts in one launch). Mode 1: the rows of A and D are split into groups of whole
  // M tiles; group_table[m_tile] names the group (-1: skip the tile) and selects that group's slice of B
  // (group * group_b_rows along B's row coordinate) and of the bias. Mode 2: every group owns a range of K
  // (rows group_table[g] .. group_table[g+1] of both MN-major operands, multiples of BLOCK_K) and a slice of D
  // (group * group_d_rows along D's rows); tiles enumerate (group, m_tile, n_tile).
  int group_mode, num_groups, group_b_rows, group_d_rows, group_bias;
  const int* group_table;
};

struct TileInfo {
  int m_tile, n_tile, kb0, kb1, group;
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers

template <int BLOCK_N, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BLOCK_M * ROW_BYTES;
  static constexpr int B_BYTES = BLOCK_N * ROW_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int OUT_BYTES = BLOCK_M * ROW_BYTES;  // one staged box: 128 rows x 128 B
  // Staging boxes for the TMA stores: two alternate; the three-stage form of the 256-wide tile (used when a second
  // output, the pre-activation values, is written) has four, so that both outputs alternate as well.
  static constexpr int NUM_OUT = (BLOCK_N == 256 && STAGES == 3) ? 4 : 2;
  static constexpr int OUT_OFF = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = OUT_OFF + NUM_OUT * OUT_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int TOTAL = BAR_OFF + NUM_BARS * 8 + 16;
};

// ---------------------------------------------------------------------------------------------
template <int BLOCK_N, int STAGES, bool TF32, bool A_MN, bool B_MN, bool ADD = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_d, const __grid_constant__ CUtensorMap map_aux,
               const GemmParams p) {
  using L = SmemLayout<BLOCK_N, STAGES>;
  constexpr int ELEM = TF32 ? 4 : 2;
  constexpr int BLOCK_K = ROW_BYTES / ELEM;   // elements of K per stage (one 128 B swizzle row)
  constexpr int UMMA_K = 32 / ELEM;
  constexpr int RUN = ROW_BYTES / ELEM;       // contiguous MN elements per 128 B row of an MN-major tile
  constexpr uint32_t TMEM_COLS = 2 * BLOCK_N <= 32 ? 32 : (2 * BLOCK_N <= 64 ? 64 : (2 * BLOCK_N <= 128 ? 128 : (2 * BLOCK_N <= 256 ? 256 : 512)));
  constexpr uint32_t IDESC = make_idesc(TF32 ? 2 : 1, A_MN, B_MN, BLOCK_M, BLOCK_N);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // 1024 B alignment for the swizzle atoms (dynamic smem base is only guaranteed 16 B aligned)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::BAR_OFF;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::BAR_OFF + L::NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::BAR_OFF + L::NUM_BARS * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_tiles * p.num_n_tiles * (p.group_mode == 2 ? p.num_groups : p.num_splits);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), EPI_THREADS);
    }
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

  // Decodes a tile index; returns false if the tile has no work (an empty group). Every role calls this with the
  // same arguments and therefore skips the same tiles.
  auto tile_info = [&](int tile, TileInfo& ti) -> bool {
    if (p.group_mode == 2) {
      const int per_group = p.num_m_tiles * p.num_n_tiles;
      ti.group = tile / per_group;
      const int t = tile - ti.group * per_group;
      ti.n_tile = t % p.num_n_tiles;
      ti.m_tile = t / p.num_n_tiles;
      ti.kb0 = __ldg(p.group_table + ti.group) / BLOCK_K;
      ti.kb1 = __ldg(p.group_table + ti.group + 1) / BLOCK_K;
      return ti.kb1 > ti.kb0;
    }
    const int split = tile % p.num_splits;
    const int t = tile / p.num_splits;
    ti.n_tile = t % p.num_n_tiles;
    ti.m_tile = t / p.num_n_tiles;
    ti.kb0 = split * p.kblocks_per_split;
    ti.kb1 = min(ti.kb0 + p.kblocks_per_split, p.total_kblocks);
    ti.group = 0;
    if (p.group_mode == 1) {
      ti.group = __ldg(p.group_table + ti.m_tile);
      return ti.group >= 0;
    }
    return true;
  };

  bool failed = false;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !failed; tile += gridDim.x) {
        TileInfo ti;
        if (!tile_info(tile, ti)) continue;
        const int m_tile = ti.m_tile, n_tile = ti.n_tile;
        const int b_row_off = (p.group_mode == 1) ? ti.group * p.group_b_rows : 0;
        for (int kb = ti.kb0; kb < ti.kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) { failed = true; break; }
          const uint32_t a_dst = smem_base + stage * L::STAGE_BYTES;
          const uint32_t b_dst = a_dst + L::A_BYTES;
          mbar_expect_tx(full_bar(stage), L::STAGE_BYTES);
          const int k0 = kb * BLOCK_K;
          if constexpr (A_MN) {
#pragma unroll
            for (int r = 0; r < BLOCK_M / RUN; ++r)
              tma_load_2d(a_dst + r * (BLOCK_K * ROW_BYTES), &map_a, full_bar(stage), m_tile * BLOCK_M + r * RUN, k0);
          } else {
            tma_load_2d(a_dst, &map_a, full_bar(stage), k0, m_tile * BLOCK_M);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int r = 0; r < BLOCK_N / RUN; ++r)
              tma_load_2d(b_dst + r * (BLOCK_K * ROW_BYTES), &map_b, full_bar(stage), n_tile * BLOCK_N + r * RUN, k0 + b_row_off);
          } else {
            tma_load_2d(b_dst, &map_b, full_bar(stage), k0, n_tile * BLOCK_N + b_row_off);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !failed; tile += gridDim.x) {
        TileInfo ti;
        if (!tile_info(tile, ti)) continue;
        const int kb0 = ti.kb0, kb1 = ti.kb1;
        const int buf = local & 1;
        const uint32_t use = (uint32_t)(local >> 1);
        if (!mbar_wait(tempty_bar(buf), (use & 1) ^ 1, abort_flag)) { failed = true; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BLOCK_N);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) { failed = true; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * L::STAGE_BYTES;
          const uint32_t b_addr = a_addr + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            constexpr uint32_t MN_SBO = TF32 ? 512 : 1024, MN_TYPE = TF32 ? 1 : 2;
            const uint64_t a_desc = A_MN ? make_smem_desc(a_addr + k * UMMA_K * ROW_BYTES, BLOCK_K * ROW_BYTES, MN_SBO, MN_TYPE)
                                         : make_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t b_desc = B_MN ? make_smem_desc(b_addr + k * UMMA_K * ROW_BYTES, BLOCK_K * ROW_BYTES, MN_SBO, MN_TYPE)
                                         : make_smem_desc(b_addr + k * 32, 16, 1024);
            tc_mma<TF32>(d_tmem, a_desc, b_desc, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));  // frees the smem stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        tc_commit(tfull_bar(buf));  // accumulator complete
        ++local;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;               // TMEM lane quarter this warp may read
    const int row = quad * 32 + lane;        // row inside the tile
    const int epi_tid = threadIdx.x - 64;
    uint8_t* out_buf[4] = {smem + L::OUT_OFF, smem + L::OUT_OFF + L::OUT_BYTES,
                           smem + L::OUT_OFF + (L::NUM_OUT == 4 ? 2 : 0) * L::OUT_BYTES,
                           smem + L::OUT_OFF + (L::NUM_OUT == 4 ? 3 : 1) * L::OUT_BYTES};
    constexpr bool AUX_ALTERNATES = L::NUM_OUT == 4;
    constexpr int COLS_PER_BOX = 32;          // accumulator columns handled per tcgen05.ld
    const int out_elem = p.out_f32 ? 4 : 2;
    const int boxes_per_store = p.out_f32 ? 1 : 2;  // 128 B rows: 32 fp32 or 64 bf16
    int local = 0;
    int flip = 0;
    for (int tile = blockIdx.x; tile < num_tiles && !failed; tile += gridDim.x) {
      TileInfo ti;
      if (!tile_info(tile, ti)) continue;
      const int m_tile = ti.m_tile, n_tile = ti.n_tile;
      const float* bias = (p.bias != nullptr) ? p.bias + (long long)ti.group * p.group_bias : nullptr;
      const int d_row_off = (p.group_mode == 2) ? ti.group * p.group_d_rows : 0;
      const int buf = local & 1;
      const uint32_t use = (uint32_t)(local >> 1);
      // every epilogue thread waits; the four warps then agree on the outcome, so that the warp-wide
      // tcgen05.ld and the named barriers below are never reached by only part of the group
      const bool ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar(buf), use & 1, abort_flag));
      if (!ok) *abort_flag = 1;
      epi_bar_sync();
      if (*abort_flag) { failed = true; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BLOCK_N);
      const int n_valid = min(BLOCK_N, p.N - n_tile * BLOCK_N);
      // Second epilogue input (p.add): this thread's 128 bytes of the NEXT 64-column group are requested while the
      // current group is converted and stored, so that only the first group of a tile waits for global memory.
      const long long add_row = (long long)m_tile * BLOCK_M + row;
      auto load_group = [&](int c_base, uint4 (&dst)[8]) {
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const int gcol = n_tile * BLOCK_N + c_base + 8 * ch;
          dst[ch] = make_uint4(0u, 0u, 0u, 0u);
          if (add_row < p.M && c_base + 8 * ch < n_valid && gcol < p.N)
            dst[ch] = *reinterpret_cast<const uint4*>(p.add + add_row * p.ld_add + gcol);
        }
      };
      uint4 add_cur[8], add_next[8];
      if (ADD) load_group(0, add_cur);
      for (int c0 = 0; c0 < BLOCK_N; c0 += COLS_PER_BOX * boxes_per_store) {
        if (c0 >= n_valid) break;  // columns beyond N: nothing to store (uniform across the CTA)
        if (ADD && c0 + 64 < n_valid) load_group(c0 + 64, add_next);
        // the staging buffer we are about to fill must have been read by its previous TMA store
        if (epi_tid == 0) {
          if (p.has_aux && !AUX_ALTERNATES) tma_wait_read<0>(); else tma_wait_read<1>();
        }
        epi_bar_sync();
        uint8_t* stage_main = (p.has_aux && !AUX_ALTERNATES) ? out_buf[0] : out_buf[flip];
        uint8_t* stage_aux = AUX_ALTERNATES ? out_buf[2 + flip] : out_buf[1];
#pragma unroll 1
        for (int half = 0; half < boxes_per_store; ++half) {
          uint32_t r[32];
          tc_ld32(t_addr + (uint32_t)(c0 + half * COLS_PER_BOX), r);
          const int gcol0 = n_tile * BLOCK_N + c0 + half * COLS_PER_BOX;
          tc_wait_ld();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
          if (p.epi != EPI_NONE && bias != nullptr) {
            if (gcol0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(bias) + 4u * gcol0) & 15u) == 0) {   // whole box, aligned: eight 16-byte loads
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 b4 = __ldg(reinterpret_cast<const float4*>(bias + gcol0) + q);
                v[4 * q] += b4.x; v[4 * q + 1] += b4.y; v[4 * q + 2] += b4.z; v[4 * q + 3] += b4.w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (gcol0 + j < p.N) v[j] += __ldg(bias + gcol0 + j);
            }
          }
          if (ADD) {
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&add_cur[ch]);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                if (p.add_mode == 0) {
                  v[8 * ch + 2 * q] += __low2float(h[q]);
                  v[8 * ch + 2 * q + 1] += __high2float(h[q]);
                } else {
                  v[8 * ch + 2 * q] *= hm_gelu_tanh_grad(__low2float(h[q]));
                  v[8 * ch + 2 * q + 1] *= hm_gelu_tanh_grad(__high2float(h[q]));
                }
              }
            }
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) add_cur[ch] = add_cur[4 + ch];   // the second half's columns move up
          }
          // 16-byte chunks of this thread's row, XOR-swizzled like the tensor map (chunk ^= row & 7)
          if (p.out_f32) {
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
              float4 o = make_float4(v[4 * ch], v[4 * ch + 1], v[4 * ch + 2], v[4 * ch + 3]);
              if (p.epi == EPI_BIAS_GELU) { o.x = hm_gelu_tanh(o.x); o.y = hm_gelu_tanh(o.y); o.z = hm_gelu_tanh(o.z); o.w = hm_gelu_tanh(o.w); }
              *reinterpret_cast<float4*>(stage_main + row * ROW_BYTES + ((ch ^ (row & 7)) << 4)) = o;
            }
          } else {
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              const int pc = (half * 4 + ch) ^ (row & 7);
              if (p.has_aux) {
                uint4 a;
                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * ch], v[8 * ch + 1]), h1 = __floats2bfloat162_rn(v[8 * ch + 2], v[8 * ch + 3]);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * ch + 4], v[8 * ch + 5]), h3 = __floats2bfloat162_rn(v[8 * ch + 6], v[8 * ch + 7]);
                a.x = *reinterpret_cast<uint32_t*>(&h0); a.y = *reinterpret_cast<uint32_t*>(&h1);
                a.z = *reinterpret_cast<uint32_t*>(&h2); a.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(stage_aux + row * ROW_BYTES + (pc << 4)) = a;
              }
              float w[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) w[j] = p.epi == EPI_BIAS_GELU ? hm_gelu_tanh(v[8 * ch + j]) : v[8 * ch + j];
              uint4 o;
              __nv_bfloat162 h0 = __floats2bfloat162_rn(w[0], w[1]), h1 = __floats2bfloat162_rn(w[2], w[3]);
              __nv_bfloat162 h2 = __floats2bfloat162_rn(w[4], w[5]), h3 = __floats2bfloat162_rn(w[6], w[7]);
              o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
              o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
              *reinterpret_cast<uint4*>(stage_main + row * ROW_BYTES + (pc << 4)) = o;
            }
          }
        }
        fence_proxy_async_smem();
        epi_bar_sync();
        if (epi_tid == 0) {
          const int gc = n_tile * BLOCK_N + c0, gr = m_tile * BLOCK_M + d_row_off;
          if (p.reduce_add) tma_reduce_add_2d(&map_d, smem_u32(stage_main), gc, gr);
          else tma_store_2d(&map_d, smem_u32(stage_main), gc, gr);
          if (p.has_aux) tma_store_2d(&map_aux, smem_u32(stage_aux), gc, gr);
          tma_commit();
        }
        if (ADD) {
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) add_cur[ch] = add_next[ch];
        }
        flip ^= 1;
        (void)out_elem;
      }
      // all of this thread's tcgen05.ld for the buffer are complete: hand the accumulator back
      tc_fence_before();
      mbar_arrive(tempty_bar(buf));
      ++local;
    }
    if (epi_tid == 0) tma_wait_all<0>();
  }

  // ------------------------------------------------------------------ teardown (every thread gets here)
  if (failed) {
    *abort_flag = 1;
    if (p.err) atomicExch(p.err, 1 + warp);
    // let copies that are still in flight land before the CTA's shared memory is released
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
// Two-CTA form (tcgen05 cta_group::2). A 128x256 tile per SM is bound by shared-memory bandwidth: every
// 128x256x16 MMA reads 12 KB of operands that TMA also had to write. Here two CTAs of a cluster (two SMs) share one
// 256x256 tile: each CTA stages its own 128 rows of A and HALF of B (128 of the 256 columns), the leader CTA issues
// one MMA that spans both SMs, and each SM keeps the accumulator rows of its own half of M in its TMEM. Per SM and
// k-block that is 32 KB written and read instead of 48 KB.
//
// Protocol (barriers live at the same shared-memory offsets in both CTAs; "leader" = cluster rank 0):
//   full[s]   (leader's, 1 arrival + bytes): both CTAs' TMA loads report their bytes to the LEADER's barrier
//   empty[s]  (each CTA's own, 1 arrival): the leader's MMA warp commits to its own and to the peer's barrier
//   tfull[b]  (each CTA's own, 1 arrival): committed by the leader when a tile's accumulation is complete
//   tempty[b] (leader's, 2 x 128 arrivals): the epilogue threads of both CTAs hand the accumulator buffer back
// All loads are unicast; every wait is bounded as in the one-CTA kernel; the two CTAs meet at a cluster barrier
// before either leaves (a CTA must not exit while its peer may still read its shared memory).
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(map), "r"(leader_bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tc_alloc_pair(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

constexpr int PAIR_N = 256;       // N of the shared tile
constexpr int PAIR_BN = 128;      // columns of B staged by each CTA
constexpr int PAIR_M = 256;       // M of the shared tile (128 rows per CTA)

template <int STAGES>
struct PairSmem {
  static constexpr int A_BYTES = BLOCK_M * ROW_BYTES;
  static constexpr int B_BYTES = PAIR_BN * ROW_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int OUT_BYTES = BLOCK_M * ROW_BYTES;
  static constexpr int OUT_OFF = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = OUT_OFF + 2 * OUT_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int TOTAL = BAR_OFF + NUM_BARS * 8 + 16;
};

template <int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
tc_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_d, const __grid_constant__ CUtensorMap map_aux,
                    const GemmParams p) {
  using L = PairSmem<STAGES>;
  constexpr int ELEM = 2;
  constexpr int BLOCK_K = ROW_BYTES / ELEM;
  constexpr int UMMA_K = 32 / ELEM;
  constexpr int RUN = ROW_BYTES / ELEM;
  constexpr int BLOCK_N = PAIR_N;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t IDESC = make_idesc(1, A_MN, B_MN, PAIR_M, PAIR_N);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::BAR_OFF;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::BAR_OFF + L::NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::BAR_OFF + L::NUM_BARS * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_tiles = p.num_m_tiles * p.num_n_tiles * (p.group_mode == 2 ? p.num_groups : p.num_splits);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 2 * EPI_THREADS);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (warp == 1) {  // the same warp of both CTAs allocates collectively
    tc_alloc_pair(smem_u32((const void*)tmem_slot), TMEM_COLS);
    tc_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs are initialised and the allocation is visible
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // false = the tile has no work (an empty group); both CTAs and all roles skip the same tiles
  auto tile_info = [&](int tile, TileInfo& ti) -> bool {
    if (p.group_mode == 2) {
      const int per_group = p.num_m_tiles * p.num_n_tiles;
      ti.group = tile / per_group;
      const int t = tile - ti.group * per_group;
      ti.n_tile = t % p.num_n_tiles;
      ti.m_tile = t / p.num_n_tiles;
      ti.kb0 = __ldg(p.group_table + ti.group) / BLOCK_K;
      ti.kb1 = __ldg(p.group_table + ti.group + 1) / BLOCK_K;
      return ti.kb1 > ti.kb0;
    }
    const int split = tile % p.num_splits;
    const int t = tile / p.num_splits;
    ti.n_tile = t % p.num_n_tiles;
    ti.m_tile = t / p.num_n_tiles;
    ti.kb0 = split * p.kblocks_per_split;
    ti.kb1 = min(ti.kb0 + p.kblocks_per_split, p.total_kblocks);
    ti.group = 0;
    return true;
  };

  bool failed = false;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const int m_off = (int)rank * BLOCK_M, n_off = (int)rank * PAIR_BN;
      for (int tile = pair_id; tile < num_tiles && !failed; tile += num_pairs) {
        TileInfo ti;
        if (!tile_info(tile, ti)) continue;
        const int m0 = ti.m_tile * PAIR_M + m_off, n0 = ti.n_tile * PAIR_N + n_off;
        for (int kb = ti.kb0; kb < ti.kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) { failed = true; break; }
          const uint32_t a_dst = smem_base + stage * L::STAGE_BYTES;
          const uint32_t b_dst = a_dst + L::A_BYTES;
          const uint32_t leader_full = map_to_cta(full_bar(stage), 0);
          if (leader) mbar_expect_tx(full_bar(stage), 2 * L::STAGE_BYTES);  // bytes of both CTAs land on this barrier
          const int k0 = kb * BLOCK_K;
          if constexpr (A_MN) {
#pragma unroll
            for (int r = 0; r < BLOCK_M / RUN; ++r)
              tma_load_2d_pair(a_dst + r * (BLOCK_K * ROW_BYTES), &map_a, leader_full, m0 + r * RUN, k0);
          } else {
            tma_load_2d_pair(a_dst, &map_a, leader_full, k0, m0);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int r = 0; r < PAIR_BN / RUN; ++r)
              tma_load_2d_pair(b_dst + r * (BLOCK_K * ROW_BYTES), &map_b, leader_full, n0 + r * RUN, k0);
          } else {
            tma_load_2d_pair(b_dst, &map_b, leader_full, k0, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      for (int tile = pair_id; tile < num_tiles && !failed; tile += num_pairs) {
        TileInfo ti;
        if (!tile_info(tile, ti)) continue;
        const int buf = local & 1;
        const uint32_t use = (uint32_t)(local >> 1);
        if (!mbar_wait(tempty_bar(buf), (use & 1) ^ 1, abort_flag)) { failed = true; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BLOCK_N);
        for (int kb = ti.kb0; kb < ti.kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) { failed = true; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * L::STAGE_BYTES;
          const uint32_t b_addr = a_addr + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            const uint64_t a_desc = A_MN ? make_smem_desc(a_addr + k * UMMA_K * ROW_BYTES, BLOCK_K * ROW_BYTES, 1024, 2)
                                         : make_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t b_desc = B_MN ? make_smem_desc(b_addr + k * UMMA_K * ROW_BYTES, BLOCK_K * ROW_BYTES, 1024, 2)
                                         : make_smem_desc(b_addr + k * 32, 16, 1024);
            tc_mma_pair(d_tmem, a_desc, b_desc, IDESC, (kb > ti.kb0 || k > 0) ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          tc_commit_pair(map_to_cta(empty_bar(stage), 0));
          tc_commit_pair(map_to_cta(empty_bar(stage), 1));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        tc_commit_pair(map_to_cta(tfull_bar(buf), 0));  // accumulator complete: tell both epilogues
        tc_commit_pair(map_to_cta(tfull_bar(buf), 1));
        ++local;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    uint8_t* out_buf[2] = {smem + L::OUT_OFF, smem + L::OUT_OFF + L::OUT_BYTES};
    constexpr int COLS_PER_BOX = 32;
    const int boxes_per_store = p.out_f32 ? 1 : 2;
    int local = 0;
    int flip = 0;
    for (int tile = pair_id; tile < num_tiles && !failed; tile += num_pairs) {
      TileInfo ti;
      if (!tile_info(tile, ti)) continue;
      const int m_tile_row = ti.m_tile * PAIR_M + (int)rank * BLOCK_M + (p.group_mode == 2 ? ti.group * p.group_d_rows : 0);
      const int n_tile = ti.n_tile;
      const float* bias = p.bias;
      const int buf = local & 1;
      const uint32_t use = (uint32_t)(local >> 1);
      const bool ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar(buf), use & 1, abort_flag));
      if (!ok) *abort_flag = 1;
      epi_bar_sync();
      if (*abort_flag) { failed = true; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BLOCK_N);
      const int n_valid = min(BLOCK_N, p.N - n_tile * BLOCK_N);
      for (int c0 = 0; c0 < BLOCK_N; c0 += COLS_PER_BOX * boxes_per_store) {
        if (c0 >= n_valid) break;
        if (epi_tid == 0) {
          if (p.has_aux) tma_wait_read<0>(); else tma_wait_read<1>();
        }
        epi_bar_sync();
        uint8_t* stage_main = p.has_aux ? out_buf[0] : out_buf[flip];
        uint8_t* stage_aux = out_buf[1];
#pragma unroll 1
        for (int half = 0; half < boxes_per_store; ++half) {
          uint32_t r[32];
          tc_ld32(t_addr + (uint32_t)(c0 + half * COLS_PER_BOX), r);
          tc_wait_ld();
          float v[32];
          const int gcol0 = n_tile * BLOCK_N + c0 + half * COLS_PER_BOX;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = __uint_as_float(r[j]) * p.alpha;
            if (p.epi != EPI_NONE && bias != nullptr && gcol0 + j < p.N) v[j] += __ldg(bias + gcol0 + j);
          }
          if (p.out_f32) {
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
              float4 o = make_float4(v[4 * ch], v[4 * ch + 1], v[4 * ch + 2], v[4 * ch + 3]);
              if (p.epi == EPI_BIAS_GELU) { o.x = hm_gelu_tanh(o.x); o.y = hm_gelu_tanh(o.y); o.z = hm_gelu_tanh(o.z); o.w = hm_gelu_tanh(o.w); }
              *reinterpret_cast<float4*>(stage_main + row * ROW_BYTES + ((ch ^ (row & 7)) << 4)) = o;
            }
          } else {
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              const int pc = (half * 4 + ch) ^ (row & 7);
              if (p.has_aux) {
                uint4 a;
                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * ch], v[8 * ch + 1]), h1 = __floats2bfloat162_rn(v[8 * ch + 2], v[8 * ch + 3]);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * ch + 4], v[8 * ch + 5]), h3 = __floats2bfloat162_rn(v[8 * ch + 6], v[8 * ch + 7]);
                a.x = *reinterpret_cast<uint32_t*>(&h0); a.y = *reinterpret_cast<uint32_t*>(&h1);
                a.z = *reinterpret_cast<uint32_t*>(&h2); a.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(stage_aux + row * ROW_BYTES + (pc << 4)) = a;
              }
              float w[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) w[j] = p.epi == EPI_BIAS_GELU ? hm_gelu_tanh(v[8 * ch + j]) : v[8 * ch + j];
              uint4 o;
              __nv_bfloat162 h0 = __floats2bfloat162_rn(w[0], w[1]), h1 = __floats2bfloat162_rn(w[2], w[3]);
              __nv_bfloat162 h2 = __floats2bfloat162_rn(w[4], w[5]), h3 = __floats2bfloat162_rn(w[6], w[7]);
              o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
              o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
              *reinterpret_cast<uint4*>(stage_main + row * ROW_BYTES + (pc << 4)) = o;
            }
          }
        }
        fence_proxy_async_smem();
        epi_bar_sync();
        if (epi_tid == 0) {
          const int gc = n_tile * BLOCK_N + c0, gr = m_tile_row;
          if (p.reduce_add) tma_reduce_add_2d(&map_d, smem_u32(stage_main), gc, gr);
          else tma_store_2d(&map_d, smem_u32(stage_main), gc, gr);
          if (p.has_aux) tma_store_2d(&map_aux, smem_u32(stage_aux), gc, gr);
          tma_commit();
        }
        flip ^= 1;
      }
      // hand this CTA's half of the accumulator buffer back to the leader's MMA warp
      tc_fence_before();
      if (leader) mbar_arrive(tempty_bar(buf));
      else mbar_arrive_remote(map_to_cta(tempty_bar(buf), 0));
      ++local;
    }
    if (epi_tid == 0) tma_wait_all<0>();
  }

  // ------------------------------------------------------------------ teardown (every thread of both CTAs gets here)
  if (failed) {
    *abort_flag = 1;
    if (p.err) atomicExch(p.err, 1 + warp);
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  cluster_sync_all();  // neither CTA leaves, or frees tensor memory, while the other may still use it
  if (warp == 1) {
    tc_fence_after();
    tc_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
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

// A tensor map is a pure function of (address, element type, extents, pitch, box, swizzle), and a training step asks
// for the same few dozen combinations over and over (weights, activations and gradients keep their addresses in the
// caching allocator), so encoded maps are kept and looked up instead of being encoded by the driver for every launch.
struct MapKey {
  const void* base;
  long long rows, cols, ld;
  int elem_bytes, box_cols, box_rows, flags;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && elem_bytes == o.elem_bytes &&
           box_cols == o.box_cols && box_rows == o.box_rows && flags == o.flags;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    unsigned long long h = 1469598103934665603ull;
    auto mix = [&h](unsigned long long v) { h = (h ^ v) * 1099511628211ull; };
    mix((unsigned long long)reinterpret_cast<uintptr_t>(k.base));
    mix((unsigned long long)k.rows); mix((unsigned long long)k.cols); mix((unsigned long long)k.ld);
    mix(((unsigned long long)(unsigned)k.elem_bytes << 32) | (unsigned)k.box_cols);
    mix(((unsigned long long)(unsigned)k.box_rows << 32) | (unsigned)k.flags);
    return (size_t)h;
  }
};
constexpr size_t MAX_CACHED_MAPS = 8192;
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;

// 2-D map over a row-major matrix [rows][cols] with leading dimension ld (elements); box = box_cols x box_rows.
int make_map(CUtensorMap* map, const void* base, int elem_bytes, bool is_f32, long long rows, long long cols,
             long long ld, int box_cols, int box_rows, bool atom32 = false) {
  const MapKey key{base, rows, cols, ld, elem_bytes, box_cols, box_rows, (is_f32 ? 1 : 0) | (atom32 ? 2 : 0)};
  static const bool use_cache = [] {  // HIVEMIND_B200_MAP_CACHE=0 encodes every map afresh (for comparison)
    const char* v = std::getenv("HIVEMIND_B200_MAP_CACHE");
    return !(v && v[0] == '0');
  }();
  if (use_cache) {
    std::lock_guard<std::mutex> guard(g_map_mutex);
    auto hit = g_map_cache.find(key);
    if (hit != g_map_cache.end()) { *map = hit->second; return 0; }
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -10;
  ensure_context_on_this_thread();
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * elem_bytes) % 16 != 0) return -11;
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)(ld * elem_bytes)};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, is_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -12;
  if (!use_cache) return 0;
  std::lock_guard<std::mutex> guard(g_map_mutex);
  if (g_map_cache.size() >= MAX_CACHED_MAPS) g_map_cache.clear();
  g_map_cache.emplace(key, *map);
  return 0;
}

struct GemmCall {
  const void *a, *b;
  void *d, *aux;
  const float* bias;
  int M, N, K;
  long long lda, ldb, ldd, ldaux;
  int a_mn, b_mn, tf32, out_f32, epi, reduce_add, splits;
  float alpha;
  int* err;
  int sms;
  int group_mode = 0, num_groups = 1;
  const int* group_table = nullptr;
  const void* add = nullptr;
  long long ldadd = 0;
  int add_mode = 0;
};

template <int BLOCK_N, int STAGES, bool TF32, bool A_MN, bool B_MN, bool ADD = false>
int launch(const GemmCall& c, cudaStream_t stream) {
  using L = SmemLayout<BLOCK_N, STAGES>;
  constexpr int ELEM = TF32 ? 4 : 2;
  constexpr int BLOCK_K = ROW_BYTES / ELEM;
  constexpr int RUN = ROW_BYTES / ELEM;
  CUtensorMap ma, mb, md, maux;
  int rc;
  // A: K-major -> matrix [M][K], box BLOCK_K x BLOCK_M. MN-major -> matrix [K][M], box RUN x BLOCK_K.
  rc = A_MN ? make_map(&ma, c.a, ELEM, TF32, c.K, c.M, c.lda, RUN, BLOCK_K, TF32)
            : make_map(&ma, c.a, ELEM, TF32, c.M, c.K, c.lda, BLOCK_K, BLOCK_M);
  if (rc) return rc;
  // grouped mode 1 stacks the groups' B matrices along B's row coordinate; mode 2 stacks the outputs along D's rows
  const long long b_groups = c.group_mode == 1 ? c.num_groups : 1, d_groups = c.group_mode == 2 ? c.num_groups : 1;
  if (c.group_mode == 2 && (!A_MN || !B_MN || (c.num_groups > 1 && c.M % BLOCK_M != 0) || c.aux)) return -17;
  if (c.group_mode == 1 && c.splits > 1) return -17;
  rc = B_MN ? make_map(&mb, c.b, ELEM, TF32, c.K * b_groups, c.N, c.ldb, RUN, BLOCK_K, TF32)
            : make_map(&mb, c.b, ELEM, TF32, c.N * b_groups, c.K, c.ldb, BLOCK_K, BLOCK_N);
  if (rc) return rc;
  const int out_elem = c.out_f32 ? 4 : 2;
  rc = make_map(&md, c.d, out_elem, c.out_f32 != 0, c.M * d_groups, c.N, c.ldd, ROW_BYTES / out_elem, BLOCK_M);
  if (rc) return rc;
  if (c.aux) {
    rc = make_map(&maux, c.aux, 2, false, c.M, c.N, c.ldaux, ROW_BYTES / 2, BLOCK_M);
    if (rc) return rc;
  } else {
    maux = md;
  }
  GemmParams p;
  p.M = c.M; p.N = c.N; p.K = c.K;
  p.num_m_tiles = (c.M + BLOCK_M - 1) / BLOCK_M;
  p.num_n_tiles = (c.N + BLOCK_N - 1) / BLOCK_N;
  p.total_kblocks = (c.K + BLOCK_K - 1) / BLOCK_K;
  int splits = c.splits < 1 ? 1 : c.splits;
  if (splits > p.total_kblocks) splits = p.total_kblocks;
  p.kblocks_per_split = (p.total_kblocks + splits - 1) / splits;
  p.num_splits = (p.total_kblocks + p.kblocks_per_split - 1) / p.kblocks_per_split;
  if (p.num_splits > 1 && !c.reduce_add) return -13;
  p.epi = c.epi; p.out_f32 = c.out_f32; p.reduce_add = c.reduce_add; p.has_aux = c.aux != nullptr;
  p.bias = c.bias; p.alpha = c.alpha; p.err = c.err;
  p.add = (const __nv_bfloat16*)c.add; p.ld_add = c.ldadd; p.add_mode = c.add_mode;
  p.group_mode = c.group_mode; p.num_groups = c.num_groups; p.group_table = c.group_table;
  p.group_b_rows = B_MN ? c.K : c.N; p.group_d_rows = c.M; p.group_bias = c.N;
  if (c.group_mode == 2) { p.num_splits = 1; p.kblocks_per_split = p.total_kblocks; }
  const int tiles = p.num_m_tiles * p.num_n_tiles * (c.group_mode == 2 ? c.num_groups : p.num_splits);
  if (tiles <= 0 || p.total_kblocks <= 0) return 0;
  const int grid = tiles < c.sms ? tiles : c.sms;
  auto kern = tc_gemm_kernel<BLOCK_N, STAGES, TF32, A_MN, B_MN, ADD>;
  const int smem = L::TOTAL + 1024;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  kern<<<grid, NUM_THREADS, smem, stream>>>(ma, mb, md, maux, p);
  return (int)cudaGetLastError();
}


template <int STAGES, bool A_MN, bool B_MN>
int launch_pair(const GemmCall& c, cudaStream_t stream) {
  using L = PairSmem<STAGES>;
  constexpr int ELEM = 2;
  constexpr int BLOCK_K = ROW_BYTES / ELEM;
  constexpr int RUN = ROW_BYTES / ELEM;
  CUtensorMap ma, mb, md, maux;
  int rc;
  rc = A_MN ? make_map(&ma, c.a, ELEM, false, c.K, c.M, c.lda, RUN, BLOCK_K)
            : make_map(&ma, c.a, ELEM, false, c.M, c.K, c.lda, BLOCK_K, BLOCK_M);
  if (rc) return rc;
  rc = B_MN ? make_map(&mb, c.b, ELEM, false, c.K, c.N, c.ldb, RUN, BLOCK_K)
            : make_map(&mb, c.b, ELEM, false, c.N, c.K, c.ldb, BLOCK_K, PAIR_BN);
  if (rc) return rc;
  const int out_elem = c.out_f32 ? 4 : 2;
  if (c.group_mode != 0 && c.group_mode != 2) return -17;
  if (c.group_mode == 2 && (!A_MN || !B_MN || c.aux || (c.num_groups > 1 && c.M % PAIR_M != 0))) return -17;
  const long long d_groups = c.group_mode == 2 ? c.num_groups : 1;
  rc = make_map(&md, c.d, out_elem, c.out_f32 != 0, c.M * d_groups, c.N, c.ldd, ROW_BYTES / out_elem, BLOCK_M);
  if (rc) return rc;
  if (c.aux) {
    rc = make_map(&maux, c.aux, 2, false, c.M, c.N, c.ldaux, ROW_BYTES / 2, BLOCK_M);
    if (rc) return rc;
  } else {
    maux = md;
  }
  GemmParams p;
  p.M = c.M; p.N = c.N; p.K = c.K;
  p.num_m_tiles = (c.M + PAIR_M - 1) / PAIR_M;
  p.num_n_tiles = (c.N + PAIR_N - 1) / PAIR_N;
  p.total_kblocks = (c.K + BLOCK_K - 1) / BLOCK_K;
  int splits = c.splits < 1 ? 1 : c.splits;
  if (splits > p.total_kblocks) splits = p.total_kblocks;
  p.kblocks_per_split = (p.total_kblocks + splits - 1) / splits;
  p.num_splits = (p.total_kblocks + p.kblocks_per_split - 1) / p.kblocks_per_split;
  if (p.num_splits > 1 && !c.reduce_add) return -13;
  p.epi = c.epi; p.out_f32 = c.out_f32; p.reduce_add = c.reduce_add; p.has_aux = c.aux != nullptr;
  p.bias = c.bias; p.alpha = c.alpha; p.err = c.err;
  p.add = (const __nv_bfloat16*)c.add; p.ld_add = c.ldadd; p.add_mode = c.add_mode;
  p.group_mode = c.group_mode; p.num_groups = c.num_groups; p.group_table = c.group_table;
  p.group_b_rows = 0; p.group_d_rows = c.M; p.group_bias = 0;
  if (c.group_mode == 2) { p.num_splits = 1; p.kblocks_per_split = p.total_kblocks; }
  const int tiles = p.num_m_tiles * p.num_n_tiles * (c.group_mode == 2 ? c.num_groups : p.num_splits);
  if (tiles <= 0 || p.total_kblocks <= 0) return 0;
  auto kern = tc_gemm_pair_kernel<STAGES, A_MN, B_MN>;
  const int smem = L::TOTAL + 1024;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // how many CTA pairs can be resident at once (SM counts per GPC need not be even)
  cfg.gridDim = dim3(2 * (c.sms / 2));
  int max_clusters = 0;
  e = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
  if (e != cudaSuccess) return (int)e;
  if (max_clusters < 1) return -18;
  int pairs = tiles < max_clusters ? tiles : max_clusters;
  cfg.gridDim = dim3(2 * pairs);
  e = cudaLaunchKernelEx(&cfg, kern, ma, mb, md, maux, p);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

template <int BLOCK_N, int STAGES, bool TF32>
int dispatch_major(const GemmCall& c, cudaStream_t s) {
  if (c.a_mn) return c.b_mn ? launch<BLOCK_N, STAGES, TF32, true, true>(c, s) : launch<BLOCK_N, STAGES, TF32, true, false>(c, s);
  return c.b_mn ? launch<BLOCK_N, STAGES, TF32, false, true>(c, s) : launch<BLOCK_N, STAGES, TF32, false, false>(c, s);
}

}  // namespace

// D = epilogue(alpha * A B^T) on tensor cores. Returns 0, a CUDA error (> 0) or a negative argument error.
//   a_mn / b_mn : 0 = operand stored [rows][K] (K contiguous), 1 = stored [K][rows] (rows contiguous)
//   tf32        : operands are fp32 and multiplied as tf32; otherwise bf16
//   out_f32     : D is fp32 (required for reduce_add); otherwise bf16
//   epi         : 0 none, 1 + bias[N], 2 gelu_tanh(. + bias[N]); aux (bf16, optional) receives the pre-GELU values
//   reduce_add  : D += result through TMA reduce-add (D must be fp32); needed when splits > 1
//   block_n     : 256, 128, 64 or 32 (N tile); err: device int set non-zero if a bounded wait ran out
HM_API int hm_tc_gemm(const void* a, const void* b, void* d, void* aux, const void* bias, int M, int N, int K,
                      long long lda, long long ldb, long long ldd, long long ldaux, int a_mn, int b_mn, int tf32,
                      int out_f32, int epi, int reduce_add, int splits, float alpha, int block_n, void* err, int sms,
                      cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (reduce_add && !out_f32) return -14;
  if (aux && out_f32) return -15;
  GemmCall c{a, b, d, aux, (const float*)bias, M, N, K, lda, ldb, ldd, ldaux, a_mn, b_mn, tf32, out_f32, epi,
             reduce_add, splits, alpha, (int*)err, sms};
  if (tf32) {
    switch (block_n) {
      case 128: return dispatch_major<128, 4, true>(c, stream);
      case 64: return dispatch_major<64, 6, true>(c, stream);
      case 32: return dispatch_major<32, 8, true>(c, stream);
      default: return -16;
    }
  }
  switch (block_n) {
    case 256: return (aux && !a_mn && !b_mn) ? launch<256, 3, false, false, false>(c, stream)
                                             : dispatch_major<256, 4, false>(c, stream);
    case 128: return dispatch_major<128, 6, false>(c, stream);
    case 64: return dispatch_major<64, 8, false>(c, stream);
    default: return -16;
  }
}

// hm_tc_gemm for bf16 operands and a bf16 result with a second input in the epilogue: `add` is a bf16 [M][N] matrix
// with row stride ldadd (elements; rows 16-byte aligned).
//   add_mode 0: D = alpha * A B^T (+ bias) + add       (input-gradient GEMM of a layer whose input also feeds a
//                                                       residual connection: the two gradients meet in the epilogue)
//   add_mode 1: D = (alpha * A B^T) * gelu_tanh'(add)  (input-gradient GEMM behind a GELU: `add` holds the
//                                                       pre-activation values)
HM_API int hm_tc_gemm_add(const void* a, const void* b, void* d, const void* add, const void* bias, int M, int N, int K,
                          long long lda, long long ldb, long long ldd, long long ldadd, int a_mn, int b_mn, int epi,
                          int add_mode, float alpha, int block_n, void* err, int sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (epi == EPI_BIAS_GELU || (ldadd % 8) != 0 || (N % 8) != 0) return -18;
  GemmCall c{a, b, d, nullptr, (const float*)bias, M, N, K, lda, ldb, ldd, 0, a_mn, b_mn, 0, 0, epi, 0, 1, alpha, (int*)err, sms};
  c.add = add;
  c.ldadd = ldadd;
  c.add_mode = add_mode;
  if (a_mn) return -18;   // the variants with a second epilogue input exist for row-major A (activations or their gradients)
  switch (block_n) {
    case 256: return b_mn ? launch<256, 4, false, false, true, true>(c, stream) : launch<256, 4, false, false, false, true>(c, stream);
    case 128: return b_mn ? launch<128, 6, false, false, true, true>(c, stream) : launch<128, 6, false, false, false, true>(c, stream);
    case 64: return b_mn ? launch<64, 8, false, false, true, true>(c, stream) : launch<64, 8, false, false, false, true>(c, stream);
    default: return -16;
  }
}

// Grouped variants of hm_tc_gemm for bf16 operands (see GemmParams for the two modes). `group_table` is a device
// array: mode 1 -> int[ceil(M / 128)] group of every M tile (-1 = skip; M is the padded row count of A and D, B is
// the stack of num_groups matrices of N x K, bias the stack of num_groups vectors of N); mode 2 -> int[num_groups + 1]
// row offsets (multiples of 64) into the shared K extent of the MN-major operands A [K][M] and B [K][N], D is the
// stack of num_groups outputs of M x N (M a multiple of 128).
HM_API int hm_tc_gemm_grouped(const void* a, const void* b, void* d, void* aux, const void* bias, int M, int N, int K,
                              long long lda, long long ldb, long long ldd, long long ldaux, int a_mn, int b_mn,
                              int out_f32, int epi, int reduce_add, float alpha, int block_n, void* err, int sms,
                              int group_mode, int num_groups, const int* group_table, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || num_groups <= 0) return 0;
  if (group_mode != 1 && group_mode != 2) return -17;
  if (group_table == nullptr) return -17;
  if (reduce_add && !out_f32) return -14;
  if (aux && out_f32) return -15;
  GemmCall c{a, b, d, aux, (const float*)bias, M, N, K, lda, ldb, ldd, ldaux, a_mn, b_mn, 0, out_f32, epi,
             reduce_add, 1, alpha, (int*)err, sms};
  c.group_mode = group_mode;
  c.num_groups = num_groups;
  c.group_table = group_table;
  switch (block_n) {
    case 256: return dispatch_major<256, 4, false>(c, stream);
    case 128: return dispatch_major<128, 6, false>(c, stream);
    case 64: return dispatch_major<64, 8, false>(c, stream);
    default: return -16;
  }
}

// hm_tc_gemm_grouped for fp32 operands multiplied as tf32 (the low-rank products of PowerSGD over many matrices of
// one shape in one launch). Same group modes and tables; K ranges of mode 2 are multiples of 32; block_n is 128, 64
// or 32; D is fp32.
HM_API int hm_tc_gemm_grouped_tf32(const void* a, const void* b, void* d, int M, int N, int K, long long lda,
                                   long long ldb, long long ldd, int a_mn, int b_mn, int reduce_add, float alpha,
                                   int block_n, void* err, int sms, int group_mode, int num_groups,
                                   const int* group_table, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || num_groups <= 0) return 0;
  if ((group_mode != 1 && group_mode != 2) || group_table == nullptr) return -17;
  GemmCall c{a, b, d, nullptr, nullptr, M, N, K, lda, ldb, ldd, 0, a_mn, b_mn, 1, 1, EPI_NONE, reduce_add, 1, alpha,
             (int*)err, sms};
  c.group_mode = group_mode;
  c.num_groups = num_groups;
  c.group_table = group_table;
  switch (block_n) {
    case 128: return dispatch_major<128, 4, true>(c, stream);
    case 64: return dispatch_major<64, 6, true>(c, stream);
    case 32: return dispatch_major<32, 8, true>(c, stream);
    default: return -16;
  }
}

// Two-CTA (cta_group::2) variant of hm_tc_gemm for bf16 operands: one 256x256 tile per pair of SMs.
// Same arguments as hm_tc_gemm without `tf32` and `block_n`. Requirements: N and M arbitrary (edges are clipped by
// TMA), the usual 16-byte alignment of leading dimensions.
HM_API int hm_tc_gemm_pair(const void* a, const void* b, void* d, void* aux, const void* bias, int M, int N, int K,
                           long long lda, long long ldb, long long ldd, long long ldaux, int a_mn, int b_mn,
                           int out_f32, int epi, int reduce_add, int splits, float alpha, void* err, int sms,
                           cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (reduce_add && !out_f32) return -14;
  if (aux && out_f32) return -15;
  GemmCall c{a, b, d, aux, (const float*)bias, M, N, K, lda, ldb, ldd, ldaux, a_mn, b_mn, 0, out_f32, epi,
             reduce_add, splits, alpha, (int*)err, sms};
  if (a_mn) return b_mn ? launch_pair<5, true, true>(c, stream) : launch_pair<5, true, false>(c, stream);
  return b_mn ? launch_pair<5, false, true>(c, stream) : launch_pair<5, false, false>(c, stream);
}

// Two-CTA variant of grouped mode 2 (per-group K ranges over MN-major operands; see hm_tc_gemm_grouped): the
// weight-gradient products of many experts in one launch. M must be a multiple of 256 when there are several groups.
HM_API int hm_tc_gemm_pair_grouped_k(const void* a, const void* b, void* d, int M, int N, int K, long long lda,
                                     long long ldb, long long ldd, int out_f32, int reduce_add, float alpha, void* err,
                                     int sms, int num_groups, const int* group_table, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || num_groups <= 0) return 0;
  if (group_table == nullptr) return -17;
  if (reduce_add && !out_f32) return -14;
  GemmCall c{a, b, d, nullptr, nullptr, M, N, K, lda, ldb, ldd, 0, 1, 1, 0, out_f32, EPI_NONE, reduce_add, 1, alpha,
             (int*)err, sms};
  c.group_mode = 2;
  c.num_groups = num_groups;
  c.group_table = group_table;
  return launch_pair<5, true, true>(c, stream);
}
