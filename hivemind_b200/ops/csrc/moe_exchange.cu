// Expert-parallel exchange over peer-mapped memory (NVLink): the all-to-all of mixture-of-experts dispatch and
// combine without a collective library. Every rank is a client (it owns token rows sorted by global expert) and a
// server (it hosts `experts_per_rank` experts). Ranks only ever WRITE their own arena; they PULL what they need from
// the arenas of their peers with plain loads:
//
//   client r:  publish rows + per-expert offsets, raise flag          (hm_mx_publish)
//   server d:  wait for every client's flag, read the counts that concern its experts, lay the rows out by
//              (expert, client) with every expert padded to whole 128-row tiles                (hm_mx_layout)
//              pull the rows from the clients' arenas                                           (hm_mx_gather)
//              run the grouped expert FFN on them (tc_gemm.cu grouped modes), raise flag        (hm_mx_publish)
//   client r:  wait for every server's flag, pull the answers for its rows back                 (hm_mx_pull)
//
// The backward pass runs the same three steps with output gradients in place of rows and input gradients in place
// of answers, reusing the layout of the forward pass. This replaces the per-row RPC fan-out of the reference
// (hivemind/moe/client/moe.py:227-243) and the server's re-batching (hivemind/moe/server/task_pool.py:161-192).
//
// Every wait on a peer's flag is bounded by `timeout_ns` on this GPU's globaltimer. A server that gives up on a
// client treats it as having sent no rows; a client that gives up on a server gets zero answers and ok[row] = 0 for
// those rows, which the combine step treats like an expert that did not respond. The server publishes the length of
// every (expert, client) segment next to its first row, so a client whose rows the server did not take (it gave up
// on that client's flag, or ran out of room) finds a shorter segment than it sent and marks the missing rows ok = 0
// instead of reading somebody else's answers.
#include "hm_common.cuh"

#define MX_MAX_RANKS 16
#define MX_TILE 128

struct HmMxPeers {
  int n_ranks, me, experts_per_rank, hidden_bytes;  // hidden_bytes: bytes per row (multiple of 16)
  unsigned long long timeout_ns;
  unsigned char* rows[MX_MAX_RANKS];        // client buffer of every rank (this phase): [cap_send][hidden]
  const int* offsets[MX_MAX_RANKS];         // client row offsets by global expert: int[E + 1]
  unsigned char* answers[MX_MAX_RANKS];     // server buffer of every rank (this phase): [cap_recv][hidden]
  const int* base_table[MX_MAX_RANKS];      // server layout of every rank: int[2][experts_per_rank][n_ranks]: first row of
                                            // every (expert, client) segment, then the segment's length
  const unsigned int* rows_flag[MX_MAX_RANKS];
  const unsigned int* answers_flag[MX_MAX_RANKS];
  int capacity;                             // rows of every answers buffer
};

// Bounded wait for *flag == want by one thread; returns false on timeout.
__device__ bool mx_wait(const unsigned int* flag, unsigned int want, unsigned long long deadline) {
  while (hm_ld_acquire_sys(flag) != want) {
    if (hm_globaltimer_ns() > deadline) return false;
    __nanosleep(200);
  }
  return true;
}

// Raise this rank's flag once everything written before on this stream is visible system-wide.
__global__ void mx_publish_kernel(unsigned int* flag, unsigned int epoch) {
  __threadfence_system();
  hm_st_release_sys(flag, epoch);
}

// Server: one block. Outputs (all in this rank's memory):
//   base_table[e][s]  first row of client s's rows for local expert e in the gathered layout
//   src_start[e][s]   first row of that segment in client s's buffer;  seg_count[e][s] its length
//   offs_pad[e]       padded start of local expert e (offs_pad[E_local] = total padded rows)
//   tile_group[m]     local expert that owns rows 128 m .. 128 m + 127, or -1
//   status[0]         bit s set if client s timed out
__global__ void __launch_bounds__(256) mx_layout_kernel(HmMxPeers p, unsigned int epoch, int* base_table,
                                                        int* src_start, int* seg_count, int* offs_pad,
                                                        int* tile_group, int max_tiles,
                                                        unsigned long long* status) {
  __shared__ int alive[MX_MAX_RANKS];
  const int R = p.n_ranks, EL = p.experts_per_rank;
  if (threadIdx.x < R) {
    const unsigned long long deadline = hm_globaltimer_ns() + p.timeout_ns;
    const bool ok = mx_wait(p.rows_flag[threadIdx.x], epoch, deadline);
    alive[threadIdx.x] = ok;
    if (!ok) atomicOr(status, 1ull << threadIdx.x);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < EL * R; i += blockDim.x) {
    const int e = i / R, s = i % R;
    const int ge = p.me * EL + e;
    int lo = 0, n = 0;
    if (alive[s]) {
      lo = p.offsets[s][ge];
      n = p.offsets[s][ge + 1] - lo;
      if (n < 0) n = 0;
    }
    src_start[i] = lo;
    seg_count[i] = n;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int cursor = 0;
    for (int e = 0; e < EL; ++e) {
      offs_pad[e] = cursor;
      for (int s = 0; s < R; ++s) {
        base_table[e * R + s] = cursor;
        if (cursor + seg_count[e * R + s] > max_tiles * MX_TILE) seg_count[e * R + s] = max(0, max_tiles * MX_TILE - cursor);
        cursor += seg_count[e * R + s];
      }
      cursor = (cursor + MX_TILE - 1) / MX_TILE * MX_TILE;
    }
    offs_pad[EL] = cursor;
  }
  __syncthreads();
  const int total = offs_pad[EL];
  for (int m = threadIdx.x; m < max_tiles; m += blockDim.x) {
    const int row = m * MX_TILE;
    int g = -1;
    if (row < total) {
      int lo = 0, hi = EL;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (offs_pad[mid] <= row) lo = mid; else hi = mid;
      }
      g = lo;
    }
    tile_group[m] = g;
  }
}

// Server: copy every (expert, client) segment from the client's arena into the gathered buffer. The grid is fixed;
// CTAs stride over the rows of each segment; one CTA moves one row per step with 16-byte loads over NVLink.
// Rows beyond `capacity` are dropped (cannot happen when the buffers are sized for the worst case).
__global__ void __launch_bounds__(128) mx_gather_kernel(HmMxPeers p, const int* __restrict__ base_table,
                                                        const int* __restrict__ src_start,
                                                        const int* __restrict__ seg_count,
                                                        unsigned char* __restrict__ gathered, int capacity) {
  const int R = p.n_ranks, EL = p.experts_per_rank;
  const int vec = p.hidden_bytes / 16;
  for (int seg = 0; seg < EL * R; ++seg) {
    const int n = seg_count[seg];
    if (n == 0) continue;
    const int s = seg % R;
    const unsigned char* src = p.rows[s] + (size_t)src_start[seg] * p.hidden_bytes;
    const int dst0 = base_table[seg];
    for (int row = blockIdx.x; row < n; row += gridDim.x) {
      if (dst0 + row >= capacity) break;
      const uint4* a = reinterpret_cast<const uint4*>(src + (size_t)row * p.hidden_bytes);
      uint4* b = reinterpret_cast<uint4*>(gathered + (size_t)(dst0 + row) * p.hidden_bytes);
      for (int i = threadIdx.x; i < vec; i += blockDim.x) b[i] = a[i];
    }
  }
}

// Client: pull the answers of my rows back. My rows are sorted by global expert (my_offsets); the rows of expert ge
// live on rank ge / EL at base_table[ge % EL][me] + (row - my_offsets[ge]).
__global__ void __launch_bounds__(128) mx_pull_kernel(HmMxPeers p, unsigned int epoch, const int* __restrict__ my_offsets,
                                                      int num_experts, unsigned char* __restrict__ out,
                                                      unsigned char* __restrict__ ok, int* __restrict__ server_state,
                                                      unsigned long long* t_start, unsigned long long* status) {
  __shared__ int state_s;
  const int EL = p.experts_per_rank;
  const int vec = p.hidden_bytes / 16;
  const int total = my_offsets[num_experts];
  for (int row = blockIdx.x; row < total; row += gridDim.x) {
    int lo = 0, hi = num_experts;  // last expert with offsets[e] <= row
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (my_offsets[mid] <= row) lo = mid; else hi = mid;
    }
    const int ge = lo, d = ge / EL;
    if (threadIdx.x == 0) {
      // one decision per server for the whole grid: 0 undecided, 1 answered, 2 gave up
      int st = *reinterpret_cast<volatile int*>(server_state + d);
      if (st == 0) {
        unsigned long long t0 = *reinterpret_cast<volatile unsigned long long*>(t_start);
        if (t0 == 0) {
          const unsigned long long now = hm_globaltimer_ns();
          const unsigned long long prev = atomicCAS(t_start, 0ull, now);
          t0 = prev == 0 ? now : prev;
        }
        const bool got = mx_wait(p.answers_flag[d], epoch, t0 + p.timeout_ns);
        atomicCAS(server_state + d, 0, got ? 1 : 2);
        st = *reinterpret_cast<volatile int*>(server_state + d);
        if (st == 2) atomicOr(status, 1ull << d);
      }
      state_s = st;
    }
    __syncthreads();
    const int st = state_s;
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * p.hidden_bytes);
    bool served = st == 1;
    int remote_row = 0;
    if (served) {
      const int seg = (ge % EL) * p.n_ranks + p.me, local = row - my_offsets[ge];
      const int* table = p.base_table[d];
      remote_row = table[seg] + local;
      served = local < table[EL * p.n_ranks + seg] && remote_row < p.capacity;   // did the server take this row?
    }
    if (served) {
      const uint4* src = reinterpret_cast<const uint4*>(p.answers[d] + (size_t)remote_row * p.hidden_bytes);
      for (int i = threadIdx.x; i < vec; i += blockDim.x) dst[i] = src[i];
    } else {
      for (int i = threadIdx.x; i < vec; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    }
    if (threadIdx.x == 0 && ok != nullptr) ok[row] = served;
    __syncthreads();
  }
}

HM_API int hm_mx_peers_size() { return (int)sizeof(HmMxPeers); }

HM_API int hm_mx_publish(unsigned int* flag, unsigned int epoch, cudaStream_t stream) {
  mx_publish_kernel<<<1, 1, 0, stream>>>(flag, epoch);
  return (int)cudaGetLastError();
}

// `peers` is a host copy of HmMxPeers (passed by value to the kernels). scratch ints: base_table[EL*R],
// src_start[EL*R], seg_count[EL*R], offs_pad[EL+1], tile_group[max_tiles]; status: 1 zeroed unsigned long long.
HM_API int hm_mx_layout(const void* peers, unsigned int epoch, int* base_table, int* src_start, int* seg_count,
                        int* offs_pad, int* tile_group, int max_tiles, unsigned long long* status,
                        cudaStream_t stream) {
  const HmMxPeers* p = (const HmMxPeers*)peers;
  if (p->n_ranks < 1 || p->n_ranks > MX_MAX_RANKS || p->hidden_bytes % 16 != 0) return -10;
  mx_layout_kernel<<<1, 256, 0, stream>>>(*p, epoch, base_table, src_start, seg_count, offs_pad, tile_group, max_tiles,
                                          status);
  return (int)cudaGetLastError();
}

HM_API int hm_mx_gather(const void* peers, const int* base_table, const int* src_start, const int* seg_count,
                        void* gathered, int capacity, int ctas, cudaStream_t stream) {
  const HmMxPeers* p = (const HmMxPeers*)peers;
  if (p->n_ranks < 1 || p->n_ranks > MX_MAX_RANKS || p->hidden_bytes % 16 != 0 || ctas < 1) return -10;
  mx_gather_kernel<<<ctas, 128, 0, stream>>>(*p, base_table, src_start, seg_count, (unsigned char*)gathered, capacity);
  return (int)cudaGetLastError();
}

// server_state: int[n_ranks] zeroed; t_start: 1 zeroed unsigned long long; status: 1 zeroed unsigned long long.
HM_API int hm_mx_pull(const void* peers, unsigned int epoch, const int* my_offsets, int num_experts, void* out,
                      unsigned char* ok, int* server_state, unsigned long long* t_start, unsigned long long* status,
                      int ctas, cudaStream_t stream) {
  const HmMxPeers* p = (const HmMxPeers*)peers;
  if (p->n_ranks < 1 || p->n_ranks > MX_MAX_RANKS || p->hidden_bytes % 16 != 0 || ctas < 1) return -10;
  mx_pull_kernel<<<ctas, 128, 0, stream>>>(*p, epoch, my_offsets, num_experts, (unsigned char*)out, ok, server_state,
                                           t_start, status);
  return (int)cudaGetLastError();
}
