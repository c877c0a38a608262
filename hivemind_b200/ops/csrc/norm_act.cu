// LayerNorm (with optional fused residual add) and bias + tanh-GELU, forward and backward.
//
// Shapes: x, y, residual are [rows, H] row-major in bf16 or fp32; gamma, beta, bias are fp32.
// One warp owns one row at a time; a lane keeps its slice of the row in registers, so the row is read
// from HBM exactly once in the forward pass and the statistics are exact two-pass (mean, then variance).
// H must be a multiple of 8 and at most 8 * 32 * HM_LN_MAXV.
//
// Reference call sites replaced: hivemind/moe/server/layers/common.py:11-12 (gelu_fast),
// :26-30 (LayerNorm(x + ffn(x)), eps 1e-12), and the LayerNorm/GELU of the user's transformer
// (examples/albert/run_trainer.py uses transformers' ALBERT).
#include "hm_common.cuh"

#define HM_LN_MAXV 8
#define HM_LN_WARPS 4

template <typename T>
__device__ __forceinline__ void ld8(const T* p, float v[8]);
template <>
__device__ __forceinline__ void ld8<float>(const float* p, float v[8]) {
  float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void ld8<__nv_bfloat16>(const __nv_bfloat16* p, float v[8]) {
  uint4 r = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    v[2 * k] = __low2float(h[k]);
    v[2 * k + 1] = __high2float(h[k]);
  }
}
template <typename T>
__device__ __forceinline__ void st8(T* p, const float v[8]);
template <>
__device__ __forceinline__ void st8<float>(float* p, const float v[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void st8<__nv_bfloat16>(__nv_bfloat16* p, const float v[8]) {
  uint4 r;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
  *reinterpret_cast<uint4*>(p) = r;
}

// y = LN(x + residual) * gamma + beta ; optionally stores z = x + residual (needed by backward when a
// residual is given), and per-row mean / rstd.
template <typename T, int NV>
__global__ void __launch_bounds__(32 * HM_LN_WARPS)
ln_fwd_kernel(const T* __restrict__ x, const T* __restrict__ residual, const float* __restrict__ gamma,
              const float* __restrict__ beta, T* __restrict__ y, T* __restrict__ z, float* __restrict__ mean_out,
              float* __restrict__ rstd_out, int rows, int H, float eps,
              const int* __restrict__ tile_group = nullptr) {
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * HM_LN_WARPS + (threadIdx.x >> 5);
  const int warps_total = gridDim.x * HM_LN_WARPS;
  const float inv_h = 1.f / (float)H;
  const float* gamma0 = gamma;
  const float* beta0 = beta;
  for (int row = warp_global; row < rows; row += warps_total) {
    if (tile_group != nullptr) {  // grouped: every 128-row tile has its own gamma / beta; tiles of group -1 are skipped
      const int g = __ldg(tile_group + (row >> 7));
      if (g < 0) continue;
      gamma = gamma0 + (size_t)g * H;
      beta = beta0 + (size_t)g * H;
    }
    const size_t base = (size_t)row * H;
    float v[NV][8];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int col = (j * 32 + lane) * 8;
      if (col < H) {
        ld8<T>(x + base + col, v[j]);
        if (residual) {
          float r[8];
          ld8<T>(residual + base + col, r);
#pragma unroll
          for (int k = 0; k < 8; ++k) v[j][k] += r[k];
          if (z) st8<T>(z + base + col, v[j]);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) s += v[j][k];
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[j][k] = 0.f;
      }
    }
    const float mean = hm_warp_sum(s) * inv_h;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int col = (j * 32 + lane) * 8;
      if (col < H) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float d = v[j][k] - mean;
          q = fmaf(d, d, q);
        }
      }
    }
    const float rstd = rsqrtf(hm_warp_sum(q) * inv_h + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int col = (j * 32 + lane) * 8;
      if (col < H) {
        float g[8], b[8], o[8];
        ld8<float>(gamma + col, g);
        ld8<float>(beta + col, b);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = fmaf((v[j][k] - mean) * rstd, g[k], b[k]);
        st8<T>(y + base + col, o);
      }
    }
  }
}

// Backward: dx = rstd * (g*dy - mean(g*dy) - xhat * mean(g*dy*xhat)); dgamma += sum dy*xhat; dbeta += sum dy.
// `zin` is the normalised input (x, or x + residual). dgamma/dbeta are fp32 buffers zeroed by the caller;
// each CTA adds its partial sums with atomics once at the end.
template <typename T, int NV>
__global__ void __launch_bounds__(32 * HM_LN_WARPS)
ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ zin, const float* __restrict__ gamma,
              const float* __restrict__ mean_in, const float* __restrict__ rstd_in, T* __restrict__ dx,
              float* __restrict__ dgamma, float* __restrict__ dbeta, int rows, int H) {
  __shared__ float sg[HM_LN_WARPS][32 * 8 + 8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warp_global = blockIdx.x * HM_LN_WARPS + warp;
  const int warps_total = gridDim.x * HM_LN_WARPS;
  const float inv_h = 1.f / (float)H;
  float ag[NV][8], ab[NV][8];
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int k = 0; k < 8; ++k) ag[j][k] = ab[j][k] = 0.f;

  for (int row = warp_global; row < rows; row += warps_total) {
    const size_t base = (size_t)row * H;
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[NV][8], gd[NV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int col = (j * 32 + lane) * 8;
      if (col < H) {
        float d[8], g[8];
        ld8<T>(dy + base + col, d);
        ld8<T>(zin + base + col, xh[j]);
        ld8<float>(gamma + col, g);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          xh[j][k] = (xh[j][k] - mean) * rstd;
          ag[j][k] = fmaf(d[k], xh[j][k], ag[j][k]);
          ab[j][k] += d[k];
          gd[j][k] = d[k] * g[k];
          s1 += gd[j][k];
          s2 = fmaf(gd[j][k], xh[j][k], s2);
        }
      }
    }
    s1 = hm_warp_sum(s1) * inv_h;
    s2 = hm_warp_sum(s2) * inv_h;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int col = (j * 32 + lane) * 8;
      if (col < H) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = rstd * (gd[j][k] - s1 - xh[j][k] * s2);
        st8<T>(dx + base + col, o);
      }
    }
  }
  // reduce the per-warp column sums inside the CTA, then one atomic per column per CTA
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int col = (j * 32 + lane) * 8;
      __syncthreads();
#pragma unroll
      for (int k = 0; k < 8; ++k) sg[warp][lane * 8 + k] = pass == 0 ? ag[j][k] : ab[j][k];
      __syncthreads();
      if (warp == 0 && col < H) {
        float* dst = pass == 0 ? dgamma : dbeta;
        if (dst) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < HM_LN_WARPS; ++w) t += sg[w][lane * 8 + k];
            atomicAdd(dst + col + k, t);
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Split LayerNorm backward (the default path). Keeping the per-column sums of dgamma / dbeta in the registers of a
// warp-per-row kernel costs ~64 registers per thread and leaves only 12 warps per SM, too few to cover HBM latency.
// Here the row pass writes dx only, and the column sums are taken by a second, column-strip pass that re-reads dy
// and the normalised input with 16-byte loads (5 tensor passes over HBM instead of 3, each near the copy rate).
template <typename T, int NV>
__global__ void __launch_bounds__(32 * HM_LN_WARPS)
ln_bwd_dx_kernel(const T* __restrict__ dy, const T* __restrict__ zin, const float* __restrict__ gamma,
                 const float* __restrict__ mean_in, const float* __restrict__ rstd_in, T* __restrict__ dx, int rows,
                 int H) {
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * HM_LN_WARPS + (threadIdx.x >> 5);
  const int warps_total = gridDim.x * HM_LN_WARPS;
  const float inv_h = 1.f / (float)H;
  for (int row = warp_global; row < rows; row += warps_total) {
    const size_t base = (size_t)row * H;
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[NV][8], gd[NV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int col = (j * 32 + lane) * 8;
      if (col < H) {
        ld8<T>(dy + base + col, gd[j]);
        ld8<T>(zin + base + col, xh[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int col = (j * 32 + lane) * 8;
      if (col < H) {
        float g[8];
        ld8<float>(gamma + col, g);  // 4 KB, stays in L1
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          xh[j][k] = (xh[j][k] - mean) * rstd;
          gd[j][k] *= g[k];
          s1 += gd[j][k];
          s2 = fmaf(gd[j][k], xh[j][k], s2);
        }
      }
    }
    s1 = hm_warp_sum(s1) * inv_h;
    s2 = hm_warp_sum(s2) * inv_h;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int col = (j * 32 + lane) * 8;
      if (col < H) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = rstd * (gd[j][k] - s1 - xh[j][k] * s2);
        st8<T>(dx + base + col, o);
      }
    }
  }
}

// Column-strip pass: block = 32 column groups (8 columns each, one 16-byte load per row) x 8 row lanes; blockIdx.y
// selects a strip of rows. MODE 0: dgamma += sum dy * xhat, dbeta += sum dy (LayerNorm). MODE 1: dx = dy * gelu'(x),
// dbias += sum dx (GELU backward; also writes dx).
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
colstrip_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, T* __restrict__ dx, float* __restrict__ out_a,
                float* __restrict__ out_b, long long rows, int H, int rows_per_strip) {
  __shared__ float red[2][8][32 * 8 + 8];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + cx) * 8;
  const long long r0 = (long long)blockIdx.y * rows_per_strip;
  const long long r1 = r0 + rows_per_strip < rows ? r0 + rows_per_strip : rows;
  float a[8], b[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) a[k] = b[k] = 0.f;
  if (col < H) {
    for (long long r = r0 + ry; r < r1; r += 8) {
      const size_t idx = (size_t)r * H + col;
      float d[8], v[8];
      ld8<T>(dy + idx, d);
      ld8<T>(x + idx, v);
      if (MODE == 0) {
        const float mean = mean_in[r], rstd = rstd_in[r];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          a[k] = fmaf(d[k], (v[k] - mean) * rstd, a[k]);
          b[k] += d[k];
        }
      } else {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          o[k] = d[k] * hm_gelu_tanh_grad(v[k]);
          a[k] += o[k];
        }
        st8<T>(dx + idx, o);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    red[0][ry][cx * 8 + k] = a[k];
    if (MODE == 0) red[1][ry][cx * 8 + k] = b[k];
  }
  __syncthreads();
  // 256 threads, 256 columns of this block: one column sum each
  const int c = threadIdx.x;
  const int gcol = blockIdx.x * 256 + c;
  if (gcol < H) {
    float ta = 0.f, tb = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      ta += red[0][w][c];
      if (MODE == 0) tb += red[1][w][c];
    }
    if (out_a) atomicAdd(out_a + gcol, ta);
    if (MODE == 0 && out_b) atomicAdd(out_b + gcol, tb);
  }
}

// ------------------------------------------------------------------------------------------------
// One-pass LayerNorm backward for bf16 rows (the default when the row fits): a CTA streams tiles of R rows of dy and
// of the normalised input into shared memory with asynchronous copies (two tiles in flight), takes the two row sums
// with one warp per row, and then switches to a column view: every thread owns eight columns, writes dx for the
// tile's rows and keeps the column sums of dy * xhat, dy and dx in registers until the CTA has run out of tiles.
// HBM sees dy and the input once and dx once; dxsum (optional) is the bias gradient of the layer whose output was
// normalised.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int R>
__global__ void __launch_bounds__(256)
ln_bwd_tile_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ zin,
                   const float* __restrict__ gamma, const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dgamma, float* __restrict__ dbeta,
                   float* __restrict__ dxsum, int rows, int H, int gp_log2) {
  extern __shared__ __align__(16) unsigned char ln_smem[];
  const int G = H >> 3;                        // 16-byte column groups per row
  const int GP = 1 << gp_log2, RP = 256 >> gp_log2;   // threads per row (power of two >= G), rows in flight in the column view
  const size_t tile_bytes = (size_t)R * H * 2;
  float* s_gamma = reinterpret_cast<float*>(ln_smem + 4 * tile_bytes);
  float* s_stat = s_gamma + H;                 // [R][4]: mean, rstd, mean(g dy), mean(g dy xhat)
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cg = tid & (GP - 1), rsub = tid >> gp_log2;
  const int num_tiles = (rows + R - 1) / R;
  const float inv_h = 1.f / (float)H;
  const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(ln_smem);

  auto issue = [&](int tile, int stage) {
    const int row0 = tile * R, nrows = min(R, rows - row0);
    const int vectors = nrows * G;             // the rows of a tile are contiguous in memory
    const char* src_d = reinterpret_cast<const char*>(dy + (size_t)row0 * H);
    const char* src_z = reinterpret_cast<const char*>(zin + (size_t)row0 * H);
    const uint32_t dst = smem_base + (uint32_t)(stage * 2 * tile_bytes);
    for (int v = tid; v < vectors; v += 256) {
      cp_async16(dst + v * 16, src_d + (size_t)v * 16);
      cp_async16(dst + (uint32_t)tile_bytes + v * 16, src_z + (size_t)v * 16);
    }
  };

  for (int i = tid; i < H; i += 256) s_gamma[i] = gamma[i];
  float g8[8], a8[8], b8[8], c8[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    g8[k] = cg < G ? gamma[cg * 8 + k] : 0.f;
    a8[k] = b8[k] = c8[k] = 0.f;
  }
  int tile = blockIdx.x, stage = 0;
  if (tile < num_tiles) issue(tile, 0);
  cp_async_commit();
  for (; tile < num_tiles; tile += gridDim.x, stage ^= 1) {
    const int next = tile + gridDim.x;
    if (next < num_tiles) issue(next, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();                        // everything but the newest group has landed: this tile is here
    __syncthreads();
    const int row0 = tile * R, nrows = min(R, rows - row0);
    const __nv_bfloat16* t_dy = reinterpret_cast<const __nv_bfloat16*>(ln_smem + stage * 2 * tile_bytes);
    const __nv_bfloat16* t_z = reinterpret_cast<const __nv_bfloat16*>(ln_smem + stage * 2 * tile_bytes + tile_bytes);
    // row view: one warp per row
    for (int r = warp; r < nrows; r += 8) {
      const float mean = mean_in[row0 + r], rstd = rstd_in[row0 + r];
      float s1 = 0.f, s2 = 0.f;
      for (int c = lane; c < G; c += 32) {
        float d[8], z[8];
        ld8<__nv_bfloat16>(t_dy + r * H + c * 8, d);
        ld8<__nv_bfloat16>(t_z + r * H + c * 8, z);
        const float4 ga = reinterpret_cast<const float4*>(s_gamma + c * 8)[0], gb = reinterpret_cast<const float4*>(s_gamma + c * 8)[1];
        const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float gd = d[k] * g[k];
          s1 += gd;
          s2 = fmaf(gd, (z[k] - mean) * rstd, s2);
        }
      }
      s1 = hm_warp_sum(s1);
      s2 = hm_warp_sum(s2);
      if (lane == 0) reinterpret_cast<float4*>(s_stat)[r] = make_float4(mean, rstd, s1 * inv_h, s2 * inv_h);
    }
    __syncthreads();
    // column view
    if (cg < G) {
      for (int r = rsub; r < nrows; r += RP) {
        const float4 st = reinterpret_cast<const float4*>(s_stat)[r];
        float d[8], z[8], o[8];
        ld8<__nv_bfloat16>(t_dy + r * H + cg * 8, d);
        ld8<__nv_bfloat16>(t_z + r * H + cg * 8, z);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float xh = (z[k] - st.x) * st.y;
          o[k] = st.y * (d[k] * g8[k] - st.z - xh * st.w);
          a8[k] = fmaf(d[k], xh, a8[k]);
          b8[k] += d[k];
          c8[k] += o[k];
        }
        st8<__nv_bfloat16>(dx + (size_t)(row0 + r) * H + cg * 8, o);
      }
    }
    __syncthreads();                           // the tile may be overwritten by the copy issued in the next iteration
  }
  cp_async_wait<0>();
  __syncthreads();
  // column sums: fold the RP row lanes through shared memory, then one atomic per column and CTA
  float* red = reinterpret_cast<float*>(ln_smem);   // [RP][GP * 8]
#pragma unroll 1
  for (int pass = 0; pass < 3; ++pass) {
    float* dst = pass == 0 ? dgamma : (pass == 1 ? dbeta : dxsum);
    if (dst == nullptr) continue;
#pragma unroll
    for (int k = 0; k < 8; ++k) red[(rsub * GP + cg) * 8 + k] = pass == 0 ? a8[k] : (pass == 1 ? b8[k] : c8[k]);
    __syncthreads();
    for (int col = tid; col < H; col += 256) {
      float t = 0.f;
      for (int rs = 0; rs < RP; ++rs) t += red[rs * GP * 8 + col];
      atomicAdd(dst + col, t);
    }
    __syncthreads();
  }
}

template <typename T>
static int colstrip_grid(long long rows, int H, int sms, dim3* grid, int* rows_per_strip) {
  const int gx = (H + 255) / 256;
  long long gy = ((long long)sms * 4 + gx - 1) / gx;
  if (gy > (rows + 7) / 8) gy = (rows + 7) / 8;
  if (gy < 1) gy = 1;
  *rows_per_strip = (int)((rows + gy - 1) / gy);
  gy = (rows + *rows_per_strip - 1) / *rows_per_strip;
  *grid = dim3(gx, (unsigned)gy);
  return 0;
}

// Grouped backward: rows come in 128-row tiles and tile_group[tile] names the parameter set (group) of the tile
// (-1: skip). A CTA walks whole tiles, keeps the column sums of one tile in registers and adds them to that group's
// dgamma / dbeta (and dxsum = column sums of dx, the bias gradient of the layer that produced the input) when the
// tile ends.
template <typename T, int NV>
__global__ void __launch_bounds__(32 * HM_LN_WARPS)
ln_bwd_grouped_kernel(const T* __restrict__ dy, const T* __restrict__ zin, const float* __restrict__ gamma0,
                      const float* __restrict__ mean_in, const float* __restrict__ rstd_in, T* __restrict__ dx,
                      float* __restrict__ dgamma, float* __restrict__ dbeta, float* __restrict__ dxsum, int rows,
                      int H, const int* __restrict__ tile_group) {
  __shared__ float sg[HM_LN_WARPS][32 * 8 + 8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_h = 1.f / (float)H;
  const int num_tiles = (rows + 127) >> 7;
  for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
    const int group = __ldg(tile_group + tile);
    if (group < 0) continue;  // uniform across the CTA
    const float* gamma = gamma0 + (size_t)group * H;
    float ag[NV][8], ab[NV][8], ac[NV][8];
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
      for (int k = 0; k < 8; ++k) ag[j][k] = ab[j][k] = ac[j][k] = 0.f;
    const int row_end = min(rows, (tile + 1) << 7);
    for (int row = (tile << 7) + warp; row < row_end; row += HM_LN_WARPS) {
      const size_t base = (size_t)row * H;
      const float mean = mean_in[row], rstd = rstd_in[row];
      float xh[NV][8], gd[NV][8];
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int col = (j * 32 + lane) * 8;
        if (col < H) {
          float d[8], g[8];
          ld8<T>(dy + base + col, d);
          ld8<T>(zin + base + col, xh[j]);
          ld8<float>(gamma + col, g);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            xh[j][k] = (xh[j][k] - mean) * rstd;
            ag[j][k] = fmaf(d[k], xh[j][k], ag[j][k]);
            ab[j][k] += d[k];
            gd[j][k] = d[k] * g[k];
            s1 += gd[j][k];
            s2 = fmaf(gd[j][k], xh[j][k], s2);
          }
        }
      }
      s1 = hm_warp_sum(s1) * inv_h;
      s2 = hm_warp_sum(s2) * inv_h;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int col = (j * 32 + lane) * 8;
        if (col < H) {
          float o[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            o[k] = rstd * (gd[j][k] - s1 - xh[j][k] * s2);
            ac[j][k] += o[k];
          }
          st8<T>(dx + base + col, o);
        }
      }
    }
#pragma unroll
    for (int pass = 0; pass < 3; ++pass) {
      float* dst0 = pass == 0 ? dgamma : (pass == 1 ? dbeta : dxsum);
      if (dst0 == nullptr) continue;
      float* dst = dst0 + (size_t)group * H;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int col = (j * 32 + lane) * 8;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 8; ++k) sg[warp][lane * 8 + k] = pass == 0 ? ag[j][k] : (pass == 1 ? ab[j][k] : ac[j][k]);
        __syncthreads();
        if (warp == 0 && col < H) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < HM_LN_WARPS; ++w) t += sg[w][lane * 8 + k];
            atomicAdd(dst + col + k, t);
          }
        }
      }
    }
    __syncthreads();
  }
}

// dx = dy * gelu'(x [+ bias]) with the bias-gradient column sums of each 128-row tile added to dbias[group].
template <typename T>
__global__ void __launch_bounds__(256)
gelu_bwd_grouped_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx,
                        float* __restrict__ dbias, long long rows, int H, const int* __restrict__ tile_group) {
  const int col = blockIdx.x * 256 + threadIdx.x;
  const int tile = blockIdx.y;
  const int group = __ldg(tile_group + tile);
  if (group < 0 || col >= H) return;
  const long long r0 = (long long)tile << 7, r1 = r0 + 128 < rows ? r0 + 128 : rows;
  float acc = 0.f;
  for (long long r = r0; r < r1; ++r) {
    const size_t idx = (size_t)r * H + col;
    float xv, dv;
    if constexpr (sizeof(T) == 2) {
      xv = __bfloat162float(x[idx]);
      dv = __bfloat162float(dy[idx]);
    } else {
      xv = x[idx];
      dv = dy[idx];
    }
    const float g = dv * hm_gelu_tanh_grad(xv);
    acc += g;
    if constexpr (sizeof(T) == 2) dx[idx] = __float2bfloat16(g);
    else dx[idx] = g;
  }
  if (dbias) atomicAdd(dbias + (size_t)group * H + col, acc);
}

// y = gelu_tanh(x + bias)
template <typename T>
__global__ void __launch_bounds__(256)
bias_gelu_fwd_kernel(const T* __restrict__ x, const float* __restrict__ bias, T* __restrict__ y, long long rows,
                     int H) {
  const long long total8 = rows * (long long)(H / 8);
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total8; i += 256LL * gridDim.x) {
    const int col = (int)(i % (H / 8)) * 8;
    float v[8], b[8];
    ld8<T>(x + i * 8, v);
    if (bias) ld8<float>(bias + col, b);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = hm_gelu_tanh(v[k] + (bias ? b[k] : 0.f));
    st8<T>(y + i * 8, v);
  }
}

// dx = dy * gelu'(x + bias); dbias += column sums of dx (fp32 atomics; zeroed by the caller).
// Grid: (ceil(H / 256), row_blocks). A thread owns one column and walks rows, so the row sum stays in a register.
template <typename T>
__global__ void __launch_bounds__(256)
bias_gelu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ bias,
                     T* __restrict__ dx, float* __restrict__ dbias, long long rows, int H) {
  const int col = blockIdx.x * 256 + threadIdx.x;
  if (col >= H) return;
  const float b = bias ? bias[col] : 0.f;
  const long long per = (rows + gridDim.y - 1) / gridDim.y;
  const long long r0 = per * blockIdx.y, r1 = r0 + per < rows ? r0 + per : rows;
  float acc = 0.f;
  for (long long r = r0; r < r1; ++r) {
    const size_t idx = (size_t)r * H + col;
    float xv, dv;
    if constexpr (sizeof(T) == 2) {
      xv = __bfloat162float(x[idx]);
      dv = __bfloat162float(dy[idx]);
    } else {
      xv = x[idx];
      dv = dy[idx];
    }
    const float g = dv * hm_gelu_tanh_grad(xv + b);
    acc += g;
    if constexpr (sizeof(T) == 2) dx[idx] = __float2bfloat16(g);
    else dx[idx] = g;
  }
  if (dbias) atomicAdd(dbias + col, acc);
}

// ------------------------------------------------------------------------------------------------
template <typename T, int NV>
static int ln_fwd_launch(const void* x, const void* res, const void* gamma, const void* beta, void* y, void* z,
                         void* mean, void* rstd, int rows, int H, float eps, int sms, cudaStream_t stream,
                         const int* tile_group = nullptr) {
  int blocks = (rows + HM_LN_WARPS - 1) / HM_LN_WARPS;
  const int cap = sms * 8;
  if (blocks > cap) blocks = cap;
  ln_fwd_kernel<T, NV><<<blocks, 32 * HM_LN_WARPS, 0, stream>>>((const T*)x, (const T*)res, (const float*)gamma,
                                                               (const float*)beta, (T*)y, (T*)z, (float*)mean,
                                                               (float*)rstd, rows, H, eps, tile_group);
  return (int)cudaGetLastError();
}
template <typename T, int NV>
static int ln_bwd_grouped_launch(const void* dy, const void* zin, const void* gamma, const void* mean,
                                 const void* rstd, void* dx, void* dgamma, void* dbeta, void* dxsum, int rows, int H,
                                 int sms, cudaStream_t stream, const int* tile_group) {
  int blocks = (rows + 127) / 128;
  const int cap = sms * 4;
  if (blocks > cap) blocks = cap;
  ln_bwd_grouped_kernel<T, NV><<<blocks, 32 * HM_LN_WARPS, 0, stream>>>(
      (const T*)dy, (const T*)zin, (const float*)gamma, (const float*)mean, (const float*)rstd, (T*)dx,
      (float*)dgamma, (float*)dbeta, (float*)dxsum, rows, H, tile_group);
  return (int)cudaGetLastError();
}
template <typename T, int NV>
static int ln_bwd_launch(const void* dy, const void* zin, const void* gamma, const void* mean, const void* rstd,
                         void* dx, void* dgamma, void* dbeta, int rows, int H, int sms, cudaStream_t stream) {
  int blocks = (rows + HM_LN_WARPS - 1) / HM_LN_WARPS;
  const int cap = sms * 8;
  if (blocks > cap) blocks = cap;
  ln_bwd_dx_kernel<T, NV><<<blocks, 32 * HM_LN_WARPS, 0, stream>>>((const T*)dy, (const T*)zin, (const float*)gamma,
                                                                  (const float*)mean, (const float*)rstd, (T*)dx, rows,
                                                                  H);
  if (dgamma != nullptr || dbeta != nullptr) {
    dim3 grid;
    int rows_per_strip;
    colstrip_grid<T>(rows, H, sms, &grid, &rows_per_strip);
    colstrip_kernel<T, 0><<<grid, 256, 0, stream>>>((const T*)dy, (const T*)zin, (const float*)mean,
                                                    (const float*)rstd, nullptr, (float*)dgamma, (float*)dbeta, rows,
                                                    H, rows_per_strip);
  }
  return (int)cudaGetLastError();
}

#define HM_LN_DISPATCH(FN, ...)                                                   \
  do {                                                                            \
    const int nv = (H + 255) / 256;                                               \
    if (H % 8 != 0 || nv > HM_LN_MAXV) return -1;                                 \
    if (dtype == HM_BF16) {                                                       \
      if (nv <= 1) return FN<__nv_bfloat16, 1>(__VA_ARGS__);                      \
      if (nv <= 2) return FN<__nv_bfloat16, 2>(__VA_ARGS__);                      \
      if (nv <= 4) return FN<__nv_bfloat16, 4>(__VA_ARGS__);                      \
      return FN<__nv_bfloat16, 8>(__VA_ARGS__);                                   \
    } else if (dtype == HM_F32) {                                                 \
      if (nv <= 1) return FN<float, 1>(__VA_ARGS__);                              \
      if (nv <= 2) return FN<float, 2>(__VA_ARGS__);                              \
      if (nv <= 4) return FN<float, 4>(__VA_ARGS__);                              \
      return FN<float, 8>(__VA_ARGS__);                                           \
    }                                                                             \
    return -2;                                                                    \
  } while (0)

HM_API int hm_layernorm_fwd(const void* x, const void* residual, const void* gamma, const void* beta, void* y, void* z,
                            void* mean, void* rstd, int rows, int H, float eps, int dtype, int sms,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  HM_LN_DISPATCH(ln_fwd_launch, x, residual, gamma, beta, y, z, mean, rstd, rows, H, eps, sms, stream);
}

HM_API int hm_layernorm_bwd(const void* dy, const void* zin, const void* gamma, const void* mean, const void* rstd,
                            void* dx, void* dgamma, void* dbeta, int rows, int H, int dtype, int sms,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  HM_LN_DISPATCH(ln_bwd_launch, dy, zin, gamma, mean, rstd, dx, dgamma, dbeta, rows, H, sms, stream);
}

// One-pass backward (bf16, H a multiple of 8 up to 2048). dgamma / dbeta / dxsum are fp32 [H] buffers that the kernel
// ADDS to (any of them may be null). Returns -1 when the shape is not covered; the caller then uses hm_layernorm_bwd.
HM_API int hm_layernorm_bwd_fused(const void* dy, const void* zin, const void* gamma, const void* mean, const void* rstd,
                                  void* dx, void* dgamma, void* dbeta, void* dxsum, int rows, int H, int dtype, int sms,
                                  cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype != HM_BF16 || H % 8 != 0 || H > 2048 || H < 64) return -1;
  int gp_log2 = 3;
  while ((1 << gp_log2) < H / 8) ++gp_log2;
  const bool small = H <= 1024;
  const int R = small ? 8 : 4;
  if ((256 >> gp_log2) > R) return -1;
  const size_t smem = (size_t)4 * R * H * 2 + (size_t)H * 4 + (size_t)R * 16;
  const int tiles = (rows + R - 1) / R;
  const int per_sm = (int)((size_t)224 * 1024 / (smem + 1024));   // 227 KB per SM, 1 KB per CTA reserved by the driver
  int blocks = sms * (per_sm < 1 ? 1 : (per_sm > 3 ? 3 : per_sm));
  if (blocks > tiles) blocks = tiles;
  cudaError_t e;
  if (small) {
    e = cudaFuncSetAttribute(ln_bwd_tile_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    ln_bwd_tile_kernel<8><<<blocks, 256, smem, stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)zin, (const float*)gamma, (const float*)mean, (const float*)rstd,
        (__nv_bfloat16*)dx, (float*)dgamma, (float*)dbeta, (float*)dxsum, rows, H, gp_log2);
  } else {
    e = cudaFuncSetAttribute(ln_bwd_tile_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    ln_bwd_tile_kernel<4><<<blocks, 256, smem, stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)zin, (const float*)gamma, (const float*)mean, (const float*)rstd,
        (__nv_bfloat16*)dx, (float*)dgamma, (float*)dbeta, (float*)dxsum, rows, H, gp_log2);
  }
  return (int)cudaGetLastError();
}

HM_API int hm_bias_gelu_fwd(const void* x, const void* bias, void* y, long long rows, int H, int dtype, int sms,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H % 8 != 0) return -1;
  const long long total8 = rows * (long long)(H / 8);
  long long blocks = (total8 + 255) / 256;
  if (blocks > (long long)sms * 16) blocks = (long long)sms * 16;
  if (dtype == HM_BF16)
    bias_gelu_fwd_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (const float*)bias,
                                                                        (__nv_bfloat16*)y, rows, H);
  else if (dtype == HM_F32)
    bias_gelu_fwd_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)x, (const float*)bias, (float*)y, rows, H);
  else
    return -2;
  return (int)cudaGetLastError();
}

HM_API int hm_bias_gelu_bwd(const void* dy, const void* x, const void* bias, void* dx, void* dbias, long long rows,
                            int H, int dtype, int sms, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (bias == nullptr && H % 8 == 0) {
    // x already holds the pre-activation (bias added by the producing GEMM): vectorised column-strip kernel
    dim3 grid;
    int rows_per_strip;
    if (dtype == HM_BF16) {
      colstrip_grid<__nv_bfloat16>(rows, H, sms, &grid, &rows_per_strip);
      colstrip_kernel<__nv_bfloat16, 1><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                                 nullptr, nullptr, (__nv_bfloat16*)dx, (float*)dbias,
                                                                 nullptr, rows, H, rows_per_strip);
    } else if (dtype == HM_F32) {
      colstrip_grid<float>(rows, H, sms, &grid, &rows_per_strip);
      colstrip_kernel<float, 1><<<grid, 256, 0, stream>>>((const float*)dy, (const float*)x, nullptr, nullptr,
                                                         (float*)dx, (float*)dbias, nullptr, rows, H, rows_per_strip);
    } else {
      return -2;
    }
    return (int)cudaGetLastError();
  }
  const int gx = (H + 255) / 256;
  int gy = (sms * 8 + gx - 1) / gx;
  if (gy > rows) gy = (int)rows;
  if (gy < 1) gy = 1;
  dim3 grid(gx, gy);
  if (dtype == HM_BF16)
    bias_gelu_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                                 (const float*)bias, (__nv_bfloat16*)dx, (float*)dbias,
                                                                 rows, H);
  else if (dtype == HM_F32)
    bias_gelu_bwd_kernel<float><<<grid, 256, 0, stream>>>((const float*)dy, (const float*)x, (const float*)bias,
                                                         (float*)dx, (float*)dbias, rows, H);
  else
    return -2;
  return (int)cudaGetLastError();
}

// Grouped variants: rows are split into 128-row tiles, tile_group[tile] selects the group's gamma / beta / bias
// (stacked [groups][H]); tiles of group -1 are not touched. Gradient buffers are fp32, stacked the same way and
// accumulated into (the caller zeroes them or passes existing gradients).
HM_API int hm_layernorm_fwd_grouped(const void* x, const void* residual, const void* gamma, const void* beta, void* y,
                                    void* z, void* mean, void* rstd, int rows, int H, float eps, int dtype,
                                    const int* tile_group, int sms, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (tile_group == nullptr) return -3;
  HM_LN_DISPATCH(ln_fwd_launch, x, residual, gamma, beta, y, z, mean, rstd, rows, H, eps, sms, stream, tile_group);
}

HM_API int hm_layernorm_bwd_grouped(const void* dy, const void* zin, const void* gamma, const void* mean,
                                    const void* rstd, void* dx, void* dgamma, void* dbeta, void* dxsum, int rows,
                                    int H, int dtype, const int* tile_group, int sms, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (tile_group == nullptr) return -3;
  // three sets of per-column accumulators live in registers: hidden sizes above 1024 would spill
  const int nv = (H + 255) / 256;
  if (H % 8 != 0 || nv > 4) return -1;
#define HM_LN_GROUPED(T)                                                                                           \
  do {                                                                                                             \
    if (nv <= 1) return ln_bwd_grouped_launch<T, 1>(dy, zin, gamma, mean, rstd, dx, dgamma, dbeta, dxsum, rows, H, \
                                                    sms, stream, tile_group);                                      \
    if (nv <= 2) return ln_bwd_grouped_launch<T, 2>(dy, zin, gamma, mean, rstd, dx, dgamma, dbeta, dxsum, rows, H, \
                                                    sms, stream, tile_group);                                      \
    return ln_bwd_grouped_launch<T, 4>(dy, zin, gamma, mean, rstd, dx, dgamma, dbeta, dxsum, rows, H, sms, stream, \
                                       tile_group);                                                                \
  } while (0)
  if (dtype == HM_BF16) HM_LN_GROUPED(__nv_bfloat16);
  if (dtype == HM_F32) HM_LN_GROUPED(float);
#undef HM_LN_GROUPED
  return -2;
}

HM_API int hm_gelu_bwd_grouped(const void* dy, const void* x, void* dx, void* dbias, long long rows, int H, int dtype,
                               const int* tile_group, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (tile_group == nullptr) return -3;
  dim3 grid((H + 255) / 256, (unsigned)((rows + 127) / 128));
  if (dtype == HM_BF16)
    gelu_bwd_grouped_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                                    (__nv_bfloat16*)dx, (float*)dbias, rows, H,
                                                                    tile_group);
  else if (dtype == HM_F32)
    gelu_bwd_grouped_kernel<float><<<grid, 256, 0, stream>>>((const float*)dy, (const float*)x, (float*)dx,
                                                            (float*)dbias, rows, H, tile_group);
  else
    return -2;
  return (int)cudaGetLastError();
}
