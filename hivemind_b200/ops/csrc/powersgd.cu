// Orthogonalisation of tall-skinny matrices for PowerSGD (P is [m, r] with r <= 64, row-major fp32).
//
// The reference runs modified Gram–Schmidt column by column on the CPU (hivemind/utils/math.py:6-14): r dependent
// steps, each a pass over the whole matrix. On the GPU the same factor Q of the thin QR decomposition (unique when
// the diagonal of R is positive, which is what Gram–Schmidt produces) is obtained with two fully parallel passes:
//   G = P^T P  (r x r, every CTA adds the contribution of its rows)
//   R = chol(G), P <- P R^{-1}
// repeated once more (CholeskyQR2) so that rounding in G does not cost orthogonality. A column whose pivot is not
// positive (a zero or dependent column) is set to zero, which is also what Gram–Schmidt with its eps yields.
// All matrices of a model are processed by one launch per pass through a table {ptr, rows} per matrix.
#include "hm_common.cuh"

#define PS_MAX_R 64
#define PS_ROWS 96    // rows per CTA in the gram and apply passes (tile + R^-1 fit 48 KB of static smem)

struct PsMat {
  float* p;
  long long rows;
  float* gram;   // [r*r] scratch, zeroed before the gram pass
  float* rinv;   // [r*r] scratch
};

// gram[a][b] += sum over this CTA's rows of P[row][a] * P[row][b]
__global__ void __launch_bounds__(256)
ps_gram_kernel(const PsMat* __restrict__ mats, const int2* __restrict__ items, int r) {
  __shared__ float tile[PS_ROWS][PS_MAX_R + 1];
  const int2 it = items[blockIdx.x];
  const PsMat m = mats[it.x];
  const long long row0 = (long long)it.y * PS_ROWS;
  const int nrows = (int)min((long long)PS_ROWS, m.rows - row0);
  for (int idx = threadIdx.x; idx < PS_ROWS * r; idx += 256) {
    const int rr = idx / r, cc = idx % r;
    tile[rr][cc] = rr < nrows ? m.p[(row0 + rr) * r + cc] : 0.f;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < r * r; e += 256) {
    const int a = e / r, b = e % r;
    if (b < a) continue;  // symmetric: upper triangle only
    float acc = 0.f;
#pragma unroll 8
    for (int rr = 0; rr < PS_ROWS; ++rr) acc = fmaf(tile[rr][a], tile[rr][b], acc);
    atomicAdd(m.gram + a * r + b, acc);
  }
}

// One CTA per matrix: Cholesky G = R^T R (upper R), then R^{-1} by back substitution. r <= 64.
__global__ void __launch_bounds__(64)
ps_chol_inv_kernel(const PsMat* __restrict__ mats, int r, float eps) {
  __shared__ float R[PS_MAX_R][PS_MAX_R + 1];
  __shared__ float Rinv[PS_MAX_R][PS_MAX_R + 1];
  __shared__ int dead[PS_MAX_R];
  const PsMat m = mats[blockIdx.x];
  const int t = threadIdx.x;
  for (int e = t; e < r * r; e += 64) {
    const int a = e / r, b = e % r;
    R[a][b] = b >= a ? m.gram[a * r + b] : 0.f;
    Rinv[a][b] = 0.f;
  }
  __syncthreads();
  // right-looking Cholesky on the upper triangle; thread t owns column t
  for (int k = 0; k < r; ++k) {
    const float pivot = R[k][k];
    const bool ok = pivot > eps * eps;
    if (t == 0) dead[k] = !ok;
    const float d = ok ? sqrtf(pivot) : 1.f;
    __syncthreads();
    if (t >= k && t < r) R[k][t] = ok ? R[k][t] / d : (t == k ? 1.f : 0.f);
    __syncthreads();
    if (t > k && t < r) {
      const float rkt = R[k][t];
      for (int i = k + 1; i <= t; ++i) R[i][t] -= R[k][i] * rkt;
    }
    __syncthreads();
  }
  // invert the upper-triangular R: column t of R^{-1} by back substitution
  if (t < r) {
    for (int i = t; i >= 0; --i) {
      float s = (i == t) ? 1.f : 0.f;
      for (int k = i + 1; k <= t; ++k) s -= R[i][k] * Rinv[k][t];
      Rinv[i][t] = s / R[i][i];
    }
  }
  __syncthreads();
  for (int e = t; e < r * r; e += 64) {
    const int a = e / r, b = e % r;
    m.rinv[e] = dead[b] ? 0.f : Rinv[a][b];  // a dead column of P becomes zero
  }
}

// P[row][:] <- P[row][:] * Rinv   (thread per output element within the CTA's row block)
__global__ void __launch_bounds__(256)
ps_apply_kernel(const PsMat* __restrict__ mats, const int2* __restrict__ items, int r) {
  __shared__ float tile[PS_ROWS][PS_MAX_R + 1];
  __shared__ float W[PS_MAX_R][PS_MAX_R + 1];
  const int2 it = items[blockIdx.x];
  const PsMat m = mats[it.x];
  const long long row0 = (long long)it.y * PS_ROWS;
  const int nrows = (int)min((long long)PS_ROWS, m.rows - row0);
  for (int e = threadIdx.x; e < r * r; e += 256) W[e / r][e % r] = m.rinv[e];
  for (int idx = threadIdx.x; idx < PS_ROWS * r; idx += 256) {
    const int rr = idx / r, cc = idx % r;
    tile[rr][cc] = rr < nrows ? m.p[(row0 + rr) * r + cc] : 0.f;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nrows * r; idx += 256) {
    const int rr = idx / r, cc = idx % r;
    float acc = 0.f;
    for (int k = 0; k <= cc; ++k) acc = fmaf(tile[rr][k], W[k][cc], acc);  // Rinv is upper triangular
    m.p[(row0 + rr) * r + cc] = acc;
  }
}

// mats: device array of PsMat; items: device int2 {matrix, row block}; one CholeskyQR sweep per call.
HM_API int hm_ps_orthogonalize_sweep(const void* mats, int num_mats, const void* items, int num_items, int r, float eps,
                                     cudaStream_t stream) {
  if (num_mats <= 0 || num_items <= 0) return 0;
  if (r > PS_MAX_R || r <= 0) return -1;
  ps_gram_kernel<<<num_items, 256, 0, stream>>>((const PsMat*)mats, (const int2*)items, r);
  ps_chol_inv_kernel<<<num_mats, 64, 0, stream>>>((const PsMat*)mats, r, eps);
  ps_apply_kernel<<<num_items, 256, 0, stream>>>((const PsMat*)mats, (const int2*)items, r);
  return (int)cudaGetLastError();
}
HM_API int hm_ps_rows_per_block() { return PS_ROWS; }
