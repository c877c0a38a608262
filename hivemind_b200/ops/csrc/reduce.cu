// Column sums of a row-major [rows, H] matrix into an fp32 vector (bias gradients:
// db = sum over tokens of dy), and the elementwise GELU-gradient product used by the linear backward.
#include "hm_common.cuh"

// out[col] += sum_r x[r][col]; `out` is zeroed (or holds a running gradient) before the launch.
// Grid (ceil(H/256), row_blocks); a thread owns one column so that loads are coalesced across the warp.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_kernel(const T* __restrict__ x, float* __restrict__ out, long long rows, int H, long long ld) {
  const int col = blockIdx.x * 256 + threadIdx.x;
  if (col >= H) return;
  const long long per = (rows + gridDim.y - 1) / gridDim.y;
  const long long r0 = per * blockIdx.y, r1 = r0 + per < rows ? r0 + per : rows;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  long long r = r0;
  for (; r + 4 <= r1; r += 4) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if constexpr (sizeof(T) == 2) acc[k] += __bfloat162float(x[(size_t)(r + k) * ld + col]);
      else acc[k] += x[(size_t)(r + k) * ld + col];
    }
  }
  for (; r < r1; ++r) {
    if constexpr (sizeof(T) == 2) acc[0] += __bfloat162float(x[(size_t)r * ld + col]);
    else acc[0] += x[(size_t)r * ld + col];
  }
  atomicAdd(out + col, (acc[0] + acc[1]) + (acc[2] + acc[3]));
}

HM_API int hm_colsum(const void* x, void* out, long long rows, int H, long long ld, int dtype, int sms,
                     cudaStream_t stream) {
  if (rows <= 0 || H <= 0) return 0;
  const int gx = (H + 255) / 256;
  long long gy = ((long long)sms * 8 + gx - 1) / gx;
  if (gy > (rows + 15) / 16) gy = (rows + 15) / 16;
  if (gy < 1) gy = 1;
  dim3 grid(gx, (unsigned)gy);
  if (dtype == HM_BF16)
    colsum_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (float*)out, rows, H, ld);
  else if (dtype == HM_F32)
    colsum_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, (float*)out, rows, H, ld);
  else
    return -2;
  return (int)cudaGetLastError();
}
