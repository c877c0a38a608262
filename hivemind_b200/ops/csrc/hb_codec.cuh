// Codec geometry and small device helpers shared by the whole-tensor codec kernels (codec.cu) and the fused
// butterfly round kernel (butterfly_round.cu). Codec math follows hivemind/compression/floating.py:18-64 and
// hivemind/compression/quantization.py:60-153.
#pragma once
#include "hm_common.cuh"

#define HB_BLOCK 4096          // block-wise quantization block
#define HB_FAIL_BIT 0x80000000u

enum HbCodec : int { HB_NONE = 0, HB_MEANSTD16 = 1, HB_FLOAT16 = 2, HB_QUANTILE8 = 3, HB_UNIFORM8 = 4, HB_BLOCKWISE8 = 5 };

__host__ __device__ inline int hb_elem_bytes(int codec) {
  return codec == HB_NONE ? 4 : ((codec == HB_FLOAT16 || codec == HB_MEANSTD16) ? 2 : 1);
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
