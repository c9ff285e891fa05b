// Per-row argmax shared by the token pick (row_argmax_kernel) and its fused form with the token all-gather
// (p2p_argmax_publish_kernel).
#pragma once

#include "nvj_common.cuh"

namespace nvj {

constexpr int kArgmaxThreads = 128;

// One decode step of a row's resident metadata: an active row (length > 0) grows by the token it has just appended;
// its position is the old length.  A row that would outgrow its block table is flagged and left alone.
__device__ __forceinline__ void advance_row(int32_t* seq_lens, int32_t* positions, int b, long long capacity, int32_t* status) {
  const int len = seq_lens[b];
  if (len <= 0) return;
  if ((long long)len + 1 > capacity) {
    if (status) atomicOr(status, NVJ_DEV_BAD_LENGTH);
    return;
  }
  if (positions) positions[b] = len;
  seq_lens[b] = len + 1;
}

// Argmax of `row_len` floats by one CTA of kArgmaxThreads threads: the first maximum wins, NaNs are never
// selected unless the whole row is NaN (then index 0).  The result is valid in thread 0.
__device__ __forceinline__ int row_argmax_cta(const float* row, int row_len) {
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  if ((row_len & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
    // 16-byte loads, four in flight per thread: the row is read in one or two round trips instead of row_len / 128
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int n4 = row_len >> 2;
    for (int base = threadIdx.x; base < n4; base += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = base + u * blockDim.x;
        v[u] = j < n4 ? row4[j] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i0 = (base + u * blockDim.x) * 4;
        const float e[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (e[c] > best || (e[c] == best && i0 + c < best_i)) { best = e[c]; best_i = i0 + c; }
      }
    }
  } else {
    for (int i = threadIdx.x; i < row_len; i += blockDim.x) {
      const float v = row[i];
      if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(kFullMask, best, o);
    const int oi = __shfl_xor_sync(kFullMask, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  __shared__ float sv[kArgmaxThreads / 32];
  __shared__ int si[kArgmaxThreads / 32];
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = best_i; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kArgmaxThreads / 32; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < best_i)) { best = sv[w]; best_i = si[w]; }
  }
  return best_i == 0x7fffffff ? 0 : best_i;
}

}  // namespace nvj
