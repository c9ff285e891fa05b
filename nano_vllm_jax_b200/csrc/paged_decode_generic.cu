// Generic paged GQA decode attention: any block size, head count and head_dim
// up to 256, cache in bf16 / f16 / f32, query in bf16 / f16 / f32.  One CTA per
// (row, query head); its four warps take every fourth key, each keeps an online
// softmax state (max, sum, accumulator) and the CTA merges the four at the end.
// This kernel serves shapes outside the specialised pipelined kernel and is the
// in-library cross-check for it; it reads K/V once per query head (through L2
// for the other heads of a group), so it is not the bandwidth path.
//
// Math follows nanovllm_jax/kv_cache.py:972-998: scores = scale * <q, k_p> for
// p < len, softmax over those keys, out = sum_p w_p v_p, all in fp32 here.

#include "paged_decode.cuh"

namespace nvj {

constexpr int kGenWarps = 4;
constexpr int kGenMaxPerLane = 8;  // head_dim <= 256

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

__device__ __forceinline__ float load_q(const void* q, long long idx, int dt) {
  if (dt == NVJ_F32) return static_cast<const float*>(q)[idx];
  if (dt == NVJ_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(q)[idx]);
  return __half2float(static_cast<const __half*>(q)[idx]);
}

template <typename KV>
__global__ void __launch_bounds__(kGenWarps * 32) decode_generic_kernel(DecodeParams p) {
  const int b = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D = p.head_dim;
  const int kvh = h / (p.num_q_heads / p.num_kv_heads);
  float* out = p.out + ((long long)b * p.num_q_heads + h) * D;
  int row = b, len;
  if (p.query_start_loc) {
    // packed prefill: find the table row of query b, cap the keys at its position
    if (b >= p.query_start_loc[p.qsl_rows]) {
      len = 0;
    } else {
      int lo = 0, hi = p.qsl_rows;  // last r with query_start_loc[r] <= b
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (p.query_start_loc[mid] <= b) lo = mid; else hi = mid;
      }
      row = lo;
      len = decode_row_len(p, row);
      const int cap = p.query_positions[b] + 1;
      len = len < cap ? len : cap;
    }
  } else {
    len = decode_row_len(p, b);
  }
  if (len <= 0) {
    for (int d = threadIdx.x; d < D; d += blockDim.x) out[d] = 0.f;
    return;
  }
  float qv[kGenMaxPerLane], acc[kGenMaxPerLane];
#pragma unroll
  for (int i = 0; i < kGenMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < D ? load_q(p.q, ((long long)b * p.num_q_heads + h) * D + d, p.q_dtype) * p.scale : 0.f;
    acc[i] = 0.f;
  }
  const KV* kc = reinterpret_cast<const KV*>(p.k_cache);
  const KV* vc = reinterpret_cast<const KV*>(p.v_cache);
  const long long tbase = decode_table_base(p, row);
  float m = -INFINITY, l = 0.f;
  for (int t = warp; t < len; t += kGenWarps) {
    const long long blk = p.block_tables[tbase + t / p.block_size];
    if (blk < 0 || blk >= p.num_blocks) {
      if (lane == 0) atomicOr(p.status, NVJ_DEV_BAD_BLOCK_ID);
      continue;
    }
    const long long row = ((blk * p.block_size + t % p.block_size) * p.num_kv_heads + kvh) * D;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kGenMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < D) s = fmaf(qv[i], to_float<KV>(kc[row + d]), s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(kFullMask, s, o);
    const float mn = fmaxf(m, s);
    const float a = __expf(m - mn), w = __expf(s - mn);
    l = l * a + w;
#pragma unroll
    for (int i = 0; i < kGenMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < D) acc[i] = fmaf(w, to_float<KV>(vc[row + d]), acc[i] * a);
    }
    m = mn;
  }
  __shared__ float s_m[kGenWarps], s_l[kGenWarps];
  __shared__ float s_acc[kGenWarps][kGenMaxPerLane * 32];
  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < kGenMaxPerLane; ++i) s_acc[warp][lane + 32 * i] = acc[i];
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < kGenWarps; ++w) M = fmaxf(M, s_m[w]);
  float L = 0.f;
  float f[kGenWarps];
#pragma unroll
  for (int w = 0; w < kGenWarps; ++w) {
    f[w] = s_m[w] == -INFINITY ? 0.f : __expf(s_m[w] - M);
    L += s_l[w] * f[w];
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < kGenWarps; ++w) o += s_acc[w][d] * f[w];
    out[d] = o * inv;
  }
}

int launch_decode_generic(const DecodeParams& p, cudaStream_t stream) {
  if (p.head_dim > kGenMaxPerLane * 32) return NVJ_ERR_UNSUPPORTED;
  if (p.num_q_heads > 65535) return NVJ_ERR_UNSUPPORTED;
  dim3 grid(p.batch, p.num_q_heads, 1);
  if (p.kv_dtype == NVJ_BF16) decode_generic_kernel<__nv_bfloat16><<<grid, kGenWarps * 32, 0, stream>>>(p);
  else if (p.kv_dtype == NVJ_F16) decode_generic_kernel<__half><<<grid, kGenWarps * 32, 0, stream>>>(p);
  else decode_generic_kernel<float><<<grid, kGenWarps * 32, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

}  // namespace nvj
