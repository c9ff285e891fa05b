// The step in front of the KV path, fused with the append: per-head RMSNorm of the query and
// key rows, partial rotary embedding, then the key and value rows go straight into their cache
// slots and the query comes out ready for attention.  Unfused, k is written after the norm,
// read and written again by the rotation, then read once more by the append; here q, k and v
// are each read once.
//
// Math, per head row x[0..D) of activation dtype bf16 (nanovllm_jax/layers.py:11-29, 49-199;
// call site nanovllm_jax/model.py:3371-3396):
//   y  = bf16( x_f32 * rsqrt(mean(x_f32^2) + eps) * (1 + w_f32) )              RMSNorm, (1 + w) form
//   c  = bf16(cos(pos * inv_freq[i])), s = bf16(sin(pos * inv_freq[i]))          i < rot / 2
//   y'[i]           = bf16( y[i] * c - y[i + rot/2] * s )                        half-split rotation
//   y'[i + rot/2]   = bf16( y[i + rot/2] * c + y[i] * s ),   y'[j >= rot] = y[j]
// The products and the sum are formed in fp32 and rounded once (what XLA does with its default
// excess-precision setting); `inv_freq` comes from the caller so that it is bit-identical to
// the framework's own table.  Positions are one row per token (text) or three rows (temporal,
// height, width) of a multimodal position id; with three rows frequency i takes its position from
// the height row when i % 3 == 1 and i < 3 * section[1], from the width row when i % 3 == 2 and
// i < 3 * section[2], else from the temporal row (the interleaved selection of layers.py:79-139).
// One warp per (token, head): D / 32 elements per lane (D = 64, 128 or 256), sum of squares by
// shuffle, the rotation partner rot / 2 elements away sits (rot / 2) / (D / 32) lanes away.
// Slots and masks are those of the plain append (kv_append.cuh).

#include "kv_append.cuh"

namespace nvj {

struct NormRopeParams {
  AppendParams a;  // slot resolution + cache pointers (new_k / new_v unused)
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const void* q_weight;
  const void* k_weight;
  const float* inv_freq;
  const int32_t* rope_positions;  // [pos_rows][tokens]
  int pos_rows, h_limit, w_limit;  // 1 or 3 rows; 3 * section[1], 3 * section[2]
  __nv_bfloat16* q_out;
  long long q_token_stride, q_head_stride, k_token_stride, v_token_stride;  // in elements
  int hq, hkv, d, rot, w_dtype;
  float eps;
};

template <int E>  // elements per lane = D / 32
__global__ void __launch_bounds__(256) qk_norm_rope_append_kernel(NormRopeParams p) {
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int heads = p.hq + 2 * p.hkv;
  if (warp >= (long long)p.a.n_tokens * heads) return;
  const int token = (int)(warp / heads), h = (int)(warp - (long long)token * heads);
  const bool is_q = h < p.hq, is_k = !is_q && h < p.hq + p.hkv;
  const int kvh = is_q ? 0 : (is_k ? h - p.hq : h - p.hq - p.hkv);

  long long slot = 0;
  if (!is_q) {
    if (lane == 0) slot = resolve_slot(p.a, token);
    slot = __shfl_sync(kFullMask, slot, 0);
    if (slot < 0) return;  // masked or padded token: nothing is written (the flag is set for a bad slot)
  }
  const __nv_bfloat16* src = is_q ? p.q + token * p.q_token_stride + h * p.q_head_stride
                                  : (is_k ? p.k + token * p.k_token_stride : p.v + token * p.v_token_stride) + (long long)kvh * p.d;
  __nv_bfloat16 raw[E];
  if (E == 8) {
    *reinterpret_cast<uint4*>(raw) = ld_nc_u4(reinterpret_cast<const uint4*>(src) + lane);
  } else {
#pragma unroll
    for (int j = 0; j < E; ++j) raw[j] = src[lane * E + j];
  }
  __nv_bfloat16* cache_dst = nullptr;
  if (!is_q) cache_dst = static_cast<__nv_bfloat16*>(is_k ? p.a.k_cache : p.a.v_cache) + (slot * p.hkv + kvh) * p.d + lane * E;

  if (!is_q && !is_k) {  // value rows are stored as they are
    if (E == 8) *reinterpret_cast<uint4*>(cache_dst) = *reinterpret_cast<const uint4*>(raw);
    else {
#pragma unroll
      for (int j = 0; j < E; ++j) cache_dst[j] = raw[j];
    }
    return;
  }

  // ---- RMSNorm in fp32, rounded to bf16
  float x[E];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < E; ++j) { x[j] = __bfloat162float(raw[j]); ss = fmaf(x[j], x[j], ss); }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(kFullMask, ss, o);
  const float r = rsqrtf(ss / (float)p.d + p.eps);
  const void* wv = is_q ? p.q_weight : p.k_weight;
  float y[E];
#pragma unroll
  for (int j = 0; j < E; ++j) {
    const int i = lane * E + j;
    const float w = p.w_dtype == NVJ_F32 ? static_cast<const float*>(wv)[i]
                                         : __bfloat162float(static_cast<const __nv_bfloat16*>(wv)[i]);
    y[j] = __bfloat162float(__float2bfloat16_rn(__fmul_rn(__fmul_rn(x[j], r), __fadd_rn(1.f, w))));
  }

  // ---- partial rotary embedding on the first `rot` elements
  const int half_lanes = (p.rot / 2) / E;  // a power of two
  float other[E];
#pragma unroll
  for (int j = 0; j < E; ++j) other[j] = __shfl_xor_sync(kFullMask, y[j], half_lanes);
  if (lane < 2 * half_lanes) {
    const bool first = lane < half_lanes;
    float pos3[3];
    pos3[0] = (float)p.rope_positions[token];
    pos3[1] = p.pos_rows == 3 ? (float)p.rope_positions[(long long)p.a.n_tokens + token] : pos3[0];
    pos3[2] = p.pos_rows == 3 ? (float)p.rope_positions[2LL * p.a.n_tokens + token] : pos3[0];
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const int i = (lane & (half_lanes - 1)) * E + j;  // index into the first half = frequency index
      const int m = i % 3;
      const float pos = (m == 1 && i < p.h_limit) ? pos3[1] : ((m == 2 && i < p.w_limit) ? pos3[2] : pos3[0]);
      const float ang = __fmul_rn(pos, p.inv_freq[i]);
      const float c = __bfloat162float(__float2bfloat16_rn(cosf(ang)));
      const float s = __bfloat162float(__float2bfloat16_rn(sinf(ang)));
      y[j] = first ? __fsub_rn(__fmul_rn(y[j], c), __fmul_rn(other[j], s))
                   : __fadd_rn(__fmul_rn(y[j], c), __fmul_rn(other[j], s));
    }
  }
  __nv_bfloat16 outv[E];
#pragma unroll
  for (int j = 0; j < E; ++j) outv[j] = __float2bfloat16_rn(y[j]);
  __nv_bfloat16* dst = is_q ? p.q_out + ((long long)token * p.hq + h) * p.d + lane * E : cache_dst;
  if (E == 8) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(outv);
  else {
#pragma unroll
    for (int j = 0; j < E; ++j) dst[j] = outv[j];
  }
}

}  // namespace nvj

extern "C" int nvj_qk_norm_rope_kv_append(const void* q, int64_t q_token_stride, int64_t q_head_stride,
                                          const void* k, int64_t k_token_stride,
                                          const void* v, int64_t v_token_stride, int act_dtype,
                                          const void* q_norm_weight, const void* k_norm_weight, int weight_dtype,
                                          float eps, const float* inv_freq, int rotary_dim,
                                          const int32_t* rope_positions, int position_rows,
                                          const int32_t* mrope_section,
                                          const int32_t* slot_mapping, const int32_t* valid_mask,
                                          const int32_t* query_start_loc, int qsl_rows, int packed,
                                          int n_rows, int n_cols,
                                          void* k_cache_layer, void* v_cache_layer, int cache_dtype,
                                          int64_t num_slots, int num_q_heads, int num_kv_heads, int head_dim,
                                          void* q_out, int32_t* status, nvj_stream_t stream) {
  using namespace nvj;
  if (n_rows < 0 || n_cols < 0 || num_slots < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 ||
      rotary_dim < 0 || rotary_dim > head_dim || (position_rows != 1 && position_rows != 3) ||
      (position_rows == 3 && !mrope_section))
    return NVJ_ERR_INVALID_ARGUMENT;
  const long long tokens = (long long)n_rows * n_cols;
  if (tokens == 0) return NVJ_OK;
  if (tokens > 0x7fffffffLL) return NVJ_ERR_TOO_LARGE;
  if (!q || !k || !v || !q_norm_weight || !k_norm_weight || !rope_positions || !slot_mapping || !k_cache_layer ||
      !v_cache_layer || !q_out || (rotary_dim > 0 && !inv_freq))
    return NVJ_ERR_INVALID_ARGUMENT;
  if (query_start_loc && qsl_rows < 0) return NVJ_ERR_INVALID_ARGUMENT;
  const int e = head_dim / 32;
  const bool shape_ok = head_dim % 32 == 0 && (e == 2 || e == 4 || e == 8) && rotary_dim % (2 * e) == 0;
  const int half_lanes = shape_ok && rotary_dim > 0 ? (rotary_dim / 2) / e : 1;
  if (act_dtype != NVJ_BF16 || cache_dtype != NVJ_BF16 || (weight_dtype != NVJ_BF16 && weight_dtype != NVJ_F32) ||
      !shape_ok || (half_lanes & (half_lanes - 1)) != 0 || half_lanes > 16)
    return NVJ_ERR_UNSUPPORTED;
  const uintptr_t align = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                          reinterpret_cast<uintptr_t>(k_cache_layer) | reinterpret_cast<uintptr_t>(v_cache_layer) |
                          reinterpret_cast<uintptr_t>(q_out);
  if (e == 8 && ((align & 15u) != 0 || ((q_token_stride | q_head_stride | k_token_stride | v_token_stride) & 7) != 0))
    return NVJ_ERR_UNSUPPORTED;
  NormRopeParams p{};
  p.a.k_cache = k_cache_layer; p.a.v_cache = v_cache_layer;
  p.a.slot_mapping = slot_mapping; p.a.valid_mask = valid_mask; p.a.query_start_loc = query_start_loc;
  p.a.status = status; p.a.num_slots = num_slots; p.a.n_tokens = (int)tokens; p.a.n_cols = n_cols;
  p.a.qsl_rows = qsl_rows; p.a.packed = packed;
  p.q = static_cast<const __nv_bfloat16*>(q); p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.q_weight = q_norm_weight; p.k_weight = k_norm_weight; p.w_dtype = weight_dtype;
  p.inv_freq = inv_freq; p.rope_positions = rope_positions; p.q_out = static_cast<__nv_bfloat16*>(q_out);
  p.pos_rows = position_rows;
  p.h_limit = position_rows == 3 ? 3 * mrope_section[1] : 0;
  p.w_limit = position_rows == 3 ? 3 * mrope_section[2] : 0;
  p.q_token_stride = q_token_stride; p.q_head_stride = q_head_stride;
  p.k_token_stride = k_token_stride; p.v_token_stride = v_token_stride;
  p.hq = num_q_heads; p.hkv = num_kv_heads; p.d = head_dim; p.rot = rotary_dim; p.eps = eps;
  const long long warps = tokens * (num_q_heads + 2 * num_kv_heads);
  const unsigned blocks = (unsigned)((warps + 7) / 8);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (e == 8) qk_norm_rope_append_kernel<8><<<blocks, 256, 0, s>>>(p);
  else if (e == 4) qk_norm_rope_append_kernel<4><<<blocks, 256, 0, s>>>(p);
  else qk_norm_rope_append_kernel<2><<<blocks, 256, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}
