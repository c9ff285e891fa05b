// Ragged packed prefill attention over the paged cache: C ABI and dispatch (tensor-core tile
// kernels for the model's shape: tcgen05 on CTA pairs, tcgen05 on single CTAs, mma.sync, in that order; the generic CUDA-core kernel for every other shape).
//
// Token i of table row r (query_start_loc[r] <= i < query_start_loc[r + 1]) sits
// at absolute position positions[i] and attends keys p < kv_lens[r], p <=
// positions[i]; tokens at or beyond query_start_loc[rows] are padding and get
// zeros (nanovllm_jax/kv_cache.py:831-849,
// nanovllm_jax/kernels/full_attention_triton.py:51-145,218-221).

#include "paged_decode.cuh"

namespace nvj {
int launch_prefill_mma(const void* q, int q_dtype, const char* k_cache, const char* v_cache,
                       long long num_blocks, const int32_t* block_tables, int table_width,
                       const int32_t* kv_lens, const int32_t* positions, const int32_t* query_start_loc,
                       int rows, int token_bucket, float scale, float* out, int32_t* status,
                       int skip_single, cudaStream_t stream);
int launch_prefill_umma2(const void* q, int q_dtype, const char* k_cache, const char* v_cache,
                         long long num_blocks, const int32_t* block_tables, int table_width,
                         const int32_t* kv_lens, const int32_t* positions, const int32_t* query_start_loc,
                         int rows, int token_bucket, float scale, float* out, int32_t* status,
                         int skip_single, int split_p, cudaStream_t stream);
int launch_prefill_umma(const void* q, int q_dtype, const char* k_cache, const char* v_cache,
                        long long num_blocks, const int32_t* block_tables, int table_width,
                        const int32_t* kv_lens, const int32_t* positions, const int32_t* query_start_loc,
                        int rows, int token_bucket, float scale, float* out, int32_t* status,
                        int skip_single, cudaStream_t stream);
}

extern "C" int nvj_paged_prefill_packed(const void* q, int q_dtype, const void* k_cache_layer,
                                        const void* v_cache_layer, int kv_dtype,
                                        int64_t num_blocks, int block_size, int num_kv_heads,
                                        int head_dim, int num_q_heads,
                                        const int32_t* block_tables, int table_width,
                                        const int32_t* kv_lens, const int32_t* positions,
                                        const int32_t* query_start_loc, int rows,
                                        int token_bucket, float scale, float* out,
                                        int32_t* status, void* workspace, size_t workspace_bytes,
                                        int variant, nvj_stream_t stream) {
  using namespace nvj;
  if (rows < 0 || token_bucket < 0 || table_width < 0 || num_blocks < 0 || block_size <= 0 ||
      num_kv_heads <= 0 || num_q_heads <= 0 || head_dim <= 0)
    return NVJ_ERR_INVALID_ARGUMENT;
  if (num_q_heads % num_kv_heads != 0 || variant < 0 || variant > 5) return NVJ_ERR_INVALID_ARGUMENT;
  if (token_bucket == 0) return NVJ_OK;
  if (!q || !k_cache_layer || !v_cache_layer || !block_tables || !kv_lens || !positions ||
      !query_start_loc || !out || !status)
    return NVJ_ERR_INVALID_ARGUMENT;
  const bool a16 = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache_layer) |
                     reinterpret_cast<uintptr_t>(v_cache_layer) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
  const bool tile_ok = kv_dtype == NVJ_BF16 && block_size == kBlk && num_kv_heads == kHkv && num_q_heads == kHq &&
                       head_dim == kD && (q_dtype == NVJ_BF16 || q_dtype == NVJ_F32) && a16;
  if (variant >= 2 && !tile_ok) return NVJ_ERR_UNSUPPORTED;
  if (tile_ok && variant != 1) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Rows that carry a single query token (the decode rows of a mixed batch) go to the pipelined
    // decode kernel when the caller lends it a decode workspace; everything else goes to the tile kernel.
    int skip_single = 0;
    const int num_ctas = decode_num_ctas();
    DecodeParams d{};
    d.batch = rows;
    if (workspace && num_ctas > 0 && rows > 0 &&
        carve_decode_workspace(d, workspace, workspace_bytes, ws_ml_bytes(num_ctas), ws_acc_bytes(num_ctas)) == NVJ_OK) {
      if (cudaMemsetAsync(out, 0, sizeof(float) * (size_t)token_bucket * kHq * kD, s) != cudaSuccess)
        return NVJ_ERR_LAUNCH;
      d.q = q;
      d.k_cache = static_cast<const char*>(k_cache_layer);
      d.v_cache = static_cast<const char*>(v_cache_layer);
      d.block_tables = block_tables;
      d.seq_lens = kv_lens;
      d.query_start_loc = query_start_loc;
      d.query_positions = positions;
      d.qsl_rows = rows;
      d.packed_rows = 1;
      d.out = out;
      d.num_blocks = num_blocks;
      d.table_width = table_width;
      d.block_size = block_size;
      d.num_kv_heads = num_kv_heads;
      d.num_q_heads = num_q_heads;
      d.head_dim = head_dim;
      d.q_dtype = q_dtype;
      d.kv_dtype = kv_dtype;
      d.scale = scale;
      // bf16 queries: the tensor-core streaming kernel (it declines without a tensor-map encoder); else the CUDA-core one
      int rc = NVJ_ERR_UNSUPPORTED;
      if (q_dtype == NVJ_BF16) {
        d.width = 1;
        rc = launch_decode_wide(d, s);
        d.width = 0;
      }
      if (rc == NVJ_ERR_UNSUPPORTED) rc = launch_decode_pipelined(d, num_ctas, s);
      if (rc != NVJ_OK) return rc;
      skip_single = 1;
    }
    const char* kc = static_cast<const char*>(k_cache_layer);
    const char* vc = static_cast<const char*>(v_cache_layer);
    // tcgen05 tiles first (CTA pairs, then single CTAs); they decline when the driver has no tensor-map
    // encoder or the scale is not positive, and the mma.sync tiles take over
    if (variant == 0 || variant == 4 || variant == 5) {
      const int rc = launch_prefill_umma2(q, q_dtype, kc, vc, num_blocks, block_tables, table_width, kv_lens, positions,
                                          query_start_loc, rows, token_bucket, scale, out, status, skip_single,
                                          variant == 5 ? 0 : 1, s);
      if (rc != NVJ_ERR_UNSUPPORTED || variant != 0) return rc;
    }
    if (variant == 0 || variant == 3) {
      const int rc = launch_prefill_umma(q, q_dtype, kc, vc, num_blocks, block_tables, table_width, kv_lens, positions,
                                         query_start_loc, rows, token_bucket, scale, out, status, skip_single, s);
      if (rc != NVJ_ERR_UNSUPPORTED || variant == 3) return rc;
    }
    return launch_prefill_mma(q, q_dtype, kc, vc, num_blocks, block_tables, table_width, kv_lens, positions,
                              query_start_loc, rows, token_bucket, scale, out, status, skip_single, s);
  }
  DecodeParams p{};
  p.q = q;
  p.k_cache = static_cast<const char*>(k_cache_layer);
  p.v_cache = static_cast<const char*>(v_cache_layer);
  p.block_tables = block_tables;
  p.seq_lens = kv_lens;
  p.query_start_loc = query_start_loc;
  p.query_positions = positions;
  p.qsl_rows = rows;
  p.out = out;
  p.status = status;
  p.num_blocks = num_blocks;
  p.batch = token_bucket;
  p.table_width = table_width;
  p.block_size = block_size;
  p.num_kv_heads = num_kv_heads;
  p.num_q_heads = num_q_heads;
  p.head_dim = head_dim;
  p.q_dtype = q_dtype;
  p.kv_dtype = kv_dtype;
  p.scale = scale;
  return launch_decode_generic(p, static_cast<cudaStream_t>(stream));
}
