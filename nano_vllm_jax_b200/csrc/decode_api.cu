// C ABI of the paged decode entry points: argument checks, workspace carving and
// kernel selection.  Nothing here allocates or synchronises.

#include "paged_decode.cuh"

namespace nvj {

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static bool pipelined_shape(const DecodeParams& p) {
  return p.kv_dtype == NVJ_BF16 && p.block_size == kBlk && p.num_kv_heads == kHkv &&
         p.num_q_heads == kHq && p.head_dim == kD && (p.q_dtype == NVJ_BF16 || p.q_dtype == NVJ_F32) &&
         aligned16(p.q) && aligned16(p.k_cache) && aligned16(p.v_cache) && aligned16(p.out) &&
         (!p.new_k || (aligned16(p.new_k) && aligned16(p.new_v)));
}

static int carve_workspace(DecodeParams& p, void* workspace, size_t bytes, int num_ctas) {
  return carve_decode_workspace(p, workspace, bytes, ws_ml_bytes(num_ctas), ws_acc_bytes(num_ctas));
}

static int run_decode(DecodeParams& p, void* workspace, size_t workspace_bytes, int variant,
                      cudaStream_t stream) {
  if (p.batch < 0 || p.table_width < 0 || p.num_blocks < 0 || p.block_size <= 0 ||
      p.num_kv_heads <= 0 || p.num_q_heads <= 0 || p.head_dim <= 0)
    return NVJ_ERR_INVALID_ARGUMENT;
  if (p.num_q_heads % p.num_kv_heads != 0) return NVJ_ERR_INVALID_ARGUMENT;
  if (variant < 0 || variant > 3) return NVJ_ERR_INVALID_ARGUMENT;
  if (p.batch == 0) return NVJ_OK;
  if (!p.q || !p.k_cache || !p.v_cache || !p.block_tables || !p.seq_lens || !p.out)
    return NVJ_ERR_INVALID_ARGUMENT;
  if (p.new_k && !p.new_v) return NVJ_ERR_INVALID_ARGUMENT;
  p.pre_append = (p.new_k && !p.positions) ? 1 : 0;
  const int num_ctas = decode_num_ctas();
  if (num_ctas <= 0) return NVJ_ERR_LAUNCH;
  const int rc = carve_workspace(p, workspace, workspace_bytes, num_ctas);
  if (rc != NVJ_OK) return rc;
  const bool fast_ok = pipelined_shape(p) && (!p.new_k || !p.kv_indptr);
  // The tensor-core streaming kernel (bf16 queries) first: one CTA per SM, whole blocks by TMA, products on
  // mma.sync tiles; it needs a tensor-map encoder from the driver.  Then the CUDA-core pipelined kernel.
  const bool mma_ok = fast_ok && p.q_dtype == NVJ_BF16;
  if ((variant == 2 && !fast_ok) || (variant == 3 && !mma_ok)) return NVJ_ERR_UNSUPPORTED;
  if (variant == 3 || (variant == 0 && mma_ok)) {
    p.width = 1;
    const int rc3 = launch_decode_wide(p, stream);
    if (rc3 != NVJ_ERR_UNSUPPORTED || variant == 3) return rc3;
    p.width = 0;
  }
  if (variant == 2 || (variant == 0 && fast_ok)) return launch_decode_pipelined(p, num_ctas, stream);
  if (p.new_k) {
    if (p.kv_indptr) return NVJ_ERR_UNSUPPORTED;
    const int a = append_decode_rows(p.new_k, p.new_v, p.pre_append ? p.seq_lens : p.positions, p.seq_lens,
                                     const_cast<char*>(p.k_cache), const_cast<char*>(p.v_cache),
                                     p.kv_dtype, p.num_blocks, p.block_size,
                                     p.num_kv_heads * p.head_dim, p.block_tables, p.table_width,
                                     p.batch, p.status, stream);
    if (a != NVJ_OK) return a;
  }
  return launch_decode_generic(p, stream);
}

}  // namespace nvj

extern "C" size_t nvj_paged_decode_workspace_bytes(int max_batch) {
  using namespace nvj;
  if (max_batch < 0) return 0;
  const int n = decode_num_ctas();
  if (n <= 0) return 0;
  return ws_header_bytes(max_batch) + ws_ml_bytes(n) + ws_acc_bytes(n);
}

extern "C" int nvj_paged_decode_workspace_init(void* workspace, size_t workspace_bytes,
                                               nvj_stream_t stream) {
  if (!workspace || workspace_bytes == 0) return NVJ_ERR_WORKSPACE;
  return cudaMemsetAsync(workspace, 0, workspace_bytes, static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? NVJ_OK
             : NVJ_ERR_LAUNCH;
}

extern "C" int nvj_paged_decode(const void* q, int q_dtype, const void* k_cache_layer,
                                const void* v_cache_layer, int kv_dtype, int64_t num_blocks,
                                int block_size, int num_kv_heads, int head_dim, int num_q_heads,
                                const int32_t* block_tables, int table_width,
                                const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                                const int32_t* seq_lens, int batch, float scale, float* out,
                                void* workspace, size_t workspace_bytes, int variant,
                                nvj_stream_t stream) {
  nvj::DecodeParams p{};
  p.q = q;
  p.k_cache = static_cast<const char*>(k_cache_layer);
  p.v_cache = static_cast<const char*>(v_cache_layer);
  p.block_tables = block_tables;
  p.kv_indptr = kv_indptr;
  p.kv_last_page_len = kv_last_page_len;
  p.seq_lens = seq_lens;
  p.out = out;
  p.num_blocks = num_blocks;
  p.batch = batch;
  p.table_width = table_width;
  p.block_size = block_size;
  p.num_kv_heads = num_kv_heads;
  p.num_q_heads = num_q_heads;
  p.head_dim = head_dim;
  p.q_dtype = q_dtype;
  p.kv_dtype = kv_dtype;
  p.scale = scale;
  return nvj::run_decode(p, workspace, workspace_bytes, variant, static_cast<cudaStream_t>(stream));
}

extern "C" int nvj_paged_decode_fused_append(const void* q, int q_dtype, const void* new_k,
                                             const void* new_v, const int32_t* positions,
                                             void* k_cache_layer, void* v_cache_layer, int kv_dtype,
                                             int64_t num_blocks, int block_size, int num_kv_heads,
                                             int head_dim, int num_q_heads,
                                             const int32_t* block_tables, int table_width,
                                             const int32_t* seq_lens, int batch, float scale,
                                             float* out, void* workspace, size_t workspace_bytes,
                                             int variant, nvj_stream_t stream) {
  if (batch > 0 && (!new_k || !new_v)) return NVJ_ERR_INVALID_ARGUMENT;
  nvj::DecodeParams p{};
  p.q = q;
  p.k_cache = static_cast<const char*>(k_cache_layer);
  p.v_cache = static_cast<const char*>(v_cache_layer);
  p.block_tables = block_tables;
  p.seq_lens = seq_lens;
  p.new_k = new_k;
  p.new_v = new_v;
  p.positions = positions;
  p.out = out;
  p.num_blocks = num_blocks;
  p.batch = batch;
  p.table_width = table_width;
  p.block_size = block_size;
  p.num_kv_heads = num_kv_heads;
  p.num_q_heads = num_q_heads;
  p.head_dim = head_dim;
  p.q_dtype = q_dtype;
  p.kv_dtype = kv_dtype;
  p.scale = scale;
  return nvj::run_decode(p, workspace, workspace_bytes, variant, static_cast<cudaStream_t>(stream));
}
