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
                         int skip_single, int split_p, float* split_area, size_t split_bytes, cudaStream_t stream);
bool prefill_umma2_usable(float scale, long long num_blocks);
int launch_prefill_umma(const void* q, int q_dtype, const char* k_cache, const char* v_cache,
                        long long num_blocks, const int32_t* block_tables, int table_width,
                        const int32_t* kv_lens, const int32_t* positions, const int32_t* query_start_loc,
                        int rows, int token_bucket, float scale, float* out, int32_t* status,
                        int skip_single, cudaStream_t stream);
}

namespace nvj {

struct PackedArgs {
  const void* q; int q_dtype;
  const void* k_cache_layer; const void* v_cache_layer; int kv_dtype;
  long long num_blocks; int block_size, num_kv_heads, head_dim, num_q_heads;
  const int32_t* block_tables; int table_width;
  const int32_t* kv_lens; const int32_t* positions; const int32_t* query_start_loc;
  int rows, token_bucket; float scale; float* out; int32_t* status;
  void* workspace; size_t workspace_bytes; int variant;
};

static int check_packed(const PackedArgs& a, bool* tile_ok) {
  if (a.rows < 0 || a.token_bucket < 0 || a.table_width < 0 || a.num_blocks < 0 || a.block_size <= 0 ||
      a.num_kv_heads <= 0 || a.num_q_heads <= 0 || a.head_dim <= 0)
    return NVJ_ERR_INVALID_ARGUMENT;
  if (a.num_q_heads % a.num_kv_heads != 0 || a.variant < 0 || a.variant > 5) return NVJ_ERR_INVALID_ARGUMENT;
  if (a.token_bucket == 0) return NVJ_OK;
  if (!a.q || !a.k_cache_layer || !a.v_cache_layer || !a.block_tables || !a.kv_lens || !a.positions ||
      !a.query_start_loc || !a.out || !a.status)
    return NVJ_ERR_INVALID_ARGUMENT;
  const bool a16 = ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k_cache_layer) |
                     reinterpret_cast<uintptr_t>(a.v_cache_layer) | reinterpret_cast<uintptr_t>(a.out)) & 15u) == 0;
  *tile_ok = a.kv_dtype == NVJ_BF16 && a.block_size == kBlk && a.num_kv_heads == kHkv && a.num_q_heads == kHq &&
             a.head_dim == kD && (a.q_dtype == NVJ_BF16 || a.q_dtype == NVJ_F32) && a16;
  if (a.variant >= 2 && !*tile_ok) return NVJ_ERR_UNSUPPORTED;
  return NVJ_OK;
}

// Rows that carry a single query token (the decode rows of a mixed batch), by the streaming decode kernel on at most
// `cta_limit` CTAs (0: one per SM).  `out` is zero where this pass writes nothing.  NVJ_ERR_WORKSPACE when the
// caller lent no usable workspace.
static int run_single_token_rows(const PackedArgs& a, int cta_limit, cudaStream_t s) {
  const int num_ctas = decode_num_ctas();
  DecodeParams d{};
  d.batch = a.rows;
  if (!a.workspace || num_ctas <= 0 || a.rows <= 0 ||
      carve_decode_workspace(d, a.workspace, a.workspace_bytes, ws_ml_bytes(num_ctas), ws_acc_bytes(num_ctas)) != NVJ_OK)
    return NVJ_ERR_WORKSPACE;
  d.q = a.q;
  d.k_cache = static_cast<const char*>(a.k_cache_layer);
  d.v_cache = static_cast<const char*>(a.v_cache_layer);
  d.block_tables = a.block_tables;
  d.seq_lens = a.kv_lens;
  d.query_start_loc = a.query_start_loc;
  d.query_positions = a.positions;
  d.qsl_rows = a.rows;
  d.packed_rows = 1;
  d.out = a.out;
  d.num_blocks = a.num_blocks;
  d.table_width = a.table_width;
  d.block_size = a.block_size;
  d.num_kv_heads = a.num_kv_heads;
  d.num_q_heads = a.num_q_heads;
  d.head_dim = a.head_dim;
  d.q_dtype = a.q_dtype;
  d.kv_dtype = a.kv_dtype;
  d.scale = a.scale;
  d.cta_limit = cta_limit;
  // bf16 queries: the tensor-core streaming kernel (it declines without a tensor-map encoder); else the CUDA-core one
  int rc = NVJ_ERR_UNSUPPORTED;
  if (a.q_dtype == NVJ_BF16) {
    d.width = 1;
    rc = launch_decode_wide(d, s);
    d.width = 0;
  }
  if (rc == NVJ_ERR_UNSUPPORTED)
    rc = launch_decode_pipelined(d, cta_limit > 0 && cta_limit < num_ctas ? cta_limit : num_ctas, s);
  return rc;
}

// Whether the CTA-pair kernel will serve this call: it and the decode-row pass zero what they do not write, so that the
// output needs no memset in front; the other tile kernels want a zeroed output when rows are left to the pass above.
static bool pair_kernel_serves(const PackedArgs& a) {
  return (a.variant == 0 || a.variant == 4 || a.variant == 5) && prefill_umma2_usable(a.scale, a.num_blocks);
}

// The query tiles: tcgen05 tiles first (CTA pairs, then single CTAs); they decline when the driver has no tensor-map
// encoder or the scale is not positive, and the mma.sync tiles take over.  With skip_single the rows of one query
// token are left to the pass above (and, unless the pair kernel serves the call, `out` has been zeroed by the caller).
static int run_tiles(const PackedArgs& a, int skip_single, cudaStream_t s) {
  const char* kc = static_cast<const char*>(a.k_cache_layer);
  const char* vc = static_cast<const char*>(a.v_cache_layer);
  const int variant = a.variant;
  if (variant == 0 || variant == 4 || variant == 5) {
    // A workspace with room between the header and the decode partials (what run_single_token_rows carves from the
    // same buffer) lets a short batch split every tile's key range over several CTA pairs.
    float* split_area = nullptr;
    size_t split_bytes = 0;
    const int num_ctas = decode_num_ctas();
    // (not in a mixed batch, whose decode rows have just been served from the same workspace: there the extra merge
    // launch costs a host-bound step more than the split saves)
    if (!skip_single && a.workspace && num_ctas > 0 && (reinterpret_cast<uintptr_t>(a.workspace) & 15u) == 0) {
      const size_t end = a.workspace_bytes / kWsAlign * kWsAlign;
      const size_t tail = ws_ml_bytes(num_ctas) + ws_acc_bytes(num_ctas), head = ws_header_bytes(a.rows);
      if (end > head + tail) {
        split_bytes = (end - head - tail) / kWsAlign * kWsAlign;
        split_area = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + end - tail - split_bytes);
      }
    }
    const int rc = launch_prefill_umma2(a.q, a.q_dtype, kc, vc, a.num_blocks, a.block_tables, a.table_width, a.kv_lens, a.positions,
                                        a.query_start_loc, a.rows, a.token_bucket, a.scale, a.out, a.status, skip_single,
                                        variant == 5 ? 0 : 1, split_area, split_bytes, s);
    if (rc != NVJ_ERR_UNSUPPORTED || variant != 0) return rc;
  }
  if (variant == 0 || variant == 3) {
    const int rc = launch_prefill_umma(a.q, a.q_dtype, kc, vc, a.num_blocks, a.block_tables, a.table_width, a.kv_lens, a.positions,
                                       a.query_start_loc, a.rows, a.token_bucket, a.scale, a.out, a.status, skip_single, s);
    if (rc != NVJ_ERR_UNSUPPORTED || variant == 3) return rc;
  }
  return launch_prefill_mma(a.q, a.q_dtype, kc, vc, a.num_blocks, a.block_tables, a.table_width, a.kv_lens, a.positions,
                            a.query_start_loc, a.rows, a.token_bucket, a.scale, a.out, a.status, skip_single, s);
}

static int run_generic(const PackedArgs& a, cudaStream_t s) {
  DecodeParams p{};
  p.q = a.q;
  p.k_cache = static_cast<const char*>(a.k_cache_layer);
  p.v_cache = static_cast<const char*>(a.v_cache_layer);
  p.block_tables = a.block_tables;
  p.seq_lens = a.kv_lens;
  p.query_start_loc = a.query_start_loc;
  p.query_positions = a.positions;
  p.qsl_rows = a.rows;
  p.out = a.out;
  p.status = a.status;
  p.num_blocks = a.num_blocks;
  p.batch = a.token_bucket;
  p.table_width = a.table_width;
  p.block_size = a.block_size;
  p.num_kv_heads = a.num_kv_heads;
  p.num_q_heads = a.num_q_heads;
  p.head_dim = a.head_dim;
  p.q_dtype = a.q_dtype;
  p.kv_dtype = a.kv_dtype;
  p.scale = a.scale;
  return launch_decode_generic(p, s);
}

}  // namespace nvj

extern "C" size_t nvj_paged_prefill_workspace_bytes(int max_rows) {
  using namespace nvj;
  if (max_rows < 0) return 0;
  const int n = decode_num_ctas();
  if (n <= 0) return 0;
  return ws_header_bytes(max_rows) + prefill_split_bytes() + ws_ml_bytes(n) + ws_acc_bytes(n);
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
  const PackedArgs a{q, q_dtype, k_cache_layer, v_cache_layer, kv_dtype, num_blocks, block_size, num_kv_heads, head_dim,
                     num_q_heads, block_tables, table_width, kv_lens, positions, query_start_loc, rows, token_bucket,
                     scale, out, status, workspace, workspace_bytes, variant};
  bool tile_ok = false;
  const int rc = check_packed(a, &tile_ok);
  if (rc != NVJ_OK || token_bucket == 0) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!tile_ok || variant == 1) return run_generic(a, s);
  // Rows that carry a single query token go to the streaming decode kernel when the caller lends it a decode
  // workspace; everything else goes to the tile kernel.
  int skip_single = 0;
  if (workspace && rows > 0) {
    if (!pair_kernel_serves(a) &&
        cudaMemsetAsync(out, 0, sizeof(float) * (size_t)token_bucket * kHq * kD, s) != cudaSuccess)
      return NVJ_ERR_LAUNCH;
    const int rc1 = run_single_token_rows(a, 0, s);
    if (rc1 == NVJ_OK) skip_single = 1;
    else if (rc1 != NVJ_ERR_WORKSPACE) return rc1;
  }
  return run_tiles(a, skip_single, s);
}

extern "C" int nvj_paged_prefill_packed_part(const void* q, int q_dtype, const void* k_cache_layer,
                                             const void* v_cache_layer, int kv_dtype,
                                             int64_t num_blocks, int block_size, int num_kv_heads,
                                             int head_dim, int num_q_heads,
                                             const int32_t* block_tables, int table_width,
                                             const int32_t* kv_lens, const int32_t* positions,
                                             const int32_t* query_start_loc, int rows,
                                             int token_bucket, float scale, float* out,
                                             int32_t* status, void* workspace, size_t workspace_bytes,
                                             int variant, int part, int cta_limit, nvj_stream_t stream) {
  using namespace nvj;
  const PackedArgs a{q, q_dtype, k_cache_layer, v_cache_layer, kv_dtype, num_blocks, block_size, num_kv_heads, head_dim,
                     num_q_heads, block_tables, table_width, kv_lens, positions, query_start_loc, rows, token_bucket,
                     scale, out, status, workspace, workspace_bytes, variant};
  if (part < 1 || part > 3 || cta_limit < 0) return NVJ_ERR_INVALID_ARGUMENT;
  bool tile_ok = false;
  const int rc = check_packed(a, &tile_ok);
  if (rc != NVJ_OK || token_bucket == 0) return rc;
  if (!tile_ok || variant == 1) return NVJ_ERR_UNSUPPORTED;  // the generic kernel serves a batch in one piece
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (part == 1) return run_single_token_rows(a, cta_limit, s);
  if (part == 2 && !pair_kernel_serves(a)) return NVJ_ERR_UNSUPPORTED;  // the other tile kernels want a zeroed output
  return run_tiles(a, part == 2 ? 1 : 0, s);
}
