/*
 * nvj_b200.h — C ABI of the B200 (sm_100a) paged KV-cache hot path.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream, launches
 * asynchronously on that stream, never synchronises the host, and returns 0 or a
 * negative nvj_status code.  No torch / JAX types appear in any signature.  The
 * functions are the plain-C form of the reference project's kernel ABI for this
 * path; the citation on each declaration names the reference interface it
 * replaces (paths are relative to the reference project root).
 *
 * Layouts (identical to the reference, nanovllm_jax/kv_cache.py:22-32):
 *   cache layer   [num_blocks, block_size, num_kv_heads, head_dim]   (one layer slice)
 *   flat slot     slot = block_id * block_size + position % block_size
 *   block tables  [rows, table_width] int32, unused entries 0
 *
 * Process state.  The compute entry points allocate nothing and keep no per-call state; what the library keeps
 * per process is (a) a cache of encoded TMA tensor maps keyed by (base address, extent), behind a mutex,
 * (b) once-per-device kernel attributes set on first use (guarded), (c) the wait limit of nvj_set_wait_limit_ns,
 * (d) the device address of the static scratch of nvj_paged_decode_static_scratch.  All entry points may be called
 * from several host threads.  The set-up calls nvj_p2p_buffer_create / open / close / destroy allocate, map and
 * synchronise by design; nothing else does.
 *
 * Device-side problems (a block id outside the pool, a wait that ran out) never
 * trap: the kernel skips the access, ORs a NVJ_DEV_* bit into a status word and
 * returns.  The status word is `int32_t* status` where a function takes one, or
 * word 0 of the decode workspace.
 */
#ifndef NVJ_B200_H_
#define NVJ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NVJ_ABI_VERSION 1

/* cudaStream_t, kept opaque so the header needs no CUDA include. */
typedef void* nvj_stream_t;

typedef enum nvj_status {
  NVJ_OK = 0,
  NVJ_ERR_INVALID_ARGUMENT = -1, /* null pointer, negative size, bad alignment   */
  NVJ_ERR_UNSUPPORTED = -2,      /* shape / dtype outside what the kernels cover */
  NVJ_ERR_LAUNCH = -3,           /* cudaGetLastError() after the launch          */
  NVJ_ERR_WORKSPACE = -4,        /* workspace missing or too small               */
  NVJ_ERR_TOO_LARGE = -5         /* size beyond a built-in limit of the entry point */
} nvj_status;

typedef enum nvj_dtype { NVJ_BF16 = 0, NVJ_F16 = 1, NVJ_F32 = 2 } nvj_dtype;

/* Bits a kernel may OR into a device status word. */
#define NVJ_DEV_TIMEOUT 1      /* a bounded wait ran out; results are invalid   */
#define NVJ_DEV_BAD_BLOCK_ID 2 /* block id / slot outside the pool; skipped     */
#define NVJ_DEV_BAD_LENGTH 4   /* seq_len beyond table_width * block_size; clipped */

int nvj_abi_version(void);
const char* nvj_status_string(int status);

/* ------------------------------------------------------------- slot mapping */

/*
 * slot[b, t] = block_tables[row, pos / bs] * bs + pos % bs for positions [n_rows, n_cols].
 * row = b when token_row_ids == NULL (nanovllm_jax/kv_cache.py:410-446, compute_slot_mapping),
 * else the token's token_row_ids entry clipped to [0, table_rows) (kv_cache.py:449-473,
 * compute_packed_slot_mapping).  A block index beyond the table is clamped to its last
 * column, as the reference's XLA gather does.
 */
int nvj_compute_slot_mapping(const int32_t* positions, const int32_t* block_tables,
                             const int32_t* token_row_ids, int n_rows, int n_cols,
                             int table_rows, int table_width, int block_size,
                             int32_t* slot_mapping, nvj_stream_t stream);

/* ------------------------------------------------------------------ append */

/*
 * Slot-mapped append of new K/V rows into one layer of the paged cache.
 * Replaces nanovllm_jax/kv_cache.py:476-564 (update_kv_cache) as called from
 * nanovllm_jax/backends.py:980-1067 (PureJAXBackend.write_kv).
 *
 *   new_k/new_v    [n_rows, n_cols, num_kv_heads, head_dim], src_dtype
 *   slot_mapping   [n_rows, n_cols] int32 flat slots
 *   valid_mask     nullable [n_rows, n_cols] int32, non-zero = write
 *   query_start_loc nullable [qsl_rows + 1] int32.  packed != 0: token i is
 *                  written iff i < query_start_loc[qsl_rows] (backends.py:1050-1054);
 *                  packed == 0: token (b, t) iff t < qsl[b+1] - qsl[b] (1055-1057).
 * A token must pass every rule that is given.  Source rows are converted to
 * cache_dtype (f32 -> bf16/f16 round-to-nearest-even; same dtype = byte copy).
 * Slots outside [0, num_slots) are skipped and flagged NVJ_DEV_BAD_BLOCK_ID.
 * Two valid tokens with the same slot: last writer unspecified (as in XLA).
 */
int nvj_kv_append(const void* new_k, const void* new_v, int src_dtype,
                  const int32_t* slot_mapping, const int32_t* valid_mask,
                  const int32_t* query_start_loc, int qsl_rows, int packed,
                  int n_rows, int n_cols,
                  void* k_cache_layer, void* v_cache_layer, int cache_dtype,
                  int64_t num_slots, int num_kv_heads, int head_dim,
                  int32_t* status, nvj_stream_t stream);

/*
 * Page-table (CSR) form of the append: page = kv_indices[kv_indptr[b] + pos / P],
 * cache[page, pos % P] = append[i].  Replaces the FP32 custom call
 * nanovllm_jax/kernels/cuda_fp32_ffi.py:323-382 (handler
 * nanovllm_jax/kernels/csrc/fp32_kv_append.cu:801-841,1563-1627) and the
 * reference nanovllm_jax/kernels/flashinfer_ffi.py:626-665.
 */
int nvj_kv_append_nhd(const void* append_key, const void* append_value, int src_dtype,
                      const int32_t* batch_indices, const int32_t* positions, int nnz,
                      void* k_cache, void* v_cache, int cache_dtype,
                      int64_t num_pages, int page_size, int num_kv_heads, int head_dim,
                      const int32_t* kv_indices, int64_t kv_indices_len,
                      const int32_t* kv_indptr, int batch,
                      const int32_t* valid_mask,
                      int32_t* status, nvj_stream_t stream);

/*
 * The step in front of the path fused with the append: per-head RMSNorm ((1 + w) form) of the
 * query and key rows, half-split rotary embedding of their first `rotary_dim` elements, then
 * key and value rows are stored at their slots and the query is returned ready for attention.
 * Replaces the sequence rms_norm(q), rms_norm(k), apply_rope(q), apply_rope(k), write_kv of
 * nanovllm_jax/model.py:3371-3396 + 3539-3550 (nanovllm_jax/layers.py:11-29, 49-199); the
 * reference lists this fusion as its roadmap item P2.2 (docs/kernel_roadmap.md:26, 416-419).
 *
 *   q        token i, head h at q + i * q_token_stride + h * q_head_stride (elements), so a
 *            query that lives inside a [tokens, heads, 2 * head_dim] query|gate projection
 *            needs no copy; k, v rows [num_kv_heads, head_dim] at token strides
 *   weights  q_norm, k_norm [head_dim], bf16 or f32
 *   inv_freq [rotary_dim / 2] f32, the framework's own 1 / theta^(2 i / rotary_dim) table
 *   rope_positions [position_rows, tokens]: one row (text) or three rows (temporal, height, width) of a
 *            multimodal position id; with three rows `mrope_section` (HOST array of 3 ints, e.g. 11 / 11 / 10)
 *            selects the row per frequency as nanovllm_jax/layers.py:79-139 does (positions are stacked x3
 *            at nanovllm_jax/model.py:3955; equal rows give the text result)
 *   slots and masks as in nvj_kv_append; q_out [tokens, num_q_heads, head_dim] bf16
 * bf16 activations and cache, head_dim 64 / 128 / 256; otherwise NVJ_ERR_UNSUPPORTED.
 */
int nvj_qk_norm_rope_kv_append(const void* q, int64_t q_token_stride, int64_t q_head_stride,
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
                               void* q_out, int32_t* status, nvj_stream_t stream);

/* ------------------------------------------------------------------ decode */

/*
 * Bytes of caller-owned scratch the decode entry points need for `max_batch`
 * rows on the current device.  The front of the buffer (64 bytes of status, 256 bytes of group
 * counters, 4 bytes per row) holds the status word and the arrival counters and must be zero before the
 * first use (nvj_paged_decode_workspace_init does that); the kernels leave them zero again on success.
 * The partial results live at the END of the buffer, so one buffer serves calls of any batch size up to
 * `max_batch`, of either decode entry point and of any width, one after another: pass the same
 * `workspace_bytes` (the buffer's size) on every call.  One workspace serves one stream at a time.
 */
size_t nvj_paged_decode_workspace_bytes(int max_batch);
int nvj_paged_decode_workspace_init(void* workspace, size_t workspace_bytes,
                                    nvj_stream_t stream);

/*
 * Width-1 paged GQA decode attention over one cache layer, online softmax,
 * fp32 accumulate, fp32 output.  Replaces nanovllm_jax/kv_cache.py:852-998
 * (paged_attention_decode), nanovllm_jax/kernels/paged_attention.py:101-194
 * and the FP32 custom call nanovllm_jax/kernels/cuda_fp32_ffi.py:527-572
 * (handler nanovllm_jax/kernels/csrc/fp32_kv_append.cu:843-957,1629-1697).
 *
 *   q            [batch, num_q_heads, head_dim], q_dtype (bf16 or f32)
 *   block_tables int32; row b starts at kv_indptr[b] when kv_indptr != NULL,
 *                else at b * table_width
 *   seq_lens     [batch] int32 keys attended per row; rows with len <= 0 get zeros
 *   kv_last_page_len nullable [batch]; with kv_indptr it clips the length to
 *                (pages - 1) * P + last_page_len as paged_attention.py:171-178 does
 *   out          [batch, num_q_heads, head_dim] float32
 *   variant      0 = auto, 1 = generic kernel; for the model's shape (bf16 cache, block_size 16,
 *                2 kv heads x 4 q heads, head_dim 256): 2 = bulk-copy pipelined kernel on the CUDA
 *                cores (bf16 or f32 queries), 3 = TMA-staged streaming kernel with the products on
 *                tensor-core tiles (bf16 queries; what auto picks first).  NVJ_ERR_UNSUPPORTED when
 *                2 or 3 is asked for another shape.
 */
int nvj_paged_decode(const void* q, int q_dtype,
                     const void* k_cache_layer, const void* v_cache_layer, int kv_dtype,
                     int64_t num_blocks, int block_size, int num_kv_heads, int head_dim,
                     int num_q_heads,
                     const int32_t* block_tables, int table_width,
                     const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                     const int32_t* seq_lens, int batch, float scale,
                     float* out,
                     void* workspace, size_t workspace_bytes,
                     int variant, nvj_stream_t stream);

/*
 * Fused decode step: write row b's new K/V at positions[b], then attend
 * seq_lens[b] keys (the new one included).  Replaces
 * nanovllm_jax/kernels/full_attention_triton.py:488-581
 * (paged_decode_attention_with_kv_append_triton) behind
 * nanovllm_jax/backends.py:1411-1442.  new_k/new_v are [batch, num_kv_heads,
 * head_dim] in the cache dtype.  Rows with seq_lens[b] <= 0 are inactive: no
 * write, zero output.  Cache contents equal nvj_kv_append followed by
 * nvj_paged_decode bit for bit.
 * positions == NULL is the pre-append form for device-resident metadata: seq_lens[b] then is the row's length BEFORE
 * this step's token, the new row goes to position seq_lens[b] and seq_lens[b] + 1 keys are attended; nothing is
 * written to seq_lens (nvj_row_argmax_advance / nvj_p2p_argmax_publish advance it at the end of the step).  A row
 * whose block table has no room left is flagged NVJ_DEV_BAD_LENGTH / NVJ_DEV_BAD_BLOCK_ID as in the other form.
 */
int nvj_paged_decode_fused_append(const void* q, int q_dtype,
                                  const void* new_k, const void* new_v,
                                  const int32_t* positions,
                                  void* k_cache_layer, void* v_cache_layer, int kv_dtype,
                                  int64_t num_blocks, int block_size, int num_kv_heads,
                                  int head_dim, int num_q_heads,
                                  const int32_t* block_tables, int table_width,
                                  const int32_t* seq_lens, int batch, float scale,
                                  float* out,
                                  void* workspace, size_t workspace_bytes,
                                  int variant, nvj_stream_t stream);

/*
 * nvj_paged_decode for callers that cannot allocate device memory (no counterpart
 * in the reference).  A custom-call handler that only receives its operands, or a
 * plugin that runs inside another runtime's memory pool, has nowhere to keep the
 * decode workspace; here it comes from a fixed array inside the library
 * (NVJ_STATIC_SCRATCH_BYTES on every GPU that loads the library), so the call
 * itself allocates nothing.  Same arguments and results as nvj_paged_decode over a
 * dense block table, minus the workspace.
 *
 *   limit        batch <= NVJ_STATIC_SCRATCH_MAX_BATCH, else NVJ_ERR_TOO_LARGE
 *   status_out   nullable device int32: receives the NVJ_DEV_* bits of this call
 *   first call   the first call on each device resolves the array's device address
 *                (cudaGetSymbolAddress); make that first call outside any stream
 *                capture.  Later calls only enqueue a small memset, the kernel and
 *                an optional 4-byte copy.
 *   sharing      every call on a device uses the same array: calls that may overlap
 *                on the GPU (different streams, no dependency) race and must be
 *                serialised by the caller.
 */
#define NVJ_STATIC_SCRATCH_MAX_BATCH 4096
#define NVJ_STATIC_SCRATCH_BYTES 5713664
int nvj_paged_decode_static_scratch(const void* q, int q_dtype,
                                    const void* k_cache_layer, const void* v_cache_layer,
                                    int kv_dtype, int64_t num_blocks, int block_size,
                                    int num_kv_heads, int head_dim, int num_q_heads,
                                    const int32_t* block_tables, int table_width,
                                    const int32_t* seq_lens, int batch, float scale,
                                    float* out, int32_t* status_out, nvj_stream_t stream);

/*
 * Paged decode attention for rows that carry 2..8 query tokens (verification of speculated
 * tokens; the reference's wide decode, nanovllm_jax/kv_cache.py:852-998 with query width T > 1,
 * reached from nanovllm_jax/backends.py:1266-1359 and nanovllm_jax/mtp/mtp_layer.py:686).
 * The rows' K/V must already be appended.  Key p of row b is visible to token t when
 * p < seq_lens[b] and (positions given) p <= positions[b, t].  The model's shape only: bf16
 * query and cache, block 16, 2 KV x 4 query heads, head_dim 256; each K/V byte is read once for
 * all of a row's tokens, the products run on the tensor cores (one 16-row tile per KV head up to width 4, two
 * from width 5 on: the tensor work per block doubles, the HBM traffic does not).
 *
 *   q          [batch, width, 8, 256] bf16
 *   positions  [batch, width] int32, nullable (no causal limit)
 *   out        [batch, width, 8 * 256] float32; rows with seq_lens <= 0 give zeros
 *   workspace  nvj_paged_decode_wide_workspace_bytes(max_batch) bytes, zeroed once
 *              (nvj_paged_decode_workspace_init) and then reused; its first word is the device
 *              status word
 * NVJ_ERR_UNSUPPORTED for width > 16 or misaligned pointers (use nvj_paged_prefill_packed with
 * rows of equal width instead); widths 9-16 (the reference verifies up to 9 tokens per row) exist on the tcgen05
 * form only.
 */
size_t nvj_paged_decode_wide_workspace_bytes(int max_batch);
/*
 * nvj_paged_decode_wide_form: the same call with the kernel chosen by the caller.  form 0 = automatic (what
 * nvj_paged_decode_wide does: widths 1-4 on mma.sync tiles, 16 query rows per warp; widths 5-8 on tcgen05, the 4 x width
 * query rows of a KV head in a 128-row tile with scores and output in tensor memory, a row cut over several CTA pairs
 * folded by a second small launch), 1 = mma.sync tiles (widths 5-8: two row tiles per warp pair, ~1.9x the width-1
 * time; NVJ_ERR_UNSUPPORTED beyond 8), 2 = tcgen05 at any width 1-16 (NVJ_ERR_UNSUPPORTED without a tensor-map
 * encoder or for scale <= 0).
 */
int nvj_paged_decode_wide_form(const void* q, const void* k_cache_layer, const void* v_cache_layer,
                               int64_t num_blocks, const int32_t* block_tables, int table_width,
                               const int32_t* seq_lens, const int32_t* positions, int batch, int width,
                               float scale, float* out, void* workspace, size_t workspace_bytes,
                               int form, nvj_stream_t stream);
int nvj_paged_decode_wide(const void* q, const void* k_cache_layer, const void* v_cache_layer,
                          int64_t num_blocks, const int32_t* block_tables, int table_width,
                          const int32_t* seq_lens, const int32_t* positions, int batch, int width,
                          float scale, float* out, void* workspace, size_t workspace_bytes,
                          nvj_stream_t stream);

/* ----------------------------------------------------------------- prefill */

/*
 * Ragged packed prefill attention over the paged cache (this chunk's rows are
 * already appended).  Token i of row r at absolute position positions[i] attends
 * keys p < kv_lens[r] and p <= positions[i]; tokens at or beyond
 * query_start_loc[rows] produce zeros.  Replaces
 * nanovllm_jax/kv_cache.py:721-849 (paged_attention_prefill_packed) and
 * nanovllm_jax/kernels/full_attention_triton.py:148-221.
 *
 *   q          [token_bucket, num_q_heads, head_dim], q_dtype
 *   out        [token_bucket, num_q_heads, head_dim] float32
 *   workspace  nullable decode workspace (nvj_paged_decode_workspace_bytes(rows)); when given,
 *              rows that hold exactly one query token (the decode rows of a mixed batch,
 *              nanovllm_jax/engine/scheduler.py:956-1032) are served by the streaming decode
 *              kernel instead of a query tile.  A workspace of nvj_paged_prefill_workspace_bytes(rows)
 *              bytes also lets the CTA-pair tile kernel (variants 0, 4, 5) split every tile's key
 *              range over several CTA pairs when the batch is too short to fill the GPU (a
 *              512-token chunk is 16 pairs on 74 pair slots): the splits park their un-normalised
 *              rows between the workspace's header and the decode partials, and a second small
 *              launch behind the tile kernel folds them (batches without single-token rows only).
 *   variant    0 = automatic; 1 = generic CUDA-core kernel (any shape or dtype); for the model's
 *              shape (bf16 cache, block 16, 2 KV x 4 query heads, head_dim 256): 2 = mma.sync
 *              tiles of 16 tokens, 3 = tcgen05 tiles of 32 tokens with accumulators in tensor
 *              memory, 4 = the same on CTA pairs (cta_group::2, 64 tokens per pair; what
 *              automatic picks first), 5 = as 4 with the softmax weights entering P V as one
 *              bf16 term instead of two (what the reference's Triton kernel does, `p.to(v.dtype)`,
 *              nanovllm_jax/kernels/full_attention_triton.py:51-145): ~1.3x faster on long
 *              prompts, max-abs error ~3e-3 instead of < 2e-3 against an fp32 softmax.
 *              NVJ_ERR_UNSUPPORTED when 2-5 is asked for another shape.
 */
size_t nvj_paged_prefill_workspace_bytes(int max_rows);
int nvj_paged_prefill_packed(const void* q, int q_dtype,
                             const void* k_cache_layer, const void* v_cache_layer, int kv_dtype,
                             int64_t num_blocks, int block_size, int num_kv_heads,
                             int head_dim, int num_q_heads,
                             const int32_t* block_tables, int table_width,
                             const int32_t* kv_lens, const int32_t* positions,
                             const int32_t* query_start_loc, int rows,
                             int token_bucket, float scale,
                             float* out, int32_t* status,
                             void* workspace, size_t workspace_bytes, int variant,
                             nvj_stream_t stream);

/*
 * The two halves of nvj_paged_prefill_packed as separate launches, for a caller that runs them side by side on two
 * streams: in a mixed batch (nanovllm_jax/engine/scheduler.py:956-1032) the decode rows and the prefill chunks
 * write different rows of `out`, and neither kernel fills the machine alone.  Same arguments; the model's shape
 * only (NVJ_ERR_UNSUPPORTED otherwise: the generic kernel serves a batch in one piece).  Neither part wants `out`
 * zeroed: each zeroes what it owns and does not write (rows without keys, padding tokens).
 *   part 1   rows that hold exactly one query token, on the streaming decode kernel with at most `cta_limit` CTAs
 *            (0 = one per SM; give the SM count minus the CTAs of part 2); `workspace` is required
 *   part 2   every other row, on the CTA-pair tile kernel (variant 0, 4 or 5; NVJ_ERR_UNSUPPORTED for another variant,
 *            or when that kernel cannot run: call nvj_paged_prefill_packed instead); `workspace` (nullable, NOT the
 *            buffer part 1 is using at the same time) only gives the key-range splits of a short batch their room
 *   part 3   all rows on the tile kernel, which then zeroes what it does not write itself (no zeroed `out` needed):
 *            a batch without decode rows that still wants the key-range splits
 * The reference runs a mixed batch through one packed attention call; the split has no counterpart there.
 */
int nvj_paged_prefill_packed_part(const void* q, int q_dtype,
                                  const void* k_cache_layer, const void* v_cache_layer, int kv_dtype,
                                  int64_t num_blocks, int block_size, int num_kv_heads,
                                  int head_dim, int num_q_heads,
                                  const int32_t* block_tables, int table_width,
                                  const int32_t* kv_lens, const int32_t* positions,
                                  const int32_t* query_start_loc, int rows,
                                  int token_bucket, float scale,
                                  float* out, int32_t* status,
                                  void* workspace, size_t workspace_bytes, int variant,
                                  int part, int cta_limit, nvj_stream_t stream);

/* ------------------------------------------------------------------ copies */

/*
 * Copy whole cache blocks dst_ids[i] <- src_ids[i] in every layer of K and V
 * (prefix reuse by copy; the oracle is cache[:, dst] = cache[:, src]).  The
 * reference shares prefix blocks by reference count
 * (nanovllm_jax/engine/block_manager.py:194-254) and has no copy; this entry
 * point serves callers that need a private copy of a shared prefix.
 * layer_stride_bytes = num_blocks * block_bytes for the contiguous 5-D cache.
 */
int nvj_copy_blocks(void* k_cache, void* v_cache, int num_layers,
                    int64_t num_blocks, int64_t block_bytes, int64_t layer_stride_bytes,
                    const int32_t* src_ids, const int32_t* dst_ids, int n_pairs,
                    int32_t* status, nvj_stream_t stream);

/*
 * GDN hybrid-state snapshot: pool[pool_slots[i]] <- table[table_slots[i]] for
 * the conv-state and recurrent-state arrays (either may be NULL).  Replaces
 * nanovllm_jax/engine/model_runner.py:3843-3854 (_get_hybrid_state).
 * row bytes: conv = layers*conv_dim*kernel*itemsize, recurrent = layers*H*Dv*Dk*4.
 */
int nvj_hybrid_snapshot(const void* conv_table, void* conv_pool, int64_t conv_row_bytes,
                        const void* rec_table, void* rec_pool, int64_t rec_row_bytes,
                        int64_t table_rows, int64_t pool_rows,
                        const int32_t* table_slots, const int32_t* pool_slots, int n,
                        int32_t* status, nvj_stream_t stream);

/*
 * GDN hybrid-state restore: table[table_slots[i]] <- pool[pool_slots[i]].
 * Replaces nanovllm_jax/engine/model_runner.py:3856-3867 (_set_hybrid_state)
 * as driven by install_cached_prefix_hybrid_states (3886-3905).
 */
int nvj_hybrid_restore(void* conv_table, const void* conv_pool, int64_t conv_row_bytes,
                       void* rec_table, const void* rec_pool, int64_t rec_row_bytes,
                       int64_t table_rows, int64_t pool_rows,
                       const int32_t* table_slots, const int32_t* pool_slots, int n,
                       int32_t* status, nvj_stream_t stream);

/*
 * The same two copies with the slot lists in HOST memory (n <= NVJ_HYBRID_HOST_SLOTS pairs, else NVJ_ERR_TOO_LARGE):
 * the indices travel in the kernel's parameters, so a restore of one sequence on a prefix hit is a single launch with
 * no host-to-device copy in front of it.  The arrays are read before the call returns.
 */
#define NVJ_HYBRID_HOST_SLOTS 24
int nvj_hybrid_snapshot_host_slots(const void* conv_table, void* conv_pool, int64_t conv_row_bytes,
                                   const void* rec_table, void* rec_pool, int64_t rec_row_bytes,
                                   int64_t table_rows, int64_t pool_rows,
                                   const int32_t* table_slots, const int32_t* pool_slots, int n,
                                   int32_t* status, nvj_stream_t stream);
int nvj_hybrid_restore_host_slots(void* conv_table, const void* conv_pool, int64_t conv_row_bytes,
                                  void* rec_table, const void* rec_pool, int64_t rec_row_bytes,
                                  int64_t table_rows, int64_t pool_rows,
                                  const int32_t* table_slots, const int32_t* pool_slots, int n,
                                  int32_t* status, nvj_stream_t stream);

/* ---------------------------------------------------- resident decode metadata */

/*
 * Advances device-resident decode metadata by one step without the host: for every row
 * with seq_lens[b] > 0, positions[b] = seq_lens[b] and seq_lens[b] += 1 (the scheduler's
 * decode batch has positions = num_tokens - 1, seq_lens = num_tokens,
 * nanovllm_jax/engine/scheduler.py:790-803).  Serves the reference's resident / static decode
 * metadata (nanovllm_jax/engine/scheduler.py:1100-1219, where the compiled executor recomputes
 * width-1 positions from seq_lens, nanovllm_jax/engine/model_executor.py:560-562), so that a
 * whole decode step can be replayed from a CUDA graph.  A row that would outgrow
 * table_width * block_size is flagged NVJ_DEV_BAD_LENGTH and not advanced.
 */
int nvj_advance_decode_metadata(int32_t* seq_lens, int32_t* positions, int batch,
                                int table_width, int block_size, int32_t* status,
                                nvj_stream_t stream);

/* ------------------------------------------------- token all-gather over NVLink */

/*
 * All-gather of n int32 per rank (the per-step output tokens) for one process per GPU on one
 * node, by peer stores into exchange buffers that the ranks map through CUDA IPC.  The reference
 * is single-device and has no counterpart; the host side that exchanges the handles is
 * nano_vllm_jax_b200/parallel.py (P2PTokenGather).
 *
 *   nvj_p2p_gather_buffer_bytes   size of one rank's exchange buffer for (world <= 16, n)
 *   nvj_p2p_buffer_create         cudaMalloc + zero + IPC handle (64 bytes) of this rank's buffer
 *   nvj_p2p_buffer_open / close   map / unmap a peer's buffer from its handle
 *   nvj_p2p_buffer_destroy        free this rank's buffer (after every peer has closed it)
 *   nvj_p2p_allgather_i32         one step, blocking: out[r * n + i] = rank r's local[i].  `peer_buffers` is a HOST array of
 *                                 `world` device pointers ([rank] = this rank's own buffer); `epoch` starts at 1 and
 *                                 grows by 1 per call on every rank, or is 0 on every call: the kernel then keeps
 *                                 the count in the rank's buffer (a launch that can be replayed from a CUDA graph).
 *                                 The kernel waits for its peers up to the wait limit (below) and then flags
 *                                 NVJ_DEV_TIMEOUT in *status and returns; with host-passed epochs the same call can
 *                                 simply be issued again.
 *
 * The split form keeps the wait out of the decode step (device-kept epochs only):
 *   nvj_p2p_argmax_publish        tokens[r] = argmax of row r of x [rows, row_len] (as nvj_row_argmax), stored locally
 *                                 and into every peer's buffer, then this rank's next epoch is published.  The publish
 *                                 waits for nobody.  rows must equal the n the buffers were sized for.  With
 *                                 `collect_out` (nullable) the same launch first collects the step before, as
 *                                 nvj_p2p_collect does: the usual form of a step, whose gathered tokens then lag by one.
 *                                 With `seq_lens` (nullable; `positions` nullable) it also advances the rows' resident
 *                                 decode metadata, as nvj_row_argmax_advance does, except that a row without room
 *                                 is only left alone, not flagged (the pre-append decode pass has flagged it).
 *   nvj_p2p_collect               waits (up to the wait limit) for the oldest published epoch not collected yet and
 *                                 writes out[r * n + i]; returns at once when there is none.  After the last step one
 *                                 call fetches the last tokens.  On a timeout NVJ_DEV_TIMEOUT is flagged in *status,
 *                                 nothing is consumed and the call can be repeated.
 * A rank must collect step k before it publishes step k + 1 (the fused form does); switch between the blocking and
 * the split form only when every published step has been collected.
 */
size_t nvj_p2p_gather_buffer_bytes(int world, int n);
int nvj_p2p_buffer_create(size_t bytes, void** dev_ptr, unsigned char* handle64);
int nvj_p2p_buffer_open(const unsigned char* handle64, void** dev_ptr);
int nvj_p2p_buffer_close(void* dev_ptr);
int nvj_p2p_buffer_destroy(void* dev_ptr);
int nvj_p2p_allgather_i32(const int32_t* local, int n, int rank, int world, void* const* peer_buffers,
                          uint32_t epoch, int32_t* out, int32_t* status, nvj_stream_t stream);
int nvj_p2p_argmax_publish(const float* x, int rows, int row_len, int32_t* tokens, int rank, int world,
                           void* const* peer_buffers, int32_t* collect_out, int32_t* seq_lens, int32_t* positions,
                           int table_width, int block_size, int32_t* status, nvj_stream_t stream);
int nvj_p2p_collect(void* own_buffer, int n, int world, int32_t* out, int32_t* status, nvj_stream_t stream);

/* ------------------------------------------------------------- bounded waits */

/*
 * No kernel of this library waits without a limit.  A wait on a CTA's own copies is bounded by a fixed 1 s; a wait
 * on another GPU (the token gather above) by the process-wide limit set here (default 1 s; 0 restores the default).
 * When a limit runs out the kernel ORs NVJ_DEV_TIMEOUT into its status word and returns; the context stays usable.
 * nvj_selftest_bounded_wait runs the mbarrier wait of the pipelined kernels on a barrier that nobody arrives on,
 * with the current limit: *status receives NVJ_DEV_TIMEOUT and *returned the number of threads that came back (64).
 * The reference has no device-side waits and no counterpart.
 */
void nvj_set_wait_limit_ns(uint64_t ns);
uint64_t nvj_get_wait_limit_ns(void);
int nvj_selftest_bounded_wait(int32_t* status, int32_t* returned, nvj_stream_t stream);

/* ------------------------------------------------------------------ host staging */

/*
 * n asynchronous copies on one stream, one cudaMemcpyAsync each, direction inferred from the pointers: a step's
 * operands from (pinned) host memory to the device, or its result back, in one call for a host loop that cannot
 * afford a framework call per operand.  `dst`, `src` and `bytes` are HOST arrays of n entries; an entry of 0 bytes is
 * skipped.  Nothing is retained: the caller keeps every buffer alive and unchanged until the stream has passed the
 * copies.  The reference stages a step's host arrays one jax.device_put at a time
 * (nanovllm_jax/engine/model_runner.py:3295, 3464-3465); no counterpart call.
 */
int nvj_copy_many_async(void* const* dst, const void* const* src, const size_t* bytes, int n,
                        nvj_stream_t stream);

/* ------------------------------------------------------------------ tokens */

/*
 * Per-row argmax over `row_len` floats -> int32 (first maximum wins).  Stand-in
 * for the sampler when one attention layer is benchmarked alone: it turns the
 * attention output of a row into the per-step token that the ranks all-gather.
 * The reference has no counterpart (it is single-device and samples from logits).
 */
int nvj_row_argmax(const float* x, int rows, int row_len, int32_t* tokens,
                   nvj_stream_t stream);

/*
 * The same token pick, and in the same launch the advance of the rows' resident decode metadata that
 * nvj_advance_decode_metadata would make (positions nullable): the tail of a decode step whose attention ran in
 * the pre-append form of nvj_paged_decode_fused_append, so that the step is two launches instead of three.
 */
int nvj_row_argmax_advance(const float* x, int rows, int row_len, int32_t* tokens, int32_t* seq_lens,
                           int32_t* positions, int table_width, int block_size, int32_t* status,
                           nvj_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* NVJ_B200_H_ */
