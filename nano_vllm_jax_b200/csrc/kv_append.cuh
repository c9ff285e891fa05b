// Slot resolution shared by the append kernels: where token i of a batch lands in one layer of
// the paged cache, under the reference's valid-token rules (nanovllm_jax/kv_cache.py:476-564,
// nanovllm_jax/backends.py:1050-1057) and its page-table form
// (nanovllm_jax/kernels/csrc/fp32_kv_append.cu:801-841).

#pragma once

#include "nvj_common.cuh"

namespace nvj {

struct AppendParams {
  const void* new_k;
  const void* new_v;
  void* k_cache;
  void* v_cache;
  const int32_t* slot_mapping;  // slot mode
  const int32_t* valid_mask;
  const int32_t* query_start_loc;
  // page-table mode
  const int32_t* batch_indices;
  const int32_t* positions;
  const int32_t* kv_indices;
  const int32_t* kv_indptr;   // null: row b's table starts at b * table_width
  const int32_t* seq_lens;    // page-table mode, optional: rows with seq_lens[b] <= 0 are skipped
  int32_t* status;
  long long num_slots;
  long long kv_indices_len;
  int n_tokens;
  int n_cols;
  int qsl_rows;
  int packed;
  int batch;
  int page_size;
  int table_width;
  int row_elems;  // num_kv_heads * head_dim
  int src_dtype;
  int dst_dtype;
};

// Returns the flat destination slot of token i, or -1 when the token is masked
// out or its slot lies outside the pool (the latter is flagged).
__device__ __forceinline__ long long resolve_slot(const AppendParams& p, int i) {
  if (p.valid_mask && p.valid_mask[i] == 0) return -1;
  long long slot;
  if (p.slot_mapping) {
    if (p.query_start_loc) {
      if (p.packed) {
        if (i >= p.query_start_loc[p.qsl_rows]) return -1;
      } else {
        const int r = i / p.n_cols, t = i - r * p.n_cols;
        if (r >= p.qsl_rows) return -1;
        if (t >= p.query_start_loc[r + 1] - p.query_start_loc[r]) return -1;
      }
    }
    slot = p.slot_mapping[i];
  } else {
    const int b = p.batch_indices ? p.batch_indices[i] : i;
    const int pos = p.positions[i];
    if (b < 0 || b >= p.batch || pos < 0) {
      if (p.status) atomicOr(p.status, NVJ_DEV_BAD_BLOCK_ID);
      return -1;
    }
    if (p.seq_lens && p.seq_lens[b] <= 0) return -1;
    // the page index is bounded by the row's own page list, so a position past it cannot reach the next row's pages
    const int page = pos / p.page_size;
    const long long first = p.kv_indptr ? (long long)p.kv_indptr[b] : (long long)b * p.table_width;
    const long long pages = p.kv_indptr ? (long long)p.kv_indptr[b + 1] - first : (long long)p.table_width;
    const long long e = first + page;
    if (page >= pages || e < 0 || e >= p.kv_indices_len) {
      if (p.status) atomicOr(p.status, NVJ_DEV_BAD_BLOCK_ID);
      return -1;
    }
    slot = (long long)p.kv_indices[e] * p.page_size + pos % p.page_size;
  }
  if (slot < 0 || slot >= p.num_slots) {
    if (p.status) atomicOr(p.status, NVJ_DEV_BAD_BLOCK_ID);
    return -1;
  }
  return slot;
}

}  // namespace nvj
