// Parameters and workspace layout shared by the paged decode kernels.
#pragma once

#include "nvj_common.cuh"

namespace nvj {

// Shape the bulk-copy pipelined kernel is specialised for (the model's
// full-attention layer: 8 query heads over 2 KV heads, head_dim 256, 16-token
// blocks, bf16 cache).
constexpr int kBlk = 16;                                // tokens per cache block
constexpr int kD = 256;                                 // head_dim
constexpr int kHkv = 2;                                 // KV heads
constexpr int kG = 4;                                   // query heads per KV head
constexpr int kHq = kHkv * kG;                          // query heads
constexpr int kRowBytes = kD * 2;                       // one (token, kv head) row, bf16
constexpr int kTokenBytes = kHkv * kRowBytes;           // 1024
constexpr int kTileBytes = kBlk * kTokenBytes;          // 16 KiB: one block of K (or of V)

struct DecodeParams {
  const void* q;
  const char* k_cache;  // one layer
  const char* v_cache;
  const int32_t* block_tables;
  const int32_t* kv_indptr;         // nullable
  const int32_t* kv_last_page_len;  // nullable
  const int32_t* seq_lens;
  // fused append (nullable)
  const void* new_k;
  const void* new_v;
  const int32_t* positions;
  // fused append without positions: seq_lens holds every row's length BEFORE this step's token; the new row goes to
  // position seq_lens[b] and seq_lens[b] + 1 keys are attended (rows with seq_lens[b] <= 0 stay inactive)
  int pre_append;
  // packed prefill through the generic kernel (nullable): query i belongs to the
  // table row r with query_start_loc[r] <= i < query_start_loc[r + 1] and attends
  // keys p <= query_positions[i]
  const int32_t* query_start_loc;
  const int32_t* query_positions;
  int qsl_rows;
  // packed_rows != 0 (pipelined kernel inside a packed batch): `batch` counts table rows; a row
  // takes part only if it holds exactly one query token, i = query_start_loc[b]; it reads q[i],
  // writes out[i] and attends min(seq_lens[b], query_positions[i] + 1) keys.  Other rows are left
  // alone (no zero fill): the prefill kernel owns them.
  int packed_rows;
  // query tokens per row of the wide kernel (2..4; 0 elsewhere): q is [batch, width, heads, dim], out
  // [batch, width, heads * dim], positions (nullable) [batch, width]
  int width;
  // upper bound on the CTAs of the streaming kernels (0: one, or two, per SM): a caller that runs another kernel
  // beside the decode pass leaves that kernel's SMs free
  int cta_limit;
  // which wide kernel serves rows of several query tokens: 0 = automatic (mma.sync tiles up to width 4, tcgen05 beyond),
  // 1 = mma.sync tiles, 2 = tcgen05
  int wide_form;
  // what a row end costs a CTA, in blocks (decode_parts.cuh); set by the launchers, the same for every kernel of a call
  int row_end_cost;
  float* out;
  // workspace
  int32_t* status;
  int32_t* counters;        // [batch] row arrival counters, zero between launches
  int32_t* group_counters;  // [kGroupCounters] group arrival counters, zero between launches
  float* part_ml;     // [ws_slots(num_ctas)][kHq][2]  (running max in log2 units, sum)
  float* part_acc;    // [ws_slots(num_ctas)][kHq][kD] un-normalised accumulators
  long long num_blocks;
  int batch;
  int table_width;
  int block_size;
  int num_kv_heads;
  int num_q_heads;
  int head_dim;
  int q_dtype;
  int kv_dtype;
  float scale;
};

// Keys row b attends: seq_lens[b], clipped to what its page list can hold.
__device__ __forceinline__ int decode_row_len(const DecodeParams& p, int b) {
  int len = p.seq_lens[b];
  if (p.pre_append && len > 0) ++len;
  if (p.packed_rows) {
    const int i = p.query_start_loc[b];
    if (p.query_start_loc[b + 1] - i != 1) return 0;
    const int cap = p.query_positions[i] + 1;
    len = len < cap ? len : cap;
  }
  int pages = p.table_width;
  if (p.kv_indptr) {
    pages = p.kv_indptr[b + 1] - p.kv_indptr[b];
    if (p.kv_last_page_len) {
      const int eff = pages > 0 ? (pages - 1) * p.block_size + p.kv_last_page_len[b] : 0;
      len = len < eff ? len : eff;
    }
  }
  const long long cap = (long long)pages * p.block_size;
  if (len > cap) {
    atomicOr(p.status, NVJ_DEV_BAD_LENGTH);
    len = (int)cap;
  }
  return len < 0 ? 0 : len;
}

// Index of row b's query / output vector.
__device__ __forceinline__ long long decode_query_index(const DecodeParams& p, int b) {
  return p.packed_rows ? (long long)p.query_start_loc[b] : (long long)b;
}

__device__ __forceinline__ long long decode_table_base(const DecodeParams& p, int b) {
  return p.kv_indptr ? (long long)p.kv_indptr[b] : (long long)b * p.table_width;
}

constexpr size_t kWsAlign = 256;
__host__ __device__ inline size_t ws_round(size_t x) { return (x + kWsAlign - 1) / kWsAlign * kWsAlign; }
// A row that is cut into more than kTreeMergeMin partials is merged in two levels: the CTAs of
// one group of kMergeGroup consecutive CTA ids fold their partials into one group partial, and
// the group that finishes last folds the group partials.  kGroupCounters arrival counters
// (two per group) follow the per-row counters; a launch never has more CTAs than they cover.
// 13: the tensor-core kernel keeps 13 parts' accumulators in flight while it folds (what its registers hold without
// spilling), so on 148 SMs both levels (13 parts, then 12 groups) are one batch of loads each.
constexpr int kMergeGroup = 13;
constexpr int kTreeMergeMin = 32;
constexpr int kGroupCounters = 64;
__host__ __device__ inline int ws_groups(int num_ctas) { return (num_ctas + kMergeGroup - 1) / kMergeGroup; }
// Partial slots: two per CTA, then two per group.
__host__ __device__ inline size_t ws_slots(int num_ctas) { return 2ull * num_ctas + 2ull * ws_groups(num_ctas); }
// Header = status word (64 B) + the group counters + one int32 counter per row.
inline size_t ws_header_bytes(int max_batch) { return ws_round(64 + sizeof(int32_t) * ((size_t)max_batch + kGroupCounters)); }
inline size_t ws_ml_bytes(int num_ctas) { return ws_round(sizeof(float) * ws_slots(num_ctas) * kHq * 2); }
inline size_t ws_acc_bytes(int num_ctas) { return ws_round(sizeof(float) * ws_slots(num_ctas) * kHq * kD); }

// Carves a decode workspace of `bytes` bytes for a call with p.batch rows whose partial results need `ml_bytes` and
// `acc_bytes`.  One buffer serves calls of any batch size, width and kernel one after another, so nothing a call
// writes may land where a later call keeps state that must start at zero:
//   [0, 64)              status word
//   [64, 320)            group arrival counters
//   [320, 320 + 4 rows)  row arrival counters
//   ... unused, or the partial outputs of the prefill kernel's key-range splits, which end where the next part begins ...
//   the last ml_bytes + acc_bytes of the buffer: partial (max, sum) pairs and accumulators
// The counters are zero before the first use and every launch leaves them zero again; the partials are always
// written before they are read.  Because the partials are anchored at the END of the buffer, a call with few rows
// cannot leave them inside the counter area of a later call with more rows (anchored behind the call's own
// counters they would: a 256-row call after a 4-row call then found garbage in its counters and never merged
// its split rows).  Callers pass the same `bytes` for every call on one buffer.
inline int carve_decode_workspace(DecodeParams& p, void* workspace, size_t bytes, size_t ml_bytes, size_t acc_bytes) {
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return NVJ_ERR_WORKSPACE;
  const size_t end = bytes / kWsAlign * kWsAlign;
  if (end < ws_header_bytes(p.batch) + ml_bytes + acc_bytes) return NVJ_ERR_WORKSPACE;
  char* w = static_cast<char*>(workspace);
  p.status = reinterpret_cast<int32_t*>(w);
  p.group_counters = reinterpret_cast<int32_t*>(w + 64);
  p.counters = reinterpret_cast<int32_t*>(w + 64 + sizeof(int32_t) * kGroupCounters);
  p.part_acc = reinterpret_cast<float*>(w + end - acc_bytes);
  p.part_ml = reinterpret_cast<float*>(w + end - acc_bytes - ml_bytes);
  return NVJ_OK;
}

// Bytes that the prefill kernel's key-range splits may need for their partial outputs on the current device.
size_t prefill_split_bytes();

int decode_num_ctas();  // 2 per SM of the current device
int launch_decode_generic(const DecodeParams& p, cudaStream_t stream);
int launch_decode_pipelined(const DecodeParams& p, int num_ctas, cudaStream_t stream);
int decode_wide_num_ctas();  // 1 per SM of the current device
int launch_decode_wide(const DecodeParams& p, cudaStream_t stream);  // tensor-core streaming kernels, width 1..8
int launch_decode_umma(const DecodeParams& p, cudaStream_t stream);  // the tcgen05 form, rows already appended
int append_decode_rows(const void* new_k, const void* new_v, const int32_t* positions,
                       const int32_t* seq_lens, void* k_cache, void* v_cache, int kv_dtype,
                       long long num_blocks, int block_size, int row_elems,
                       const int32_t* block_tables, int table_width, int batch, int32_t* status,
                       cudaStream_t stream);

}  // namespace nvj
