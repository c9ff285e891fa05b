// Slot-mapped append of new K/V rows into one layer of the paged cache.
//
// HBM-bound byte movement: one warp moves one token (its K row and its V row,
// num_kv_heads * head_dim elements each) with 16-byte vector accesses; a scalar
// kernel covers shapes whose rows are not a multiple of 16 bytes.  Semantics
// follow the reference's masked scatter (nanovllm_jax/kv_cache.py:476-564 with
// the valid masks of nanovllm_jax/backends.py:1050-1057) and its page-table
// form (nanovllm_jax/kernels/csrc/fp32_kv_append.cu:801-841).

#include "kv_append.cuh"

namespace nvj {

// Same-dtype rows, row bytes a multiple of 16: pure 16-byte copies.
__global__ void __launch_bounds__(256) append_copy16_kernel(AppendParams p, int row_bytes) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= p.n_tokens) return;
  long long slot = 0;
  if (lane == 0) slot = resolve_slot(p, warp);
  slot = __shfl_sync(kFullMask, slot, 0);
  if (slot < 0) return;
  const int chunks = row_bytes >> 4;
  const uint4* sk = reinterpret_cast<const uint4*>(static_cast<const char*>(p.new_k) + (long long)warp * row_bytes);
  const uint4* sv = reinterpret_cast<const uint4*>(static_cast<const char*>(p.new_v) + (long long)warp * row_bytes);
  uint4* dk = reinterpret_cast<uint4*>(static_cast<char*>(p.k_cache) + slot * row_bytes);
  uint4* dv = reinterpret_cast<uint4*>(static_cast<char*>(p.v_cache) + slot * row_bytes);
  for (int c = lane; c < chunks; c += 32) {
    const uint4 a = ld_nc_u4(sk + c);
    const uint4 b = ld_nc_u4(sv + c);
    dk[c] = a;
    dv[c] = b;
  }
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_f16(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// f32 source rows narrowed to a 16-bit cache dtype, 8 elements per lane step.
template <bool kToBf16>
__global__ void __launch_bounds__(256) append_narrow_kernel(AppendParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= p.n_tokens) return;
  long long slot = 0;
  if (lane == 0) slot = resolve_slot(p, warp);
  slot = __shfl_sync(kFullMask, slot, 0);
  if (slot < 0) return;
  const int groups = p.row_elems >> 3;
  const float4* sk = reinterpret_cast<const float4*>(static_cast<const float*>(p.new_k) + (long long)warp * p.row_elems);
  const float4* sv = reinterpret_cast<const float4*>(static_cast<const float*>(p.new_v) + (long long)warp * p.row_elems);
  uint4* dk = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.k_cache) + slot * p.row_elems);
  uint4* dv = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.v_cache) + slot * p.row_elems);
  for (int g = lane; g < groups; g += 32) {
    const float4 a0 = sk[2 * g], a1 = sk[2 * g + 1];
    const float4 b0 = sv[2 * g], b1 = sv[2 * g + 1];
    uint4 ok, ov;
    if (kToBf16) {
      ok = make_uint4(pack_bf16(a0.x, a0.y), pack_bf16(a0.z, a0.w), pack_bf16(a1.x, a1.y), pack_bf16(a1.z, a1.w));
      ov = make_uint4(pack_bf16(b0.x, b0.y), pack_bf16(b0.z, b0.w), pack_bf16(b1.x, b1.y), pack_bf16(b1.z, b1.w));
    } else {
      ok = make_uint4(pack_f16(a0.x, a0.y), pack_f16(a0.z, a0.w), pack_f16(a1.x, a1.y), pack_f16(a1.z, a1.w));
      ov = make_uint4(pack_f16(b0.x, b0.y), pack_f16(b0.z, b0.w), pack_f16(b1.x, b1.y), pack_f16(b1.z, b1.w));
    }
    dk[g] = ok;
    dv[g] = ov;
  }
}

__device__ __forceinline__ float load_as_float(const void* base, long long idx, int dt) {
  if (dt == NVJ_F32) return static_cast<const float*>(base)[idx];
  if (dt == NVJ_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
  return __half2float(static_cast<const __half*>(base)[idx]);
}
__device__ __forceinline__ void store_from_float(void* base, long long idx, int dt, float v) {
  if (dt == NVJ_F32) static_cast<float*>(base)[idx] = v;
  else if (dt == NVJ_BF16) static_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
  else static_cast<__half*>(base)[idx] = __float2half_rn(v);
}

// Any shape, any dtype pair: one warp per token, element-wise.
__global__ void __launch_bounds__(256) append_scalar_kernel(AppendParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= p.n_tokens) return;
  long long slot = 0;
  if (lane == 0) slot = resolve_slot(p, warp);
  slot = __shfl_sync(kFullMask, slot, 0);
  if (slot < 0) return;
  const long long s0 = (long long)warp * p.row_elems, d0 = slot * p.row_elems;
  if (p.src_dtype == p.dst_dtype) {
    const int es = dtype_size(p.src_dtype);
    const char* sk = static_cast<const char*>(p.new_k) + s0 * es;
    const char* sv = static_cast<const char*>(p.new_v) + s0 * es;
    char* dk = static_cast<char*>(p.k_cache) + d0 * es;
    char* dv = static_cast<char*>(p.v_cache) + d0 * es;
    for (int c = lane; c < p.row_elems * es; c += 32) {
      dk[c] = sk[c];
      dv[c] = sv[c];
    }
  } else {
    for (int e = lane; e < p.row_elems; e += 32) {
      store_from_float(p.k_cache, d0 + e, p.dst_dtype, load_as_float(p.new_k, s0 + e, p.src_dtype));
      store_from_float(p.v_cache, d0 + e, p.dst_dtype, load_as_float(p.new_v, s0 + e, p.src_dtype));
    }
  }
}

// slot[i] = block_table[row(i), pos / bs] * bs + pos % bs; row(i) is the token's own row
// (rectangular batches) or its clipped token_row_ids entry (packed batches).
__global__ void __launch_bounds__(256)
slot_mapping_kernel(const int32_t* positions, const int32_t* block_tables, const int32_t* token_row_ids,
                    int n_rows, int n_cols, int table_rows, int table_width, int block_size,
                    int32_t* slots) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_rows * n_cols) return;
  int row = token_row_ids ? token_row_ids[i] : i / n_cols;
  row = row < 0 ? 0 : (row >= table_rows ? table_rows - 1 : row);
  const int pos = positions[i];
  // floor division and a non-negative remainder, as jnp's // and % give for a negative position
  // (nanovllm_jax/kv_cache.py:432-435); C's / and % would round toward zero
  int col = pos / block_size, off = pos % block_size;
  if (off < 0) { off += block_size; --col; }
  // a negative block index wraps around once as NumPy / jnp indexing does, then the gather clamps
  if (col < 0) col += table_width;
  col = col < 0 ? 0 : (col >= table_width ? table_width - 1 : col);
  slots[i] = block_tables[(long long)row * table_width + col] * block_size + off;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int launch_append(const AppendParams& p, cudaStream_t stream) {
  if (p.n_tokens == 0) return NVJ_OK;
  const int threads = 256;
  const int blocks = (p.n_tokens * 32 + threads - 1) / threads;
  const int src_es = dtype_size(p.src_dtype), dst_es = dtype_size(p.dst_dtype);
  const bool ptrs_ok = aligned16(p.new_k) && aligned16(p.new_v) && aligned16(p.k_cache) && aligned16(p.v_cache);
  if (p.src_dtype == p.dst_dtype && ptrs_ok && (p.row_elems * src_es) % 16 == 0) {
    append_copy16_kernel<<<blocks, threads, 0, stream>>>(p, p.row_elems * src_es);
  } else if (p.src_dtype == NVJ_F32 && dst_es == 2 && ptrs_ok && p.row_elems % 8 == 0) {
    if (p.dst_dtype == NVJ_BF16) append_narrow_kernel<true><<<blocks, threads, 0, stream>>>(p);
    else append_narrow_kernel<false><<<blocks, threads, 0, stream>>>(p);
  } else {
    append_scalar_kernel<<<blocks, threads, 0, stream>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

static bool dtype_ok(int dt) { return dt == NVJ_BF16 || dt == NVJ_F16 || dt == NVJ_F32; }

// Append one new row per decode row at positions[b] through the dense block
// table; used by the fused decode entry point when the generic kernel runs.
int append_decode_rows(const void* new_k, const void* new_v, const int32_t* positions,
                       const int32_t* seq_lens, void* k_cache, void* v_cache, int kv_dtype,
                       long long num_blocks, int block_size, int row_elems,
                       const int32_t* block_tables, int table_width, int batch, int32_t* status,
                       cudaStream_t stream) {
  AppendParams p{};
  p.new_k = new_k;
  p.new_v = new_v;
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.positions = positions;
  p.kv_indices = block_tables;
  p.seq_lens = seq_lens;
  p.status = status;
  p.num_slots = num_blocks * block_size;
  p.kv_indices_len = (long long)batch * table_width;
  p.n_tokens = batch;
  p.n_cols = 1;
  p.batch = batch;
  p.page_size = block_size;
  p.table_width = table_width;
  p.row_elems = row_elems;
  p.src_dtype = kv_dtype;
  p.dst_dtype = kv_dtype;
  return launch_append(p, stream);
}

}  // namespace nvj

extern "C" int nvj_kv_append(const void* new_k, const void* new_v, int src_dtype,
                             const int32_t* slot_mapping, const int32_t* valid_mask,
                             const int32_t* query_start_loc, int qsl_rows, int packed,
                             int n_rows, int n_cols, void* k_cache_layer, void* v_cache_layer,
                             int cache_dtype, int64_t num_slots, int num_kv_heads, int head_dim,
                             int32_t* status, nvj_stream_t stream) {
  using namespace nvj;
  if (n_rows < 0 || n_cols < 0 || num_slots < 0 || num_kv_heads <= 0 || head_dim <= 0)
    return NVJ_ERR_INVALID_ARGUMENT;
  if (!dtype_ok(src_dtype) || !dtype_ok(cache_dtype)) return NVJ_ERR_UNSUPPORTED;
  if ((long long)n_rows * n_cols > 0x7fffffffLL / 32) return NVJ_ERR_UNSUPPORTED;
  if (n_rows * n_cols == 0) return NVJ_OK;
  if (!new_k || !new_v || !slot_mapping || !k_cache_layer || !v_cache_layer)
    return NVJ_ERR_INVALID_ARGUMENT;
  if (query_start_loc && qsl_rows < 0) return NVJ_ERR_INVALID_ARGUMENT;
  AppendParams p{};
  p.new_k = new_k;
  p.new_v = new_v;
  p.k_cache = k_cache_layer;
  p.v_cache = v_cache_layer;
  p.slot_mapping = slot_mapping;
  p.valid_mask = valid_mask;
  p.query_start_loc = query_start_loc;
  p.status = status;
  p.num_slots = num_slots;
  p.n_tokens = n_rows * n_cols;
  p.n_cols = n_cols;
  p.qsl_rows = qsl_rows;
  p.packed = packed;
  p.page_size = 1;
  p.row_elems = num_kv_heads * head_dim;
  p.src_dtype = src_dtype;
  p.dst_dtype = cache_dtype;
  return launch_append(p, static_cast<cudaStream_t>(stream));
}

extern "C" int nvj_kv_append_nhd(const void* append_key, const void* append_value, int src_dtype,
                                 const int32_t* batch_indices, const int32_t* positions, int nnz,
                                 void* k_cache, void* v_cache, int cache_dtype, int64_t num_pages,
                                 int page_size, int num_kv_heads, int head_dim,
                                 const int32_t* kv_indices, int64_t kv_indices_len,
                                 const int32_t* kv_indptr, int batch, const int32_t* valid_mask,
                                 int32_t* status, nvj_stream_t stream) {
  using namespace nvj;
  if (nnz < 0 || num_pages < 0 || page_size <= 0 || num_kv_heads <= 0 || head_dim <= 0 ||
      batch < 0 || kv_indices_len < 0)
    return NVJ_ERR_INVALID_ARGUMENT;
  if (!dtype_ok(src_dtype) || !dtype_ok(cache_dtype)) return NVJ_ERR_UNSUPPORTED;
  if (nnz > 0x7fffffff / 32) return NVJ_ERR_UNSUPPORTED;
  if (nnz == 0) return NVJ_OK;
  if (!append_key || !append_value || !batch_indices || !positions || !k_cache || !v_cache ||
      !kv_indices || !kv_indptr)
    return NVJ_ERR_INVALID_ARGUMENT;
  AppendParams p{};
  p.new_k = append_key;
  p.new_v = append_value;
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.valid_mask = valid_mask;
  p.batch_indices = batch_indices;
  p.positions = positions;
  p.kv_indices = kv_indices;
  p.kv_indptr = kv_indptr;
  p.status = status;
  p.num_slots = num_pages * page_size;
  p.kv_indices_len = kv_indices_len;
  p.n_tokens = nnz;
  p.n_cols = 1;
  p.batch = batch;
  p.page_size = page_size;
  p.row_elems = num_kv_heads * head_dim;
  p.src_dtype = src_dtype;
  p.dst_dtype = cache_dtype;
  return launch_append(p, static_cast<cudaStream_t>(stream));
}

extern "C" int nvj_compute_slot_mapping(const int32_t* positions, const int32_t* block_tables,
                                        const int32_t* token_row_ids, int n_rows, int n_cols,
                                        int table_rows, int table_width, int block_size,
                                        int32_t* slot_mapping, nvj_stream_t stream) {
  if (n_rows < 0 || n_cols < 0 || table_rows <= 0 || table_width <= 0 || block_size <= 0)
    return NVJ_ERR_INVALID_ARGUMENT;
  const long long n = (long long)n_rows * n_cols;
  if (n == 0) return NVJ_OK;
  if (n > 0x7fffffffLL) return NVJ_ERR_UNSUPPORTED;
  if (!positions || !block_tables || !slot_mapping) return NVJ_ERR_INVALID_ARGUMENT;
  nvj::slot_mapping_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      positions, block_tables, token_row_ids, n_rows, n_cols, table_rows, table_width, block_size,
      slot_mapping);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}
