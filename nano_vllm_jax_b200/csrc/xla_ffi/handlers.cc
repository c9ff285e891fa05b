// XLA-FFI custom-call handlers (api_version 1) over the C ABI of include/nvj_b200.h: one thin adapter per entry
// point.  They replace, operand for operand where the reference has one, the handlers NanoVllmJaxFp32KvAppend and
// NanoVllmJaxFp32PagedDecodeAttention of nanovllm_jax/kernels/csrc/fp32_kv_append.cu:1563-1697 and serve the other
// operations of the path (fused append + decode, wide decode, packed prefill, block copy, GDN state snapshot /
// restore, slot mapping, resident-metadata advance, token pick) to `jax.ffi.ffi_call`.
//
// NOT COMPILED BY THE BUILD (see ffi_util.h).  Conventions of every handler:
//   * static scalars (scale, layer_id, block_size, packed, variant) are attributes; everything else is a buffer;
//   * caches, workspaces and other in-place operands are aliased to results by the Python side
//     (`input_output_aliases`), and the handler writes through the result buffer;
//   * a `status` result (s32[1]) is cleared here and receives the NVJ_DEV_* bits of the call;
//   * the decode workspace is an operand (u8[n], zeros) aliased to a result: a handler only ever sees the
//     buffers XLA hands it.  NvjB200PagedDecodeAttention, which keeps the reference's operand list, uses the
//     library's built-in scratch instead (nvj_paged_decode_static_scratch).

#include <cuda_runtime_api.h>

#include "ffi_util.h"

using namespace nvj_xla;

namespace {

XLA_FFI_Error* ClearStatus(XLA_FFI_CallFrame* frame, XLA_FFI_Buffer* status, nvj_stream_t stream) {
  if (!IsI32(status, 1) || status->dims[0] < 1) return Invalid(frame, "status must be s32[1]");
  if (cudaMemsetAsync(status->data, 0, sizeof(int32_t), static_cast<cudaStream_t>(stream)) != cudaSuccess)
    return MakeError(frame->api, XLA_FFI_Error_Code_INTERNAL, "cudaMemsetAsync(status) failed");
  return nullptr;
}

// [num_pages, page_size, num_kv_heads, head_dim] of one layer slice
struct Nhd {
  int64_t pages, page_size, kv_heads, head_dim;
};
bool NhdOf(const XLA_FFI_Buffer* b, Nhd* s) {
  if (b == nullptr || b->rank != 4 || FloatDtype(b) < 0) return false;
  *s = {b->dims[0], b->dims[1], b->dims[2], b->dims[3]};
  return true;
}

}  // namespace

// slot_mapping = NvjB200ComputeSlotMapping(positions s32[R, C], block_tables s32[rows, W] [, token_row_ids s32[R, C]])
//   attrs: block_size
extern "C" XLA_FFI_Error* NvjB200ComputeSlotMapping(XLA_FFI_CallFrame* frame) {
  NVJ_XLA_PROLOGUE("NvjB200ComputeSlotMapping", 2, 1, 1);
  XLA_FFI_Buffer *positions = Arg(frame, 0), *tables = Arg(frame, 1), *row_ids = Arg(frame, 2), *slots = Ret(frame, 0);
  int32_t block_size = 0;
  if (!IsI32(positions, 2) || !IsI32(tables, 2) || !IsI32(slots, 2) || !SameShape(positions, slots))
    return Invalid(frame, "positions, slot_mapping s32[R, C] and block_tables s32[rows, W] expected");
  if (row_ids != nullptr && (!IsI32(row_ids, 2) || !SameShape(row_ids, positions)))
    return Invalid(frame, "token_row_ids must have the shape of positions");
  if (!IntAttr(frame, "block_size", &block_size)) return Invalid(frame, "attribute block_size (s32) is required");
  return FromStatus(frame, "nvj_compute_slot_mapping",
                    nvj_compute_slot_mapping(static_cast<const int32_t*>(positions->data), static_cast<const int32_t*>(tables->data),
                                             row_ids ? static_cast<const int32_t*>(row_ids->data) : nullptr,
                                             (int)positions->dims[0], (int)positions->dims[1], (int)tables->dims[0],
                                             (int)tables->dims[1], block_size, static_cast<int32_t*>(slots->data), stream));
}

// k_layer, v_layer, status = NvjB200KvAppend(new_k [R, C, Hkv, D], new_v, slot_mapping s32[R, C], k_layer, v_layer,
//                                            query_start_loc s32[rows + 1] [, valid_mask s32[R, C]])
//   attrs: packed (0 | 1); aliases {3: 0, 4: 1}.  k_layer / v_layer: [slots, Hkv, D] or [NB, bs, Hkv, D].
extern "C" XLA_FFI_Error* NvjB200KvAppend(XLA_FFI_CallFrame* frame) {
  NVJ_XLA_PROLOGUE("NvjB200KvAppend", 6, 1, 3);
  XLA_FFI_Buffer *new_k = Arg(frame, 0), *new_v = Arg(frame, 1), *slots = Arg(frame, 2), *qsl = Arg(frame, 5), *mask = Arg(frame, 6);
  XLA_FFI_Buffer *k_out = Ret(frame, 0), *v_out = Ret(frame, 1), *status = Ret(frame, 2);
  int32_t packed = 0;
  if (new_k == nullptr || new_k->rank != 4 || FloatDtype(new_k) < 0 || !SameShape(new_k, new_v))
    return Invalid(frame, "new_k and new_v must be [rows, cols, kv_heads, head_dim] of one floating type");
  if (!IsI32(slots, 2) || slots->dims[0] != new_k->dims[0] || slots->dims[1] != new_k->dims[1])
    return Invalid(frame, "slot_mapping must be s32[rows, cols]");
  if (FloatDtype(k_out) < 0 || !SameShape(k_out, v_out) || (k_out->rank != 3 && k_out->rank != 4))
    return Invalid(frame, "cache layers must be [slots, kv_heads, head_dim] or [blocks, block_size, kv_heads, head_dim]");
  const int64_t kv_heads = k_out->dims[k_out->rank - 2], head_dim = k_out->dims[k_out->rank - 1];
  if (new_k->dims[2] != kv_heads || new_k->dims[3] != head_dim) return Invalid(frame, "new rows do not match the cache heads");
  if (!IsI32(qsl, 1) || qsl->dims[0] < 1) return Invalid(frame, "query_start_loc must be s32[rows + 1]");
  if (mask != nullptr && (!IsI32(mask, 2) || !SameShape(mask, slots))) return Invalid(frame, "valid_mask must be s32[rows, cols]");
  if (!IntAttr(frame, "packed", &packed)) return Invalid(frame, "attribute packed (s32) is required");
  if (XLA_FFI_Error* error = ClearStatus(frame, status, stream)) return error;
  return FromStatus(frame, "nvj_kv_append",
                    nvj_kv_append(new_k->data, new_v->data, FloatDtype(new_k), static_cast<const int32_t*>(slots->data),
                                  mask ? static_cast<const int32_t*>(mask->data) : nullptr, static_cast<const int32_t*>(qsl->data),
                                  (int)qsl->dims[0] - 1, packed, (int)new_k->dims[0], (int)new_k->dims[1], k_out->data, v_out->data,
                                  FloatDtype(k_out), Elements(k_out) / (kv_heads * head_dim), (int)kv_heads, (int)head_dim,
                                  static_cast<int32_t*>(status->data), stream));
}

// k_cache, v_cache = NvjB200KvAppendNhd(append_key [nnz, Hkv, D], append_value, batch_indices s32[nnz], positions s32[nnz],
//                                       k_cache [NB, P, Hkv, D], v_cache, kv_indices s32[total], kv_indptr s32[B + 1],
//                                       kv_last_page_len s32[B] [, valid_mask s32[nnz]])
//   The operand list of the reference's NanoVllmJaxFp32KvAppend (fp32_kv_append.cu:1584-1593); aliases {4: 0, 5: 1}.
extern "C" XLA_FFI_Error* NvjB200KvAppendNhd(XLA_FFI_CallFrame* frame) {
  NVJ_XLA_PROLOGUE("NvjB200KvAppendNhd", 9, 1, 2);
  XLA_FFI_Buffer *key = Arg(frame, 0), *value = Arg(frame, 1), *rows = Arg(frame, 2), *positions = Arg(frame, 3);
  XLA_FFI_Buffer *indices = Arg(frame, 6), *indptr = Arg(frame, 7), *last = Arg(frame, 8), *mask = Arg(frame, 9);
  XLA_FFI_Buffer *k_out = Ret(frame, 0), *v_out = Ret(frame, 1);
  Nhd c;
  if (!NhdOf(k_out, &c) || !SameShape(k_out, v_out)) return Invalid(frame, "caches must be [pages, page_size, kv_heads, head_dim]");
  if (key == nullptr || key->rank != 3 || FloatDtype(key) < 0 || !SameShape(key, value) || key->dims[1] != c.kv_heads ||
      key->dims[2] != c.head_dim)
    return Invalid(frame, "append_key / append_value must be [nnz, kv_heads, head_dim]");
  const int64_t nnz = key->dims[0];
  if (!IsI32(rows, 1) || !IsI32(positions, 1) || rows->dims[0] != nnz || positions->dims[0] != nnz)
    return Invalid(frame, "batch_indices and positions must be s32[nnz]");
  if (!IsI32(indices, 1) || !IsI32(indptr, 1) || !IsI32(last, 1) || indptr->dims[0] != last->dims[0] + 1)
    return Invalid(frame, "page metadata must be s32: kv_indices [total], kv_indptr [B + 1], kv_last_page_len [B]");
  if (mask != nullptr && (!IsI32(mask, 1) || mask->dims[0] != nnz)) return Invalid(frame, "valid_mask must be s32[nnz]");
  return FromStatus(frame, "nvj_kv_append_nhd",
                    nvj_kv_append_nhd(key->data, value->data, FloatDtype(key), static_cast<const int32_t*>(rows->data),
                                      static_cast<const int32_t*>(positions->data), (int)nnz, k_out->data, v_out->data,
                                      FloatDtype(k_out), c.pages, (int)c.page_size, (int)c.kv_heads, (int)c.head_dim,
                                      static_cast<const int32_t*>(indices->data), indices->dims[0],
                                      static_cast<const int32_t*>(indptr->data), (int)last->dims[0],
                                      mask ? static_cast<const int32_t*>(mask->data) : nullptr, nullptr, stream));
}

// q_out, k_layer, v_layer, status = NvjB200QkNormRopeKvAppend(q bf16[T, Hq, D], k bf16[T, Hkv, D], v, q_norm [D], k_norm [D],
//                                       inv_freq f32[rot / 2], rope_positions s32[P, T], slot_mapping s32[T], k_layer, v_layer,
//                                       query_start_loc s32[rows + 1])
//   attrs: eps (f32), packed (s32), and for P = 3 position rows mrope_t, mrope_h, mrope_w (s32); aliases {8: 1, 9: 2}.
extern "C" XLA_FFI_Error* NvjB200QkNormRopeKvAppend(XLA_FFI_CallFrame* frame) {
  NVJ_XLA_PROLOGUE("NvjB200QkNormRopeKvAppend", 11, 0, 4);
  XLA_FFI_Buffer *q = Arg(frame, 0), *k = Arg(frame, 1), *v = Arg(frame, 2), *qw = Arg(frame, 3), *kw = Arg(frame, 4);
  XLA_FFI_Buffer *inv = Arg(frame, 5), *pos = Arg(frame, 6), *slots = Arg(frame, 7), *qsl = Arg(frame, 10);
  XLA_FFI_Buffer *q_out = Ret(frame, 0), *k_out = Ret(frame, 1), *v_out = Ret(frame, 2), *status = Ret(frame, 3);
  if (q == nullptr || q->rank != 3 || k == nullptr || k->rank != 3 || !SameShape(k, v) || !SameShape(q, q_out) ||
      FloatDtype(q) != NVJ_BF16 || FloatDtype(k) != NVJ_BF16 || q->dims[0] != k->dims[0] || q->dims[2] != k->dims[2])
    return Invalid(frame, "q [T, Hq, D] and k, v [T, Hkv, D] must be bf16 with equal T and D");
  const int64_t tokens = q->dims[0], hq = q->dims[1], hkv = k->dims[1], d = q->dims[2];
  if (FloatDtype(qw) < 0 || !SameShape(qw, kw) || qw->rank != 1 || qw->dims[0] != d) return Invalid(frame, "norm weights must be [D]");
  if (!Is(inv, XLA_FFI_DataType_F32, 1)) return Invalid(frame, "inv_freq must be f32[rotary_dim / 2]");
  if (!IsI32(pos, 2) || pos->dims[1] != tokens || (pos->dims[0] != 1 && pos->dims[0] != 3))
    return Invalid(frame, "rope_positions must be s32[1, T] (text) or s32[3, T] (temporal, height, width)");
  if (!IsI32(slots, 1) || slots->dims[0] != tokens || !IsI32(qsl, 1)) return Invalid(frame, "slot_mapping s32[T], query_start_loc s32[rows + 1]");
  if (FloatDtype(k_out) != NVJ_BF16 || !SameShape(k_out, v_out)) return Invalid(frame, "cache layers must be bf16 and of equal shape");
  float eps = 1e-6f;
  int32_t packed = 1, sec[3] = {0, 0, 0};
  FloatAttr(frame, "eps", &eps);
  IntAttr(frame, "packed", &packed);
  if (pos->dims[0] == 3 && !(IntAttr(frame, "mrope_t", &sec[0]) && IntAttr(frame, "mrope_h", &sec[1]) && IntAttr(frame, "mrope_w", &sec[2])))
    return Invalid(frame, "three position rows need the attributes mrope_t, mrope_h, mrope_w");
  if (XLA_FFI_Error* error = ClearStatus(frame, status, stream)) return error;
  return FromStatus(frame, "nvj_qk_norm_rope_kv_append",
                    nvj_qk_norm_rope_kv_append(q->data, hq * d, d, k->data, hkv * d, v->data, hkv * d, NVJ_BF16, qw->data, kw->data,
                                               FloatDtype(qw), eps, static_cast<const float*>(inv->data), (int)inv->dims[0] * 2,
                                               static_cast<const int32_t*>(pos->data), (int)pos->dims[0], sec,
                                               static_cast<const int32_t*>(slots->data), nullptr,
                                               static_cast<const int32_t*>(qsl->data), (int)qsl->dims[0] - 1, packed, 1, (int)tokens,
                                               k_out->data, v_out->data, NVJ_BF16, Elements(k_out) / (hkv * d), (int)hq, (int)hkv,
                                               (int)d, q_out->data, static_cast<int32_t*>(status->data), stream));
}

// out = NvjB200PagedDecodeAttention(q [B, Hq, D], k_cache [NB, P, Hkv, D], v_cache, kv_indptr s32[B + 1], kv_indices s32[B * W],
//                                   kv_last_page_len s32[B], seq_lens s32[B])       attrs: softmax_scale (f32)
//   The reference's NanoVllmJaxFp32PagedDecodeAttention operand list (fp32_kv_append.cu:1650-1659) with the scale as
//   an attribute.  Like the reference it reads kv_indices as a dense [B, W] table (W = total / B) and needs no
//   workspace operand: the scratch is the library's built-in array, so at most NVJ_STATIC_SCRATCH_MAX_BATCH rows and
//   one such call in flight per device.  out is f32[B, Hq, D].
extern "C" XLA_FFI_Error* NvjB200PagedDecodeAttention(XLA_FFI_CallFrame* frame) {
  NVJ_XLA_PROLOGUE("NvjB200PagedDecodeAttention", 7, 0, 1);
  XLA_FFI_Buffer *q = Arg(frame, 0), *k = Arg(frame, 1), *v = Arg(frame, 2), *indptr = Arg(frame, 3), *indices = Arg(frame, 4);
  XLA_FFI_Buffer *last = Arg(frame, 5), *lens = Arg(frame, 6), *out = Ret(frame, 0);
  Nhd c;
  if (!NhdOf(k, &c) || !SameShape(k, v)) return Invalid(frame, "caches must be [pages, page_size, kv_heads, head_dim]");
  if (q == nullptr || q->rank != 3 || FloatDtype(q) < 0 || q->dims[2] != c.head_dim || q->dims[1] % c.kv_heads != 0)
    return Invalid(frame, "q must be [batch, q_heads, head_dim] with q_heads a multiple of kv_heads");
  const int64_t batch = q->dims[0];
  if (!IsI32(indptr, 1) || indptr->dims[0] != batch + 1 || !IsI32(indices, 1) || !IsI32(last, 1) || last->dims[0] != batch ||
      !IsI32(lens, 1) || lens->dims[0] != batch || (batch > 0 && indices->dims[0] % batch != 0))
    return Invalid(frame, "kv_indptr s32[B + 1], kv_indices s32[B * W], kv_last_page_len s32[B], seq_lens s32[B] expected");
  if (!Is(out, XLA_FFI_DataType_F32, 3) || out->dims[0] != batch || out->dims[1] != q->dims[1] || out->dims[2] != q->dims[2])
    return Invalid(frame, "out must be f32[batch, q_heads, head_dim]");
  float scale = 0.f;
  if (!FloatAttr(frame, "softmax_scale", &scale)) return Invalid(frame, "attribute softmax_scale (f32) is required");
  return FromStatus(frame, "nvj_paged_decode_static_scratch",
                    nvj_paged_decode_static_scratch(q->data, FloatDtype(q), k->data, v->data, FloatDtype(k), c.pages, (int)c.page_size,
                                                    (int)c.kv_heads, (int)c.head_dim, (int)q->dims[1],
                                                    static_cast<const int32_t*>(indices->data),
                                                    batch > 0 ? (int)(indices->dims[0] / batch) : 0,
                                                    static_cast<const int32_t*>(lens->data), (int)batch, scale,
                                                    static_cast<float*>(out->data), nullptr, stream));
}

// out, workspace = NvjB200PagedDecodeCsr(q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, seq_lens, workspace u8[n])
//   attrs: softmax_scale (f32), variant (s32, optional).  Ragged page lists (kv_indptr need not be uniform); aliases {7: 1}.
extern "C" XLA_FFI_Error* NvjB200PagedDecodeCsr(XLA_FFI_CallFrame* frame) {
  NVJ_XLA_PROLOGUE("NvjB200PagedDecodeCsr", 8, 0, 2);
  XLA_FFI_Buffer *q = Arg(frame, 0), *k = Arg(frame, 1), *v = Arg(frame, 2), *indptr = Arg(frame, 3), *indices = Arg(frame, 4);
  XLA_FFI_Buffer *last = Arg(frame, 5), *lens = Arg(frame, 6), *out = Ret(frame, 0), *ws = Ret(frame, 1);
  Nhd c;
  if (!NhdOf(k, &c) || !SameShape(k, v) || q == nullptr || q->rank != 3 || FloatDtype(q) < 0 || q->dims[2] != c.head_dim)
    return Invalid(frame, "q [B, Hq, D] and caches [pages, page_size, kv_heads, D] expected");
  const int64_t batch = q->dims[0];
  if (!IsI32(indptr, 1) || indptr->dims[0] != batch + 1 || !IsI32(indices, 1) || !IsI32(last, 1) || !IsI32(lens, 1) ||
      last->dims[0] != batch || lens->dims[0] != batch)
    return Invalid(frame, "page metadata must be s32 of the documented shapes");
  if (!Is(out, XLA_FFI_DataType_F32, 3) || !Is(ws, XLA_FFI_DataType_U8, 1)) return Invalid(frame, "out f32[B, Hq, D], workspace u8[n]");
  float scale = 0.f;
  int32_t variant = 0;
  if (!FloatAttr(frame, "softmax_scale", &scale)) return Invalid(frame, "attribute softmax_scale (f32) is required");
  IntAttr(frame, "variant", &variant);
  return FromStatus(frame, "nvj_paged_decode",
                    nvj_paged_decode(q->data, FloatDtype(q), k->data, v->data, FloatDtype(k), c.pages, (int)c.page_size, (int)c.kv_heads,
                                     (int)c.head_dim, (int)q->dims[1], static_cast<const int32_t*>(indices->data), 0,
                                     static_cast<const int32_t*>(indptr->data), static_cast<const int32_t*>(last->data),
                                     static_cast<const int32_t*>(lens->data), (int)batch, scale, static_cast<float*>(out->data),
                                     ws->data, (size_t)ws->dims[0], variant, stream));
}

// out, k_cache, v_cache, workspace = NvjB200PagedDecodeWithKvAppend(query [B, 1, Hq, D], new_k [B, 1, Hkv, D], new_v,
//                                        k_cache [L, NB, P, Hkv, D], v_cache, block_table s32[B, W], seq_lens s32[B],
//                                        positions s32[B, 1], workspace u8[n])
//   attrs: layer_id (s32), scale (f32), variant (s32, optional).  Operand order of the reference's fused Triton call
//   (nanovllm_jax/kernels/full_attention_triton.py:488-581); aliases {3: 1, 4: 2, 8: 3}; out is f32[B, 1, Hq * D].
//   query must already be in the cache dtype (or f32), new_k / new_v in the cache dtype.
extern "C" XLA_FFI_Error* NvjB200PagedDecodeWithKvAppend(XLA_FFI_CallFrame* frame) {
  NVJ_XLA_PROLOGUE("NvjB200PagedDecodeWithKvAppend", 9, 0, 4);
  XLA_FFI_Buffer *q = Arg(frame, 0), *nk = Arg(frame, 1), *nv = Arg(frame, 2), *table = Arg(frame, 5), *lens = Arg(frame, 6);
  XLA_FFI_Buffer *pos = Arg(frame, 7), *out = Ret(frame, 0), *k_out = Ret(frame, 1), *v_out = Ret(frame, 2), *ws = Ret(frame, 3);
  if (q == nullptr || q->rank != 4 || q->dims[1] != 1 || FloatDtype(q) < 0) return Invalid(frame, "decode query must have shape [batch, 1, heads, head_dim]");
  if (k_out == nullptr || k_out->rank != 5 || FloatDtype(k_out) < 0 || !SameShape(k_out, v_out))
    return Invalid(frame, "k/v cache must have shape [layers, pages, page_size, kv_heads, head_dim]");
  const int64_t batch = q->dims[0], hq = q->dims[2], d = q->dims[3];
  const int64_t layers = k_out->dims[0], pages = k_out->dims[1], page = k_out->dims[2], hkv = k_out->dims[3];
  if (nk == nullptr || nk->rank != 4 || !SameShape(nk, nv) || nk->dims[0] != batch || nk->dims[1] != 1 || nk->dims[2] != hkv ||
      nk->dims[3] != d || nk->dtype != k_out->dtype || k_out->dims[4] != d || hq % hkv != 0)
    return Invalid(frame, "new_k/new_v must have shape [batch, 1, kv_heads, head_dim] in the cache dtype");
  if (!IsI32(table, 2) || table->dims[0] != batch || !IsI32(lens, 1) || lens->dims[0] != batch || !IsI32(pos, 2) ||
      pos->dims[0] != batch || pos->dims[1] != 1)
    return Invalid(frame, "block_table s32[B, W], seq_lens s32[B], positions s32[B, 1] expected");
  if (!Is(out, XLA_FFI_DataType_F32, 3) || out->dims[0] != batch || out->dims[2] != hq * d || !Is(ws, XLA_FFI_DataType_U8, 1))
    return Invalid(frame, "out must be f32[B, 1, Hq * D] and workspace u8[n]");
  int32_t layer = -1, variant = 0;
  float scale = 0.f;
  if (!IntAttr(frame, "layer_id", &layer) || !FloatAttr(frame, "scale", &scale)) return Invalid(frame, "attributes layer_id (s32) and scale (f32) are required");
  if (layer < 0 || layer >= layers) return Invalid(frame, "layer_id is out of range for cache");
  IntAttr(frame, "variant", &variant);
  const int64_t layer_bytes = pages * page * hkv * d * (FloatDtype(k_out) == NVJ_F32 ? 4 : 2);
  return FromStatus(frame, "nvj_paged_decode_fused_append",
                    nvj_paged_decode_fused_append(q->data, FloatDtype(q), nk->data, nv->data, static_cast<const int32_t*>(pos->data),
                                                  static_cast<char*>(k_out->data) + layer * layer_bytes,
                                                  static_cast<char*>(v_out->data) + layer * layer_bytes, FloatDtype(k_out), pages,
                                                  (int)page, (int)hkv, (int)d, (int)hq, static_cast<const int32_t*>(table->data),
                                                  (int)table->dims[1], static_cast<const int32_t*>(lens->data), (int)batch, scale,
                                                  static_cast<float*>(out->data), ws->data, (size_t)ws->dims[0], variant, stream));
}

// out, workspace = NvjB200PagedDecodeWide(q bf16[B, T, 8, 256], k_layer bf16[NB, 16, 2, 256], v_layer, block_table s32[B, W],
//                                         seq_lens s32[B], positions s32[B, T], workspace u8[n])      attrs: scale (f32)
//   out f32[B, T, 2048]; aliases {6: 1}.  Widths the streaming kernel does not take are UNIMPLEMENTED: use the packed prefill.
extern "C" XLA_FFI_Error* NvjB200PagedDecodeWide(XLA_FFI_CallFrame* frame) {
  NVJ_XLA_PROLOGUE("NvjB200PagedDecodeWide", 7, 0, 2);
  XLA_FFI_Buffer *q = Arg(frame, 0), *k = Arg(frame, 1), *v = Arg(frame, 2), *table = Arg(frame, 3), *lens = Arg(frame, 4);
  XLA_FFI_Buffer *pos = Arg(frame, 5), *out = Ret(frame, 0), *ws = Ret(frame, 1);
  Nhd c;
  if (q == nullptr || q->rank != 4 || FloatDtype(q) != NVJ_BF16 || q->dims[2] != 8 || q->dims[3] != 256 || !NhdOf(k, &c) ||
      !SameShape(k, v) || FloatDtype(k) != NVJ_BF16 || c.page_size != 16 || c.kv_heads != 2 || c.head_dim != 256)
    return MakeError(frame->api, XLA_FFI_Error_Code_UNIMPLEMENTED, "wide decode serves bf16 [B, T, 8, 256] over a bf16 cache [NB, 16, 2, 256]");
  const int64_t batch = q->dims[0], width = q->dims[1];
  if (!IsI32(table, 2) || table->dims[0] != batch || !IsI32(lens, 1) || lens->dims[0] != batch || !IsI32(pos, 2) ||
      pos->dims[0] != batch || pos->dims[1] != width)
    return Invalid(frame, "block_table s32[B, W], seq_lens s32[B], positions s32[B, T] expected");
  if (!Is(out, XLA_FFI_DataType_F32, 3) || out->dims[0] != batch || out->dims[1] != width || out->dims[2] != 2048 ||
      !Is(ws, XLA_FFI_DataType_U8, 1))
    return Invalid(frame, "out must be f32[B, T, 2048] and workspace u8[n]");
  float scale = 0.f;
  if (!FloatAttr(frame, "scale", &scale)) return Invalid(frame, "attribute scale (f32) is required");
  return FromStatus(frame, "nvj_paged_decode_wide",
                    nvj_paged_decode_wide(q->data, k->data, v->data, c.pages, static_cast<const int32_t*>(table->data), (int)table->dims[1],
                                          static_cast<const int32_t*>(lens->data), static_cast<const int32_t*>(pos->data), (int)batch,
                                          (int)width, scale, static_cast<float*>(out->data), ws->data, (size_t)ws->dims[0], stream));
}

// out, status, workspace = NvjB200PackedPrefillAttention(query [1, T, Hq, D], k_layer [NB, P, Hkv, D], v_layer, block_table s32[rows, W],
//                                       kv_lens s32[rows], positions s32[1, T], query_start_loc s32[rows + 1], workspace u8[n])
//   attrs: scale (f32), variant (s32, optional).  Operand order of the reference's packed Triton call
//   (nanovllm_jax/kernels/full_attention_triton.py:148-221); out f32[1, T, Hq * D]; aliases {7: 2}.
extern "C" XLA_FFI_Error* NvjB200PackedPrefillAttention(XLA_FFI_CallFrame* frame) {
  NVJ_XLA_PROLOGUE("NvjB200PackedPrefillAttention", 8, 0, 3);
  XLA_FFI_Buffer *q = Arg(frame, 0), *k = Arg(frame, 1), *v = Arg(frame, 2), *table = Arg(frame, 3), *lens = Arg(frame, 4);
  XLA_FFI_Buffer *pos = Arg(frame, 5), *qsl = Arg(frame, 6), *out = Ret(frame, 0), *status = Ret(frame, 1), *ws = Ret(frame, 2);
  Nhd c;
  if (q == nullptr || q->rank != 4 || q->dims[0] != 1 || FloatDtype(q) < 0) return Invalid(frame, "packed prefill query must have shape [1, token_bucket, heads, head_dim]");
  if (!NhdOf(k, &c) || !SameShape(k, v) || q->dims[3] != c.head_dim || q->dims[2] % c.kv_heads != 0)
    return Invalid(frame, "query / cache shapes do not agree");
  const int64_t tokens = q->dims[1], hq = q->dims[2];
  if (!IsI32(table, 2) || !IsI32(lens, 1) || lens->dims[0] != table->dims[0]) return Invalid(frame, "kv_lens shape must align with block_table rows");
  if (!IsI32(pos, 2) || pos->dims[0] != 1 || pos->dims[1] != tokens) return Invalid(frame, "packed positions must have shape [1, token_bucket]");
  if (!IsI32(qsl, 1) || qsl->dims[0] != table->dims[0] + 1) return Invalid(frame, "query_start_loc must have shape [rows + 1]");
  if (!Is(out, XLA_FFI_DataType_F32, 3) || out->dims[1] != tokens || out->dims[2] != hq * c.head_dim || !Is(ws, XLA_FFI_DataType_U8, 1))
    return Invalid(frame, "out must be f32[1, T, Hq * D] and workspace u8[n]");
  float scale = 0.f;
  int32_t variant = 0;
  if (!FloatAttr(frame, "scale", &scale)) return Invalid(frame, "attribute scale (f32) is required");
  IntAttr(frame, "variant", &variant);
  if (XLA_FFI_Error* error = ClearStatus(frame, status, stream)) return error;
  return FromStatus(frame, "nvj_paged_prefill_packed",
                    nvj_paged_prefill_packed(q->data, FloatDtype(q), k->data, v->data, FloatDtype(k), c.pages, (int)c.page_size,
                                             (int)c.kv_heads, (int)c.head_dim, (int)hq, static_cast<const int32_t*>(table->data),
                                             (int)table->dims[1], static_cast<const int32_t*>(lens->data),
                                             static_cast<const int32_t*>(pos->data), static_cast<const int32_t*>(qsl->data),
                                             (int)table->dims[0], (int)tokens, scale, static_cast<float*>(out->data),
                                             static_cast<int32_t*>(status->data), ws->dims[0] > 0 ? ws->data : nullptr,
                                             (size_t)ws->dims[0], variant, stream));
}

// k_cache, v_cache, status = NvjB200CopyBlocks(k_cache [L, NB, P, Hkv, D], v_cache, src_ids s32[n], dst_ids s32[n])   aliases {0: 0, 1: 1}
extern "C" XLA_FFI_Error* NvjB200CopyBlocks(XLA_FFI_CallFrame* frame) {
  NVJ_XLA_PROLOGUE("NvjB200CopyBlocks", 4, 0, 3);
  XLA_FFI_Buffer *src = Arg(frame, 2), *dst = Arg(frame, 3), *k_out = Ret(frame, 0), *v_out = Ret(frame, 1), *status = Ret(frame, 2);
  if (k_out == nullptr || k_out->rank != 5 || FloatDtype(k_out) < 0 || !SameShape(k_out, v_out))
    return Invalid(frame, "caches must be [layers, blocks, block_size, kv_heads, head_dim] of equal shape");
  if (!IsI32(src, 1) || !IsI32(dst, 1) || src->dims[0] != dst->dims[0]) return Invalid(frame, "src_ids and dst_ids must be s32[n]");
  const int64_t block_bytes = k_out->dims[2] * k_out->dims[3] * k_out->dims[4] * (FloatDtype(k_out) == NVJ_F32 ? 4 : 2);
  if (XLA_FFI_Error* error = ClearStatus(frame, status, stream)) return error;
  return FromStatus(frame, "nvj_copy_blocks",
                    nvj_copy_blocks(k_out->data, v_out->data, (int)k_out->dims[0], k_out->dims[1], block_bytes, k_out->dims[1] * block_bytes,
                                    static_cast<const int32_t*>(src->data), static_cast<const int32_t*>(dst->data), (int)src->dims[0],
                                    static_cast<int32_t*>(status->data), stream));
}

namespace {
int64_t RowBytes(const XLA_FFI_Buffer* b) {
  int64_t n = 1;
  for (int64_t i = 1; i < b->rank; ++i) n *= b->dims[i];
  const int64_t item = (b->dtype == XLA_FFI_DataType_F32 || b->dtype == XLA_FFI_DataType_S32) ? 4 : 2;
  return n * item;
}

// conv_dst, rec_dst, status = copy(conv_table, conv_pool, rec_table, rec_pool, table_slots s32[n], pool_slots s32[n])
XLA_FFI_Error* HybridCopy(XLA_FFI_CallFrame* frame, const char* name, bool restore) {
  NVJ_XLA_PROLOGUE(name, 6, 0, 3);
  XLA_FFI_Buffer *conv_table = Arg(frame, 0), *conv_pool = Arg(frame, 1), *rec_table = Arg(frame, 2), *rec_pool = Arg(frame, 3);
  XLA_FFI_Buffer *table_slots = Arg(frame, 4), *pool_slots = Arg(frame, 5), *status = Ret(frame, 2);
  // the destination arrays are the aliased results: pools for a snapshot ({1: 0, 3: 1}), tables for a restore ({0: 0, 2: 1})
  XLA_FFI_Buffer *conv_dst = Ret(frame, 0), *rec_dst = Ret(frame, 1);
  if (conv_table->rank < 2 || rec_table->rank < 2 || RowBytes(conv_table) != RowBytes(conv_pool) || RowBytes(rec_table) != RowBytes(rec_pool))
    return Invalid(frame, "table and pool rows must have the same size");
  if (!IsI32(table_slots, 1) || !IsI32(pool_slots, 1) || table_slots->dims[0] != pool_slots->dims[0])
    return Invalid(frame, "table_slots and pool_slots must be s32[n]");
  if (XLA_FFI_Error* error = ClearStatus(frame, status, stream)) return error;
  const int n = (int)table_slots->dims[0];
  const int32_t *ts = static_cast<const int32_t*>(table_slots->data), *ps = static_cast<const int32_t*>(pool_slots->data);
  const int rc = restore ? nvj_hybrid_restore(conv_dst->data, conv_pool->data, RowBytes(conv_table), rec_dst->data, rec_pool->data,
                                              RowBytes(rec_table), rec_table->dims[0], rec_pool->dims[0], ts, ps, n,
                                              static_cast<int32_t*>(status->data), stream)
                         : nvj_hybrid_snapshot(conv_table->data, conv_dst->data, RowBytes(conv_table), rec_table->data, rec_dst->data,
                                               RowBytes(rec_table), rec_table->dims[0], rec_pool->dims[0], ts, ps, n,
                                               static_cast<int32_t*>(status->data), stream);
  return FromStatus(frame, name, rc);
}
}  // namespace

extern "C" XLA_FFI_Error* NvjB200HybridSnapshot(XLA_FFI_CallFrame* frame) { return HybridCopy(frame, "NvjB200HybridSnapshot", false); }
extern "C" XLA_FFI_Error* NvjB200HybridRestore(XLA_FFI_CallFrame* frame) { return HybridCopy(frame, "NvjB200HybridRestore", true); }

// seq_lens, positions, status = NvjB200AdvanceDecodeMetadata(seq_lens s32[B], positions s32[B, 1])
//   attrs: table_width, block_size (s32); aliases {0: 0, 1: 1}
extern "C" XLA_FFI_Error* NvjB200AdvanceDecodeMetadata(XLA_FFI_CallFrame* frame) {
  NVJ_XLA_PROLOGUE("NvjB200AdvanceDecodeMetadata", 2, 0, 3);
  XLA_FFI_Buffer *lens = Ret(frame, 0), *pos = Ret(frame, 1), *status = Ret(frame, 2);
  int32_t width = 0, block = 0;
  if (!IsI32(lens, 1) || pos == nullptr || pos->dtype != XLA_FFI_DataType_S32 || Elements(pos) != lens->dims[0])
    return Invalid(frame, "seq_lens s32[B] and positions s32[B, 1] expected");
  if (!IntAttr(frame, "table_width", &width) || !IntAttr(frame, "block_size", &block)) return Invalid(frame, "attributes table_width and block_size (s32) are required");
  if (XLA_FFI_Error* error = ClearStatus(frame, status, stream)) return error;
  return FromStatus(frame, "nvj_advance_decode_metadata",
                    nvj_advance_decode_metadata(static_cast<int32_t*>(lens->data), static_cast<int32_t*>(pos->data), (int)lens->dims[0], width,
                                                block, static_cast<int32_t*>(status->data), stream));
}

// tokens s32[rows] = NvjB200RowArgmax(x f32[rows, n])
extern "C" XLA_FFI_Error* NvjB200RowArgmax(XLA_FFI_CallFrame* frame) {
  NVJ_XLA_PROLOGUE("NvjB200RowArgmax", 1, 0, 1);
  XLA_FFI_Buffer *x = Arg(frame, 0), *tokens = Ret(frame, 0);
  if (!Is(x, XLA_FFI_DataType_F32, 2) || !IsI32(tokens, 1) || tokens->dims[0] != x->dims[0]) return Invalid(frame, "x f32[rows, n] -> tokens s32[rows]");
  return FromStatus(frame, "nvj_row_argmax",
                    nvj_row_argmax(static_cast<const float*>(x->data), (int)x->dims[0], (int)x->dims[1], static_cast<int32_t*>(tokens->data), stream));
}
