"""CPU oracle for the paged KV-cache hot path.  TEST INFRASTRUCTURE ONLY.

A NumPy (+ ml_dtypes.bfloat16) restatement of the reference's pure-JAX paged
path.  Only tests, the smoke check and the benchmark's CPU-baseline leg may
import this module; the product never does.

Reference functions restated (paths relative to the reference project root):
  compute_slot_mapping            nanovllm_jax/kv_cache.py:410-446
  compute_packed_slot_mapping     nanovllm_jax/kv_cache.py:449-473
  update_kv_cache                 nanovllm_jax/kv_cache.py:476-564
  write_kv valid masks            nanovllm_jax/backends.py:1050-1057
  paged_attention (legacy)        nanovllm_jax/kv_cache.py:567-647
  paged_attention_prefill         nanovllm_jax/kv_cache.py:650-718
  paged_attention_prefill_packed  nanovllm_jax/kv_cache.py:721-849
  paged_attention_decode          nanovllm_jax/kv_cache.py:852-998
  NHD / CSR helpers and decode    nanovllm_jax/kernels/paged_attention.py:23-54,101-194
  NHD append                      nanovllm_jax/kernels/flashinfer_ffi.py:626-665

Pinning.  The integer paths (slot arithmetic, masks, scatter semantics) are pinned
by the known answers of the reference's own tests (tests/test_oracle_pins.py
lists them with their source lines).  The reference stores NO golden vectors for
attention values, and JAX is not installed where this was written, so the
floating-point results are "parity unpinned": they are cross-checked only
against an independent dense float64 attention (oracle/dense_ref.py), which is
the same check the reference's tests make (paged == dense).

Numeric modes of the attention functions:
  mode="fp32"  inputs widened to float32, everything computed in float32.  This
               is the contract the CUDA kernels are gated on (max-abs 2e-2).
  mode="ref"   results rounded to the dtype JAX type promotion would give after
               each array-level operation (bf16 q with a bf16 cache: scores,
               weights and output are bf16).  An approximation of XLA's rounding
               points, reported beside the gate, never gated on.
"""

from __future__ import annotations

import numpy as np

try:  # bf16 on the host
    from ml_dtypes import bfloat16
except Exception:  # pragma: no cover - ml_dtypes is part of the image
    bfloat16 = None

MASK_VALUE = -1e10  # the reference fills masked scores with -1e10, not -inf


# --------------------------------------------------------------------------- slots

def compute_slot_mapping(positions, block_table, block_size):
    """slot[b, t] = block_table[b, pos // bs] * bs + pos % bs."""
    positions = np.asarray(positions)
    block_table = np.asarray(block_table)
    rows = np.arange(positions.shape[0])[:, None]
    blocks = block_table[rows, positions // block_size]
    return (blocks * block_size + positions % block_size).astype(np.int32)


def compute_packed_slot_mapping(positions, block_table, token_row_ids, block_size):
    """Packed form: the table row of each token comes from token_row_ids (clipped)."""
    positions = np.asarray(positions)
    token_row_ids = np.asarray(token_row_ids)
    block_table = np.asarray(block_table)
    if positions.shape != token_row_ids.shape:
        raise ValueError("positions and token_row_ids must have matching shapes")
    if block_table.ndim != 2:
        raise ValueError("block_table must be a 2D tensor [batch, max_blocks_per_seq]")
    if block_size <= 0:
        raise ValueError("block_size must be positive")
    rows = np.clip(token_row_ids, 0, block_table.shape[0] - 1)
    blocks = block_table[rows, positions // block_size]
    return (blocks * block_size + positions % block_size).astype(np.int32)


def write_kv_valid_mask(slot_mapping_shape, query_start_loc, packed):
    """Valid-token mask PureJAXBackend.write_kv derives from the metadata."""
    qsl = np.asarray(query_start_loc).astype(np.int64)
    n = int(np.prod(slot_mapping_shape))
    if packed:
        return (np.arange(n).reshape(slot_mapping_shape) < qsl[-1])
    qlen = np.diff(qsl)
    return np.arange(slot_mapping_shape[1])[None, :] < qlen[:, None]


# --------------------------------------------------------------------------- append

def _layer_view(cache, layer_idx):
    if layer_idx < 0:
        raise ValueError("layer_idx must be non-negative")
    if cache.ndim not in (4, 5):
        raise ValueError(f"Unsupported KV cache rank: {cache.ndim}")
    if layer_idx >= cache.shape[0]:
        raise ValueError(f"layer_idx {layer_idx} is out of bounds for {cache.shape[0]} layers")
    layer = cache[layer_idx]
    return layer.reshape(-1, layer.shape[-2], layer.shape[-1])  # flat slots, a view


def update_kv_cache(k_cache, v_cache, slot_mapping, new_k, new_v, layer_idx=0, valid_mask=None):
    """Scatter new rows into copies of the caches; masked tokens are dropped.

    Later tokens win on duplicate slots here (XLA leaves that unspecified).
    """
    if k_cache.shape != v_cache.shape:
        raise ValueError("k_cache and v_cache must have the same shape")
    k_out, v_out = k_cache.copy(), v_cache.copy()
    kf, vf = _layer_view(k_out, layer_idx), _layer_view(v_out, layer_idx)
    slots = np.asarray(slot_mapping).reshape(-1)
    nk = np.asarray(new_k).astype(kf.dtype).reshape(-1, kf.shape[1], kf.shape[2])
    nv = np.asarray(new_v).astype(vf.dtype).reshape(-1, vf.shape[1], vf.shape[2])
    keep = np.ones(slots.shape, bool) if valid_mask is None else np.asarray(valid_mask).reshape(-1).astype(bool)
    for i in np.nonzero(keep)[0]:
        s = int(slots[i])
        if 0 <= s < kf.shape[0]:
            kf[s] = nk[i]
            vf[s] = nv[i]
    return k_out, v_out


def kv_append_paged_nhd(append_key, append_value, batch_indices, positions, k_cache, v_cache,
                        kv_indices, kv_indptr, kv_last_page_len=None, valid_mask=None):
    """Page-table form on one layer slice [pages, P, Hkv, D]."""
    if k_cache.shape != v_cache.shape:
        raise ValueError("k_cache and v_cache must have the same shape")
    k_out, v_out = k_cache.copy(), v_cache.copy()
    page_size = k_cache.shape[1]
    positions = np.asarray(positions).astype(np.int64)
    pages = np.asarray(kv_indices)[np.asarray(kv_indptr)[np.asarray(batch_indices)] + positions // page_size]
    for i in range(len(positions)):
        if valid_mask is not None and not valid_mask[i]:
            continue
        k_out[pages[i], positions[i] % page_size] = append_key[i]
        v_out[pages[i], positions[i] % page_size] = append_value[i]
    return k_out, v_out


def copy_blocks(k_cache, v_cache, src_ids, dst_ids):
    """cache[:, dst] = cache[:, src] for 5-D caches (prefix reuse by copy)."""
    k_out, v_out = k_cache.copy(), v_cache.copy()
    k_out[:, dst_ids] = k_cache[:, src_ids]
    v_out[:, dst_ids] = v_cache[:, src_ids]
    return k_out, v_out


# --------------------------------------------------------------------------- attention

def _result_dtype(q, k):
    """dtype JAX promotion gives q (x) k."""
    f32 = np.dtype(np.float32)
    if q.dtype == f32 or k.dtype == f32:
        return f32
    if q.dtype == k.dtype:
        return q.dtype
    return f32  # bf16 x f16 promotes to f32


def _round(x, dtype, mode):
    if mode == "ref" and np.dtype(dtype) != np.dtype(np.float32):
        return x.astype(dtype).astype(np.float32)
    return x


def _gather_window(cache, layer_idx, block_table, block_size, max_kv_len):
    """[rows, max_kv_len, Hkv, D] window addressed through the block table."""
    flat = _layer_view(np.asarray(cache), layer_idx)
    pos = np.arange(max_kv_len)
    slots = np.asarray(block_table)[:, pos // block_size].astype(np.int64) * block_size + pos % block_size
    return flat[slots]


def _masked_attention(q, k, v, mask, scale, groups, mode):
    """q [B,T,Hq,D], k/v [B,S,Hkv,D], mask [B,T,S] -> [B,T,Hq*D] (float32 array)."""
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]
    rdt = _result_dtype(q, k)
    qf = q.astype(np.float32).reshape(B, T, Hkv, groups, D)
    kf = k.astype(np.float32)
    vf = v.astype(np.float32)
    # batched GEMM form of einsum("btkgd,bskd->btkgs")
    S = k.shape[1]
    qm = qf.transpose(0, 2, 1, 3, 4).reshape(B, Hkv, T * groups, D)
    scores = np.matmul(qm, kf.transpose(0, 2, 3, 1)).reshape(B, Hkv, T, groups, S).transpose(0, 2, 1, 3, 4)
    scores = _round(scores, rdt, mode)
    scores = _round(scores * np.float32(scale), rdt, mode)
    scores = np.where(mask[:, :, None, None, :], scores, np.float32(MASK_VALUE))
    scores = _round(scores, rdt, mode)
    mx = scores.max(axis=-1, keepdims=True)
    e = _round(np.exp(_round(scores - mx, rdt, mode)), rdt, mode)
    w = _round(e / _round(e.sum(axis=-1, keepdims=True), rdt, mode), rdt, mode)
    # batched GEMM form of einsum("btkgs,bskd->btkgd")
    wm = w.transpose(0, 2, 1, 3, 4).reshape(B, Hkv, T * groups, S)
    out = np.matmul(wm, vf.transpose(0, 2, 1, 3)).reshape(B, Hkv, T, groups, D).transpose(0, 2, 1, 3, 4)
    out = _round(out, rdt, mode)
    return out.reshape(B, T, Hq * D), rdt


def _finish(out, rdt, mode):
    return out.astype(rdt) if mode == "ref" else out.astype(np.float32)


def paged_attention_decode(query, k_cache, v_cache, block_table, kv_lens, block_size, scale,
                           num_key_value_groups, max_kv_len=None, layer_idx=0, positions=None,
                           mode="fp32"):
    query = np.asarray(query)
    block_table = np.asarray(block_table)
    kv_lens = np.asarray(kv_lens)
    batch, query_len = query.shape[:2]
    if query_len < 1:
        raise ValueError("decode attention requires query_len >= 1")
    if block_table.ndim != 2:
        raise ValueError("block_tables must be a 2D tensor [batch, max_blocks_per_seq]")
    if block_table.shape[0] != batch:
        raise ValueError(f"query batch {batch} must match block_tables batch {block_table.shape[0]}")
    if kv_lens.shape[0] != batch:
        raise ValueError("seq_lens shape must align with query batch")
    if positions is not None and tuple(np.shape(positions)) != (batch, query_len):
        raise ValueError("positions must have shape [batch, query_len]")
    if positions is None and query_len != 1:
        raise ValueError("positions are required for multi-token decode attention")
    if block_size <= 0:
        raise ValueError("block_size must be positive")
    if max_kv_len is None:
        max_kv_len = block_table.shape[1] * block_size
    if max_kv_len <= 0:
        raise ValueError("max_kv_len must be positive")
    if max_kv_len > block_table.shape[1] * block_size:
        raise ValueError("max_kv_len exceeds the physical cache span covered by block_tables")
    k = _gather_window(k_cache, layer_idx, block_table, block_size, max_kv_len)
    v = _gather_window(v_cache, layer_idx, block_table, block_size, max_kv_len)
    key_pos = np.arange(max_kv_len)
    mask = np.broadcast_to((key_pos[None, :] < kv_lens[:, None])[:, None, :], (batch, query_len, max_kv_len))
    if positions is not None:
        mask = mask & (key_pos[None, None, :] <= np.asarray(positions)[:, :, None])
    out, rdt = _masked_attention(query, k, v, mask, scale, num_key_value_groups, mode)
    return _finish(out, rdt, mode)


def paged_attention_prefill(query, k_cache, v_cache, block_table, kv_lens, positions, block_size,
                            scale, num_key_value_groups, layer_idx=0, mode="fp32"):
    """Rectangular prefill with a cached prefix: same masks as multi-token decode."""
    return paged_attention_decode(query, k_cache, v_cache, block_table, kv_lens, block_size, scale,
                                  num_key_value_groups, layer_idx=layer_idx, positions=positions,
                                  mode=mode)


def paged_attention(query, k_cache, v_cache, slot_mapping, kv_lens, scale, num_key_value_groups,
                    layer_idx=0, mode="fp32"):
    """Legacy prefill: keys gathered by slot_mapping, plain causal mask, no length mask."""
    query = np.asarray(query)
    B, T = query.shape[:2]
    kf = _layer_view(np.asarray(k_cache), layer_idx)[np.asarray(slot_mapping)]
    vf = _layer_view(np.asarray(v_cache), layer_idx)[np.asarray(slot_mapping)]
    mask = np.broadcast_to(np.tril(np.ones((T, T), bool))[None], (B, T, T))
    out, rdt = _masked_attention(query, kf, vf, mask, scale, num_key_value_groups, mode)
    return _finish(out, rdt, mode)


def paged_attention_prefill_packed(query, k_cache, v_cache, block_table, kv_lens, positions,
                                   token_row_ids, query_start_loc, block_size, scale,
                                   num_key_value_groups, layer_idx=0, max_query_len=None, mode="fp32"):
    """Ragged packed prefill: [1, T, Hq, D] -> [1, T, Hq*D]; padded tokens give 0.

    The pure-JAX path casts q to the cache dtype and returns the cache dtype
    (kv_cache.py:834-843); mode="ref" does the same, mode="fp32" returns float32.
    """
    query = np.asarray(query)
    positions = np.asarray(positions)
    block_table = np.asarray(block_table)
    kv_lens = np.asarray(kv_lens)
    qsl = np.asarray(query_start_loc).astype(np.int64)
    if query.ndim != 4 or query.shape[0] != 1:
        raise ValueError("packed prefill query must have shape [1, token_bucket, heads, head_dim]")
    if positions.shape != np.shape(token_row_ids) or positions.shape[0] != 1:
        raise ValueError("packed positions and token_row_ids must have shape [1, token_bucket]")
    if block_table.ndim != 2:
        raise ValueError("block_table must be a 2D tensor [batch, max_blocks_per_seq]")
    if kv_lens.shape[0] != block_table.shape[0]:
        raise ValueError("kv_lens shape must align with block_table rows")
    _, T, Hq, D = query.shape
    max_kv_len = block_table.shape[1] * block_size
    kwin = _gather_window(k_cache, layer_idx, block_table, block_size, max_kv_len)
    vwin = _gather_window(v_cache, layer_idx, block_table, block_size, max_kv_len)
    cache_dtype = kwin.dtype
    out = np.zeros((T, Hq * D), np.float32)
    key_pos = np.arange(max_kv_len)
    for r in range(block_table.shape[0]):
        lo, hi = int(qsl[r]), int(qsl[r + 1])
        hi = min(hi, T)
        if hi <= lo:
            continue
        q_r = query[0, lo:hi][None]
        if mode == "ref":
            q_r = q_r.astype(cache_dtype)
        mask = (key_pos[None, :] < kv_lens[r]) & (key_pos[None, :] <= positions[0, lo:hi, None])
        o, _ = _masked_attention(q_r, kwin[r][None], vwin[r][None], mask[None], scale,
                                 num_key_value_groups, mode)
        out[lo:hi] = o[0]
    res = out.reshape(1, T, Hq * D)
    return res.astype(cache_dtype) if mode == "ref" else res


# --------------------------------------------------------------------------- NHD / CSR forms

def kv_last_page_len_from_seq_lens(seq_lens, page_size):
    if page_size <= 0:
        raise ValueError("page_size must be positive")
    seq_lens = np.asarray(seq_lens).astype(np.int32)
    return np.where(seq_lens > 0, (seq_lens - 1) % page_size + 1, 0).astype(np.int32)


def dense_block_tables_to_kv_indptr(block_tables):
    block_tables = np.asarray(block_tables)
    if block_tables.ndim != 2:
        raise ValueError("block_tables must have shape [batch, max_pages_per_sequence]")
    b, w = block_tables.shape
    return block_tables.reshape(-1).astype(np.int32), (np.arange(b + 1) * w).astype(np.int32)


def paged_decode_attention_gqa_nhd(q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len,
                                   seq_lens, softmax_scale, max_pages_per_sequence=None, mode="fp32"):
    """CSR form on one layer slice: q [B,Hq,D] -> [B,Hq,D]."""
    q = np.asarray(q)
    kv_indptr = np.asarray(kv_indptr)
    kv_indices = np.asarray(kv_indices)
    B, Hq, D = q.shape
    P, Hkv = k_cache.shape[1], k_cache.shape[2]
    if max_pages_per_sequence is None:
        max_pages_per_sequence = kv_indices.shape[0] // B
    W = int(max_pages_per_sequence)
    counts = kv_indptr[1:] - kv_indptr[:-1]
    pos = np.arange(W * P)
    page_off = np.minimum((pos // P)[None, :], np.maximum(counts, 1)[:, None] - 1)
    pages = kv_indices[kv_indptr[:-1, None] + page_off]
    k = np.asarray(k_cache)[pages, (pos % P)[None, :]]
    v = np.asarray(v_cache)[pages, (pos % P)[None, :]]
    eff = np.where(counts > 0, (counts - 1) * P + np.asarray(kv_last_page_len), 0)
    eff = np.minimum(eff, np.asarray(seq_lens))
    mask = (pos[None, :] < eff[:, None])[:, None, :]
    out, rdt = _masked_attention(q[:, None], k, v, mask, softmax_scale, Hq // Hkv, mode)
    return _finish(out, rdt, mode).reshape(B, Hq, D)
