"""Paged KV-cache interface: the reference's `kv_cache.py` names on torch CUDA tensors.

Same containers, function names, argument orders and error behaviour as
nanovllm_jax/kv_cache.py, so callers of the reference module (the backend, and
the direct callers model_jit.py:388-421, chunked_prefill.py:214-229) read the
same.  Differences that follow from running on torch + hand-written kernels:

* arrays are torch CUDA tensors; every function launches sm_100a kernels through
  the C ABI and there is no CPU path;
* the reference is functional and gets in-place reuse from buffer donation
  (model_executor.py:638-641); here the caches are updated in place and the same
  tensors are returned;
* attention accumulates in fp32.  Outputs follow the reference's dtype promotion
  (bf16 q with a bf16 cache gives bf16) unless `out_dtype` is given; the backend
  asks for fp32 like the reference's accelerated routes do.
"""

from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, List, Optional, Tuple

import torch

from .kernels import paged_kv as _k


@dataclass
class KVCacheSpec:
    """Logical KV cache shape requested by the engine (kv_cache.py:9-19)."""

    num_layers: int
    num_blocks: int
    block_size: int
    num_kv_heads: int
    head_dim: int
    dtype: Any = torch.float32
    max_kv_cache_bytes: Optional[int] = None


@dataclass
class KVCacheStorage:
    """Physical arrays `[num_layers, num_blocks, block_size, num_kv_heads, head_dim]` (kv_cache.py:22-32)."""

    k_cache: torch.Tensor
    v_cache: torch.Tensor


@dataclass
class AttentionMetadata:
    """Per-step paged/ragged attention metadata (kv_cache.py:51-64).

    `slot_mapping` may be given as a zero-argument callable; it is then computed when first read.  A width-1 decode
    step that goes through the fused append + attention kernel never reads it (the kernel resolves the slots from the
    block table itself), so the step is spared a launch.
    """

    slot_mapping: torch.Tensor
    block_tables: torch.Tensor
    seq_lens: torch.Tensor
    query_start_loc: torch.Tensor
    num_prefill_tokens: int
    num_decode_tokens: int
    positions: Optional[torch.Tensor] = None
    max_kv_len: Optional[int] = None
    token_row_ids: Optional[torch.Tensor] = None
    max_query_len: Optional[int] = None
    # not in the reference: the caller's own count of 1-token rows in a packed batch (None = not told)
    single_token_rows: Optional[int] = None
    # not in the reference: 64-token query tiles the other rows of that batch make up (sum of ceil(len / 64); None = not told)
    query_tile_pairs: Optional[int] = None


def _read_slot_mapping(self):
    value = self.__dict__.get("slot_mapping")
    if value is not None and not isinstance(value, torch.Tensor) and callable(value):
        value = value()
        self.__dict__["slot_mapping"] = value
    return value


def _store_slot_mapping(self, value):
    self.__dict__["slot_mapping"] = value


AttentionMetadata.slot_mapping = property(_read_slot_mapping, _store_slot_mapping)


@dataclass
class BlockTables:
    """Host-side allocation state snapshot (kv_cache.py:67-73)."""

    tables: List[List[int]]
    ref_counts: Optional[Any] = None
    hashes: Optional[Any] = None


@dataclass
class HybridLayerState:
    """GDN conv / recurrent state kept apart from the KV storage (kv_cache.py:76-81)."""

    conv_state: Optional[torch.Tensor] = None
    recurrent_state: Optional[torch.Tensor] = None


@dataclass
class KVCacheState:
    """Cache arrays plus block table, lengths and slot mapping (kv_cache.py:84-139)."""

    k_cache: torch.Tensor
    v_cache: torch.Tensor
    block_table: torch.Tensor
    kv_lens: torch.Tensor
    slot_mapping: torch.Tensor
    conv_state: Optional[torch.Tensor] = None
    recurrent_state: Optional[torch.Tensor] = None

    @property
    def storage(self) -> KVCacheStorage:
        return KVCacheStorage(self.k_cache, self.v_cache)

    @property
    def attention_metadata(self) -> AttentionMetadata:
        batch, query_len = self.slot_mapping.shape
        qsl = torch.arange(batch + 1, dtype=torch.int32, device=self.slot_mapping.device) * query_len
        return AttentionMetadata(self.slot_mapping, self.block_table, self.kv_lens, qsl,
                                 int(batch * query_len), 0, None)

    @property
    def hybrid_state(self) -> HybridLayerState:
        return HybridLayerState(self.conv_state, self.recurrent_state)

    def replace(self, **kwargs) -> "KVCacheState":
        return replace(self, **kwargs)


def _itemsize(dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def estimate_kv_cache_bytes(spec: KVCacheSpec) -> int:
    """Total bytes of the K and V arrays (kv_cache.py:142-152)."""
    n = spec.num_layers * spec.num_blocks * spec.block_size * spec.num_kv_heads * spec.head_dim
    return int(n * _itemsize(spec.dtype) * 2)


def cap_num_kv_cache_blocks(spec: KVCacheSpec) -> int:
    """Largest block count within `max_kv_cache_bytes` (kv_cache.py:155-170)."""
    if spec.max_kv_cache_bytes is None:
        return spec.num_blocks
    per_block = estimate_kv_cache_bytes(replace(spec, num_blocks=1))
    if per_block <= 0:
        raise ValueError("Invalid KV cache spec: bytes_per_block must be positive")
    capped = spec.max_kv_cache_bytes // per_block
    if capped < 1:
        raise ValueError("max_kv_cache_bytes is too small for one KV block "
                         f"({spec.max_kv_cache_bytes} < {per_block})")
    return min(spec.num_blocks, int(capped))


def init_kv_cache(num_blocks, block_size, num_kv_heads, head_dim, max_seqs, max_blocks_per_seq,
                  num_layers=24, dtype=torch.float32, max_kv_cache_bytes=None, device="cuda") -> KVCacheState:
    """Zero-filled caches and tables (kv_cache.py:216-271)."""
    spec = KVCacheSpec(num_layers, num_blocks, block_size, num_kv_heads, head_dim, dtype, max_kv_cache_bytes)
    nb = cap_num_kv_cache_blocks(spec)
    shape = (num_layers, nb, block_size, num_kv_heads, head_dim)
    return KVCacheState(
        k_cache=torch.zeros(shape, dtype=dtype, device=device),
        v_cache=torch.zeros(shape, dtype=dtype, device=device),
        block_table=torch.zeros((max_seqs, max_blocks_per_seq), dtype=torch.int32, device=device),
        kv_lens=torch.zeros(max_seqs, dtype=torch.int32, device=device),
        slot_mapping=torch.zeros((max_seqs, 1), dtype=torch.int32, device=device),
    )


def init_hybrid_state(config, batch_size: int = 1, dtype=None, device="cuda") -> HybridLayerState:
    """Zero GDN state tables `[S, L_lin, conv_dim, K]` and `[S, L_lin, Hv, Dv, Dk]` fp32 (kv_cache.py:379-407)."""
    if dtype is None:
        dtype = getattr(config, "get_dtype", lambda: torch.float32)()
    key_dim = config.linear_num_key_heads * config.linear_key_head_dim
    value_dim = config.linear_num_value_heads * config.linear_value_head_dim
    n_lin = sum(1 for lt in config.layer_types if lt == "linear_attention")
    conv = torch.zeros((batch_size, n_lin, key_dim * 2 + value_dim, config.linear_conv_kernel_size),
                       dtype=dtype, device=device)
    rec = torch.zeros((batch_size, n_lin, config.linear_num_value_heads, config.linear_value_head_dim,
                       config.linear_key_head_dim), dtype=torch.float32, device=device)
    return HybridLayerState(conv, rec)


def _resolve_kv_layer(cache: torch.Tensor, layer_idx: int) -> Tuple[torch.Tensor, bool]:
    """One layer of a 5-D `[L, NB, bs, Hkv, D]` or flat 4-D `[L, slots, Hkv, D]` cache (kv_cache.py:341-369)."""
    if layer_idx < 0:
        raise ValueError("layer_idx must be non-negative")
    if cache.ndim not in (4, 5):
        raise ValueError(f"Unsupported KV cache rank: {cache.ndim}")
    if layer_idx >= cache.shape[0]:
        raise ValueError(f"layer_idx {layer_idx} is out of bounds for {cache.shape[0]} layers")
    return cache[layer_idx], cache.ndim == 4


def _paged_layer(cache: torch.Tensor, layer_idx: int, block_size: int) -> torch.Tensor:
    """Layer slice viewed as `[pages, block_size, Hkv, D]` whatever the cache rank."""
    layer, flat = _resolve_kv_layer(cache, layer_idx)
    if flat:
        if layer.shape[0] % block_size != 0:
            raise ValueError("flat cache slot count must be a multiple of block_size")
        layer = layer.view(layer.shape[0] // block_size, block_size, layer.shape[1], layer.shape[2])
    elif layer.shape[1] != block_size:
        raise ValueError("block_size must match the cache page size")
    return layer


def compute_slot_mapping(positions, block_table, block_size, is_prefill: bool = True):
    """slot = block_table[b, pos // bs] * bs + pos % bs for positions `[B, T]` (kv_cache.py:410-446)."""
    return _k.compute_slot_mapping(positions.to(torch.int32), block_table.to(torch.int32), block_size)


def compute_packed_slot_mapping(positions, block_table, token_row_ids, block_size):
    """Packed `[1, T]` form; the table row of each token is its (clipped) row id (kv_cache.py:449-473)."""
    if positions.shape != token_row_ids.shape:
        raise ValueError("positions and token_row_ids must have matching shapes")
    if block_table.ndim != 2:
        raise ValueError("block_table must be a 2D tensor [batch, max_blocks_per_seq]")
    if block_size <= 0:
        raise ValueError("block_size must be positive")
    return _k.compute_slot_mapping(positions.to(torch.int32), block_table.to(torch.int32), block_size,
                                   token_row_ids.to(torch.int32))


def update_kv_cache(k_cache, v_cache, slot_mapping, new_k, new_v, layer_idx: int = 0, valid_mask=None):
    """Write new K/V rows at their slots (kv_cache.py:476-564); in place, returns the same tensors.

    With `valid_mask=None` every token of `slot_mapping` is written, padded ones
    included, as in the reference.  Duplicate valid slots: winner unspecified.
    """
    if k_cache.shape != v_cache.shape:
        raise ValueError("k_cache and v_cache must have the same shape")
    k_layer, _ = _resolve_kv_layer(k_cache, layer_idx)
    v_layer, _ = _resolve_kv_layer(v_cache, layer_idx)
    sm = slot_mapping.to(torch.int32)
    if sm.ndim != 2:
        sm = sm.reshape(1, -1)
    _k.kv_append_slots(new_k, new_v, sm, k_layer, v_layer, valid_mask=valid_mask)
    return k_cache, v_cache


def _promoted(query, cache, out_dtype):
    return out_dtype if out_dtype is not None else torch.promote_types(query.dtype, cache.dtype)


def paged_attention_decode(query, k_cache, v_cache, block_table, kv_lens, block_size, scale,
                           num_key_value_groups, max_kv_len=None, layer_idx: int = 0, positions=None,
                           out_dtype=None):
    """Decode attention over a bounded paged window (kv_cache.py:852-998) -> `[B, T, Hq*D]`.

    Query width > 1 (speculative verification, rectangular prefill) applies the causal mask
    p <= positions[b, t]; such a batch travels the packed prefill route with rows of equal width.
    """
    batch, query_len, num_heads, head_dim = query.shape
    if query_len < 1:
        raise ValueError("decode attention requires query_len >= 1")
    if block_table.ndim != 2:
        raise ValueError("block_tables must be a 2D tensor [batch, max_blocks_per_seq]")
    if block_table.shape[0] != batch:
        raise ValueError(f"query batch {batch} must match block_tables batch {block_table.shape[0]}")
    if kv_lens.shape[0] != batch:
        raise ValueError("seq_lens shape must align with query batch")
    if positions is not None and tuple(positions.shape) != (batch, query_len):
        raise ValueError("positions must have shape [batch, query_len]")
    if positions is None and query_len != 1:
        raise ValueError("positions are required for multi-token decode attention")
    if block_size <= 0:
        raise ValueError("block_size must be positive")
    window = block_table.shape[1] * block_size
    if max_kv_len is None:
        max_kv_len = window
    if max_kv_len <= 0:
        raise ValueError("max_kv_len must be positive")
    if max_kv_len > window:
        raise ValueError("max_kv_len exceeds the physical cache span covered by block_tables")
    k_layer = _paged_layer(k_cache, layer_idx, block_size)
    v_layer = _paged_layer(v_cache, layer_idx, block_size)
    if max_kv_len > k_layer.shape[0] * block_size:
        raise ValueError("max_kv_len exceeds the physical cache slot capacity")
    if num_heads != k_layer.shape[2] * num_key_value_groups:
        raise ValueError("num_key_value_groups does not match the head counts")
    lens = kv_lens.to(torch.int32).clamp(max=int(max_kv_len))
    tables = block_table.to(torch.int32)
    if positions is not None and query_len > 1 and _k.wide_decode_supported(query, k_layer):
        # 2..4 query tokens per row: the streaming kernel of the width-1 path with the products on the tensor cores
        out = _k.paged_decode_attention_wide(query, k_layer, v_layer, tables, lens, positions, scale)
        return out.to(_promoted(query, k_cache, out_dtype))
    if positions is not None and query_len > 1:
        # a rectangular batch is a packed batch with rows of equal width: K/V of a row are then read once for all
        # of its query tokens (tensor-core tiles for the model's shape) instead of once per token
        qsl = torch.arange(batch + 1, dtype=torch.int32, device=query.device) * query_len
        out = _k.packed_paged_prefill_attention(query.reshape(1, batch * query_len, num_heads, head_dim), k_layer, v_layer,
                                                tables.contiguous(), lens.contiguous(),
                                                positions.to(torch.int32).reshape(1, -1), qsl, block_size, scale,
                                                num_key_value_groups)
        return out.reshape(batch, query_len, num_heads * head_dim).to(_promoted(query, k_cache, out_dtype))
    if positions is not None:
        lens = torch.minimum(lens, positions.to(torch.int32).reshape(-1) + 1)
    out = _k.paged_decode_attention(query.reshape(batch * query_len, num_heads, head_dim), k_layer, v_layer,
                                    tables, lens, scale)
    return out.reshape(batch, query_len, num_heads * head_dim).to(_promoted(query, k_cache, out_dtype))


def paged_attention_prefill(query, k_cache, v_cache, block_table, kv_lens, positions, block_size, scale,
                            num_key_value_groups, layer_idx: int = 0, out_dtype=None):
    """Rectangular prefill with a cached prefix (kv_cache.py:650-718): same masks as wide decode."""
    return paged_attention_decode(query, k_cache, v_cache, block_table, kv_lens, block_size, scale,
                                  num_key_value_groups, layer_idx=layer_idx, positions=positions,
                                  out_dtype=out_dtype)


def paged_attention(query, k_cache, v_cache, slot_mapping, kv_lens, scale, num_key_value_groups,
                    layer_idx: int = 0, out_dtype=None):
    """Legacy prefill (kv_cache.py:567-647): keys of row b are the slots slot_mapping[b, :], causal mask.

    Each row's slot list is read as a block table of one-token pages and the batch travels the packed
    prefill route as `batch` rows of `seq_len` tokens, so token t of row b attends slot_mapping[b, 0..t];
    the metadata built for it is O(batch * seq_len).
    """
    batch, seq_len, num_heads, head_dim = query.shape
    k_layer, _ = _resolve_kv_layer(k_cache, layer_idx)
    v_layer, _ = _resolve_kv_layer(v_cache, layer_idx)
    hkv = k_layer.shape[-2]
    k1 = k_layer.reshape(-1, 1, hkv, head_dim)
    v1 = v_layer.reshape(-1, 1, hkv, head_dim)
    dev = query.device
    positions = torch.arange(seq_len, dtype=torch.int32, device=dev).repeat(batch)[None]
    qsl = torch.arange(batch + 1, dtype=torch.int32, device=dev) * seq_len
    lens = torch.full((batch,), seq_len, dtype=torch.int32, device=dev)
    out = _k.packed_paged_prefill_attention(query.reshape(1, batch * seq_len, num_heads, head_dim), k1, v1,
                                            slot_mapping.to(torch.int32), lens, positions, qsl, 1, scale,
                                            num_key_value_groups, seq_len, num_decode_rows=0)
    return out.reshape(batch, seq_len, num_heads * head_dim).to(_promoted(query, k_cache, out_dtype))


def paged_attention_prefill_packed(query, k_cache, v_cache, block_table, kv_lens, positions, token_row_ids,
                                   query_start_loc, block_size, scale, num_key_value_groups,
                                   layer_idx: int = 0, max_query_len=None, use_triton=None, out_dtype=None,
                                   num_decode_rows=None, query_tile_pairs=None):
    """Ragged packed prefill over the paged cache (kv_cache.py:721-849) -> `[1, T, Hq*D]`.

    `use_triton` is accepted for signature compatibility and ignored: there is one
    route.  The pure reference path returns the cache dtype; so does this unless
    `out_dtype` is given.
    """
    if query.ndim != 4 or query.shape[0] != 1:
        raise ValueError("packed prefill query must have shape [1, token_bucket, heads, head_dim]")
    if positions.shape != token_row_ids.shape or positions.shape[0] != 1:
        raise ValueError("packed positions and token_row_ids must have shape [1, token_bucket]")
    if block_table.ndim != 2:
        raise ValueError("block_table must be a 2D tensor [batch, max_blocks_per_seq]")
    if kv_lens.shape[0] != block_table.shape[0]:
        raise ValueError("kv_lens shape must align with block_table rows")
    k_layer = _paged_layer(k_cache, layer_idx, block_size)
    v_layer = _paged_layer(v_cache, layer_idx, block_size)
    out = _k.packed_paged_prefill_attention(query, k_layer, v_layer, block_table.to(torch.int32),
                                            kv_lens.to(torch.int32), positions.to(torch.int32),
                                            query_start_loc.to(torch.int32), block_size, scale,
                                            num_key_value_groups, max_query_len, num_decode_rows=num_decode_rows,
                                            query_tile_pairs=query_tile_pairs)
    return out.to(out_dtype if out_dtype is not None else k_cache.dtype)
