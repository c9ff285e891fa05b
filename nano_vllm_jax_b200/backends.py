"""The backend boundary of the full-attention KV path, served by the sm_100a kernels.

`B200Backend` has the KV/attention methods of the reference's `InferenceBackend`
protocol (nanovllm_jax/backends.py:639-711) with the signatures of its
`PureJAXBackend` (859-1461): allocate_kv_cache, build_attention_metadata,
write_kv, attention, write_kv_and_attention.  The model's full-attention block
(nanovllm_jax/model.py:3517-3550) and the executor's metadata build
(nanovllm_jax/engine/model_executor.py:430-441) call exactly these.  The GDN
compute methods of the protocol are outside this path and absent here.

In the reference a new implementation is chosen with one string per operation
(`full_attention_kv_append_impl`, `full_attention_decode_impl`,
`full_attention_prefill_impl`, backends.py:121-192) or by `select_backend`
(3174-3205); the value that selects this backend is "b200" in all of them.
"""

from __future__ import annotations

import os
from dataclasses import replace
from typing import Optional

import torch

from . import kv_cache as kvc
from .kernels import paged_kv as _k
from .kv_cache import AttentionMetadata, KVCacheSpec, KVCacheStorage

B200_IMPL = "b200"

_CACHE_DTYPES = {"default": None, "bf16": torch.bfloat16, "bfloat16": torch.bfloat16,
                 "fp16": torch.float16, "float16": torch.float16, "fp32": torch.float32,
                 "float32": torch.float32}


def normalize_full_attention_impl(value: Optional[str]) -> str:
    """Accepts the impl strings a config may carry for this path; only "b200" has a route here."""
    v = (value or B200_IMPL).strip().lower()
    if v != B200_IMPL:
        raise ValueError(f"unsupported full-attention implementation {value!r}: this backend provides 'b200'")
    return v


_CACHE_DTYPE_ENV = "NANO_VLLM_JAX_FULL_ATTN_KV_CACHE_DTYPE"
_OFF_VALUES = {"", "0", "false", "no", "off", "none"}


def full_attention_kv_cache_dtype(default_dtype, config=None):
    """`full_attention_kv_cache_dtype` override (backends.py:100-118): default | bf16 | fp16 | fp32 | off.

    As in the reference (backends.py:74-80) the environment variable
    NANO_VLLM_JAX_FULL_ATTN_KV_CACHE_DTYPE wins over the config attribute.
    """
    env = os.environ.get(_CACHE_DTYPE_ENV)
    if env is not None:
        name = env.strip().lower()
    elif config is not None and hasattr(config, "full_attention_kv_cache_dtype"):
        name = str(getattr(config, "full_attention_kv_cache_dtype") or "default").strip().lower()
    else:
        name = "default"
    if name == "default" or name in _OFF_VALUES:
        return default_dtype
    if name not in _CACHE_DTYPES:
        raise ValueError(f"Unknown {_CACHE_DTYPE_ENV}={name!r}; expected fp32, bf16, fp16, default, or off")
    return _CACHE_DTYPES[name]


class B200Backend:
    """KV-cache and attention operations on one B200, in place on torch CUDA tensors."""

    name = "b200"

    def __init__(self, config=None, device: str | torch.device = "cuda"):
        self.config = config
        self.device = torch.device(device)
        self._decode_qsl: dict = {}  # (rows, device) -> arange(rows + 1) of a decode batch
        for field in ("full_attention_kv_append_impl", "full_attention_decode_impl", "full_attention_prefill_impl"):
            if config is not None and getattr(config, field, None) not in (None, "", "reference", B200_IMPL):
                normalize_full_attention_impl(getattr(config, field))

    # ---- allocation (backends.py:868-891)
    def allocate_kv_cache(self, spec: KVCacheSpec, max_seqs: int, max_blocks_per_seq: int) -> KVCacheStorage:
        dtype = full_attention_kv_cache_dtype(spec.dtype, self.config)
        capped = replace(spec, dtype=dtype)
        capped = replace(capped, num_blocks=kvc.cap_num_kv_cache_blocks(capped))
        state = kvc.init_kv_cache(capped.num_blocks, capped.block_size, capped.num_kv_heads, capped.head_dim,
                                  max_seqs, max_blocks_per_seq, num_layers=capped.num_layers, dtype=dtype,
                                  max_kv_cache_bytes=capped.max_kv_cache_bytes, device=self.device)
        return state.storage

    # ---- metadata (backends.py:910-978)
    def build_attention_metadata(self, positions, block_tables, seq_lens, block_size, is_prefill,
                                 query_start_loc=None, num_prefill_tokens=None, num_decode_tokens=None,
                                 token_row_ids=None, max_query_len=None, query_lens_host=None) -> AttentionMetadata:
        # `query_lens_host` (the scheduler's host-side query lengths, engine/scheduler.py `query_lens_host`) is an
        # optional extension: it tells a packed batch how many rows hold a single token without a device read
        if positions.ndim != 2:
            raise ValueError("positions must be a 2D tensor [batch, query_len]")
        if block_tables.ndim != 2:
            raise ValueError("block_tables must be a 2D tensor [batch, max_blocks_per_seq]")
        if token_row_ids is not None:
            if not is_prefill:
                raise ValueError("token_row_ids are only supported for packed prefill")
            if token_row_ids.shape != positions.shape:
                raise ValueError("token_row_ids and positions must have matching shapes")
            if seq_lens.shape[0] != block_tables.shape[0]:
                raise ValueError("seq_lens shape must align with packed prefill rows")
            slot_mapping = kvc.compute_packed_slot_mapping(positions, block_tables, token_row_ids, block_size)
        else:
            if positions.shape[0] != block_tables.shape[0]:
                raise ValueError("positions and block_tables batch dimensions must match")
            if positions.shape[0] != seq_lens.shape[0]:
                raise ValueError("positions and seq_lens batch dimensions must match")
            if is_prefill:
                slot_mapping = kvc.compute_slot_mapping(positions, block_tables, block_size, is_prefill)
            else:  # decode: made when first read (the fused append + decode kernel never reads it)
                slot_mapping = lambda: kvc.compute_slot_mapping(positions, block_tables, block_size, is_prefill)  # noqa: E731
        batch, query_len = positions.shape
        if query_start_loc is None:
            if is_prefill:
                query_start_loc = torch.cat([torch.zeros(1, dtype=torch.int32, device=seq_lens.device),
                                             torch.cumsum(seq_lens.to(torch.int32), 0).to(torch.int32)])
            else:  # one query token per row: a constant per batch size, built once
                key = (int(seq_lens.shape[0]), seq_lens.device)
                query_start_loc = self._decode_qsl.get(key)
                if query_start_loc is None:
                    query_start_loc = torch.arange(key[0] + 1, dtype=torch.int32, device=seq_lens.device)
                    if not (seq_lens.is_cuda and torch.cuda.is_current_stream_capturing()):
                        self._decode_qsl[key] = query_start_loc
        return AttentionMetadata(
            slot_mapping=slot_mapping, block_tables=block_tables, seq_lens=seq_lens,
            query_start_loc=query_start_loc,
            num_prefill_tokens=(batch * query_len if is_prefill else 0) if num_prefill_tokens is None else num_prefill_tokens,
            num_decode_tokens=(0 if is_prefill else batch) if num_decode_tokens is None else num_decode_tokens,
            positions=positions,
            max_kv_len=block_tables.shape[1] * block_size if not is_prefill else None,
            token_row_ids=token_row_ids,
            max_query_len=max_query_len if max_query_len is not None else query_len,
            single_token_rows=(sum(1 for n in query_lens_host if int(n) == 1)
                               if (query_lens_host is not None and token_row_ids is not None) else None),
            query_tile_pairs=(sum(-(-int(n) // 64) for n in query_lens_host if int(n) > 1)
                              if (query_lens_host is not None and token_row_ids is not None) else None))

    # ---- append (backends.py:980-1067)
    def write_kv(self, layer_id, k, v, cache: KVCacheStorage, metadata: AttentionMetadata) -> KVCacheStorage:
        k_layer, _ = kvc._resolve_kv_layer(cache.k_cache, layer_id)
        v_layer, _ = kvc._resolve_kv_layer(cache.v_cache, layer_id)
        sm = metadata.slot_mapping.to(torch.int32)
        _k.kv_append_slots(k, v, sm, k_layer, v_layer,
                           query_start_loc=metadata.query_start_loc.to(torch.int32),
                           packed=metadata.token_row_ids is not None)
        return KVCacheStorage(cache.k_cache, cache.v_cache)

    # ---- attention (backends.py:1069-1250)
    def attention(self, layer_id, query, cache: KVCacheStorage, metadata: AttentionMetadata, block_size,
                  scale, num_key_value_groups, is_prefill):
        f32 = torch.float32
        if is_prefill:
            if metadata.token_row_ids is not None:
                if metadata.positions is None:
                    raise ValueError("metadata.positions is required for packed prefill attention")
                return kvc.paged_attention_prefill_packed(
                    query, cache.k_cache, cache.v_cache, metadata.block_tables, metadata.seq_lens,
                    metadata.positions, metadata.token_row_ids, metadata.query_start_loc, block_size, scale,
                    num_key_value_groups, layer_idx=layer_id, max_query_len=metadata.max_query_len, out_dtype=f32,
                    num_decode_rows=metadata.single_token_rows, query_tile_pairs=metadata.query_tile_pairs)
            if metadata.positions is None:
                return kvc.paged_attention(query, cache.k_cache, cache.v_cache, metadata.slot_mapping,
                                           metadata.seq_lens, scale, num_key_value_groups, layer_idx=layer_id,
                                           out_dtype=f32)
            return kvc.paged_attention_prefill(query, cache.k_cache, cache.v_cache, metadata.block_tables,
                                               metadata.seq_lens, metadata.positions, block_size, scale,
                                               num_key_value_groups, layer_idx=layer_id, out_dtype=f32)
        if metadata.positions is None:
            raise ValueError("metadata.positions is required for decode attention")
        if metadata.positions.shape[0] != metadata.block_tables.shape[0]:
            raise ValueError("positions and block_tables batch dimensions must match")
        return kvc.paged_attention_decode(query, cache.k_cache, cache.v_cache, metadata.block_tables,
                                          metadata.seq_lens, block_size, scale, num_key_value_groups,
                                          layer_idx=layer_id, max_kv_len=metadata.max_kv_len,
                                          positions=metadata.positions, out_dtype=f32)

    # ---- fused boundary (backends.py:1252-1461)
    def write_kv_and_attention(self, layer_id, query, k, v, cache: KVCacheStorage, metadata: AttentionMetadata,
                               block_size, scale, num_key_value_groups, is_prefill):
        fused = (not is_prefill and query.shape[1] == 1 and k.shape[1] == 1 and v.shape[1] == 1
                 and cache.k_cache.ndim == 5 and metadata.positions is not None)
        if fused:
            out, k_cache, v_cache = _k.paged_decode_attention_with_kv_append(
                query, k, v, cache.k_cache, cache.v_cache, metadata.block_tables.to(torch.int32),
                metadata.seq_lens.to(torch.int32), metadata.positions, layer_id, block_size, scale,
                num_key_value_groups)
            return KVCacheStorage(k_cache, v_cache), out
        storage = self.write_kv(layer_id, k, v, cache, metadata)
        out = self.attention(layer_id, query, storage, metadata, block_size, scale, num_key_value_groups, is_prefill)
        return storage, out


def select_backend(name: Optional[str] = None, config=None, device="cuda") -> B200Backend:
    """Counterpart of backends.py:3174-3205 with a single choice."""
    if name not in (None, "", "auto", "b200", "gpu", "cuda"):
        raise ValueError(f"unknown backend {name!r}: this package provides 'b200'")
    return B200Backend(config=config, device=device)
