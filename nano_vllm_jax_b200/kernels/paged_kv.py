"""Kernel-ABI wrappers: torch CUDA tensors in, C-ABI calls out.

These functions keep the names, argument orders and aliasing of the reference's
kernel-level ABI for one NHD layer slice `[num_pages, page_size, num_kv_heads,
head_dim]`:

  kv_append_paged_nhd                    nanovllm_jax/kernels/cuda_fp32_ffi.py:323-382
  kv_append_paged_nhd_from_metadata      nanovllm_jax/kernels/cuda_fp32_ffi.py:427-472
  paged_decode_attention_gqa_nhd         nanovllm_jax/kernels/cuda_fp32_ffi.py:527-572
  paged_decode_attention_with_kv_append  nanovllm_jax/kernels/full_attention_triton.py:488-581
  packed_paged_prefill_attention         nanovllm_jax/kernels/full_attention_triton.py:148-221
  kv_last_page_len_from_seq_lens,
  dense_block_tables_to_kv_indptr        nanovllm_jax/kernels/paged_attention.py:23-54

The reference's custom calls alias the cache inputs to the outputs
(`input_output_aliases`); here the caches are updated in place and the same
tensors are returned.  Every function launches on the current CUDA stream and
does not synchronise, unless `NVJ_CHECK_STATUS=1` asks for the device status
word to be read back after each call (tests do).
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .. import _lib
from .._lib import NVJ_BF16, NVJ_F16, NVJ_F32, NvjError, check

_DTYPES = {torch.bfloat16: NVJ_BF16, torch.float16: NVJ_F16, torch.float32: NVJ_F32}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype}") from None


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _cuda(name: str, t: torch.Tensor) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    return t


def _i32(name: str, t: torch.Tensor) -> torch.Tensor:
    _cuda(name, t)
    if t.dtype != torch.int32:
        raise ValueError(f"{name} must have dtype int32")
    return t.contiguous()


def _strict() -> bool:
    return os.environ.get("NVJ_CHECK_STATUS", "0") == "1"


def _poison() -> bool:
    # Debug aid (tests set it): fill output buffers with NaN before a launch so that an
    # element the kernel fails to write cannot pass for a result left by an earlier call.
    return os.environ.get("NVJ_POISON_OUTPUT", "0") == "1"


class DeviceStatusError(NvjError):
    """A kernel flagged a device-side problem (bad block id, bad length, timeout)."""


def _raise_status(word: int, what: str) -> None:
    names = [n for bit, n in ((1, "timeout"), (2, "block id or slot outside the pool"),
                              (4, "sequence length beyond the block table")) if word & bit]
    raise DeviceStatusError(f"{what}: device status {word} ({', '.join(names)})")


# --------------------------------------------------------------------------- workspaces

class _Workspace:
    """Decode scratch + status word for one (device, stream)."""

    def __init__(self, device: torch.device, max_batch: int):
        lib = _lib.load()
        with torch.cuda.device(device):  # one buffer serves the width-1 and the wide kernel (never in flight together)
            nbytes = max(int(lib.nvj_paged_decode_workspace_bytes(int(max_batch))),
                         int(lib.nvj_paged_decode_wide_workspace_bytes(int(max_batch))),
                         int(lib.nvj_paged_prefill_workspace_bytes(int(max_batch))))
        if nbytes <= 0:
            raise NvjError("nvj_paged_decode_workspace_bytes failed (no CUDA device?)")
        self.max_batch = int(max_batch)
        self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        self.nbytes = nbytes

    def status_tensor(self) -> torch.Tensor:
        return self.buf[:4].view(torch.int32)


_workspaces: dict[tuple[int, int], _Workspace] = {}
# Workspaces that a larger one has replaced.  They are kept until the process ends: a CUDA graph captured on
# the stream while the smaller buffer was current still holds its address, and a freed buffer could be handed
# to another tensor by the caching allocator before that graph is replayed.
_retired_workspaces: list[_Workspace] = []
_status_words: dict[tuple[int, int], torch.Tensor] = {}


def _workspace(device: torch.device, batch: int) -> _Workspace:
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream(device))
    ws = _workspaces.get(key)
    if ws is None or ws.max_batch < batch:
        if ws is not None:
            _retired_workspaces.append(ws)
        ws = _Workspace(device, max(batch, 256, 2 * (ws.max_batch if ws else 0)))
        _workspaces[key] = ws
    return ws


def _status_word(device: torch.device) -> torch.Tensor:
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream(device))
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = t
    return t


def _check_word(t: torch.Tensor, what: str, ws: Optional[_Workspace] = None) -> None:
    word = int(t.item())
    if word:
        if ws is not None:
            ws.buf.zero_()  # counters may be left mid-flight after a flagged launch
        else:
            t.zero_()
        _raise_status(word, what)


def check_device_status(device=None) -> None:
    """Synchronise and raise if any kernel on `device`'s current stream flagged a problem."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream(device))
    if key in _workspaces:
        _check_word(_workspaces[key].status_tensor(), "paged decode", _workspaces[key])
    if key in _status_words:
        _check_word(_status_words[key], "paged kv")


# --------------------------------------------------------------------------- metadata helpers

def kv_last_page_len_from_seq_lens(seq_lens: torch.Tensor, page_size: int) -> torch.Tensor:
    if page_size <= 0:
        raise ValueError("page_size must be positive")
    seq_lens = seq_lens.to(torch.int32)
    return torch.where(seq_lens > 0, (seq_lens - 1) % page_size + 1, torch.zeros_like(seq_lens)).to(torch.int32)


def dense_block_tables_to_kv_indptr(block_tables: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    if block_tables.ndim != 2:
        raise ValueError("block_tables must have shape [batch, max_pages_per_sequence]")
    batch, width = block_tables.shape
    kv_indices = block_tables.reshape(-1).to(torch.int32)
    kv_indptr = torch.arange(batch + 1, dtype=torch.int32, device=block_tables.device) * width
    return kv_indices, kv_indptr


def _check_nhd_cache(k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
    _cuda("k_cache", k_cache)
    _cuda("v_cache", v_cache)
    if k_cache.shape != v_cache.shape:
        raise ValueError("k_cache and v_cache must have the same shape")
    if k_cache.ndim != 4:
        raise ValueError("k_cache must have NHD shape [num_pages, page_size, num_kv_heads, head_dim]")
    if k_cache.dtype != v_cache.dtype:
        raise ValueError("k_cache and v_cache must have the same dtype")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("cache layer slices must be contiguous")


# --------------------------------------------------------------------------- slot mapping

def compute_slot_mapping(positions, block_table, block_size, token_row_ids=None):
    """int32 slots for positions `[rows, cols]`; packed batches pass `token_row_ids` of the same shape."""
    lib = _lib.load()
    positions = _i32("positions", positions)
    block_table = _i32("block_table", block_table)
    if positions.ndim != 2 or block_table.ndim != 2:
        raise ValueError("positions and block_table must be 2D")
    rid = None
    if token_row_ids is not None:
        rid = _i32("token_row_ids", token_row_ids)
        if rid.shape != positions.shape:
            raise ValueError("positions and token_row_ids must have matching shapes")
    elif positions.shape[0] > block_table.shape[0]:
        raise ValueError("positions and block_tables batch dimensions must match")
    out = torch.empty(positions.shape, dtype=torch.int32, device=positions.device)
    check(lib.nvj_compute_slot_mapping(_ptr(positions), _ptr(block_table), _ptr(rid), positions.shape[0],
                                       positions.shape[1], block_table.shape[0], block_table.shape[1],
                                       int(block_size), _ptr(out), _stream(positions.device)),
          "nvj_compute_slot_mapping")
    return out


# --------------------------------------------------------------------------- append

def kv_append_slots(new_k, new_v, slot_mapping, k_cache_layer, v_cache_layer, *, valid_mask=None,
                    query_start_loc=None, packed=False):
    """Slot-mapped append into one layer (flat `[slots, Hkv, D]` or `[NB, bs, Hkv, D]`), in place.

    new_k/new_v `[rows, cols, Hkv, D]`; slot_mapping `[rows, cols]` int32.  The
    valid rules are those of nvj_kv_append (explicit mask and/or query_start_loc).
    """
    lib = _lib.load()
    _cuda("new_k", new_k)
    _cuda("k_cache_layer", k_cache_layer)
    if new_k.shape != new_v.shape:
        raise ValueError("new_k and new_v must have the same shape")
    if k_cache_layer.shape != v_cache_layer.shape:
        raise ValueError("k_cache and v_cache must have the same shape")
    hkv, d = k_cache_layer.shape[-2], k_cache_layer.shape[-1]
    if tuple(new_k.shape[-2:]) != (hkv, d):
        raise ValueError("new_k trailing dimensions must match cache [num_kv_heads, head_dim]")
    if not (k_cache_layer.is_contiguous() and v_cache_layer.is_contiguous()):
        raise ValueError("cache layer slices must be contiguous")
    slot_mapping = _i32("slot_mapping", slot_mapping)
    n_tokens = slot_mapping.numel()
    if new_k.numel() != n_tokens * hkv * d:
        raise ValueError("slot_mapping and new_k must describe the same number of tokens")
    rows, cols = (slot_mapping.shape if slot_mapping.ndim == 2 else (1, n_tokens))
    new_k, new_v = new_k.contiguous(), new_v.contiguous()
    vm = None
    if valid_mask is not None:
        vm = _cuda("valid_mask", valid_mask).reshape(-1).to(torch.int32).contiguous()
        if vm.numel() != n_tokens:
            raise ValueError("valid_mask must have the shape of slot_mapping")
    qsl, qsl_rows = None, 0
    if query_start_loc is not None:
        qsl = _i32("query_start_loc", query_start_loc)
        qsl_rows = qsl.numel() - 1
    num_slots = k_cache_layer.numel() // (hkv * d)
    st = _status_word(k_cache_layer.device)
    rc = lib.nvj_kv_append(_ptr(new_k), _ptr(new_v), _dt(new_k), _ptr(slot_mapping), _ptr(vm), _ptr(qsl),
                           qsl_rows, 1 if packed else 0, rows, cols, _ptr(k_cache_layer),
                           _ptr(v_cache_layer), _dt(k_cache_layer), num_slots, hkv, d, _ptr(st),
                           _stream(k_cache_layer.device))
    check(rc, "nvj_kv_append")
    if _strict():
        _check_word(st, "nvj_kv_append")
    return k_cache_layer, v_cache_layer


def kv_append_paged_nhd(append_key, append_value, batch_indices, positions, k_cache, v_cache,
                        kv_indices, kv_indptr, kv_last_page_len, valid_mask=None):
    """Page-table append on one NHD layer slice, in place; returns (k_cache, v_cache)."""
    lib = _lib.load()
    _check_nhd_cache(k_cache, v_cache)
    _cuda("append_key", append_key)
    if append_key.shape != append_value.shape:
        raise ValueError("append_key and append_value must have the same shape")
    if append_key.ndim != 3:
        raise ValueError("append_key must have shape [nnz_tokens, num_kv_heads, head_dim]")
    if tuple(append_key.shape[1:]) != tuple(k_cache.shape[2:]):
        raise ValueError("append_key trailing dimensions must match cache [num_kv_heads, head_dim]")
    nnz = append_key.shape[0]
    batch_indices = _i32("batch_indices", batch_indices)
    positions = _i32("positions", positions)
    if batch_indices.shape != (nnz,) or positions.shape != (nnz,):
        raise ValueError("batch_indices and positions must both have shape [nnz_tokens]")
    kv_indices = _i32("kv_indices", kv_indices)
    kv_indptr = _i32("kv_indptr", kv_indptr)
    _i32("kv_last_page_len", kv_last_page_len)
    if kv_indices.ndim != 1 or kv_indptr.ndim != 1 or kv_last_page_len.ndim != 1:
        raise ValueError("page metadata tensors must be rank-1")
    vm = None
    if valid_mask is not None:
        vm = _i32("valid_mask", valid_mask)
        if vm.shape != (nnz,):
            raise ValueError("valid_mask must have shape [nnz_tokens]")
    pages, page_size, hkv, d = k_cache.shape
    st = _status_word(k_cache.device)
    ak, av = append_key.contiguous(), append_value.contiguous()
    rc = lib.nvj_kv_append_nhd(_ptr(ak), _ptr(av), _dt(ak), _ptr(batch_indices), _ptr(positions), nnz,
                               _ptr(k_cache), _ptr(v_cache), _dt(k_cache), pages, page_size, hkv, d,
                               _ptr(kv_indices), kv_indices.numel(), _ptr(kv_indptr),
                               kv_indptr.numel() - 1, _ptr(vm), _ptr(st), _stream(k_cache.device))
    check(rc, "nvj_kv_append_nhd")
    if _strict():
        _check_word(st, "nvj_kv_append_nhd")
    return k_cache, v_cache


def kv_append_paged_nhd_from_metadata(k, v, k_cache_layer, v_cache_layer, metadata, *, page_size):
    """Append rectangular scheduled K/V `[B, T, Hkv, D]` using ragged metadata (padded tokens masked)."""
    if metadata.positions is None:
        raise ValueError("metadata.positions is required for the paged KV append")
    batch, query_len = k.shape[:2]
    if batch * query_len == 0:
        return k_cache_layer, v_cache_layer
    dev = k.device
    query_lens = torch.diff(metadata.query_start_loc.to(torch.int32))
    valid = torch.arange(query_len, dtype=torch.int32, device=dev)[None, :] < query_lens[:, None]
    batch_indices = torch.arange(batch, dtype=torch.int32, device=dev).repeat_interleave(query_len)
    kv_indices, kv_indptr = dense_block_tables_to_kv_indptr(metadata.block_tables)
    return kv_append_paged_nhd(
        k.reshape(batch * query_len, *k.shape[2:]), v.reshape(batch * query_len, *v.shape[2:]),
        batch_indices, metadata.positions.reshape(-1).to(torch.int32), k_cache_layer, v_cache_layer,
        kv_indices, kv_indptr, kv_last_page_len_from_seq_lens(metadata.seq_lens, page_size),
        valid.reshape(-1).to(torch.int32))


# --------------------------------------------------------------------------- decode

def _decode_call(q3, k_layer, v_layer, block_tables, table_width, kv_indptr, kv_last_page_len,
                 seq_lens, scale, variant, new_k=None, new_v=None, positions=None):
    lib = _lib.load()
    _check_nhd_cache(k_layer, v_layer)
    _cuda("q", q3)
    if q3.ndim != 3:
        raise ValueError("q must have shape [batch, num_q_heads, head_dim]")
    batch, hq, d = q3.shape
    pages, page_size, hkv, dk = k_layer.shape
    if d != dk:
        raise ValueError("q and cache head_dim must match")
    if hq % hkv != 0:
        raise ValueError("num_q_heads must be divisible by num_kv_heads")
    if q3.dtype not in _DTYPES:
        raise ValueError(f"unsupported q dtype {q3.dtype}")
    q3 = q3.contiguous()
    seq_lens = _i32("seq_lens", seq_lens)
    if seq_lens.shape != (batch,):
        raise ValueError("seq_lens must have shape [batch]")
    block_tables = _i32("block_tables", block_tables)
    out = torch.empty((batch, hq, d), dtype=torch.float32, device=q3.device)
    if batch == 0:
        return out
    if _poison():
        out.fill_(float("nan"))
    ws = _workspace(q3.device, batch)
    stream = _stream(q3.device)
    if new_k is None:
        rc = lib.nvj_paged_decode(_ptr(q3), _dt(q3), _ptr(k_layer), _ptr(v_layer), _dt(k_layer), pages,
                                  page_size, hkv, d, hq, _ptr(block_tables), table_width,
                                  _ptr(kv_indptr), _ptr(kv_last_page_len), _ptr(seq_lens), batch,
                                  float(scale), _ptr(out), _ptr(ws.buf), ws.nbytes, int(variant), stream)
        what = "nvj_paged_decode"
    else:
        rc = lib.nvj_paged_decode_fused_append(_ptr(q3), _dt(q3), _ptr(new_k), _ptr(new_v), _ptr(positions),
                                               _ptr(k_layer), _ptr(v_layer), _dt(k_layer), pages,
                                               page_size, hkv, d, hq, _ptr(block_tables), table_width,
                                               _ptr(seq_lens), batch, float(scale), _ptr(out),
                                               _ptr(ws.buf), ws.nbytes, int(variant), stream)
        what = "nvj_paged_decode_fused_append"
    check(rc, what)
    if _strict():
        _check_word(ws.status_tensor(), what, ws)
    return out


WIDE_DECODE_MAX_WIDTH = 16


def wide_decode_supported(q, k_layer) -> bool:
    """Whether `paged_decode_attention_wide` takes this batch: 2..16 query tokens per row, the model's shape, bf16."""
    return (q.ndim == 4 and 2 <= q.shape[1] <= WIDE_DECODE_MAX_WIDTH and q.dtype == torch.bfloat16
            and k_layer.dtype == torch.bfloat16 and tuple(q.shape[2:]) == (8, 256) and tuple(k_layer.shape[1:]) == (16, 2, 256))


def paged_decode_attention_wide(q, k_layer, v_layer, block_table, seq_lens, positions, scale, *, form=0):
    """Decode attention for rows of 2..16 query tokens: q `[B, T, 8, 256]` bf16 -> `[B, T, 8 * 256]` fp32.

    Token t of row b sees keys p < seq_lens[b] with p <= positions[b, t] (the reference's wide decode,
    nanovllm_jax/kv_cache.py:852-998); K and V of a row are read once for all of its tokens.
    `form`: 0 automatic (mma.sync tiles up to 4 tokens per row, tcgen05 beyond), 1 mma.sync tiles (up to 8 tokens),
    2 tcgen05.
    """
    if not wide_decode_supported(q, k_layer):
        raise ValueError("paged_decode_attention_wide: 2..16 bf16 query tokens per row over the bf16 cache [NB, 16, 2, 256]")
    lib = _lib.load()
    batch, width = int(q.shape[0]), int(q.shape[1])
    q = q.contiguous()
    tables = block_table.to(torch.int32).contiguous()
    lens = seq_lens.to(torch.int32).contiguous()
    pos = None if positions is None else positions.to(torch.int32).reshape(batch, width).contiguous()
    out = torch.empty((batch, width, 8 * 256), dtype=torch.float32, device=q.device)
    ws = _workspace(q.device, batch)
    _lib.check(lib.nvj_paged_decode_wide_form(q.data_ptr(), k_layer.data_ptr(), v_layer.data_ptr(), int(k_layer.shape[0]),
                                              tables.data_ptr(), int(tables.shape[1]), lens.data_ptr(),
                                              0 if pos is None else pos.data_ptr(), batch, width, float(scale), out.data_ptr(),
                                              ws.buf.data_ptr(), ws.nbytes, int(form), _stream(q.device)),
               "nvj_paged_decode_wide_form")
    if _strict():
        _check_word(ws.status_tensor(), "paged decode (wide)", ws)
    return out


def paged_decode_attention(q, k_layer, v_layer, block_table, seq_lens, scale, *, variant=0):
    """Width-1 decode over a dense block table: q `[B, Hq, D]` -> fp32 `[B, Hq, D]`."""
    if block_table.ndim != 2:
        raise ValueError("block_tables must be a 2D tensor [batch, max_blocks_per_seq]")
    if block_table.shape[0] != q.shape[0]:
        raise ValueError(f"query batch {q.shape[0]} must match block_tables batch {block_table.shape[0]}")
    return _decode_call(q, k_layer, v_layer, block_table, block_table.shape[1], None, None, seq_lens,
                        scale, variant)


STATIC_SCRATCH_MAX_BATCH = 4096


def paged_decode_attention_no_alloc(q, k_layer, v_layer, block_table, seq_lens, scale, out, status_out=None):
    """Width-1 decode that allocates nothing: every buffer, `out` included, comes from the caller.

    For hosts that may not allocate device memory while a step runs (a handler that
    only sees its operands, a plugin inside another runtime's memory pool): the
    decode workspace is a fixed array inside the library instead of a tensor.  The
    array is shared by all calls on a device, so calls must not overlap on the GPU;
    at most `STATIC_SCRATCH_MAX_BATCH` rows.  `status_out` (optional int32[1] CUDA
    tensor) receives the device status bits; nothing is read back here.
    """
    lib = _lib.load()
    _check_nhd_cache(k_layer, v_layer)
    _cuda("q", q)
    if q.ndim != 3 or block_table.ndim != 2 or block_table.shape[0] != q.shape[0]:
        raise ValueError("q must be [batch, heads, head_dim] and block_table [batch, width]")
    batch, hq, d = q.shape
    pages, page_size, hkv, dk = k_layer.shape
    if d != dk:
        raise ValueError("q and cache head_dim must match")
    if hq % hkv != 0:
        raise ValueError("num_q_heads must be divisible by num_kv_heads")
    if q.dtype not in _DTYPES:
        raise ValueError(f"unsupported q dtype {q.dtype}")
    if tuple(out.shape) != (batch, hq, d) or out.dtype != torch.float32 or not out.is_cuda or not out.is_contiguous():
        raise ValueError("out must be a contiguous float32 CUDA tensor [batch, heads, head_dim]")
    if not q.is_contiguous():
        raise ValueError("q must be contiguous (this call makes no copies)")
    # nothing may be copied or converted here: the operands are used where they lie
    for name, t in (("block_table", block_table), ("seq_lens", seq_lens)):
        _cuda(name, t)
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous int32 tensor (this call makes no copies)")
    if tuple(seq_lens.shape) != (batch,):
        raise ValueError("seq_lens must have shape [batch]")
    tensors = [k_layer, v_layer, out, block_table, seq_lens]
    if status_out is not None:
        if (not isinstance(status_out, torch.Tensor) or not status_out.is_cuda or status_out.dtype != torch.int32
                or status_out.numel() < 1 or not status_out.is_contiguous()):
            raise ValueError("status_out must be a CUDA int32 tensor with at least one element")
        tensors.append(status_out)
    if any(t.device != q.device for t in tensors):
        raise ValueError("all tensors must live on the device of q")
    rc = lib.nvj_paged_decode_static_scratch(_ptr(q), _dt(q), _ptr(k_layer), _ptr(v_layer), _dt(k_layer), pages,
                                             page_size, hkv, d, hq, _ptr(block_table), block_table.shape[1],
                                             _ptr(seq_lens), batch, float(scale), _ptr(out), _ptr(status_out),
                                             _stream(q.device))
    check(rc, "nvj_paged_decode_static_scratch")
    return out


def paged_decode_attention_gqa_nhd(q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len,
                                   seq_lens, softmax_scale, *, variant=0):
    """CSR page-table decode on one NHD layer slice: q `[B, Hq, D]` -> fp32 `[B, Hq, D]`."""
    batch = q.shape[0]
    kv_indptr = _i32("kv_indptr", kv_indptr)
    kv_indices = _i32("kv_indices", kv_indices)
    kv_last_page_len = _i32("kv_last_page_len", kv_last_page_len)
    if kv_indptr.shape != (batch + 1,):
        raise ValueError("kv_indptr must have shape [batch + 1]")
    if kv_indices.ndim != 1:
        raise ValueError("kv_indices must have shape [total_pages]")
    if kv_last_page_len.shape != (batch,):
        raise ValueError("kv_last_page_len must have shape [batch]")
    return _decode_call(q, k_cache, v_cache, kv_indices, 0, kv_indptr, kv_last_page_len, seq_lens,
                        softmax_scale, variant)


def paged_decode_attention_with_kv_append(query, new_k, new_v, k_cache, v_cache, block_table, seq_lens,
                                          positions, layer_id, block_size, scale,
                                          num_key_value_groups, *, variant=0):
    """Fused decode step on the 5-D caches: returns (out `[B, 1, Hq*D]` fp32, k_cache, v_cache).

    `positions=None` is the pre-append form for device-resident metadata: `seq_lens` then holds the rows' lengths
    before this step's token (the token goes to position `seq_lens[b]`, `seq_lens[b] + 1` keys are attended) and is
    not written; `row_argmax(..., advance=...)` or the token gather's publish advances it at the end of the step."""
    if query.ndim != 4 or query.shape[1] != 1 or new_k.shape[1] != 1 or new_v.shape[1] != 1:
        raise ValueError("fused decode attention supports only width-1 decode")
    if k_cache.ndim != 5 or v_cache.ndim != 5:
        raise ValueError("fused decode attention requires cache shape "
                         "[num_layers, num_pages, page_size, num_kv_heads, head_dim]")
    if not 0 <= layer_id < k_cache.shape[0]:
        raise ValueError(f"layer_idx {layer_id} is out of bounds for {k_cache.shape[0]} layers")
    if k_cache.shape[2] != block_size:
        raise ValueError("block_size must match the cache page size")
    batch, _, hq, d = query.shape
    if hq != k_cache.shape[3] * num_key_value_groups:
        raise ValueError("num_key_value_groups does not match the head counts")
    dt = k_cache.dtype
    nk = new_k[:, 0].to(dt).contiguous()
    nv = new_v[:, 0].to(dt).contiguous()
    q3 = query[:, 0]
    if q3.dtype not in (torch.float32, dt):
        q3 = q3.to(dt)
    pos = None if positions is None else _i32("positions", positions.reshape(batch).to(torch.int32))
    out = _decode_call(q3, k_cache[layer_id], v_cache[layer_id], block_table, block_table.shape[1],
                       None, None, seq_lens, scale, variant, nk, nv, pos)
    return out.reshape(batch, 1, hq * d), k_cache, v_cache


# --------------------------------------------------------------------------- prefill

def packed_paged_prefill_attention(query, k_cache_layer, v_cache_layer, block_table, kv_lens, positions,
                                   query_start_loc, block_size, scale, num_key_value_groups,
                                   max_query_len=None, variant=None, num_decode_rows=None, query_tile_pairs=None):
    """Ragged packed prefill: query `[1, T, Hq, D]` -> fp32 `[1, T, Hq*D]`, padded tokens 0.

    `variant`: 0 automatic, 1 generic, 2 mma.sync tiles, 3 tcgen05 tiles, 4 tcgen05 tiles on CTA pairs, 5 = 4 with
    bf16-rounded softmax weights in P V (default: the
    `NVJ_PREFILL_VARIANT` environment variable, else 0).  `num_decode_rows`: how many rows hold a single query
    token (the scheduler's `num_decode_tokens` of a mixed batch); 0 spares the launch that serves such rows,
    None (unknown) keeps it.  `query_tile_pairs`: how many 64-token tiles the other rows make up (sum of
    ceil(len / 64) over them), for the split of the SMs between the two kernels of a mixed batch; None = an upper bound.
    """
    lib = _lib.load()
    _check_nhd_cache(k_cache_layer, v_cache_layer)
    if query.ndim != 4 or query.shape[0] != 1:
        raise ValueError("packed prefill query must have shape [1, token_bucket, heads, head_dim]")
    if positions.ndim != 2 or positions.shape[0] != 1 or positions.shape[1] != query.shape[1]:
        raise ValueError("packed positions and token_row_ids must have shape [1, token_bucket]")
    if block_table.ndim != 2:
        raise ValueError("block_table must be a 2D tensor [batch, max_blocks_per_seq]")
    if kv_lens.shape[0] != block_table.shape[0]:
        raise ValueError("kv_lens shape must align with block_table rows")
    _, tokens, hq, d = query.shape
    pages, page_size, hkv, dk = k_cache_layer.shape
    if page_size != block_size or d != dk or hq != hkv * num_key_value_groups:
        raise ValueError("query / cache shapes do not agree")
    q = _cuda("query", query)[0].contiguous()
    block_table = _i32("block_table", block_table)
    kv_lens = _i32("kv_lens", kv_lens)
    pos = _i32("positions", positions.reshape(-1))
    qsl = _i32("query_start_loc", query_start_loc)
    rows = block_table.shape[0]
    if qsl.numel() != rows + 1:
        raise ValueError("query_start_loc must have shape [rows + 1]")
    out = torch.empty((tokens, hq, d), dtype=torch.float32, device=q.device)
    if _poison():
        out.fill_(float("nan"))
    st = _status_word(q.device)
    variant = int(os.environ.get("NVJ_PREFILL_VARIANT", "0")) if variant is None else int(variant)
    model_shape = (k_cache_layer.dtype == torch.bfloat16 and (page_size, hkv, d, hq) == (16, 2, 256, 8)
                   and q.dtype in (torch.bfloat16, torch.float32))

    def call(fn, ws, *extra):
        return fn(_ptr(q), _dt(q), _ptr(k_cache_layer), _ptr(v_cache_layer), _dt(k_cache_layer), pages, page_size, hkv, d, hq,
                  _ptr(block_table), block_table.shape[1], _ptr(kv_lens), _ptr(pos), _ptr(qsl), rows, tokens, float(scale),
                  _ptr(out), _ptr(st), _ptr(ws.buf) if ws else None, ws.nbytes if ws else 0, variant, *extra,
                  _stream(q.device))

    # A mixed batch (decode rows + prefill chunks, counts known on the host): the two kinds of row are served by two
    # kernels that write different rows of `out` and neither fills the machine, so they can run side by side on two
    # streams, the decode pass leaving the tile kernel's SMs free.  That pays when the launches come from a CUDA graph
    # (one 6-layer step: 328 -> 229 us); launched eagerly the extra stream bookkeeping costs the host more than the
    # overlap saves, so the fork is taken only while the current stream is being captured (NVJ_MIXED_SIDE_BY_SIDE=1
    # forces it, =0 forbids it).
    mixed = model_shape and variant in (0, 4, 5) and num_decode_rows is not None and 0 < num_decode_rows < rows
    mode = os.environ.get("NVJ_MIXED_SIDE_BY_SIDE", "auto")
    side_by_side = mixed and (mode == "1" or (mode != "0" and torch.cuda.is_current_stream_capturing()))
    if side_by_side:
        cur = torch.cuda.current_stream(q.device)
        side = _side_stream(q.device)
        sms = torch.cuda.get_device_properties(q.device).multi_processor_count
        pairs = -(-(tokens - num_decode_rows) // 64) + (rows - num_decode_rows)  # at most: every chunk may end a tile early
        if query_tile_pairs is not None:
            pairs = max(1, min(pairs, int(query_tile_pairs)))
        tile_ctas = 4 * pairs  # CTA pairs x 2 KV heads
        cta_limit = max(sms // 2, sms - tile_ctas)
        side.wait_stream(cur)
        # The decode rows are the longer of the two: they stay on the current stream and the tiles go to the side
        # stream, so that the fork and the join are paid on the shorter branch (the other way round the same step
        # measured 254 instead of 233 us).  No workspace for the tiles: key-range splits would ask for the SMs the
        # decode pass is running on.  (Starting the decode pass under the caller's append, as a programmatic dependent
        # launch that waits in front of its first K/V read, was measured too: 272 us, not kept.)
        with torch.cuda.stream(side):
            rc2 = call(lib.nvj_paged_prefill_packed_part, None, 2, 0)
        if rc2 == _lib.NVJ_ERR_UNSUPPORTED:  # the CTA-pair kernel cannot run here: the batch in one piece after all
            cur.wait_stream(side)
            ws = _workspace(q.device, rows)
            check(call(lib.nvj_paged_prefill_packed, ws), "nvj_paged_prefill_packed")
        else:
            ws = _workspace(q.device, rows)
            rc1 = call(lib.nvj_paged_prefill_packed_part, ws, 1, cta_limit)
            cur.wait_stream(side)
            check(rc1, "nvj_paged_prefill_packed_part (decode rows)")
            check(rc2, "nvj_paged_prefill_packed_part (tiles)")
    elif model_shape and variant != 1 and num_decode_rows == 0 and os.environ.get("NVJ_PREFILL_KEY_SPLITS", "1") != "0":
        # no decode rows: the tile kernel alone (it zero-fills what it does not write), with the workspace lent for
        # the key-range splits of a short batch
        ws = _workspace(q.device, rows)
        check(call(lib.nvj_paged_prefill_packed_part, ws, 3, 0), "nvj_paged_prefill_packed_part (tiles, all rows)")
    else:
        ws = _workspace(q.device, rows) if (num_decode_rows is None or num_decode_rows > 0) else None
        check(call(lib.nvj_paged_prefill_packed, ws), "nvj_paged_prefill_packed")
    if _strict():
        _check_word(st, "nvj_paged_prefill_packed")
        if ws is not None:
            _check_word(ws.status_tensor(), "nvj_paged_prefill_packed (decode rows)", ws)
    return out.reshape(1, tokens, hq * d)


_side_streams: dict[int, "torch.cuda.Stream"] = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    """One extra stream per device for work that runs beside the current stream (forked and joined inside a call)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    s = _side_streams.get(idx)
    if s is None:
        s = torch.cuda.Stream(device)
        _side_streams[idx] = s
    return s


# --------------------------------------------------------------------------- norm + rope + append

_inv_freq_tables: dict[tuple, torch.Tensor] = {}


def rope_inv_freq(rope_theta: float, rotary_dim: int, device) -> torch.Tensor:
    """`1 / theta^(arange(0, rot, 2) / rot)` in fp32, formed as the reference forms it (layers.py:97, 143-145)."""
    device = torch.device(device)
    key = (float(rope_theta), int(rotary_dim), device.index)
    t = _inv_freq_tables.get(key)
    if t is None:
        import numpy as np
        inv = np.float32(1.0) / (np.float32(rope_theta) ** (np.arange(0, rotary_dim, 2, dtype=np.float32) / np.float32(rotary_dim)))
        t = torch.from_numpy(inv.astype(np.float32)).to(device)
        _inv_freq_tables[key] = t
    return t


def qk_norm_rope_kv_append(query, k, v, q_norm_weight, k_norm_weight, positions, slot_mapping, k_cache_layer,
                           v_cache_layer, *, eps=1e-6, rope_theta=1e7, rotary_dim=64, valid_mask=None,
                           query_start_loc=None, packed=False, mrope_section=(11, 11, 10)):
    """RMSNorm(q), RMSNorm(k), partial RoPE on both, K/V rows into their slots; returns the query for attention.

    query `[rows, cols, Hq, D]` (may be a strided view, e.g. the first half of a `[.., Hq, 2 D]` query|gate
    projection), k, v `[rows, cols, Hkv, D]`, slot_mapping `[rows, cols]` int32; the cache layer is updated in place.
    positions: `[rows, cols]` int32 (text), or `[3, rows, cols]` (temporal, height, width rows of a multimodal
    position id, nanovllm_jax/model.py:3955) combined per frequency by `mrope_section` as
    nanovllm_jax/layers.py:79-139 does.  Fuses nanovllm_jax/model.py:3371-3396 with the append of 3539-3550.
    """
    lib = _lib.load()
    for name, t in (("query", query), ("k", k), ("v", v), ("k_cache_layer", k_cache_layer), ("v_cache_layer", v_cache_layer)):
        _cuda(name, t)
    if query.ndim != 4 or k.ndim != 4 or k.shape != v.shape or query.shape[:2] != k.shape[:2]:
        raise ValueError("query [rows, cols, Hq, D] and k, v [rows, cols, Hkv, D] must agree in rows and cols")
    rows, cols, hq, d = query.shape
    hkv = k.shape[2]
    if tuple(k_cache_layer.shape[-2:]) != (hkv, d) or k_cache_layer.shape != v_cache_layer.shape:
        raise ValueError("cache layer trailing dimensions must be [num_kv_heads, head_dim]")
    if not (k_cache_layer.is_contiguous() and v_cache_layer.is_contiguous()):
        raise ValueError("cache layer slices must be contiguous")
    if query.stride(3) != 1 or k.stride(3) != 1 or v.stride(3) != 1:
        raise ValueError("the head dimension must be contiguous")

    def token_strides(t, heads):
        # tokens must be evenly spaced: [rows, cols] collapses to one token axis
        if rows * cols > 1 and cols > 1 and rows > 1 and t.stride(0) != t.stride(1) * cols:
            return None
        tok = t.stride(1) if cols > 1 else (t.stride(0) if rows > 1 else heads * d)
        return tok, t.stride(2)

    qs = token_strides(query, hq)
    if qs is None:
        query = query.contiguous()
        qs = (hq * d, d)
    ks, vs = token_strides(k, hkv), token_strides(v, hkv)
    if ks is None or ks[1] != d:
        k = k.contiguous(); ks = (hkv * d, d)
    if vs is None or vs[1] != d:
        v = v.contiguous(); vs = (hkv * d, d)
    slot_mapping = _i32("slot_mapping", slot_mapping)
    pos_rows = 3 if positions.ndim == 3 else 1
    if pos_rows == 3 and (positions.shape[0] != 3 or len(mrope_section) != 3):
        raise ValueError("multimodal positions must have shape [3, rows, cols] and mrope_section three entries")
    pos = _i32("positions", positions).reshape(-1)
    if slot_mapping.numel() != rows * cols or pos.numel() != pos_rows * rows * cols:
        raise ValueError("positions [rows, cols] (or [3, rows, cols]) and slot_mapping [rows, cols] expected")
    import ctypes
    sections = (ctypes.c_int32 * 3)(*[int(x) for x in mrope_section]) if pos_rows == 3 else None
    vm = None
    if valid_mask is not None:
        vm = _cuda("valid_mask", valid_mask).reshape(-1).to(torch.int32).contiguous()
    qsl, qsl_rows = None, 0
    if query_start_loc is not None:
        qsl = _i32("query_start_loc", query_start_loc)
        qsl_rows = qsl.numel() - 1
    qw, kw = q_norm_weight.contiguous(), k_norm_weight.contiguous()
    if qw.dtype != kw.dtype or qw.numel() != d or kw.numel() != d:
        raise ValueError("q_norm and k_norm weights must be [head_dim] of one dtype")
    inv = rope_inv_freq(rope_theta, rotary_dim, query.device) if rotary_dim > 0 else None
    q_out = torch.empty((rows, cols, hq, d), dtype=query.dtype, device=query.device)
    num_slots = k_cache_layer.numel() // (hkv * d)
    st = _status_word(query.device)
    rc = lib.nvj_qk_norm_rope_kv_append(_ptr(query), qs[0], qs[1], _ptr(k), ks[0], _ptr(v), vs[0], _dt(query),
                                        _ptr(qw), _ptr(kw), _dt(qw), float(eps), _ptr(inv), int(rotary_dim), _ptr(pos),
                                        pos_rows, sections, _ptr(slot_mapping), _ptr(vm), _ptr(qsl), qsl_rows, 1 if packed else 0,
                                        rows, cols, _ptr(k_cache_layer), _ptr(v_cache_layer), _dt(k_cache_layer),
                                        num_slots, hq, hkv, d, _ptr(q_out), _ptr(st), _stream(query.device))
    check(rc, "nvj_qk_norm_rope_kv_append")
    if _strict():
        _check_word(st, "nvj_qk_norm_rope_kv_append")
    return q_out, k_cache_layer, v_cache_layer


# --------------------------------------------------------------------------- copies / tokens

def copy_blocks(k_cache, v_cache, src_ids, dst_ids):
    """cache[:, dst] = cache[:, src] on the 5-D caches, in place (src and dst sets disjoint)."""
    lib = _lib.load()
    if k_cache.ndim != 5 or k_cache.shape != v_cache.shape:
        raise ValueError("copy_blocks requires 5-D caches of equal shape")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("caches must be contiguous")
    src_ids, dst_ids = _i32("src_ids", src_ids), _i32("dst_ids", dst_ids)
    if src_ids.shape != dst_ids.shape or src_ids.ndim != 1:
        raise ValueError("src_ids and dst_ids must be rank-1 and of equal length")
    layers, nb = k_cache.shape[:2]
    block_bytes = k_cache[0, 0].numel() * k_cache.element_size()
    st = _status_word(k_cache.device)
    rc = lib.nvj_copy_blocks(_ptr(k_cache), _ptr(v_cache), layers, nb, block_bytes, nb * block_bytes,
                             _ptr(src_ids), _ptr(dst_ids), src_ids.numel(), _ptr(st), _stream(k_cache.device))
    check(rc, "nvj_copy_blocks")
    if _strict():
        _check_word(st, "nvj_copy_blocks")
    return k_cache, v_cache


def _row_bytes(t):
    return 0 if t is None else t[0].numel() * t.element_size()


HYBRID_HOST_SLOTS = 24


def hybrid_copy(conv_table, rec_table, conv_pool, rec_pool, table_slots, pool_slots, *, restore: bool):
    """Snapshot (table -> pool) or restore (pool -> table) GDN state rows, in place.

    `table_slots` / `pool_slots`: int32 CUDA tensors, or plain Python sequences of at most `HYBRID_HOST_SLOTS`
    ints, which ride in the kernel's parameters (no index upload in front of the launch).
    """
    lib = _lib.load()
    for name, t in (("conv_table", conv_table), ("rec_table", rec_table), ("conv_pool", conv_pool), ("rec_pool", rec_pool)):
        if t is not None and not (t.is_cuda and t.is_contiguous()):
            raise ValueError(f"{name} must be a contiguous CUDA tensor")
    ref_t = rec_table if rec_table is not None else conv_table
    ref_p = rec_pool if rec_pool is not None else conv_pool
    if ref_t is None or ref_p is None:
        return
    if _row_bytes(conv_table) != _row_bytes(conv_pool) or _row_bytes(rec_table) != _row_bytes(rec_pool):
        raise ValueError("table and pool rows must have the same size")
    st = _status_word(ref_t.device)
    if not isinstance(table_slots, torch.Tensor):
        import ctypes
        n = len(table_slots)
        if n != len(pool_slots) or n > HYBRID_HOST_SLOTS:
            raise ValueError(f"host slot lists must have equal length of at most {HYBRID_HOST_SLOTS}")
        t_arr, p_arr = (ctypes.c_int32 * n)(*[int(x) for x in table_slots]), (ctypes.c_int32 * n)(*[int(x) for x in pool_slots])
        fn = lib.nvj_hybrid_restore_host_slots if restore else lib.nvj_hybrid_snapshot_host_slots
        rc = fn(_ptr(conv_table), _ptr(conv_pool), _row_bytes(conv_table), _ptr(rec_table), _ptr(rec_pool),
                _row_bytes(rec_table), ref_t.shape[0], ref_p.shape[0], t_arr, p_arr, n, _ptr(st), _stream(ref_t.device))
    else:
        table_slots, pool_slots = _i32("table_slots", table_slots), _i32("pool_slots", pool_slots)
        fn = lib.nvj_hybrid_restore if restore else lib.nvj_hybrid_snapshot
        rc = fn(_ptr(conv_table), _ptr(conv_pool), _row_bytes(conv_table), _ptr(rec_table), _ptr(rec_pool),
                _row_bytes(rec_table), ref_t.shape[0], ref_p.shape[0], _ptr(table_slots), _ptr(pool_slots),
                table_slots.numel(), _ptr(st), _stream(ref_t.device))
    check(rc, "nvj_hybrid_restore" if restore else "nvj_hybrid_snapshot")
    if _strict():
        _check_word(st, "hybrid state copy")


def _advance_args(advance, rows):
    """(seq_lens, positions or None, table_width, block_size) of a step's resident metadata, checked."""
    seq_lens, positions, table_width, block_size = advance
    seq_lens = _i32("seq_lens", seq_lens)
    if seq_lens.shape != (rows,) or not seq_lens.is_contiguous():
        raise ValueError("advance: seq_lens must be a contiguous int32 [rows] tensor")
    if positions is not None:
        positions = _i32("positions", positions)
        if positions.numel() != rows or not positions.is_contiguous():
            raise ValueError("advance: positions must be a contiguous int32 tensor of one entry per row")
    return seq_lens, positions, int(table_width), int(block_size)


class CopyList:
    """A fixed list of copies `dst[i] <- src[i]` issued by one library call (`nvj_copy_many_async`).

    Built once for tensors whose addresses stay put (a pipeline slot's device buffers and its pinned result);
    `sources` / `targets` may be replaced per call by tensors of the same sizes.  The caller keeps every tensor alive
    and unchanged until the stream has passed the copies; pageable host memory makes a copy synchronous.
    """

    def __init__(self, dsts, srcs):
        if len(dsts) != len(srcs):
            raise ValueError("as many sources as targets")
        self.n = len(dsts)
        self._dst = (ctypes.c_void_p * self.n)()
        self._src = (ctypes.c_void_p * self.n)()
        self._bytes = (ctypes.c_size_t * self.n)()
        for i, (d, s) in enumerate(zip(dsts, srcs)):
            self._set(i, d, s)

    def _set(self, i, d, s):
        if not (d.is_contiguous() and s.is_contiguous()):
            raise ValueError("copies are between contiguous tensors")
        nbytes = d.numel() * d.element_size()
        if nbytes != s.numel() * s.element_size() or d.dtype != s.dtype:
            raise ValueError("source and target of a copy must have the same dtype and size")
        self._dst[i], self._src[i], self._bytes[i] = d.data_ptr(), s.data_ptr(), nbytes

    def set_source(self, i, s):
        """Replace source i by a contiguous tensor of the same byte size (its dtype is the caller's to check)."""
        if s.numel() * s.element_size() != self._bytes[i] or not s.is_contiguous():
            raise ValueError("a replaced source must be contiguous and of the size the list was built with")
        self._src[i] = s.data_ptr()

    def issue(self, stream) -> None:
        """Enqueue the copies on `stream` (a `torch.cuda.Stream`)."""
        check(_lib.load().nvj_copy_many_async(self._dst, self._src, self._bytes, self.n, stream.cuda_stream),
              "nvj_copy_many_async")


def row_argmax(x: torch.Tensor, out: torch.Tensor | None = None, advance=None) -> torch.Tensor:
    """int32 argmax of each row of a float32 `[rows, n]` tensor (first maximum wins).

    `advance=(seq_lens, positions, table_width, block_size)` also advances the rows' resident decode metadata in the
    same launch, as `advance_decode_metadata` would (positions may be None): the tail of a pre-append decode step."""
    lib = _lib.load()
    _cuda("x", x)
    if x.dtype != torch.float32 or x.ndim != 2:
        raise ValueError("row_argmax expects a float32 [rows, n] tensor")
    x = x.contiguous()
    if out is None:
        out = torch.empty(x.shape[0], dtype=torch.int32, device=x.device)
    elif out.dtype != torch.int32 or out.shape != (x.shape[0],) or not out.is_contiguous() or out.device != x.device:
        raise ValueError("row_argmax: out must be a contiguous int32 [rows] tensor on x's device")
    if advance is None:
        check(lib.nvj_row_argmax(_ptr(x), x.shape[0], x.shape[1], _ptr(out), _stream(x.device)), "nvj_row_argmax")
        return out
    seq_lens, positions, table_width, block_size = _advance_args(advance, x.shape[0])
    st = _status_word(x.device)
    check(lib.nvj_row_argmax_advance(_ptr(x), x.shape[0], x.shape[1], _ptr(out), _ptr(seq_lens), _ptr(positions),
                                     table_width, block_size, _ptr(st), _stream(x.device)), "nvj_row_argmax_advance")
    if _strict():
        _check_word(st, "nvj_row_argmax_advance")
    return out
