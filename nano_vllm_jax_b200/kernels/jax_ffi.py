"""`jax.ffi` binding of the sm_100a kernels: the route a JAX host takes into this library.

Mirrors the reference's own custom-call module, nanovllm_jax/kernels/cuda_fp32_ffi.py: the handlers
in `csrc/xla_ffi/` are compiled against `jax.ffi.include_dir()` on first use (:121-178), the shared
object is loaded with RTLD_GLOBAL and every handler registered once under a lock with
`jax.ffi.register_ffi_target(name, jax.ffi.pycapsule(fn), platform="gpu", api_version=1)` (:181-256),
and each public function checks its operands, then builds a `jax.ffi.ffi_call` with the caches aliased
to the results (`input_output_aliases`, :360-382, :558-572).  Function names, argument orders and error
texts follow the reference:

  kv_append_paged_nhd                    cuda_fp32_ffi.py:323-382   (kv_append_paged_nhd_fp32)
  paged_decode_attention_gqa_nhd         cuda_fp32_ffi.py:527-572   (paged_decode_attention_gqa_nhd_fp32)
  paged_decode_attention_with_kv_append  full_attention_triton.py:488-581
  packed_paged_prefill_attention         full_attention_triton.py:148-221
  copy_blocks, row_argmax                no counterpart in the reference

JAX is not installed where this library is built and measured, so nothing here has been executed:
importing the module is safe without JAX, every entry point raises `KernelBackendUnavailable` when
`import jax` fails (the reference's error type for a missing optional dependency,
nanovllm_jax/kernels/registry.py:55-113), and the torch / ctypes binding in `paged_kv.py` is what
the tests and benchmarks use.
"""

from __future__ import annotations

import ctypes
import subprocess
import threading
from pathlib import Path
from typing import Any

from .. import _lib
from .. import build as _build

XLA_SOURCES = _build.CSRC / "xla_ffi"
XLA_LIB_PATH = _build.PKG_DIR / "libnvj_b200_xla.so"

# target name registered with XLA -> exported handler symbol in csrc/xla_ffi/handlers.cc
TARGETS = {
    "nvj_b200_compute_slot_mapping": "NvjB200ComputeSlotMapping",
    "nvj_b200_kv_append": "NvjB200KvAppend",
    "nvj_b200_kv_append_nhd": "NvjB200KvAppendNhd",
    "nvj_b200_qk_norm_rope_kv_append": "NvjB200QkNormRopeKvAppend",
    "nvj_b200_paged_decode_attention": "NvjB200PagedDecodeAttention",
    "nvj_b200_paged_decode_csr": "NvjB200PagedDecodeCsr",
    "nvj_b200_paged_decode_with_kv_append": "NvjB200PagedDecodeWithKvAppend",
    "nvj_b200_paged_decode_wide": "NvjB200PagedDecodeWide",
    "nvj_b200_packed_prefill_attention": "NvjB200PackedPrefillAttention",
    "nvj_b200_copy_blocks": "NvjB200CopyBlocks",
    "nvj_b200_hybrid_snapshot": "NvjB200HybridSnapshot",
    "nvj_b200_hybrid_restore": "NvjB200HybridRestore",
    "nvj_b200_advance_decode_metadata": "NvjB200AdvanceDecodeMetadata",
    "nvj_b200_row_argmax": "NvjB200RowArgmax",
}

_REGISTER_LOCK = threading.Lock()
_REGISTERED = False
_LOADED_LIBS: list = []


class KernelBackendUnavailable(RuntimeError):
    """An optional dependency of this route (JAX, its FFI headers, nvcc) is missing."""


def _jax():
    try:
        import jax
        import jax.numpy as jnp
    except Exception as exc:  # ModuleNotFoundError on this image
        raise KernelBackendUnavailable(f"the jax.ffi route needs JAX: {exc}") from exc
    return jax, jnp


def build_xla_ffi_library(force: bool = False) -> Path:
    """Compile csrc/xla_ffi/*.cc against the XLA FFI headers and link it to the kernel library."""
    jax, _ = _jax()
    kernels = _build.build()
    sources = sorted(XLA_SOURCES.glob("*.cc"))
    newest = max(p.stat().st_mtime for p in sources + list(XLA_SOURCES.glob("*.h")))
    if not force and XLA_LIB_PATH.exists() and XLA_LIB_PATH.stat().st_mtime > max(newest, kernels.stat().st_mtime):
        return XLA_LIB_PATH
    nvcc = _build.nvcc_path()
    if nvcc is None:
        raise KernelBackendUnavailable("nvcc not found: cannot build the XLA-FFI adapter")
    cmd = [nvcc, "-std=c++17", "-O2", "-shared", "-Xcompiler", "-fPIC", "-I", jax.ffi.include_dir(), "-I", str(_build.INCLUDE),
           "-I", str(XLA_SOURCES), "-o", str(XLA_LIB_PATH), *[str(p) for p in sources], str(kernels),
           "-Xlinker", f"-rpath={kernels.parent}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("Failed to build the XLA-FFI adapter with nvcc:\n" + (proc.stdout + proc.stderr)[-12000:])
    return XLA_LIB_PATH


def _register_targets() -> None:
    global _REGISTERED
    if _REGISTERED:
        return
    with _REGISTER_LOCK:
        if _REGISTERED:
            return
        jax, _ = _jax()
        _lib.load()  # the kernels, RTLD_GLOBAL
        library = ctypes.CDLL(str(build_xla_ffi_library()), mode=ctypes.RTLD_GLOBAL)
        for target, symbol in TARGETS.items():
            jax.ffi.register_ffi_target(target, jax.ffi.pycapsule(getattr(library, symbol)), platform="gpu", api_version=1)
        _LOADED_LIBS.append(library)
        _REGISTERED = True


def _as_jax_array(name: str, value: Any):
    _, jnp = _jax()
    try:
        return jnp.asarray(value)
    except Exception as exc:
        raise ValueError(f"{name} must be array-like") from exc


def _i32(name: str, value: Any):
    _, jnp = _jax()
    arr = _as_jax_array(name, value)
    if arr.dtype != jnp.int32:
        raise ValueError(f"{name} must have dtype int32")
    return arr


def decode_workspace(max_batch: int):
    """Zeroed scratch operand of the decode and prefill calls, sized by the library for `max_batch` rows.  Inside
    `jax.jit` this is a constant-shaped `jnp.zeros`, so every call starts from cleared counters."""
    _, jnp = _jax()
    lib = _lib.load()
    nbytes = max(int(lib.nvj_paged_decode_workspace_bytes(int(max_batch))), int(lib.nvj_paged_decode_wide_workspace_bytes(int(max_batch))))
    return jnp.zeros((nbytes,), dtype=jnp.uint8)


# --------------------------------------------------------------------------- append

def _validate_kv_append_inputs(append_key, append_value, batch_indices, positions, k_cache, v_cache, kv_indices, kv_indptr,
                               kv_last_page_len, valid_mask):
    if k_cache.shape != v_cache.shape:
        raise ValueError("k_cache and v_cache must have the same shape")
    if k_cache.ndim != 4:
        raise ValueError("k_cache must have NHD shape [num_pages, page_size, num_kv_heads, head_dim]")
    if append_key.shape != append_value.shape:
        raise ValueError("append_key and append_value must have the same shape")
    if append_key.ndim != 3:
        raise ValueError("append_key must have shape [nnz_tokens, num_kv_heads, head_dim]")
    if tuple(append_key.shape[1:]) != tuple(k_cache.shape[2:]):
        raise ValueError("append_key trailing dimensions must match cache [num_kv_heads, head_dim]")
    nnz = append_key.shape[0]
    if batch_indices.shape != (nnz,) or positions.shape != (nnz,):
        raise ValueError("batch_indices and positions must both have shape [nnz_tokens]")
    if kv_indices.ndim != 1 or kv_indptr.ndim != 1 or kv_last_page_len.ndim != 1:
        raise ValueError("page metadata tensors must be rank-1")
    if valid_mask is not None and valid_mask.shape != (nnz,):
        raise ValueError("valid_mask must have shape [nnz_tokens]")


def kv_append_paged_nhd(append_key, append_value, batch_indices, positions, k_cache, v_cache, kv_indices, kv_indptr,
                        kv_last_page_len, valid_mask=None):
    """Page-table append on one NHD layer slice; returns (k_cache, v_cache) aliased to the inputs."""
    jax, _ = _jax()
    append_key = _as_jax_array("append_key", append_key)
    append_value = _as_jax_array("append_value", append_value)
    batch_indices, positions = _i32("batch_indices", batch_indices), _i32("positions", positions)
    k_cache, v_cache = _as_jax_array("k_cache", k_cache), _as_jax_array("v_cache", v_cache)
    kv_indices, kv_indptr = _i32("kv_indices", kv_indices), _i32("kv_indptr", kv_indptr)
    kv_last_page_len = _i32("kv_last_page_len", kv_last_page_len)
    valid_mask = None if valid_mask is None else _i32("valid_mask", valid_mask)
    _validate_kv_append_inputs(append_key, append_value, batch_indices, positions, k_cache, v_cache, kv_indices, kv_indptr,
                               kv_last_page_len, valid_mask)
    _register_targets()
    call = jax.ffi.ffi_call("nvj_b200_kv_append_nhd",
                            (jax.ShapeDtypeStruct(k_cache.shape, k_cache.dtype), jax.ShapeDtypeStruct(v_cache.shape, v_cache.dtype)),
                            has_side_effect=True, input_output_aliases={4: 0, 5: 1})
    args = (append_key, append_value, batch_indices, positions, k_cache, v_cache, kv_indices, kv_indptr, kv_last_page_len)
    if valid_mask is not None:
        args = (*args, valid_mask)
    return call(*args)


# --------------------------------------------------------------------------- decode

def paged_decode_attention_gqa_nhd(q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, seq_lens, softmax_scale):
    """Decode attention over an NHD paged cache: q `[B, Hq, D]` -> float32 `[B, Hq, D]`.

    Operand list of the reference's `paged_decode_attention_gqa_nhd_fp32`; `kv_indices` is read as a dense `[B, W]`
    table.  The scratch is the library's built-in array (at most 4096 rows, one call in flight per device).
    """
    jax, jnp = _jax()
    import numpy as np
    q, k_cache, v_cache = _as_jax_array("q", q), _as_jax_array("k_cache", k_cache), _as_jax_array("v_cache", v_cache)
    kv_indptr, kv_indices = _i32("kv_indptr", kv_indptr), _i32("kv_indices", kv_indices)
    kv_last_page_len, seq_lens = _i32("kv_last_page_len", kv_last_page_len), _i32("seq_lens", seq_lens)
    if q.ndim != 3:
        raise ValueError("q must have shape [batch, num_q_heads, head_dim]")
    if k_cache.ndim != 4 or k_cache.shape != v_cache.shape:
        raise ValueError("k_cache must have NHD shape [num_pages, page_size, num_kv_heads, head_dim]")
    batch = q.shape[0]
    if kv_indptr.shape != (batch + 1,):
        raise ValueError("kv_indptr must have shape [batch + 1]")
    if kv_last_page_len.shape != (batch,) or seq_lens.shape != (batch,):
        raise ValueError("kv_last_page_len and seq_lens must have shape [batch]")
    _register_targets()
    call = jax.ffi.ffi_call("nvj_b200_paged_decode_attention", jax.ShapeDtypeStruct(q.shape, jnp.float32), has_side_effect=False)
    return call(q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, seq_lens, softmax_scale=np.float32(softmax_scale))


def paged_decode_attention_with_kv_append(query, new_k, new_v, k_cache, v_cache, block_table, seq_lens, positions, *, layer_id,
                                          block_size, scale, num_key_value_groups):
    """Append width-1 K/V and run paged decode attention in one launch: (out `[B, 1, Hq*D]` f32, k_cache, v_cache)."""
    jax, jnp = _jax()
    import numpy as np
    if query.ndim != 4 or query.shape[1] != 1:
        raise ValueError("decode query must have shape [batch, 1, heads, head_dim]")
    if new_k.ndim != 4 or new_k.shape[1] != 1 or new_v.shape != new_k.shape:
        raise ValueError("new_k/new_v must have shape [batch, 1, kv_heads, head_dim]")
    if k_cache.ndim != 5 or v_cache.shape != k_cache.shape:
        raise ValueError("k/v cache must have shape [layers, pages, page_size, kv_heads, head_dim]")
    if block_table.ndim != 2:
        raise ValueError("block_table must have shape [batch, max_blocks_per_seq]")
    batch, _, num_heads, head_dim = query.shape
    if block_table.shape[0] != batch:
        raise ValueError("query and block_table batch sizes must match")
    if layer_id < 0 or layer_id >= k_cache.shape[0]:
        raise ValueError("layer_id is out of range for cache")
    if k_cache.shape[2] != block_size:
        raise ValueError("cache page size must match block_size")
    if num_heads != k_cache.shape[3] * num_key_value_groups:
        raise ValueError("num_key_value_groups must match query/KV head counts")
    if positions.shape != (batch, 1):
        raise ValueError("positions must have shape [batch, 1]")
    cache_dtype = k_cache.dtype
    query = query.astype(cache_dtype) if cache_dtype in (jnp.bfloat16, jnp.float16) else query
    workspace = decode_workspace(batch)
    _register_targets()
    call = jax.ffi.ffi_call("nvj_b200_paged_decode_with_kv_append",
                            (jax.ShapeDtypeStruct((batch, 1, num_heads * head_dim), jnp.float32),
                             jax.ShapeDtypeStruct(k_cache.shape, k_cache.dtype), jax.ShapeDtypeStruct(v_cache.shape, v_cache.dtype),
                             jax.ShapeDtypeStruct(workspace.shape, workspace.dtype)),
                            has_side_effect=True, input_output_aliases={3: 1, 4: 2, 8: 3})
    out, k_out, v_out, _ = call(query, new_k.astype(cache_dtype), new_v.astype(cache_dtype), k_cache, v_cache,
                                block_table.astype(jnp.int32), seq_lens.astype(jnp.int32), positions.astype(jnp.int32), workspace,
                                layer_id=np.int32(layer_id), scale=np.float32(scale))
    return out, k_out, v_out


# --------------------------------------------------------------------------- prefill

def packed_paged_prefill_attention(query, k_cache_layer, v_cache_layer, block_table, kv_lens, positions, query_start_loc, *,
                                   block_size, scale, num_key_value_groups, max_query_len=None):
    """Ragged packed prefill over the paged cache: query `[1, T, Hq, D]` -> float32 `[1, T, Hq*D]`, padded tokens 0."""
    jax, jnp = _jax()
    import numpy as np
    if query.ndim != 4 or query.shape[0] != 1:
        raise ValueError("packed prefill query must have shape [1, token_bucket, heads, head_dim]")
    if positions.ndim != 2 or positions.shape[0] != 1 or positions.shape[1] != query.shape[1]:
        raise ValueError("packed positions and token_row_ids must have shape [1, token_bucket]")
    if block_table.ndim != 2:
        raise ValueError("block_table must be a 2D tensor [batch, max_blocks_per_seq]")
    if kv_lens.shape[0] != block_table.shape[0]:
        raise ValueError("kv_lens shape must align with block_table rows")
    _, tokens, hq, d = query.shape
    if k_cache_layer.shape[1] != block_size or k_cache_layer.shape[3] != d or hq != k_cache_layer.shape[2] * num_key_value_groups:
        raise ValueError("query / cache shapes do not agree")
    cache_dtype = k_cache_layer.dtype
    query = query.astype(cache_dtype) if cache_dtype in (jnp.bfloat16, jnp.float16) else query
    workspace = decode_workspace(block_table.shape[0])
    _register_targets()
    call = jax.ffi.ffi_call("nvj_b200_packed_prefill_attention",
                            (jax.ShapeDtypeStruct((1, tokens, hq * d), jnp.float32), jax.ShapeDtypeStruct((1,), jnp.int32),
                             jax.ShapeDtypeStruct(workspace.shape, workspace.dtype)),
                            has_side_effect=False, input_output_aliases={7: 2})
    out, _, _ = call(query, k_cache_layer, v_cache_layer, block_table.astype(jnp.int32), kv_lens.astype(jnp.int32),
                     positions.astype(jnp.int32), query_start_loc.astype(jnp.int32), workspace, scale=np.float32(scale))
    return out


# --------------------------------------------------------------------------- copies / tokens

def copy_blocks(k_cache, v_cache, src_ids, dst_ids):
    """cache[:, dst] = cache[:, src] on the 5-D caches; returns (k_cache, v_cache) aliased to the inputs."""
    jax, jnp = _jax()
    if k_cache.ndim != 5 or k_cache.shape != v_cache.shape:
        raise ValueError("copy_blocks requires 5-D caches of equal shape")
    _register_targets()
    call = jax.ffi.ffi_call("nvj_b200_copy_blocks",
                            (jax.ShapeDtypeStruct(k_cache.shape, k_cache.dtype), jax.ShapeDtypeStruct(v_cache.shape, v_cache.dtype),
                             jax.ShapeDtypeStruct((1,), jnp.int32)),
                            has_side_effect=True, input_output_aliases={0: 0, 1: 1})
    k_out, v_out, _ = call(k_cache, v_cache, _i32("src_ids", src_ids), _i32("dst_ids", dst_ids))
    return k_out, v_out


def row_argmax(x):
    """int32 argmax of each row of a float32 `[rows, n]` array (first maximum wins)."""
    jax, jnp = _jax()
    x = _as_jax_array("x", x)
    if x.ndim != 2 or x.dtype != jnp.float32:
        raise ValueError("row_argmax expects a float32 [rows, n] array")
    _register_targets()
    return jax.ffi.ffi_call("nvj_b200_row_argmax", jax.ShapeDtypeStruct((x.shape[0],), jnp.int32), has_side_effect=False)(x)
