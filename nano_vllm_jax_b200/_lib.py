"""ctypes binding of `libnvj_b200.so` (the C ABI declared in `include/nvj_b200.h`).

The library is the product: there is no Python or CPU fallback.  Loading fails
loudly when the shared object is missing and cannot be built, and every wrapper
raises on a non-zero status.
"""

from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_uint32, c_uint64, c_void_p

from . import build as _build

NVJ_BF16, NVJ_F16, NVJ_F32 = 0, 1, 2
NVJ_DEV_TIMEOUT, NVJ_DEV_BAD_BLOCK_ID, NVJ_DEV_BAD_LENGTH = 1, 2, 4
NVJ_ERR_UNSUPPORTED = -2  # a kernel declined the call (shape, dtype, alignment, a missing driver feature)

# name -> (restype, argtypes); one entry per declaration in include/nvj_b200.h
SIGNATURES = {
    "nvj_abi_version": (c_int, []),
    "nvj_status_string": (c_char_p, [c_int]),
    "nvj_compute_slot_mapping": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                         c_void_p, c_void_p]),
    "nvj_kv_append": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                              c_int, c_int, c_void_p, c_void_p, c_int, c_int64, c_int, c_int,
                              c_void_p, c_void_p]),
    "nvj_qk_norm_rope_kv_append": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int,
                                           c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                           c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                           c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int,
                                           c_void_p, c_void_p, c_void_p]),
    "nvj_kv_append_nhd": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                  c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int,
                                  c_void_p, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "nvj_paged_decode_workspace_bytes": (c_size_t, [c_int]),
    "nvj_paged_decode_workspace_init": (c_int, [c_void_p, c_size_t, c_void_p]),
    "nvj_paged_decode_wide_workspace_bytes": (c_size_t, [c_int]),
    "nvj_paged_decode_wide": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_void_p, c_void_p,
                                      c_int, c_int, c_float, c_void_p, c_void_p, c_size_t, c_void_p]),
    "nvj_paged_decode_wide_form": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_void_p, c_void_p,
                                           c_int, c_int, c_float, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "nvj_paged_decode": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int64, c_int, c_int,
                                 c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                 c_float, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "nvj_paged_decode_fused_append": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_int, c_int64, c_int, c_int,
                                              c_int, c_int, c_void_p, c_int, c_void_p, c_int,
                                              c_float, c_void_p, c_void_p, c_size_t, c_int,
                                              c_void_p]),
    "nvj_paged_decode_static_scratch": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int64, c_int,
                                                c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int,
                                                c_float, c_void_p, c_void_p, c_void_p]),
    "nvj_paged_prefill_packed": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int64, c_int,
                                         c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                         c_void_p, c_int, c_int, c_float, c_void_p, c_void_p,
                                         c_void_p, c_size_t, c_int, c_void_p]),
    "nvj_paged_prefill_packed_part": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int64, c_int,
                                              c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                              c_void_p, c_int, c_int, c_float, c_void_p, c_void_p,
                                              c_void_p, c_size_t, c_int, c_int, c_int, c_void_p]),
    "nvj_copy_blocks": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p,
                                c_void_p, c_int, c_void_p, c_void_p]),
    "nvj_hybrid_snapshot": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64,
                                    c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "nvj_hybrid_restore": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64,
                                   c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "nvj_hybrid_snapshot_host_slots": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64,
                                               c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "nvj_hybrid_restore_host_slots": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64,
                                              c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "nvj_advance_decode_metadata": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "nvj_p2p_gather_buffer_bytes": (c_size_t, [c_int, c_int]),
    "nvj_p2p_buffer_create": (c_int, [c_size_t, c_void_p, c_void_p]),
    "nvj_p2p_buffer_open": (c_int, [c_void_p, c_void_p]),
    "nvj_p2p_buffer_close": (c_int, [c_void_p]),
    "nvj_p2p_buffer_destroy": (c_int, [c_void_p]),
    "nvj_p2p_allgather_i32": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_uint32, c_void_p, c_void_p, c_void_p]),
    "nvj_p2p_argmax_publish": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_int, c_int, c_void_p, c_void_p]),
    "nvj_p2p_collect": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "nvj_set_wait_limit_ns": (None, [c_uint64]),
    "nvj_get_wait_limit_ns": (c_uint64, []),
    "nvj_selftest_bounded_wait": (c_int, [c_void_p, c_void_p, c_void_p]),
    "nvj_paged_prefill_workspace_bytes": (c_size_t, [c_int]),
    "nvj_copy_many_async": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "nvj_row_argmax": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "nvj_row_argmax_advance": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
}

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


class NvjError(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def library_path() -> str:
    return str(_build.LIB_PATH)


def load() -> ctypes.CDLL:
    """Load (building first if the shared object is absent) and type the library."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if os.environ.get("NVJ_FORCE_REBUILD", "0") == "1" or not _build.LIB_PATH.exists():
            _build.build(force=True)
        lib = ctypes.CDLL(str(_build.LIB_PATH), mode=ctypes.RTLD_GLOBAL)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here = header and library disagree
            fn.restype = restype
            fn.argtypes = argtypes
        if lib.nvj_abi_version() != 1:
            raise NvjError("libnvj_b200.so has an unexpected ABI version")
        _lib = lib
        return lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().nvj_status_string(status).decode()
        raise NvjError(f"{what}: {msg} (status {status})")
