"""Shared builders for the parity tests: seeded synthetic caches, tables and queries."""

from __future__ import annotations

import numpy as np
import torch
from ml_dtypes import bfloat16

BS, HQ, HKV, D = 16, 8, 2, 256
SCALE = 1.0 / 16.0


def to_torch(a: np.ndarray, device="cuda") -> torch.Tensor:
    """NumPy (incl. ml_dtypes bfloat16) -> torch tensor on `device`, bit-exact."""
    if a.dtype == bfloat16:
        return torch.from_numpy(a.view(np.uint16).copy()).view(torch.bfloat16).to(device)
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def to_numpy(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(bfloat16)
    return t.numpy()


def bits(a: np.ndarray) -> np.ndarray:
    """Integer view for bit-exact comparisons (NaN-safe)."""
    a = np.ascontiguousarray(a)
    return a.view({2: np.uint16, 4: np.uint32, 1: np.uint8, 8: np.uint64}[a.dtype.itemsize])


def decode_case(seed, num_blocks, batch, ctx_lo, ctx_hi, *, layers=1, width=None, hq=HQ, hkv=HKV, d=D,
                bs=BS, dtype=bfloat16, empty_rows=()):
    """Seeded decode step: filled cache, scattered disjoint block tables, q and new k/v rows.

    seq_lens = ctx + 1 and positions = ctx (the step's own token is attended), as
    the scheduler builds a decode batch.  Rows listed in `empty_rows` are padding
    (seq_len 0, table all zero).
    """
    rng = np.random.default_rng(seed)
    ctx = rng.integers(ctx_lo, ctx_hi + 1, size=batch)
    seq_lens = (ctx + 1).astype(np.int32)
    for r in empty_rows:
        seq_lens[r] = 0
    need = -(-seq_lens // bs)
    w = int(max(1, need.max())) if width is None else width
    perm = rng.permutation(num_blocks)
    assert need.sum() <= num_blocks
    tables = np.zeros((batch, w), np.int32)
    o = 0
    for b in range(batch):
        tables[b, :need[b]] = perm[o:o + need[b]]
        o += need[b]
    shape = (layers, num_blocks, bs, hkv, d)
    k_cache = rng.standard_normal(shape, dtype=np.float32).astype(dtype)
    v_cache = rng.standard_normal(shape, dtype=np.float32).astype(dtype)
    q = rng.standard_normal((batch, 1, hq, d), dtype=np.float32).astype(dtype)
    new_k = rng.standard_normal((batch, 1, hkv, d), dtype=np.float32).astype(dtype)
    new_v = rng.standard_normal((batch, 1, hkv, d), dtype=np.float32).astype(dtype)
    positions = np.maximum(seq_lens - 1, 0).astype(np.int32)[:, None]
    return dict(k_cache=k_cache, v_cache=v_cache, q=q, new_k=new_k, new_v=new_v, tables=tables,
                seq_lens=seq_lens, positions=positions, bs=bs, groups=hq // hkv)
