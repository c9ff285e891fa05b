"""CPU oracle for the step in front of the KV path.  TEST INFRASTRUCTURE ONLY.

NumPy (+ ml_dtypes.bfloat16) restatement of what the reference's full-attention block does to
the projected query and key before `write_kv_and_attention` (paths relative to the reference
project root):
  rms_norm      nanovllm_jax/layers.py:11-29      fp32 norm, (1 + weight) form, cast back
  apply_rope    nanovllm_jax/layers.py:49-199     half-split rotation of the first
                                                  int(head_dim * partial_rotary_factor) dims;
                                                  cos / sin rounded to the input dtype first
  call site     nanovllm_jax/model.py:3371-3396   norm in [B, T, H, D], rope on q and k
Only tests, the smoke check and benchmark CPU legs may import this module.

Pinning: the reference holds no vectors for these functions and cannot be imported where this
was written (it needs JAX), so the values are "parity unpinned".  The rounding points of bf16
arithmetic in the reference depend on XLA's excess-precision setting: with the default (allowed)
`x1 * cos - x2 * sin` is formed in fp32 and rounded once, `excess_precision=False` here rounds
after every multiply and add instead.  Positions are `[B, T]` (text) or `[3, B, T]` (temporal,
height, width rows of a multimodal position id) with the interleaved selection of
layers.py:79-139; equal rows give the text result.
"""

from __future__ import annotations

import numpy as np

from .kv_cache_ref import update_kv_cache

try:
    from ml_dtypes import bfloat16
except ImportError:  # pragma: no cover
    bfloat16 = None


def rms_norm(x, weight, eps=1e-6):
    """layers.py:11-29."""
    xf = np.asarray(x).astype(np.float32)
    mean_sq = np.mean(np.square(xf), axis=-1, keepdims=True, dtype=np.float32)
    x_norm = xf * (np.float32(1.0) / np.sqrt(mean_sq + np.float32(eps)))
    out = x_norm * (np.float32(1.0) + np.asarray(weight).astype(np.float32))
    return out.astype(np.asarray(x).dtype)


def rope_inv_freq(rope_theta, rotary_dim):
    """layers.py:97 / 143-145: 1 / theta^(arange(0, dim, 2) / dim), fp32."""
    return (np.float32(1.0) / (np.float32(rope_theta) ** (np.arange(0, rotary_dim, 2, dtype=np.float32) / np.float32(rotary_dim)))).astype(np.float32)


def mrope_freqs(positions, inv_freq, mrope_section):
    """layers.py:86-139: frequencies `[B, T, dim / 2]` from positions `[3, B, T]`: the temporal row's, with the
    entries `arange(1, 3 * section[1], 3)` taken from the height row and `arange(2, 3 * section[2], 3)` from the
    width row (indices beyond dim / 2 dropped)."""
    positions = np.asarray(positions).astype(np.float32)
    freqs = positions[..., None] * inv_freq[None, None, None, :]  # [3, B, T, dim / 2]
    out = freqs[0].copy()
    for row in (1, 2):
        idx = np.arange(row, mrope_section[row] * 3, 3)
        idx = idx[idx < inv_freq.shape[0]]
        out[:, :, idx] = freqs[row][:, :, idx]
    return out


def apply_rope(x, positions, head_dim, rope_theta, partial_rotary_factor=1.0, excess_precision=True,
               mrope_section=None):
    """layers.py:49-199 for x `[B, T, H, D]` ("BTHD") and positions `[B, T]` or, with `mrope_section`, `[3, B, T]`."""
    x = np.asarray(x)
    dt = x.dtype
    dim = int(head_dim * partial_rotary_factor)
    n = dim // 2
    positions = np.asarray(positions)
    if mrope_section is not None and len(mrope_section) == 3:
        if positions.ndim == 2:
            positions = np.stack([positions] * 3)
        freqs = mrope_freqs(positions, rope_inv_freq(rope_theta, dim), mrope_section)
    else:
        if positions.ndim == 3:
            positions = positions[0]
        freqs = positions.astype(np.float32)[..., None] * rope_inv_freq(rope_theta, dim)[None, None, :]
    cos = np.cos(freqs).astype(np.float32)[:, :, None, :].astype(dt)
    sin = np.sin(freqs).astype(np.float32)[:, :, None, :].astype(dt)
    x1, x2 = x[..., :n], x[..., n:dim]
    if excess_precision:
        c, s = cos.astype(np.float32), sin.astype(np.float32)
        a, b = x1.astype(np.float32), x2.astype(np.float32)
        first, second = (a * c - b * s).astype(dt), (b * c + a * s).astype(dt)
    else:  # every array operation rounds to the input dtype
        first = ((x1 * cos).astype(dt) - (x2 * sin).astype(dt)).astype(dt)
        second = ((x2 * cos).astype(dt) + (x1 * sin).astype(dt)).astype(dt)
    return np.concatenate([first, second, x[..., dim:]], axis=-1).astype(dt)


def qk_norm_rope_kv_append(query, k, v, q_norm_weight, k_norm_weight, positions, slot_mapping, k_cache, v_cache,
                           layer_idx=0, eps=1e-6, rope_theta=1e7, partial_rotary_factor=0.25, valid_mask=None,
                           excess_precision=True, mrope_section=None):
    """model.py:3371-3396 followed by the append of 3539-3550: returns (query', k_cache', v_cache')."""
    d = np.asarray(query).shape[-1]
    q = apply_rope(rms_norm(query, q_norm_weight, eps), positions, d, rope_theta, partial_rotary_factor, excess_precision,
                   mrope_section)
    kk = apply_rope(rms_norm(k, k_norm_weight, eps), positions, d, rope_theta, partial_rotary_factor, excess_precision,
                    mrope_section)
    nk, nv = update_kv_cache(k_cache, v_cache, slot_mapping, kk, v, layer_idx, valid_mask=valid_mask)
    return q, nk, nv
