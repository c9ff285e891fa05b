"""A 6-layer all-full-attention stand-in model around the KV path (test infrastructure).

The model itself is outside the path; this is the thinnest stack that drives the
path the way the reference's `full_attention_block` does
(nanovllm_jax/model.py:3199-3591): RMSNorm in the (1 + w) form, q_proj producing
query and gate, per-head RMSNorm on q/k, partial RoPE on the first 64 dims,
`backend.write_kv_and_attention`, sigmoid gate, o_proj, SiLU-gated MLP, tied
LM head, greedy argmax.  Projection weights follow the reference's weight-free
tests, N(0,1) * hidden^-0.5 (nanovllm_jax/model.py:1009-1046); norm gains are 1.
All dense math runs in torch (fp32) on the GPU; only the attention backend differs
between the two runs that are compared (the B200 kernels vs the CPU oracle).
"""

from __future__ import annotations

import numpy as np
import torch

from helpers import to_numpy, to_torch
from nano_vllm_jax_b200.kv_cache import KVCacheStorage
from oracle import kv_cache_ref as R

HIDDEN, HQ, HKV, D, INTER, VOCAB, LAYERS = 1024, 8, 2, 256, 3584, 4096, 6
ROT, THETA, EPS = 64, 1e7, 1e-6
SCALE = D ** -0.5


def make_weights(seed, device="cuda"):
    g = torch.Generator(device=device).manual_seed(seed)
    s = HIDDEN ** -0.5

    def w(*shape):
        return (torch.randn(shape, generator=g, device=device) * s).to(torch.bfloat16)

    layers = [dict(wq=w(HIDDEN, HQ * 2 * D), wk=w(HIDDEN, HKV * D), wv=w(HIDDEN, HKV * D), wo=w(HQ * D, HIDDEN),
                   wg=w(HIDDEN, INTER), wu=w(HIDDEN, INTER), wd=w(INTER, HIDDEN)) for _ in range(LAYERS)]
    return dict(emb=w(VOCAB, HIDDEN), layers=layers)


def rmsnorm(x, dim_weight=0.0):
    # (1 + w) form with w = 0.  The reference's weight-free tests set w = 1, which doubles every
    # normalised activation: scores then have a standard deviation of 4, the softmax is nearly
    # one-hot and a 6-layer random stack amplifies 1e-6 attention differences into 0.1 logit
    # differences, so no two numeric paths could be compared through it.
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + EPS) * (1.0 + dim_weight)).to(x.dtype)


def rope(x, positions):
    """Half-split rotation of the first 64 dims (nanovllm_jax/layers.py:79-198); x [T, H, D]."""
    inv = THETA ** (-torch.arange(0, ROT, 2, device=x.device, dtype=torch.float32) / ROT)
    ang = positions.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    x1, x2 = xf[..., :ROT // 2], xf[..., ROT // 2:ROT]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin, xf[..., ROT:]], dim=-1).to(x.dtype)


class OracleAttention:
    """`write_kv_and_attention` served by the CPU oracle on NumPy mirrors of the caches."""

    def __init__(self, k_cache, v_cache):
        self.k, self.v = to_numpy(k_cache), to_numpy(v_cache)
        self.errors = []  # when used as a shadow: max-abs attention difference per layer call

    def write_kv_and_attention(self, layer_id, query, k, v, cache, metadata, block_size, scale, groups, is_prefill):
        sl = slice(layer_id, layer_id + 1)
        slots = to_numpy(metadata.slot_mapping)
        packed = metadata.token_row_ids is not None
        valid = R.write_kv_valid_mask(slots.shape, to_numpy(metadata.query_start_loc), packed)
        nk, nv = R.update_kv_cache(self.k[sl], self.v[sl], slots, to_numpy(k), to_numpy(v), 0, valid_mask=valid)
        self.k[sl], self.v[sl] = nk, nv
        tables, lens = to_numpy(metadata.block_tables), to_numpy(metadata.seq_lens)
        if packed:
            out = R.paged_attention_prefill_packed(to_numpy(query), nk, nv, tables, lens, to_numpy(metadata.positions),
                                                   to_numpy(metadata.token_row_ids), to_numpy(metadata.query_start_loc),
                                                   block_size, scale, groups)
        else:
            out = R.paged_attention_decode(to_numpy(query), nk, nv, tables, lens, block_size, scale, groups,
                                           positions=to_numpy(metadata.positions))
        return cache, to_torch(out.astype(np.float32))


def forward(weights, attn, backend, cache: KVCacheStorage, batch, block_size=16, shadow=None, shadow_tol=2e-2):
    """One engine step: returns (greedy token per table row [rows], last-token logits [rows, VOCAB]).

    `shadow`, if given, is a second attention backend that is handed exactly the same q/k/v at every
    layer; its output must agree with `attn`'s within `shadow_tol` on the real tokens (its caches can
    then be compared bit for bit with `attn`'s afterwards).
    """
    tokens, positions = batch.tokens, batch.positions
    md = backend.build_attention_metadata(positions, batch.block_tables, batch.seq_lens, block_size, batch.is_prefill,
                                          query_start_loc=batch.query_start_loc, token_row_ids=batch.token_row_ids,
                                          query_lens_host=batch.query_lens_host if batch.token_row_ids is not None else None)
    shape = tokens.shape  # [1, T] packed or [B, 1] decode
    flat_tok, flat_pos = tokens.reshape(-1).long(), positions.reshape(-1)
    # Dense math in fp32 on the bf16-valued weights; only q/k/v are rounded to bf16, at the boundary
    # of the path.  (With a bf16 residual stream a 1e-6 attention difference flips roundings that a
    # random 6-layer stack amplifies to 0.05 in the logits: the comparison would measure the
    # stand-in's own rounding, not the path.)
    bf = torch.bfloat16
    x = weights["emb"][flat_tok].float()
    n = x.shape[0]
    for li, lw in enumerate(weights["layers"]):
        h = rmsnorm(x)
        qg = (h @ lw["wq"].float()).view(n, HQ, 2 * D)
        q, gate = qg[..., :D], qg[..., D:]
        k = (h @ lw["wk"].float()).view(n, HKV, D)
        v = (h @ lw["wv"].float()).view(n, HKV, D).to(bf)
        q, k = rope(rmsnorm(q), flat_pos).to(bf), rope(rmsnorm(k), flat_pos).to(bf)
        cache, out = attn.write_kv_and_attention(li, q.reshape(*shape, HQ, D).contiguous(), k.reshape(*shape, HKV, D).contiguous(),
                                                 v.reshape(*shape, HKV, D).contiguous(), cache, md, block_size, SCALE,
                                                 HQ // HKV, batch.is_prefill)
        if shadow is not None:
            _, ref = shadow.write_kv_and_attention(li, q.reshape(*shape, HQ, D).contiguous(), k.reshape(*shape, HKV, D).contiguous(),
                                                   v.reshape(*shape, HKV, D).contiguous(), cache, md, block_size, SCALE,
                                                   HQ // HKV, batch.is_prefill)
            if batch.token_row_ids is not None:
                real = torch.arange(n, device=x.device) < batch.query_start_loc[-1]
            else:
                real = batch.seq_lens > 0
            err = float((out.reshape(n, -1)[real].float() - ref.reshape(n, -1)[real].float()).abs().max())
            assert err <= shadow_tol, f"layer {li}: attention differs from the oracle by {err}"
            if getattr(shadow, "errors", None) is not None:
                shadow.errors.append(err)
        o = out.reshape(n, HQ * D).float() * torch.sigmoid(gate.reshape(n, HQ * D))
        x = x + o @ lw["wo"].float()
        h2 = rmsnorm(x)
        x = x + (torch.nn.functional.silu(h2 @ lw["wg"].float()) * (h2 @ lw["wu"].float())) @ lw["wd"].float()
    if batch.token_row_ids is not None:
        last = (batch.query_start_loc[1:] - 1).long().clamp(min=0)  # last token of every row
    else:
        last = torch.arange(n, device=x.device)
    logits = rmsnorm(x[last]) @ weights["emb"].float().t()
    return logits.argmax(-1), logits
