"""Byte cap and cache-dtype override of the KV-cache allocation (no GPU needed: allocation only).

Restates the reference's own cases: tests/test_backend_boundaries.py:165-216 of the reference
(`test_kv_cache_block_count_is_capped_by_bytes`, `test_full_attention_kv_cache_dtype_override`,
`..._default_config_uses_spec_dtype`) for nanovllm_jax/kv_cache.py:142-170 and
nanovllm_jax/backends.py:100-118, 868-891.
"""

from types import SimpleNamespace

import pytest
import torch

from nano_vllm_jax_b200.backends import B200Backend, full_attention_kv_cache_dtype
from nano_vllm_jax_b200.kv_cache import KVCacheSpec, cap_num_kv_cache_blocks, estimate_kv_cache_bytes, init_kv_cache

ENV = "NANO_VLLM_JAX_FULL_ATTN_KV_CACHE_DTYPE"


def _spec(**kw):
    base = dict(num_layers=2, num_blocks=100, block_size=4, num_kv_heads=1, head_dim=8, dtype=torch.float32,
                max_kv_cache_bytes=None)
    base.update(kw)
    return KVCacheSpec(**base)


def test_estimate_counts_k_and_v_of_every_layer():
    assert estimate_kv_cache_bytes(_spec()) == 2 * 100 * 4 * 1 * 8 * 4 * 2
    assert estimate_kv_cache_bytes(_spec(dtype=torch.bfloat16)) == 2 * 100 * 4 * 1 * 8 * 2 * 2


def test_kv_cache_block_count_is_capped_by_bytes():
    spec = _spec(max_kv_cache_bytes=2 * 2 * 4 * 1 * 8 * 4 * 2)  # room for exactly two blocks
    assert cap_num_kv_cache_blocks(spec) == 2
    assert cap_num_kv_cache_blocks(_spec(max_kv_cache_bytes=2 * 2 * 4 * 1 * 8 * 4 * 2 + 511)) == 2  # floor
    assert cap_num_kv_cache_blocks(_spec()) == 100                                  # no cap given
    assert cap_num_kv_cache_blocks(_spec(max_kv_cache_bytes=1 << 40)) == 100        # cap above the request


def test_cap_too_small_for_one_block_is_an_error():
    per_block = estimate_kv_cache_bytes(_spec(num_blocks=1))
    with pytest.raises(ValueError, match="too small for one KV block"):
        cap_num_kv_cache_blocks(_spec(max_kv_cache_bytes=per_block - 1))
    assert cap_num_kv_cache_blocks(_spec(max_kv_cache_bytes=per_block)) == 1


def test_init_kv_cache_allocates_the_capped_count_zero_filled():
    state = init_kv_cache(100, 4, 1, 8, max_seqs=3, max_blocks_per_seq=5, num_layers=2, dtype=torch.float32,
                          max_kv_cache_bytes=3 * 2 * 4 * 1 * 8 * 4 * 2, device="cpu")
    assert tuple(state.k_cache.shape) == (2, 3, 4, 1, 8) and state.v_cache.shape == state.k_cache.shape
    assert not state.k_cache.any() and not state.v_cache.any()
    assert tuple(state.block_table.shape) == (3, 5) and state.block_table.dtype == torch.int32
    assert tuple(state.kv_lens.shape) == (3,)


def test_backend_allocation_applies_cap_after_the_dtype_override(monkeypatch):
    # 4096 bytes hold 16 fp32 blocks of this spec but 32 bf16 ones: the cap is evaluated on the overridden dtype
    monkeypatch.setenv(ENV, "bf16")
    spec = _spec(num_blocks=100, block_size=2, max_kv_cache_bytes=4096)
    cache = B200Backend(device="cpu").allocate_kv_cache(spec, max_seqs=1, max_blocks_per_seq=4)
    assert cache.k_cache.dtype == torch.bfloat16 and cache.v_cache.dtype == torch.bfloat16
    assert cache.k_cache.shape[1] == 4096 // (2 * 2 * 1 * 8 * 2 * 2) == 32
    monkeypatch.setenv(ENV, "default")
    cache = B200Backend(device="cpu").allocate_kv_cache(spec, max_seqs=1, max_blocks_per_seq=4)
    assert cache.k_cache.dtype == torch.float32 and cache.k_cache.shape[1] == 4096 // (2 * 2 * 1 * 8 * 4 * 2) == 16


def test_full_attention_kv_cache_dtype_override(monkeypatch):
    monkeypatch.setenv(ENV, "bf16")
    cache = B200Backend(device="cpu").allocate_kv_cache(_spec(num_blocks=4, block_size=2, max_kv_cache_bytes=4096),
                                                        max_seqs=1, max_blocks_per_seq=4)
    assert cache.k_cache.dtype == torch.bfloat16 and cache.v_cache.dtype == torch.bfloat16


def test_full_attention_kv_cache_dtype_default_config_uses_spec_dtype(monkeypatch):
    monkeypatch.delenv(ENV, raising=False)
    config = SimpleNamespace(full_attention_kv_cache_dtype="default")
    cache = B200Backend(config, device="cpu").allocate_kv_cache(_spec(num_blocks=4, block_size=2, max_kv_cache_bytes=4096),
                                                                max_seqs=1, max_blocks_per_seq=4)
    assert cache.k_cache.dtype == torch.float32 and cache.v_cache.dtype == torch.float32


def test_dtype_names_config_and_environment_precedence(monkeypatch):
    monkeypatch.delenv(ENV, raising=False)
    f32 = torch.float32
    for name, want in (("bf16", torch.bfloat16), ("bfloat16", torch.bfloat16), ("fp16", torch.float16),
                       ("float16", torch.float16), ("fp32", f32), ("float32", f32), ("default", torch.float16),
                       ("off", torch.float16), (None, torch.float16)):
        assert full_attention_kv_cache_dtype(torch.float16, SimpleNamespace(full_attention_kv_cache_dtype=name)) == want
    assert full_attention_kv_cache_dtype(f32, None) == f32
    monkeypatch.setenv(ENV, "FP16 ")  # the environment wins over the config, case and blanks ignored
    assert full_attention_kv_cache_dtype(f32, SimpleNamespace(full_attention_kv_cache_dtype="bf16")) == torch.float16
    monkeypatch.setenv(ENV, "int8")
    with pytest.raises(ValueError, match="expected fp32, bf16, fp16, default, or off"):
        full_attention_kv_cache_dtype(f32, None)
