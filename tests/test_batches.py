"""Batch layouts the scheduler hands to the path (host logic, CPU tensors)."""

import pytest

from nano_vllm_jax_b200.engine.block_manager import BlockManager
from nano_vllm_jax_b200.engine.scheduled_batch import (build_decode_batch, build_mixed_prefill_decode_batch,
                                                       build_packed_prefill_batch)
from nano_vllm_jax_b200.engine.sequence import Sequence


def _alloc(bm, tokens, seq_id):
    s = Sequence(tokens, seq_id=seq_id)
    bm.allocate(s, use_prefix_cache=False)
    return s


def test_decode_batch_layout_and_padding():
    # scheduler.py:790-803, 859-870
    bm = BlockManager(16, 2)
    a, b = _alloc(bm, [5, 6, 7], 1), _alloc(bm, [8], 2)
    batch = build_decode_batch([a, b], batch_size_bucket=4, device="cpu")
    assert batch.tokens.tolist() == [[7], [8], [0], [0]]
    assert batch.positions.tolist() == [[2], [0], [0], [0]]
    assert batch.seq_lens.tolist() == [3, 1, 0, 0]
    assert batch.query_start_loc.tolist() == [0, 1, 2, 2, 2]
    assert batch.seq_ids.tolist() == [1, 2, -1, -1]
    assert batch.block_tables.tolist()[0] == a.block_table and batch.block_tables.tolist()[2] == [0, 0]
    assert not batch.is_prefill and batch.num_decode_tokens == 2


def test_uncached_suffix_prefill_positions():
    # tests/test_backend_boundaries.py:678-693 in the reference: num_cached_tokens=2 -> positions [[2,3]], seq_lens [4]
    bm = BlockManager(8, 2)
    s = _alloc(bm, [1, 2, 3, 4], 3)
    s.num_cached_tokens = 2
    batch = build_packed_prefill_batch([s], device="cpu")
    assert batch.positions.tolist() == [[2, 3]]
    assert batch.seq_lens.tolist() == [4]
    assert batch.tokens.tolist() == [[3, 4]]


def test_mixed_batch_rows_and_token_row_ids():
    # tests/test_device_token_carry.py:551-574 in the reference: query_lens (1,1,3,3), row ids [0,1,2,2,2,3,3,3]
    bm = BlockManager(32, 2)
    d0, d1 = _alloc(bm, [1, 2, 3], 10), _alloc(bm, [4, 5], 11)
    p0, p1 = _alloc(bm, [6, 7, 8, 9], 12), _alloc(bm, [1, 1, 1], 13)
    batch = build_mixed_prefill_decode_batch(decode_seqs=[d0, d1], prefill_seqs=[p0, p1], prefill_chunk_lens=[3, 3],
                                             token_bucket=10, device="cpu")
    assert batch.query_lens_host == (1, 1, 3, 3)
    assert batch.token_row_ids.tolist() == [[0, 1, 2, 2, 2, 3, 3, 3, 0, 0]]
    assert batch.positions.tolist() == [[2, 1, 0, 1, 2, 0, 1, 2, 0, 0]]
    assert batch.seq_lens.tolist() == [3, 2, 3, 3]
    assert batch.is_prefill and batch.mixed_prefill_decode and batch.packed_prefill
    assert batch.prefill_is_final == [True, True, False, True]
    with pytest.raises(ValueError):
        build_mixed_prefill_decode_batch(decode_seqs=[], prefill_seqs=[p0], prefill_chunk_lens=[1], device="cpu")


def test_packed_bucket_overflow_is_an_error():
    bm = BlockManager(8, 2)
    s = _alloc(bm, [1, 2, 3, 4], 1)
    with pytest.raises(ValueError):
        build_packed_prefill_batch([s], token_bucket=2, device="cpu")
