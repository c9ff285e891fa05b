"""Host-side prefix reuse: the reference's own block-manager cases, restated.

Source of every case: tests/test_backend_boundaries.py:4178-4313 in the reference
(refcounts, used-block hits, no sharing before publish, hybrid allow-list, tail
hashing), plus a known-answer test of the chained xxh64 digest.
"""

import numpy as np
import xxhash

from nano_vllm_jax_b200.engine.block_manager import BlockManager
from nano_vllm_jax_b200.engine.sequence import SamplingParams, Sequence


def _seq(tokens, seq_id):
    return Sequence(tokens, SamplingParams(temperature=0.0), seq_id=seq_id)


def test_hash_is_xxh64_of_prefix_bytes_then_int64_tokens():
    # block_manager.py:49-56
    toks = [1, 2, 3]
    assert BlockManager.compute_hash(toks) == xxhash.xxh64(np.array(toks, np.int64).tobytes()).intdigest()
    h0 = BlockManager.compute_hash(toks)
    expect = xxhash.xxh64(h0.to_bytes(8, "little") + np.array([4, 5], np.int64).tobytes()).intdigest()
    assert BlockManager.compute_hash([4, 5], h0) == expect
    # published xxh64 test vector (empty input, seed 0)
    assert xxhash.xxh64(b"").intdigest() == 0xEF46DB3751D8E999


def test_prefix_cache_shares_blocks_and_refcounts():
    bm = BlockManager(num_blocks=6, block_size=2)
    a, b = _seq([1, 2, 9], 1), _seq([1, 2, 7], 2)
    bm.allocate(a)
    bm.record_computed_prefix(a, 2, publish=True)
    bm.allocate(b)
    shared = a.block_table[0]
    assert shared == b.block_table[0]
    assert bm.blocks[shared].ref_count == 2
    bm.deallocate(a)
    assert bm.blocks[shared].ref_count == 1


def test_used_full_block_hit_needs_no_free_block():
    bm = BlockManager(num_blocks=1, block_size=2)
    a, b = _seq([1, 2], 1), _seq([1, 2], 2)
    bm.allocate(a)
    bm.record_computed_prefix(a, 2, publish=True)
    assert len(bm.free_block_ids) == 0
    assert bm.can_allocate(b)
    bm.allocate(b)
    assert a.block_table == b.block_table == [0]
    assert bm.blocks[0].ref_count == 2


def test_uncomputed_allocation_is_not_shared():
    bm = BlockManager(num_blocks=2, block_size=2)
    a, b = _seq([1, 2], 1), _seq([1, 2], 2)
    bm.allocate(a)
    assert bm.can_allocate(b)
    bm.allocate(b)
    assert a.block_table != b.block_table
    assert b.num_cached_tokens == 0


def test_hybrid_allowlist_requires_final_prefix_hash():
    bm = BlockManager(num_blocks=6, block_size=2)
    a, b = _seq([1, 2, 3, 4], 1), _seq([1, 2, 3, 4, 5], 2)
    bm.allocate(a)
    final = bm.record_computed_prefix(a, 4, publish=True)
    assert final is not None
    assert bm.cached_prefix_info(b, cacheable_hashes=set()) == (0, None)
    assert bm.cached_prefix_info(b, cacheable_hashes={final}) == (4, final)
    bm.allocate(b, cacheable_hashes={final})
    assert b.block_table[:2] == a.block_table
    assert b.num_cached_tokens == 4
    assert b.cached_prefix_hash == final


def test_no_prefix_cache_keeps_repeated_prompts_on_unique_blocks():
    bm = BlockManager(num_blocks=4, block_size=2)
    a, b = _seq([1, 2], 1), _seq([1, 2], 2)
    bm.allocate(a, use_prefix_cache=False)
    bm.allocate(b, use_prefix_cache=False)
    assert a.block_table != b.block_table
    assert bm.blocks[a.block_table[0]].ref_count == 1
    assert bm.blocks[b.block_table[0]].ref_count == 1
    assert bm.blocks[a.block_table[0]].hash != -1
    assert bm.blocks[b.block_table[0]].hash != -1
    assert bm.hash_to_block_id == {}


def test_no_prefix_cache_requires_free_blocks():
    bm = BlockManager(num_blocks=1, block_size=2)
    a, b = _seq([1, 2], 1), _seq([1, 2], 2)
    bm.allocate(a, use_prefix_cache=False)
    assert len(bm.free_block_ids) == 0
    assert not bm.can_allocate(b, use_prefix_cache=False)


def test_completed_tail_is_hashed_before_next_block():
    bm = BlockManager(num_blocks=3, block_size=2)
    s = _seq([1], 1)
    bm.allocate(s, use_prefix_cache=False)
    assert bm.blocks[s.block_table[-1]].hash == -1
    s.append_token(2)
    bm.may_append_slots(s, 1)
    done = s.block_table[-1]
    assert bm.blocks[done].hash != -1
    s.append_token(3)
    bm.may_append_slots(s, 1)
    assert len(s.block_table) == 2 and s.block_table[0] == done


def test_freed_cached_block_is_reused_then_evicted_on_overwrite():
    # block_manager.py:58-77 — a free block keeps its digest until it is handed out for new content
    bm = BlockManager(num_blocks=2, block_size=2)
    a = _seq([1, 2], 1)
    bm.allocate(a)
    h = bm.record_computed_prefix(a, 2, publish=True)
    blk = a.block_table[0]
    bm.deallocate(a)
    b = _seq([1, 2, 3], 2)
    bm.allocate(b)                      # hit on a free cached block: reused without clearing
    assert b.block_table[0] == blk and b.num_cached_tokens == 2 and b.cached_prefix_hash == h
    bm.deallocate(b)
    c, d = _seq([7, 8], 3), _seq([9, 9], 4)
    bm.allocate(c)
    bm.allocate(d)                      # both blocks overwritten: the stale digest must be gone
    assert h not in bm.hash_to_block_id


def test_lookahead_reserve_and_trim():
    bm = BlockManager(num_blocks=4, block_size=2)
    s = _seq([1, 2], 1)
    bm.allocate(s, use_prefix_cache=False)
    s.append_token(3)
    assert bm.can_append_slots(s, 3)
    bm.may_append_slots(s, 3)           # 3 tokens now + 2 look-ahead -> 5 tokens -> 3 blocks
    assert len(s.block_table) == 3
    bm.trim_append_slots(s, 1)
    assert len(s.block_table) == 2
    assert bm.stats() == {"total_blocks": 4, "free_blocks": 2, "used_blocks": 2}
