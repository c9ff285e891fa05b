"""Bookkeeping of the prefix-state snapshot pool (host logic; the copy kernel is replaced by an indexing stand-in).

The reference keeps an unbounded dict of states (nanovllm_jax/engine/scheduler.py:67-69, 239-279); the pool here is
bounded, so these cases cover what a bounded pool adds: eviction order, rows that must not be evicted, and what is
published when a snapshot cannot be stored.
"""

from types import SimpleNamespace

import pytest

from nano_vllm_jax_b200.engine import prefix_state as PS


@pytest.fixture()
def pool(monkeypatch):
    calls = []

    def fake_copy(conv_t, rec_t, conv_p, rec_p, table_slots, pool_slots, *, restore):
        ts, ps = table_slots.tolist(), pool_slots.tolist()
        calls.append((list(ts), list(ps), restore))
        assert len(set(ps if not restore else ts)) == len(ps), "two pairs of one launch write the same row"
        for t, p in zip(ts, ps):
            if restore:
                rec_t[t] = rec_p[p]
            else:
                rec_p[p] = rec_t[t]

    monkeypatch.setattr(PS._k, "hybrid_copy", fake_copy)
    table = PS.HybridStateTable(None, (2, 3), max_slots=8, device="cpu")
    for sid in range(8):
        table.rec[table.slot(sid)] = float(sid + 1)
    return PS.PrefixStateCache(table, capacity=2), calls


def test_more_new_hashes_than_rows_in_one_batch_never_reuses_a_row_of_that_batch(pool):
    cache, calls = pool
    stored = cache.snapshot([0, 1, 2, 3], [100, 101, 102, 103])
    assert stored == [True, True, False, False]          # two rows: the first two are kept, the rest skipped
    assert len(calls[-1][1]) == 2 and len(set(calls[-1][1])) == 2
    assert 100 in cache and 101 in cache and 102 not in cache and 103 not in cache
    cache.restore([4], [100])
    assert float(cache.table.rec[cache.table.slot(4)].min()) == 1.0   # sequence 0's state, not overwritten by 2 or 3


def test_lru_entry_goes_first_and_the_same_hash_twice_in_a_batch_is_copied_once(pool):
    cache, calls = pool
    cache.snapshot([0], [100])
    cache.snapshot([1], [101])
    cache.restore([5], [100])                              # 100 becomes the most recently used
    assert cache.snapshot([2, 3], [102, 102]) == [True, True]
    assert len(calls[-1][0]) == 1                          # one copy for the repeated hash
    assert 101 not in cache and 100 in cache and 102 in cache


def test_pinned_hash_survives_until_its_sequence_is_seeded(pool):
    cache, _ = pool
    cache.snapshot([0], [100])
    cache.snapshot([1], [101])
    waiting = SimpleNamespace(seq_id=6, cached_prefix_hash=100, num_cached_tokens=16, cached_prefix_hybrid_seeded=False)
    cache.pin_for([waiting])
    cache.pin_for([waiting])                               # idempotent per sequence
    assert cache.snapshot([2], [102]) == [True]            # evicts 101, the only entry that may go
    assert 100 in cache and 101 not in cache
    assert cache.snapshot([3], [103]) == [True]            # evicts 102
    assert 100 in cache
    cache.install_cached_prefix_hybrid_states([waiting])
    assert waiting.cached_prefix_hybrid_seeded and float(cache.table.rec[cache.table.slot(6)].max()) == 1.0
    cache.snapshot([4], [104])                             # now 100 is the least recently used... but was just restored
    cache.snapshot([5], [105])
    assert 100 not in cache                                # the pin is gone: it can be dropped again


def test_everything_pinned_skips_the_snapshot_and_the_prefix_is_not_published(pool):
    cache, _ = pool
    cache.snapshot([0, 1], [100, 101])
    cache.pin(100); cache.pin(101)
    published = []
    bm = SimpleNamespace(record_computed_prefix=lambda seq, computed, publish: 777,
                         publish_computed_prefix=lambda seq, computed: published.append(seq.seq_id))
    seq = SimpleNamespace(seq_id=2, num_prompt_tokens=32, num_cached_tokens=0)
    cache.record_computed_prefix_states(bm, [seq], [16])
    assert published == [] and 777 not in cache
    cache.unpin(101)
    cache.record_computed_prefix_states(bm, [seq], [16])
    assert published == [2] and 777 in cache and 101 not in cache


def test_missing_state_is_a_runtime_error_as_in_the_reference(pool):
    cache, _ = pool
    with pytest.raises(RuntimeError, match="missing hybrid prefix state"):
        cache.restore([0], [999])
