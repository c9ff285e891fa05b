"""Pin the CPU oracle to the known answers of the reference's own tests.

Each test cites the reference test it restates (paths relative to the reference
project root).  The reference stores no golden vectors for this path; its tests
build small deterministic inputs and assert hand-computed indices or that two
implementations agree.  The same inputs and the same expected values are used
here against `oracle/kv_cache_ref.py`.
"""

import numpy as np
import pytest
from ml_dtypes import bfloat16

from oracle import kv_cache_ref as R
from oracle.dense_ref import dense_gqa_attention


def test_slot_mapping_position_25_non_identity_tables():
    # tests/test_kv_cache.py:366-422 — tables [[5,2,8,1,3],[7,4,6,0,9]], pos 25, bs 16 -> 41 and 73
    table = np.array([[5, 2, 8, 1, 3], [7, 4, 6, 0, 9]], np.int32)
    slots = R.compute_slot_mapping(np.array([[25], [25]], np.int32), table, 16)
    assert slots.tolist() == [[41], [73]]


def test_slot_mapping_identity_table():
    # tests/test_kv_cache.py:272-319 — blocks [0,1,2], pos 25 -> block 1, slot 9
    slots = R.compute_slot_mapping(np.array([[25]]), np.array([[0, 1, 2]]), 16)
    assert slots.tolist() == [[1 * 16 + 9]]


def test_packed_slot_mapping_padding_aliases_a_real_slot():
    # tests/test_backend_boundaries.py:1441-1459 — expected [[6, 7, 12, 6]]
    slots = R.compute_packed_slot_mapping(np.array([[0, 1, 2, 0]], np.int32), np.array([[3, 4], [5, 6]], np.int32),
                                          np.array([[0, 0, 1, 0]], np.int32), 2)
    assert slots.tolist() == [[6, 7, 12, 6]]


def test_packed_slot_mapping_shape_errors():
    with pytest.raises(ValueError):
        R.compute_packed_slot_mapping(np.zeros((1, 3), np.int32), np.zeros((2, 2), np.int32), np.zeros((1, 4), np.int32), 2)
    with pytest.raises(ValueError):
        R.compute_packed_slot_mapping(np.zeros((1, 3), np.int32), np.zeros((2,), np.int32), np.zeros((1, 3), np.int32), 2)


def test_masked_update_preserves_invalid_and_duplicate_slots():
    # tests/test_kv_cache.py:627-677 — slots [[2,2,3,5]], valid [[1,0,1,0]]
    nb, bs, hkv, d = 4, 8, 2, 3
    n = nb * bs * hkv * d
    k0 = np.arange(n, dtype=np.float32).reshape(1, nb, bs, hkv, d)
    v0 = (np.arange(n, dtype=np.float32) + 1000.0).reshape(1, nb, bs, hkv, d)
    rng = np.random.default_rng(0)
    nk = rng.standard_normal((1, 4, hkv, d)).astype(np.float32)
    nv = rng.standard_normal((1, 4, hkv, d)).astype(np.float32)
    k1, v1 = R.update_kv_cache(k0, v0, np.array([[2, 2, 3, 5]], np.int32), nk, nv, 0,
                               valid_mask=np.array([[1, 0, 1, 0]], bool))
    kf, vf = k1[0].reshape(-1, hkv, d), v1[0].reshape(-1, hkv, d)
    np.testing.assert_array_equal(kf[2], nk[0, 0])
    np.testing.assert_array_equal(kf[3], nk[0, 2])
    np.testing.assert_array_equal(kf[5], k0[0].reshape(-1, hkv, d)[5])
    np.testing.assert_array_equal(vf[2], nv[0, 0])
    np.testing.assert_array_equal(vf[3], nv[0, 2])
    np.testing.assert_array_equal(vf[5], v0[0].reshape(-1, hkv, d)[5])
    untouched = np.ones(nb * bs, bool)
    untouched[[2, 3]] = False
    np.testing.assert_array_equal(kf[untouched], k0[0].reshape(-1, hkv, d)[untouched])
    assert k0[0, 0, 2, 0, 0] == 12.0  # inputs are not modified (functional update)


def test_nhd_append_equals_canonical_update():
    # tests/test_nhd_kv_cache.py:140-184 — 2 rows x 2 tokens, tables [[3,1],[2,4]]
    pages, P, hkv, d = 6, 2, 2, 4
    rng = np.random.default_rng(1)
    k0 = rng.standard_normal((1, pages, P, hkv, d)).astype(np.float32)
    v0 = rng.standard_normal((1, pages, P, hkv, d)).astype(np.float32)
    tables = np.array([[3, 1], [2, 4]], np.int32)
    positions = np.array([[0, 1], [2, 3]], np.int32)
    nk = rng.standard_normal((2, 2, hkv, d)).astype(np.float32)
    nv = rng.standard_normal((2, 2, hkv, d)).astype(np.float32)
    slots = R.compute_slot_mapping(positions, tables, P)
    ck, cv = R.update_kv_cache(k0, v0, slots, nk, nv, 0)
    idx, ptr = R.dense_block_tables_to_kv_indptr(tables)
    nk_, nv_ = R.kv_append_paged_nhd(nk.reshape(4, hkv, d), nv.reshape(4, hkv, d), np.array([0, 0, 1, 1]),
                                     positions.reshape(-1), k0[0], v0[0], idx, ptr,
                                     R.kv_last_page_len_from_seq_lens(np.array([2, 4]), P))
    np.testing.assert_array_equal(nk_, ck[0])
    np.testing.assert_array_equal(nv_, cv[0])


def test_write_kv_valid_masks():
    # backends.py:1050-1057 — packed: i < qsl[-1]; dense: t < query_len[b]
    assert R.write_kv_valid_mask((1, 6), [0, 3, 4, 4], packed=True).tolist() == [[True] * 4 + [False] * 2]
    assert R.write_kv_valid_mask((3, 2), [0, 2, 3, 3], packed=False).tolist() == [[True, True], [True, False], [False, False]]


def test_last_page_len_and_indptr():
    # kernels/paged_attention.py:23-54
    assert R.kv_last_page_len_from_seq_lens(np.array([0, 1, 16, 17, 31]), 16).tolist() == [0, 1, 16, 1, 15]
    idx, ptr = R.dense_block_tables_to_kv_indptr(np.array([[3, 1, 5], [2, 4, 0]]))
    assert idx.tolist() == [3, 1, 5, 2, 4, 0] and ptr.tolist() == [0, 3, 6]


def _paged_setup(seed, dtype=np.float32, nb=6, bs=4, hkv=2, groups=2, d=8):
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((1, nb, bs, hkv, d)).astype(dtype)
    v = rng.standard_normal((1, nb, bs, hkv, d)).astype(dtype)
    return rng, k, v


def _dense_from_pages(cache, table_row, n, bs):
    flat = cache[0].reshape(-1, cache.shape[-2], cache.shape[-1])
    pos = np.arange(n)
    return flat[table_row[pos // bs] * bs + pos % bs]


def test_decode_paged_equals_dense_noncontiguous_tables():
    # tests/test_backend_boundaries.py:315-378 — tables [[3,1,5],[2,4,0]], fp32, tol 1e-6
    rng, k, v = _paged_setup(2)
    tables = np.array([[3, 1, 5], [2, 4, 0]], np.int32)
    lens = np.array([7, 10], np.int32)
    q = rng.standard_normal((2, 1, 4, 8)).astype(np.float32)
    out = R.paged_attention_decode(q, k, v, tables, lens, 4, 0.35, 2)
    for b in range(2):
        ref = dense_gqa_attention(q[b], _dense_from_pages(k, tables[b], lens[b], 4),
                                  _dense_from_pages(v, tables[b], lens[b], 4), 0.35, 2)
        np.testing.assert_allclose(out[b, 0], ref.reshape(-1), rtol=1e-5, atol=1e-6)


def test_decode_nhd_abi_equals_canonical():
    # tests/test_paged_attention_abi.py:20-97 — B2, P4, Hq4/Hkv2, D8, lens [7,10]
    rng, k, v = _paged_setup(3)
    tables = np.array([[3, 1, 5], [2, 4, 0]], np.int32)
    lens = np.array([7, 10], np.int32)
    q = rng.standard_normal((2, 4, 8)).astype(np.float32)
    idx, ptr = R.dense_block_tables_to_kv_indptr(tables)
    a = R.paged_decode_attention_gqa_nhd(q, k[0], v[0], ptr, idx, R.kv_last_page_len_from_seq_lens(lens, 4), lens, 0.5)
    b = R.paged_attention_decode(q[:, None], k, v, tables, lens, 4, 0.5, 2)
    np.testing.assert_allclose(a.reshape(2, -1), b[:, 0], rtol=1e-6, atol=1e-6)


def test_decode_independent_of_pool_size():
    # tests/test_kv_cache.py:479-558 — same sequence in a 4-block and an 8-block pool
    rng = np.random.default_rng(4)
    small = rng.standard_normal((1, 4, 4, 2, 8)).astype(np.float32)
    smallv = rng.standard_normal((1, 4, 4, 2, 8)).astype(np.float32)
    big = np.concatenate([small, rng.standard_normal((1, 4, 4, 2, 8)).astype(np.float32)], axis=1)
    bigv = np.concatenate([smallv, rng.standard_normal((1, 4, 4, 2, 8)).astype(np.float32)], axis=1)
    q = rng.standard_normal((1, 1, 4, 8)).astype(np.float32)
    t = np.array([[2, 0, 3]], np.int32)
    a = R.paged_attention_decode(q, small, smallv, t, np.array([9]), 4, 0.3, 2)
    b = R.paged_attention_decode(q, big, bigv, t, np.array([9]), 4, 0.3, 2)
    np.testing.assert_allclose(a, b, rtol=1e-6, atol=1e-6)


def test_gqa_grouping_equals_repeated_kv_heads():
    # tests/test_kv_cache.py:561-624 — Hq 8 / Hkv 2 grouped == KV heads repeated 4x
    rng = np.random.default_rng(5)
    k = rng.standard_normal((1, 4, 4, 2, 8)).astype(np.float32)
    v = rng.standard_normal((1, 4, 4, 2, 8)).astype(np.float32)
    q = rng.standard_normal((1, 1, 8, 8)).astype(np.float32)
    t = np.array([[1, 3, 0]], np.int32)
    a = R.paged_attention_decode(q, k, v, t, np.array([11]), 4, 0.3, 4)
    b = R.paged_attention_decode(q, np.repeat(k, 4, axis=3), np.repeat(v, 4, axis=3), t, np.array([11]), 4, 0.3, 1)
    np.testing.assert_allclose(a, b, rtol=1e-6, atol=1e-6)


def test_packed_prefill_equals_dense_rows_and_zero_padding():
    # tests/test_backend_boundaries.py:1462-1529 — rows of 3 and 2 tokens plus one pad token, atol 1e-6
    rng, k, v = _paged_setup(6, bs=2, nb=8)
    tables = np.array([[3, 4], [5, 6]], np.int32)
    kv_lens = np.array([3, 2], np.int32)
    positions = np.array([[0, 1, 2, 0, 1, 0]], np.int32)
    rows = np.array([[0, 0, 0, 1, 1, 0]], np.int32)
    qsl = np.array([0, 3, 5], np.int32)
    q = rng.standard_normal((1, 6, 4, 8)).astype(np.float32)
    out = R.paged_attention_prefill_packed(q, k, v, tables, kv_lens, positions, rows, qsl, 2, 0.4, 2)
    for r, (lo, hi) in enumerate([(0, 3), (3, 5)]):
        ref = dense_gqa_attention(q[0, lo:hi], _dense_from_pages(k, tables[r], kv_lens[r], 2),
                                  _dense_from_pages(v, tables[r], kv_lens[r], 2), 0.4, 2,
                                  query_positions=positions[0, lo:hi])
        np.testing.assert_allclose(out[0, lo:hi], ref.reshape(hi - lo, -1), rtol=1e-5, atol=1e-6)
    assert not out[0, 5].any()


def test_wide_decode_uses_positions_as_causal_mask():
    # kv_cache.py:972-977 — query t attends p <= positions[b, t]
    rng, k, v = _paged_setup(7)
    tables = np.array([[4, 2, 0]], np.int32)
    q = rng.standard_normal((1, 3, 4, 8)).astype(np.float32)
    pos = np.array([[6, 7, 8]], np.int32)
    out = R.paged_attention_decode(q, k, v, tables, np.array([9]), 4, 0.3, 2, positions=pos)
    ref = dense_gqa_attention(q[0], _dense_from_pages(k, tables[0], 9, 4), _dense_from_pages(v, tables[0], 9, 4),
                              0.3, 2, query_positions=pos[0])
    np.testing.assert_allclose(out[0], ref.reshape(3, -1), rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        R.paged_attention_decode(q, k, v, tables, np.array([9]), 4, 0.3, 2)  # width 3 without positions


def test_ref_mode_rounds_to_bf16_and_stays_near_fp32_mode():
    rng = np.random.default_rng(8)
    k = rng.standard_normal((1, 8, 16, 2, 64)).astype(bfloat16)
    v = rng.standard_normal((1, 8, 16, 2, 64)).astype(bfloat16)
    q = rng.standard_normal((2, 1, 8, 64)).astype(bfloat16)
    t = np.array([[1, 5, 2], [7, 0, 3]], np.int32)
    lens = np.array([33, 48])
    a = R.paged_attention_decode(q, k, v, t, lens, 16, 0.125, 4, mode="ref")
    b = R.paged_attention_decode(q, k, v, t, lens, 16, 0.125, 4, mode="fp32")
    assert a.dtype == bfloat16 and b.dtype == np.float32
    assert np.abs(a.astype(np.float32) - b).max() < 3e-2


def test_copy_blocks_oracle():
    rng = np.random.default_rng(9)
    k = rng.standard_normal((2, 6, 2, 1, 4)).astype(np.float32)
    v = rng.standard_normal((2, 6, 2, 1, 4)).astype(np.float32)
    k1, v1 = R.copy_blocks(k, v, [0, 2], [5, 4])
    np.testing.assert_array_equal(k1[:, 5], k[:, 0])
    np.testing.assert_array_equal(v1[:, 4], v[:, 2])
    np.testing.assert_array_equal(k1[:, :4], k[:, :4])


def test_mrope_row_selection_matches_the_interleaved_layout_of_the_reference():
    # layers.py:86-139 with mrope_section (11, 11, 10) over 32 frequencies: the height row supplies indices
    # 1, 4, ..., 31 (11 of them), the width row 2, 5, ..., 29 (10), the temporal row the other 11
    from oracle import norm_rope_ref as N
    inv = np.ones(32, np.float32)                      # unit frequencies: the result IS the selected position
    pos = np.stack([np.full((1, 2), 100), np.full((1, 2), 200), np.full((1, 2), 300)]).astype(np.int32)
    got = N.mrope_freqs(pos, inv, (11, 11, 10))[0, 0]
    want = np.full(32, 100.0, np.float32)
    want[1::3] = 200.0
    want[2:30:3] = 300.0
    np.testing.assert_array_equal(got, want)
    assert (got == 100).sum() == 11 and (got == 200).sum() == 11 and (got == 300).sum() == 10
    # equal rows are the text case, bit for bit
    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, 5, 3, 256), dtype=np.float32).astype(N.bfloat16)
    p = rng.integers(0, 5000, size=(2, 5)).astype(np.int32)
    a = N.apply_rope(x, p, 256, 1e7, 0.25)
    b = N.apply_rope(x, np.stack([p, p, p]), 256, 1e7, 0.25, mrope_section=(11, 11, 10))
    c = N.apply_rope(x, p, 256, 1e7, 0.25, mrope_section=(11, 11, 10))
    np.testing.assert_array_equal(a.view(np.uint16), b.view(np.uint16))
    np.testing.assert_array_equal(a.view(np.uint16), c.view(np.uint16))
