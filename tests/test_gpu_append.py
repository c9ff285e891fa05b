"""KV append on the GPU through the C ABI: bit-exact against the CPU oracle."""

import numpy as np
import pytest
import torch
from ml_dtypes import bfloat16

from helpers import bits, decode_case, to_numpy, to_torch
from oracle import kv_cache_ref as R

pytestmark = pytest.mark.gpu


def _kv():
    from nano_vllm_jax_b200 import kv_cache
    return kv_cache


def _assert_same(a_t, b_np):
    np.testing.assert_array_equal(bits(to_numpy(a_t)), bits(b_np))


def test_masked_duplicates_known_answer():
    # reference tests/test_kv_cache.py:627-677: slots [[2,2,3,5]], valid [[1,0,1,0]], fp32, odd row size (scalar kernel)
    nb, bs, hkv, d = 4, 8, 2, 3
    n = nb * bs * hkv * d
    k0 = np.arange(n, dtype=np.float32).reshape(1, nb, bs, hkv, d)
    v0 = k0 + 1000.0
    rng = np.random.default_rng(0)
    nk = rng.standard_normal((1, 4, hkv, d)).astype(np.float32)
    nv = rng.standard_normal((1, 4, hkv, d)).astype(np.float32)
    slots = np.array([[2, 2, 3, 5]], np.int32)
    valid = np.array([[1, 0, 1, 0]], bool)
    ek, ev = R.update_kv_cache(k0, v0, slots, nk, nv, 0, valid_mask=valid)
    kc, vc = to_torch(k0), to_torch(v0)
    rk, rv = _kv().update_kv_cache(kc, vc, to_torch(slots), to_torch(nk), to_torch(nv), 0, valid_mask=to_torch(valid))
    assert rk is kc and rv is vc  # updated in place, same tensors returned
    _assert_same(kc, ek)
    _assert_same(vc, ev)


@pytest.mark.parametrize("layer", [0, 2])
def test_decode_append_config1_bit_exact(layer):
    c = decode_case(1, 256, 4, 64, 512, layers=3)
    slots = R.compute_slot_mapping(c["positions"], c["tables"], 16)
    ek, ev = R.update_kv_cache(c["k_cache"], c["v_cache"], slots, c["new_k"], c["new_v"], layer)
    kc, vc = to_torch(c["k_cache"]), to_torch(c["v_cache"])
    kv = _kv()
    s = kv.compute_slot_mapping(to_torch(c["positions"]), to_torch(c["tables"]), 16)
    np.testing.assert_array_equal(to_numpy(s), slots)
    kv.update_kv_cache(kc, vc, s, to_torch(c["new_k"]), to_torch(c["new_v"]), layer)
    _assert_same(kc, ek)
    _assert_same(vc, ev)


def test_backend_write_kv_masks_padded_rows_and_tokens():
    # reference tests/test_cuda_fp32_ffi.py:127-195: layer 1 of 3, padded rows, sentinel-filled caches
    from nano_vllm_jax_b200.backends import B200Backend
    from nano_vllm_jax_b200.kv_cache import KVCacheStorage
    rng = np.random.default_rng(3)
    L, nb, bs, hkv, d = 3, 12, 16, 2, 256
    k0 = np.full((L, nb, bs, hkv, d), -1.0, np.float32).astype(bfloat16)
    v0 = np.full((L, nb, bs, hkv, d), -2.0, np.float32).astype(bfloat16)
    tables = np.array([[3, 1, 0], [2, 4, 0], [0, 0, 0]], np.int32)
    positions = np.array([[15, 16, 17], [5, 0, 0], [0, 0, 0]], np.int32)  # row 1 has one real token, row 2 is padding
    qsl = np.array([0, 3, 4, 4], np.int32)
    seq_lens = np.array([18, 6, 0], np.int32)
    nk = rng.standard_normal((3, 3, hkv, d)).astype(bfloat16)
    nv = rng.standard_normal((3, 3, hkv, d)).astype(bfloat16)
    slots = R.compute_slot_mapping(positions, tables, bs)
    ek, ev = R.update_kv_cache(k0, v0, slots, nk, nv, 1, valid_mask=R.write_kv_valid_mask(slots.shape, qsl, False))
    be = B200Backend()
    md = be.build_attention_metadata(to_torch(positions), to_torch(tables), to_torch(seq_lens), bs, True,
                                     query_start_loc=to_torch(qsl))
    np.testing.assert_array_equal(to_numpy(md.slot_mapping), slots)
    cache = KVCacheStorage(to_torch(k0), to_torch(v0))
    out = be.write_kv(1, to_torch(nk), to_torch(nv), cache, md)
    _assert_same(out.k_cache, ek)
    _assert_same(out.v_cache, ev)
    assert float(out.k_cache[0].float().max()) == -1.0  # other layers untouched


def test_packed_append_drops_tokens_beyond_query_start_loc():
    # reference tests/test_backend_boundaries.py:1441-1459: padding token aliases slot 6 and must not overwrite it
    from nano_vllm_jax_b200.backends import B200Backend
    from nano_vllm_jax_b200.kv_cache import KVCacheStorage
    rng = np.random.default_rng(4)
    nb, bs, hkv, d = 8, 2, 2, 8
    k0 = rng.standard_normal((1, nb, bs, hkv, d)).astype(np.float32)
    v0 = rng.standard_normal((1, nb, bs, hkv, d)).astype(np.float32)
    tables = np.array([[3, 4], [5, 6]], np.int32)
    positions = np.array([[0, 1, 2, 0]], np.int32)
    rows = np.array([[0, 0, 1, 0]], np.int32)
    qsl = np.array([0, 2, 3], np.int32)
    nk = rng.standard_normal((1, 4, hkv, d)).astype(np.float32)
    nv = rng.standard_normal((1, 4, hkv, d)).astype(np.float32)
    slots = R.compute_packed_slot_mapping(positions, tables, rows, bs)
    assert slots.tolist() == [[6, 7, 12, 6]]
    ek, ev = R.update_kv_cache(k0, v0, slots, nk, nv, 0, valid_mask=R.write_kv_valid_mask(slots.shape, qsl, True))
    be = B200Backend()
    md = be.build_attention_metadata(to_torch(positions), to_torch(tables), to_torch(np.array([2, 3], np.int32)), bs,
                                     True, query_start_loc=to_torch(qsl), token_row_ids=to_torch(rows))
    assert to_numpy(md.slot_mapping).tolist() == [[6, 7, 12, 6]]
    out = be.write_kv(0, to_torch(nk), to_torch(nv), KVCacheStorage(to_torch(k0), to_torch(v0)), md)
    _assert_same(out.k_cache, ek)
    _assert_same(out.v_cache, ev)


def test_nhd_page_table_append_equals_canonical():
    # reference tests/test_nhd_kv_cache.py:140-184 and tests/test_cuda_fp32_ffi.py:83-125 (D=256, arange payloads)
    from nano_vllm_jax_b200.kernels import paged_kv as K
    pages, P, hkv, d = 6, 16, 2, 256
    k0 = np.full((pages, P, hkv, d), -1.0, np.float32)
    v0 = np.full((pages, P, hkv, d), -2.0, np.float32)
    tables = np.array([[3, 1], [2, 4]], np.int32)
    bi = np.array([0, 0, 1, 1], np.int32)
    pos = np.array([15, 16, 0, 31], np.int32)
    nk = np.arange(4 * hkv * d, dtype=np.float32).reshape(4, hkv, d)
    nv = nk + 0.5
    idx, ptr = R.dense_block_tables_to_kv_indptr(tables)
    lpl = R.kv_last_page_len_from_seq_lens(np.array([17, 32]), P)
    ek, ev = R.kv_append_paged_nhd(nk, nv, bi, pos, k0, v0, idx, ptr, lpl)
    kc, vc = to_torch(k0), to_torch(v0)
    K.kv_append_paged_nhd(to_torch(nk), to_torch(nv), to_torch(bi), to_torch(pos), kc, vc, to_torch(idx),
                          to_torch(ptr), to_torch(lpl))
    _assert_same(kc, ek)
    _assert_same(vc, ev)
    # with a valid mask: token 1 dropped
    vm = np.array([1, 0, 1, 1], np.int32)
    ek, ev = R.kv_append_paged_nhd(nk, nv, bi, pos, k0, v0, idx, ptr, lpl, valid_mask=vm)
    kc, vc = to_torch(k0), to_torch(v0)
    K.kv_append_paged_nhd(to_torch(nk), to_torch(nv), to_torch(bi), to_torch(pos), kc, vc, to_torch(idx),
                          to_torch(ptr), to_torch(lpl), to_torch(vm))
    _assert_same(kc, ek)
    _assert_same(vc, ev)


def test_fp32_rows_are_rounded_to_the_cache_dtype_like_astype():
    # kv_cache.py:522-523: new rows are cast to the cache dtype (round to nearest even)
    rng = np.random.default_rng(5)
    k0 = np.zeros((1, 4, 16, 2, 256), np.float32).astype(bfloat16)
    nk = rng.standard_normal((2, 3, 2, 256)).astype(np.float32)
    nk[0, 0, 0, :4] = [1.00390625, 1.01171875, -0.0, 3.0e38]  # ties and a near-overflow value
    nv = rng.standard_normal((2, 3, 2, 256)).astype(np.float32)
    slots = np.array([[0, 1, 2], [40, 41, 63]], np.int32)
    ek, ev = R.update_kv_cache(k0, k0, slots, nk, nv, 0)
    kc, vc = to_torch(k0), to_torch(k0.copy())
    _kv().update_kv_cache(kc, vc, to_torch(slots), to_torch(nk), to_torch(nv), 0)
    _assert_same(kc, ek)
    _assert_same(vc, ev)


def test_empty_and_out_of_range():
    from nano_vllm_jax_b200.kernels import paged_kv as K
    k0 = np.zeros((1, 2, 16, 2, 256), np.float32).astype(bfloat16)
    kc, vc = to_torch(k0), to_torch(k0.copy())
    e = torch.zeros((0, 1, 2, 256), dtype=torch.bfloat16, device="cuda")
    K.kv_append_slots(e, e, torch.zeros((0, 1), dtype=torch.int32, device="cuda"), kc[0], vc[0])  # no-op
    one = torch.ones((1, 1, 2, 256), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(K.DeviceStatusError):  # slot 32 is outside a 32-slot pool: skipped and flagged, no fault
        K.kv_append_slots(one, one, torch.tensor([[32]], dtype=torch.int32, device="cuda"), kc[0], vc[0])
    assert float(kc.float().abs().max()) == 0.0
    K.kv_append_slots(one, one, torch.tensor([[31]], dtype=torch.int32, device="cuda"), kc[0], vc[0])
    assert float(kc[0, 1, 15].float().min()) == 1.0


def test_slot_mapping_of_negative_positions_floors_like_the_reference():
    # jnp's // and % floor (nanovllm_jax/kv_cache.py:432-435): position -1 is offset bs - 1 of block index -1,
    # which indexes the table's last column; C's / and % would give column 0, offset -1
    tables = np.array([[3, 1, 7], [2, 4, 6]], np.int32)
    positions = np.array([[-1, 0, 17], [-16, -17, 33]], np.int32)
    want = R.compute_slot_mapping(positions, tables, 16)
    np.testing.assert_array_equal(want, [[7 * 16 + 15, 48, 17], [6 * 16, 4 * 16 + 15, 6 * 16 + 1]])
    got = _kv().compute_slot_mapping(to_torch(positions), to_torch(tables), 16)
    np.testing.assert_array_equal(to_numpy(got), want)
    rid = np.array([[1, 1, 0, 0, 1, 0]], np.int32)
    ppos = positions.reshape(1, -1)
    np.testing.assert_array_equal(to_numpy(_kv().compute_packed_slot_mapping(to_torch(ppos), to_torch(tables), to_torch(rid), 16)),
                                  R.compute_packed_slot_mapping(ppos, tables, rid, 16))


def test_page_table_append_does_not_reach_into_the_next_rows_pages():
    # row 0 owns 2 pages; a position in "page 2" must be flagged and dropped, not written into row 1's first page
    from nano_vllm_jax_b200.kernels import paged_kv as K
    k0 = np.zeros((6, 4, 1, 8), np.float32)
    kc, vc = to_torch(k0), to_torch(k0.copy())
    one = torch.ones((1, 1, 8), dtype=torch.float32, device="cuda")
    indices = to_torch(np.array([0, 1, 2, 3], np.int32))
    indptr = to_torch(np.array([0, 2, 4], np.int32))
    last = to_torch(np.array([4, 4], np.int32))
    with pytest.raises(K.DeviceStatusError):
        K.kv_append_paged_nhd(one, one, to_torch(np.array([0], np.int32)), to_torch(np.array([8], np.int32)), kc, vc,
                              indices, indptr, last)
    assert float(kc.abs().max()) == 0.0 and float(vc.abs().max()) == 0.0
    K.kv_append_paged_nhd(one, one, to_torch(np.array([0], np.int32)), to_torch(np.array([7], np.int32)), kc, vc,
                          indices, indptr, last)
    assert float(kc[1, 3].min()) == 1.0 and float(kc.sum()) == 8.0
