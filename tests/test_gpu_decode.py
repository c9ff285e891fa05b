"""Paged GQA decode attention on the GPU through the C ABI, against the CPU oracle.

Tolerances: the contract is max-abs 2e-2 against the oracle's fp32 mode (bf16
storage, fp32 accumulate).  Both kernels accumulate in fp32, so the tests also
hold them to a tighter regression bound TIGHT.  Cache contents are compared bit
for bit.
"""

import numpy as np
import pytest
import torch
from ml_dtypes import bfloat16

from helpers import BS, SCALE, bits, decode_case, to_numpy, to_torch
from oracle import kv_cache_ref as R

pytestmark = pytest.mark.gpu

CONTRACT = 2e-2
TIGHT = 2e-3
GENERIC, PIPELINED, TENSOR = 1, 2, 3


def _K():
    from nano_vllm_jax_b200.kernels import paged_kv as K
    return K


def _run(c, variant, layer=0):
    K = _K()
    out = K.paged_decode_attention(to_torch(c["q"][:, 0]), to_torch(c["k_cache"][layer]), to_torch(c["v_cache"][layer]),
                                   to_torch(c["tables"]), to_torch(c["seq_lens"]), SCALE, variant=variant)
    torch.cuda.synchronize()
    return to_numpy(out).reshape(out.shape[0], -1)


def _oracle(c, layer=0):
    return R.paged_attention_decode(c["q"], c["k_cache"], c["v_cache"], c["tables"], c["seq_lens"], c["bs"], SCALE,
                                    c["groups"], layer_idx=layer)[:, 0]


def _check(out, ref, active):
    err = np.abs(out[active] - ref[active]).max()
    assert err <= CONTRACT, f"contract broken: max-abs {err}"
    assert err <= TIGHT, f"regression bound broken: max-abs {err}"


@pytest.mark.parametrize("variant", [GENERIC, PIPELINED, TENSOR])
def test_config1_single_layer_decode(variant):
    c = decode_case(1, 256, 4, 64, 512)
    out = _run(c, variant)
    _check(out, _oracle(c), np.ones(4, bool))


@pytest.mark.parametrize("variant", [GENERIC, PIPELINED, TENSOR])
def test_every_length_from_0_to_3_blocks_plus_1(variant):
    # one batch row per length 0 .. 3*bs+1: empty rows, partial last blocks of every size, exact multiples
    n = 3 * BS + 2
    c = decode_case(2, 512, n, 3 * BS, 3 * BS)  # four blocks per row, then every length up to them
    c["seq_lens"] = np.arange(n, dtype=np.int32)
    out = _run(c, variant)
    ref = _oracle(c)
    active = c["seq_lens"] > 0
    _check(out, ref, active)
    assert not out[~active].any()  # rows with seq_len 0 are defined to be zeros


@pytest.mark.parametrize("variant", [GENERIC, PIPELINED, TENSOR])
def test_padded_rows_interleaved_and_layer_offset(variant):
    c = decode_case(3, 300, 9, 20, 200, layers=2, empty_rows=(0, 4, 8))
    out = _run(c, variant, layer=1)
    ref = _oracle(c, layer=1)
    active = c["seq_lens"] > 0
    _check(out, ref, active)
    assert not out[~active].any()


@pytest.mark.parametrize("variant", [PIPELINED, TENSOR])
def test_rows_split_across_many_ctas(variant):
    # 3 rows of ~4000 keys = ~750 blocks over the CTAs: every row is finished by a cross-CTA merge
    c = decode_case(4, 900, 3, 3900, 4095)
    out = _run(c, variant)
    _check(out, _oracle(c), np.ones(3, bool))
    again = _run(c, variant)  # arrival counters were left at zero: a second launch gives the same bits
    np.testing.assert_array_equal(bits(out), bits(again))


@pytest.mark.parametrize("variant", [PIPELINED, TENSOR])
@pytest.mark.parametrize("lens", [(20000,), (9000, 30, 9000, 700, 5), (3000, 12000, 1, 6000)])
def test_few_long_rows_are_merged_in_two_levels(lens, variant):
    # rows cut into more than 32 partials: groups of 13 CTAs fold first, the last group folds the groups;
    # short rows between them share CTAs and groups with the long ones
    c = decode_case(9, 2600, len(lens), 1, 1)
    rng = np.random.default_rng(9)
    c["seq_lens"] = np.asarray(lens, np.int32)
    need = -(-c["seq_lens"] // BS)
    c["tables"] = np.zeros((len(lens), int(need.max())), np.int32)
    perm, o = rng.permutation(2600), 0
    for b in range(len(lens)):
        c["tables"][b, :need[b]] = perm[o:o + need[b]]
        o += need[b]
    out = _run(c, variant)
    _check(out, _oracle(c), np.ones(len(lens), bool))
    again = _run(c, variant)  # row and group counters were left at zero
    np.testing.assert_array_equal(bits(out), bits(again))


@pytest.mark.parametrize("variant", [PIPELINED, TENSOR])
def test_mixed_short_and_long_rows(variant):
    c = decode_case(5, 4096, 40, 1, 1500)
    out = _run(c, variant)
    ref = _oracle(c)
    _check(out, ref, np.ones(40, bool))
    gen = _run(c, GENERIC)
    assert np.abs(gen - out).max() <= TIGHT


def test_long_ranges_refill_the_block_id_ring():
    # > 512 blocks per CTA (the look-ahead ring is refilled in flight): 48 rows x ~56k keys
    rows, ctx = 48, 56000
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rows = max(rows, (2 * sms * 600) // (ctx // BS) + 1)
    nb = rows * (ctx // BS + 2)
    rng = np.random.default_rng(6)
    lens = rng.integers(ctx - 500, ctx, size=rows).astype(np.int32)
    need = -(-lens // BS)
    w = int(need.max())
    perm = rng.permutation(nb)
    tables = np.zeros((rows, w), np.int32)
    o = 0
    for b in range(rows):
        tables[b, :need[b]] = perm[o:o + need[b]]
        o += need[b]
    g = torch.Generator(device="cuda").manual_seed(6)
    kc = torch.randn((nb, BS, 2, 256), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    vc = torch.randn((nb, BS, 2, 256), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    q = torch.randn((rows, 8, 256), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    K = _K()
    t_tables, t_lens = to_torch(tables), to_torch(lens)
    fast = K.paged_decode_attention(q, kc, vc, t_tables, t_lens, SCALE, variant=PIPELINED)
    tensor = K.paged_decode_attention(q, kc, vc, t_tables, t_lens, SCALE, variant=TENSOR)
    slow = K.paged_decode_attention(q, kc, vc, t_tables, t_lens, SCALE, variant=GENERIC)
    torch.cuda.synchronize()
    assert float((fast - slow).abs().max()) <= TIGHT
    assert float((tensor - slow).abs().max()) <= TIGHT
    # two rows against the CPU oracle (the gather of all rows would need tens of GB on the host)
    for b in (0, rows - 1):
        blocks = tables[b, :need[b]]
        k_np = to_numpy(kc[to_torch(blocks).long()])[None]
        v_np = to_numpy(vc[to_torch(blocks).long()])[None]
        ref = R.paged_attention_decode(to_numpy(q[b])[None, None], k_np, v_np, np.arange(need[b], dtype=np.int32)[None],
                                       lens[b:b + 1], BS, SCALE, 4)[0, 0]
        assert np.abs(to_numpy(fast[b]).reshape(-1) - ref).max() <= TIGHT


@pytest.mark.parametrize("variant", [GENERIC, PIPELINED, TENSOR])
def test_fused_append_cache_bit_exact_and_attention(variant):
    K = _K()
    c = decode_case(7, 2048, 33, 1, 900, layers=2, empty_rows=(5,))
    layer = 1
    slots = R.compute_slot_mapping(c["positions"], c["tables"], BS)
    valid = (c["seq_lens"] > 0)[:, None]
    ek, ev = R.update_kv_cache(c["k_cache"], c["v_cache"], slots, c["new_k"], c["new_v"], layer, valid_mask=valid)
    ref = R.paged_attention_decode(c["q"], ek, ev, c["tables"], c["seq_lens"], BS, SCALE, 4, layer_idx=layer)
    kc, vc = to_torch(c["k_cache"]), to_torch(c["v_cache"])
    out, rk, rv = K.paged_decode_attention_with_kv_append(
        to_torch(c["q"]), to_torch(c["new_k"]), to_torch(c["new_v"]), kc, vc, to_torch(c["tables"]),
        to_torch(c["seq_lens"]), to_torch(c["positions"]), layer, BS, SCALE, 4, variant=variant)
    torch.cuda.synchronize()
    assert rk is kc and rv is vc and out.shape == (33, 1, 2048) and out.dtype == torch.float32
    np.testing.assert_array_equal(bits(to_numpy(kc)), bits(ek))
    np.testing.assert_array_equal(bits(to_numpy(vc)), bits(ev))
    active = c["seq_lens"] > 0
    _check(to_numpy(out)[:, 0], ref[:, 0], active)
    assert not to_numpy(out)[~active].any()


@pytest.mark.parametrize("variant", [PIPELINED, TENSOR])
def test_fused_equals_append_then_decode_bitwise(variant):
    K = _K()
    from nano_vllm_jax_b200 import kv_cache as kv
    c = decode_case(8, 2048, 64, 100, 400)
    kc1, vc1 = to_torch(c["k_cache"]), to_torch(c["v_cache"])
    kc2, vc2 = to_torch(c["k_cache"]), to_torch(c["v_cache"])
    out1, _, _ = K.paged_decode_attention_with_kv_append(
        to_torch(c["q"]), to_torch(c["new_k"]), to_torch(c["new_v"]), kc1, vc1, to_torch(c["tables"]),
        to_torch(c["seq_lens"]), to_torch(c["positions"]), 0, BS, SCALE, 4, variant=variant)
    s = kv.compute_slot_mapping(to_torch(c["positions"]), to_torch(c["tables"]), BS)
    kv.update_kv_cache(kc2, vc2, s, to_torch(c["new_k"]), to_torch(c["new_v"]), 0)
    out2 = K.paged_decode_attention(to_torch(c["q"][:, 0]), kc2[0], vc2[0], to_torch(c["tables"]),
                                    to_torch(c["seq_lens"]), SCALE, variant=variant)
    torch.cuda.synchronize()
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert torch.equal(out1.reshape(64, 8, 256), out2)


@pytest.mark.parametrize("variant", [GENERIC, PIPELINED, TENSOR])
def test_csr_page_table_form(variant):
    # reference tests/test_paged_attention_abi.py:100-151 shape: P16, Hq8/Hkv2, D256, lens [17, 31]
    K = _K()
    c = decode_case(9, 64, 2, 1, 1)
    c["seq_lens"] = np.array([17, 31], np.int32)
    c["tables"] = np.array([[3, 1], [2, 4]], np.int32)
    idx, ptr = R.dense_block_tables_to_kv_indptr(c["tables"])
    lpl = R.kv_last_page_len_from_seq_lens(c["seq_lens"], BS)
    ref = R.paged_decode_attention_gqa_nhd(c["q"][:, 0], c["k_cache"][0], c["v_cache"][0], ptr, idx, lpl, c["seq_lens"], SCALE)
    out = K.paged_decode_attention_gqa_nhd(to_torch(c["q"][:, 0]), to_torch(c["k_cache"][0]), to_torch(c["v_cache"][0]),
                                           to_torch(ptr), to_torch(idx), to_torch(lpl), to_torch(c["seq_lens"]), SCALE,
                                           variant=variant)
    assert out.shape == (2, 8, 256) and out.dtype == torch.float32
    assert np.abs(to_numpy(out) - ref).max() <= TIGHT
    # last-page length shorter than seq_lens clips the attended keys (paged_attention.py:171-178)
    lpl2 = np.array([1, 10], np.int32)
    ref2 = R.paged_decode_attention_gqa_nhd(c["q"][:, 0], c["k_cache"][0], c["v_cache"][0], ptr, idx, lpl2, c["seq_lens"], SCALE)
    out2 = K.paged_decode_attention_gqa_nhd(to_torch(c["q"][:, 0]), to_torch(c["k_cache"][0]), to_torch(c["v_cache"][0]),
                                            to_torch(ptr), to_torch(idx), to_torch(lpl2), to_torch(c["seq_lens"]), SCALE,
                                            variant=variant)
    assert np.abs(to_numpy(out2) - ref2).max() <= TIGHT


def test_fp32_small_shapes_generic_kernel():
    # reference tests/test_paged_attention_abi.py:20-97: B2, P4, Hq4/Hkv2, D8, lens [7,10], fp32, tol 1e-6 there
    from nano_vllm_jax_b200 import kv_cache as kv
    rng = np.random.default_rng(10)
    k = rng.standard_normal((1, 6, 4, 2, 8)).astype(np.float32)
    v = rng.standard_normal((1, 6, 4, 2, 8)).astype(np.float32)
    q = rng.standard_normal((2, 1, 4, 8)).astype(np.float32)
    tables = np.array([[3, 1, 5], [2, 4, 0]], np.int32)
    lens = np.array([7, 10], np.int32)
    ref = R.paged_attention_decode(q, k, v, tables, lens, 4, 0.35, 2)
    out = kv.paged_attention_decode(to_torch(q), to_torch(k), to_torch(v), to_torch(tables), to_torch(lens), 4, 0.35, 2)
    assert out.dtype == torch.float32 and out.shape == (2, 1, 32)
    np.testing.assert_allclose(to_numpy(out), ref, rtol=1e-5, atol=2e-6)
    # flat 4-D cache rank is the same memory (kv_cache.py:341-369)
    out4 = kv.paged_attention_decode(to_torch(q), to_torch(k.reshape(1, 24, 2, 8)), to_torch(v.reshape(1, 24, 2, 8)),
                                     to_torch(tables), to_torch(lens), 4, 0.35, 2)
    assert torch.equal(out, out4)


def test_wide_decode_with_positions_and_reference_dtype():
    from nano_vllm_jax_b200 import kv_cache as kv
    c = decode_case(11, 128, 3, 40, 90)
    rng = np.random.default_rng(11)
    q = rng.standard_normal((3, 4, 8, 256)).astype(bfloat16)
    pos = (c["seq_lens"][:, None] - 4 + np.arange(4)[None, :]).astype(np.int32)
    ref = R.paged_attention_decode(q, c["k_cache"], c["v_cache"], c["tables"], c["seq_lens"], BS, SCALE, 4, positions=pos)
    out = kv.paged_attention_decode(to_torch(q), to_torch(c["k_cache"]), to_torch(c["v_cache"]), to_torch(c["tables"]),
                                    to_torch(c["seq_lens"]), BS, SCALE, 4, positions=to_torch(pos))
    assert out.dtype == torch.bfloat16  # promotion of bf16 q with a bf16 cache, as in the reference
    assert np.abs(to_numpy(out.float()) - ref).max() <= CONTRACT
    out32 = kv.paged_attention_decode(to_torch(q), to_torch(c["k_cache"]), to_torch(c["v_cache"]), to_torch(c["tables"]),
                                      to_torch(c["seq_lens"]), BS, SCALE, 4, positions=to_torch(pos), out_dtype=torch.float32)
    assert np.abs(to_numpy(out32) - ref).max() <= TIGHT
    with pytest.raises(ValueError):
        kv.paged_attention_decode(to_torch(q), to_torch(c["k_cache"]), to_torch(c["v_cache"]), to_torch(c["tables"]),
                                  to_torch(c["seq_lens"]), BS, SCALE, 4)


def test_legacy_prefill_gathers_keys_by_slot_mapping():
    # kv_cache.py:567-647: token t of row b attends the slots slot_mapping[b, 0..t], wherever they sit in the cache
    from nano_vllm_jax_b200 import kv_cache as kv
    rng = np.random.default_rng(13)
    k = rng.standard_normal((2, 64, 4, 2, 64)).astype(np.float32)
    v = rng.standard_normal((2, 64, 4, 2, 64)).astype(np.float32)
    slots = rng.permutation(64 * 4)[: 3 * 21].reshape(3, 21).astype(np.int32)
    q = rng.standard_normal((3, 21, 8, 64)).astype(np.float32)
    lens = np.full(3, 21, np.int32)
    ref = R.paged_attention(q, k, v, slots, lens, 0.125, 4, layer_idx=1)
    out = kv.paged_attention(to_torch(q), to_torch(k), to_torch(v), to_torch(slots), to_torch(lens), 0.125, 4, layer_idx=1)
    assert out.shape == (3, 21, 8 * 64)
    np.testing.assert_allclose(to_numpy(out), ref, rtol=1e-5, atol=3e-6)


def test_rectangular_prefill_with_rows_padded_at_position_zero():
    # rows of a rectangular [B, T] prefill are padded with (token 0, position 0): positions do not grow along a row,
    # and the key range of a query tile is set by the token that sees the most keys, wherever it sits
    from nano_vllm_jax_b200 import kv_cache as kv
    c = decode_case(12, 256, 3, 150, 400)
    rng = np.random.default_rng(12)
    width = 70
    q = rng.standard_normal((3, width, 8, 256)).astype(bfloat16)
    real = np.array([70, 41, 9])
    pos = np.zeros((3, width), np.int32)
    for r in range(3):
        pos[r, :real[r]] = c["seq_lens"][r] - real[r] + np.arange(real[r])
    ref = R.paged_attention_prefill(q, c["k_cache"], c["v_cache"], c["tables"], c["seq_lens"], pos, BS, SCALE, 4)
    out = kv.paged_attention_prefill(to_torch(q), to_torch(c["k_cache"]), to_torch(c["v_cache"]), to_torch(c["tables"]),
                                     to_torch(c["seq_lens"]), to_torch(pos), BS, SCALE, 4, out_dtype=torch.float32)
    assert out.shape == (3, width, 2048)
    assert np.abs(to_numpy(out) - ref).max() <= TIGHT


@pytest.mark.parametrize("variant", [GENERIC, PIPELINED, TENSOR])
def test_block_id_outside_the_pool_is_flagged_not_read(variant):
    K = _K()
    c = decode_case(12, 64, 2, 30, 60)
    c["tables"][1, 1] = 64  # one past the last block
    with pytest.raises(K.DeviceStatusError):
        _run(c, variant)
    c["tables"][1, 1] = 5
    out = _run(c, variant)  # the workspace was reset by the failed check: the next launch is clean
    _check(out, _oracle(c), np.ones(2, bool))


def test_validation_errors_match_the_reference_messages():
    from nano_vllm_jax_b200 import kv_cache as kv
    c = decode_case(13, 16, 2, 5, 9)
    args = [to_torch(c["q"]), to_torch(c["k_cache"]), to_torch(c["v_cache"]), to_torch(c["tables"]), to_torch(c["seq_lens"])]
    with pytest.raises(ValueError, match="block_size must be positive"):
        kv.paged_attention_decode(*args, 0, SCALE, 4)
    with pytest.raises(ValueError, match="out of bounds"):
        kv.paged_attention_decode(*args, BS, SCALE, 4, layer_idx=3)
    with pytest.raises(ValueError, match="must match block_tables batch"):
        kv.paged_attention_decode(args[0], args[1], args[2], args[3][:1], args[4], BS, SCALE, 4)
    with pytest.raises(ValueError, match="max_kv_len exceeds"):
        kv.paged_attention_decode(*args, BS, SCALE, 4, max_kv_len=10 ** 6)
    with pytest.raises(ValueError, match="CUDA tensor"):
        kv.paged_attention_decode(args[0].cpu(), *args[1:], BS, SCALE, 4)


def test_fused_append_position_beyond_the_table_is_flagged_on_the_generic_route_too():
    # a shape only the generic kernel serves (fp32, block 4): the append in front of it must treat a position past
    # the row's table as the fused kernels do (flag, no write), not write into the next row's block
    K = _K()
    rng = np.random.default_rng(14)
    L, nb, bs, hkv, d = 1, 8, 4, 1, 8
    k0 = np.zeros((L, nb, bs, hkv, d), np.float32)
    kc, vc = to_torch(k0), to_torch(k0.copy())
    q = to_torch(rng.standard_normal((2, 1, 2, d)).astype(np.float32))
    nk = torch.ones((2, 1, hkv, d), dtype=torch.float32, device="cuda")
    tables = to_torch(np.array([[1, 2], [3, 4]], np.int32))
    lens = to_torch(np.array([5, 5], np.int32))
    bad_pos = to_torch(np.array([[8], [4]], np.int32))   # row 0: block index 2 of a 2-wide table
    with pytest.raises(K.DeviceStatusError):
        K.paged_decode_attention_with_kv_append(q, nk, nk, kc, vc, tables, lens, bad_pos, 0, bs, 0.3, 2)
    torch.cuda.synchronize()
    assert float(kc[0, 3].abs().max()) == 0.0            # row 1's first block untouched by row 0
    assert float(kc[0, 4, 0].min()) == 1.0               # row 1's own token landed


@pytest.mark.parametrize("variant", [PIPELINED, TENSOR])
def test_one_workspace_serves_small_and_large_batches_in_turn(variant):
    # A call with few rows leaves partial results in the workspace; they must not sit where a later call with more
    # rows keeps its arrival counters (that once left every split row beyond ~110 of a 256-row call unwritten).
    K = _K()
    small = decode_case(15, 3000, 4, 9000, 10000)       # 4 long rows: every CTA writes partials
    large = decode_case(16, 9000, 256, 300, 500)        # 256 rows, most of them split over two CTAs
    wide_q = np.random.default_rng(17).standard_normal((4, 3, 8, 256), dtype=np.float32).astype(bfloat16)
    for _ in range(2):
        _check(_run(small, variant), _oracle(small), np.ones(4, bool))
        _check(_run(large, variant), _oracle(large), np.ones(256, bool))
        # a wide call (larger partial area) in between, then the large batch again
        K.paged_decode_attention_wide(to_torch(wide_q), to_torch(small["k_cache"][0]), to_torch(small["v_cache"][0]),
                                      to_torch(small["tables"]), to_torch(small["seq_lens"]), None, SCALE)
        _check(_run(large, variant), _oracle(large), np.ones(256, bool))
