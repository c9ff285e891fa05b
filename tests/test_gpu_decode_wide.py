"""Decode attention for rows of 2..8 query tokens (speculative verification) on the GPU, through the C ABI,
against the CPU oracle's wide decode (nanovllm_jax/kv_cache.py:852-998 restated in oracle/kv_cache_ref.py).

Tolerance: the contract is max-abs 2e-2 against the oracle's fp32 mode; the kernel is also held to 2e-3.
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


def _case(seed, num_blocks, lens, width, causal=True):
    c = decode_case(seed, num_blocks, len(lens), 1, 1)
    rng = np.random.default_rng(seed)
    lens = np.asarray(lens, np.int32)
    need = -(-lens // BS)
    tables = np.zeros((len(lens), max(1, int(need.max()))), np.int32)
    perm, o = rng.permutation(num_blocks), 0
    for b in range(len(lens)):
        tables[b, :need[b]] = perm[o:o + need[b]]
        o += need[b]
    q = rng.standard_normal((len(lens), width, 8, 256), dtype=np.float32).astype(bfloat16)
    if causal:  # the row's last `width` tokens are the queries
        pos = np.maximum(lens[:, None] - width + np.arange(width)[None, :], 0).astype(np.int32)
    else:
        pos = rng.integers(0, np.maximum(lens, 1)[:, None], size=(len(lens), width)).astype(np.int32)
    return c, q, tables, lens, pos


FORMS = pytest.mark.parametrize("form", [1, 2], ids=["mma_sync", "tcgen05"])


def _run(c, q, tables, lens, pos, form=0):
    from nano_vllm_jax_b200.kernels import paged_kv as K
    out = K.paged_decode_attention_wide(to_torch(q), to_torch(c["k_cache"][0]), to_torch(c["v_cache"][0]), to_torch(tables),
                                        to_torch(lens), None if pos is None else to_torch(pos), SCALE, form=form)
    torch.cuda.synchronize()
    return to_numpy(out)


def _oracle(c, q, tables, lens, pos):
    return R.paged_attention_decode(q, c["k_cache"], c["v_cache"], tables, lens, BS, SCALE, 4, positions=pos)


@FORMS
@pytest.mark.parametrize("width", [2, 3, 4, 5, 6, 7, 8])
def test_every_length_around_the_block_boundaries(width, form):
    lens = list(range(width, 3 * BS + 3)) + [5 * BS - 1, 5 * BS, 5 * BS + 1, 8 * BS + 7]  # beyond one 64-key tile too
    c, q, tables, lens, pos = _case(20 + width, 512, lens, width)
    out = _run(c, q, tables, lens, pos, form)
    err = np.abs(out - _oracle(c, q, tables, lens, pos)).max()
    assert err <= TIGHT, err


@FORMS
@pytest.mark.parametrize("width", [4, 7])
def test_scattered_positions_and_rows_without_keys(width, form):
    # positions anywhere inside the row (not only the tail), two rows of length 0 between live ones
    lens = [700, 0, 33, 1500, 0, 16, 257]
    c, q, tables, lens, pos = _case(31, 512, lens, width, causal=False)
    out = _run(c, q, tables, lens, pos, form)
    ref = _oracle(c, q, tables, lens, pos)
    live = lens > 0
    assert np.abs(out[live] - ref[live]).max() <= TIGHT
    assert not out[~live].any()  # defined as zeros (the reference leaves such rows undefined)


@FORMS
@pytest.mark.parametrize("width", [3, 8])
@pytest.mark.parametrize("lens", [(20000,), (9000, 30, 9000, 700, 5), (3000, 12000, 2, 6000)])
def test_long_rows_are_split_over_ctas_and_merged(lens, width, form):
    c, q, tables, lens, pos = _case(9, 2600, lens, width)
    lens = np.maximum(lens, width)
    pos = np.maximum(lens[:, None] - width + np.arange(width)[None, :], 0).astype(np.int32)
    out = _run(c, q, tables, lens, pos, form)
    assert np.abs(out - _oracle(c, q, tables, lens, pos)).max() <= TIGHT
    again = _run(c, q, tables, lens, pos, form)  # counters were left at zero; the merge order is fixed
    np.testing.assert_array_equal(bits(out), bits(again))


@FORMS
@pytest.mark.parametrize("width", [4, 6])
def test_no_positions_means_no_causal_limit_and_matches_the_packed_route(width, form):
    from nano_vllm_jax_b200.kernels import paged_kv as K
    lens = [300, 1000, 64, 129]
    c, q, tables, lens, pos = _case(41, 256, lens, width)
    out = _run(c, q, tables, lens, None, form)
    full = np.broadcast_to(lens[:, None] - 1, pos.shape).astype(np.int32)
    assert np.abs(out - _oracle(c, q, tables, lens, full)).max() <= TIGHT
    # the same batch as a packed batch of equal-width rows on the prefill tiles
    qsl = torch.arange(len(lens) + 1, dtype=torch.int32, device="cuda") * width
    packed = K.packed_paged_prefill_attention(to_torch(q).reshape(1, -1, 8, 256), to_torch(c["k_cache"][0]), to_torch(c["v_cache"][0]),
                                              to_torch(tables), to_torch(lens), to_torch(pos).reshape(1, -1), qsl, BS, SCALE, 4)
    causal = _run(c, q, tables, lens, pos, form)
    assert np.abs(to_numpy(packed).reshape(causal.shape) - causal).max() <= TIGHT


def test_refusals():
    from nano_vllm_jax_b200.kernels import paged_kv as K
    c, q, tables, lens, pos = _case(5, 64, [40, 50], 16)
    q9 = np.concatenate([q, q[:, :1]], axis=1)  # 17 tokens per row
    with pytest.raises(ValueError):
        K.paged_decode_attention_wide(to_torch(q9), to_torch(c["k_cache"][0]), to_torch(c["v_cache"][0]), to_torch(tables),
                                      to_torch(lens), None, SCALE)
    with pytest.raises(ValueError):
        K.paged_decode_attention_wide(to_torch(q).float(), to_torch(c["k_cache"][0]), to_torch(c["v_cache"][0]), to_torch(tables),
                                      to_torch(lens), None, SCALE)


@pytest.mark.parametrize("width", [5, 8])
def test_the_two_forms_agree_on_a_batch_of_many_rows(width):
    """What the automatic choice takes at these widths (tcgen05) against the mma.sync form, 96 rows of 600..2500 tokens:
    most rows lie inside one CTA pair's range, some are cut over two and folded by the merge launch."""
    rng = np.random.default_rng(77)
    lens = rng.integers(600, 2501, size=96)
    c, q, tables, lens, pos = _case(13, 96 * 160, lens, width)
    auto = _run(c, q, tables, lens, pos, 0)
    mma = _run(c, q, tables, lens, pos, 1)
    assert np.abs(auto - mma).max() <= TIGHT
    rows = [0, 17, 95]
    ref = _oracle({"k_cache": c["k_cache"], "v_cache": c["v_cache"]}, q[rows], tables[rows], lens[rows], pos[rows])
    assert np.abs(auto[rows] - ref).max() <= TIGHT


@pytest.mark.parametrize("width", [9, 12, 16])
def test_rows_of_nine_to_sixteen_tokens_take_the_tcgen05_form(width):
    """The reference verifies up to 9 tokens per row (kv_cache.py:972-977); the second half of the query rows sits in
    the next 32 TMEM lanes and has a softmax warp of its own."""
    lens = list(range(width, 2 * BS + 2)) + [5 * BS, 5 * BS + 1, 700, 2600, 9000]
    c, q, tables, lens, pos = _case(50 + width, 1024, lens, width)
    out = _run(c, q, tables, lens, pos, 0)
    assert np.abs(out - _oracle(c, q, tables, lens, pos)).max() <= TIGHT
    from nano_vllm_jax_b200._lib import NvjError
    with pytest.raises(NvjError):  # the mma.sync form ends at 8
        _run(c, q, tables, lens, pos, 1)
