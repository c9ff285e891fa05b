"""RMSNorm + partial RoPE + KV append in one kernel against the CPU oracle of the same sequence."""

import numpy as np
import pytest
import torch
from ml_dtypes import bfloat16

from helpers import BS, bits, to_numpy, to_torch
from oracle import kv_cache_ref as R
from oracle import norm_rope_ref as N

pytestmark = pytest.mark.gpu


def _ulp_diff(a, b):
    """Distance in bf16 steps between two bf16 arrays (sign-magnitude bit patterns made monotonic)."""
    def key(x):
        u = bits(x).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(a) - key(b))


def _case(seed, rows, cols, nb, hq=8, hkv=2, d=256, max_pos=4000):
    rng = np.random.default_rng(seed)
    qg = (rng.standard_normal((rows, cols, hq, 2 * d), dtype=np.float32) * 1.7).astype(bfloat16)  # query|gate projection
    k = (rng.standard_normal((rows, cols, hkv, d), dtype=np.float32) * 0.6).astype(bfloat16)
    v = rng.standard_normal((rows, cols, hkv, d), dtype=np.float32).astype(bfloat16)
    qw = (rng.standard_normal(d, dtype=np.float32) * 0.2).astype(bfloat16)
    kw = (rng.standard_normal(d, dtype=np.float32) * 0.2).astype(bfloat16)
    pos = rng.integers(0, max_pos, size=(rows, cols)).astype(np.int32)
    slots = rng.permutation(nb * BS)[: rows * cols].reshape(rows, cols).astype(np.int32)
    kc = rng.standard_normal((1, nb, BS, hkv, d), dtype=np.float32).astype(bfloat16)
    vc = rng.standard_normal((1, nb, BS, hkv, d), dtype=np.float32).astype(bfloat16)
    return dict(qg=qg, k=k, v=v, qw=qw, kw=kw, pos=pos, slots=slots, kc=kc, vc=vc, d=d)


@pytest.mark.parametrize("rows,cols,d,rot", [(37, 1, 256, 64), (1, 300, 256, 64), (5, 9, 128, 32), (3, 4, 64, 64)])
def test_fused_norm_rope_append_matches_the_oracle(rows, cols, d, rot):
    from nano_vllm_jax_b200.kernels import paged_kv as K
    c = _case(rows * 7 + cols, rows, cols, 64, d=d, max_pos=40000)
    q_view = c["qg"][..., :d]  # the query half of the projection: a strided view, as in the model
    ref_q, ref_k, ref_v = N.qk_norm_rope_kv_append(q_view, c["k"], c["v"], c["qw"], c["kw"], c["pos"], c["slots"],
                                                   c["kc"], c["vc"], partial_rotary_factor=rot / d)
    t_qg = to_torch(c["qg"])
    kc, vc = to_torch(c["kc"]), to_torch(c["vc"])
    q_out, _, _ = K.qk_norm_rope_kv_append(t_qg[..., :d], to_torch(c["k"]), to_torch(c["v"]), to_torch(c["qw"]), to_torch(c["kw"]),
                                           to_torch(c["pos"]), to_torch(c["slots"]), kc[0], vc[0], rotary_dim=rot)
    torch.cuda.synchronize()
    # V rows are copies: bit-exact, and nothing but the addressed slots changed
    np.testing.assert_array_equal(bits(to_numpy(vc)), bits(ref_v))
    # K and q: the same roundings as the oracle up to the last bf16 step where a sum of squares or a cosine differs in its last fp32 bit
    # K and q: the same roundings as the oracle except where a sum of squares, a cosine or a sine differs in its last
    # fp32 bit and flips a bf16 rounding: rare, and then one bf16 step of the operands (a rotated element that nearly
    # cancels is many steps of ITSELF away, so the bound is taken against the head row's magnitude)
    for name, got, want in (("q", to_numpy(q_out), ref_q), ("k cache", to_numpy(kc), ref_k)):
        g, w = got.astype(np.float32), want.astype(np.float32)
        bound = 2.0 ** -7 * np.abs(w).max(axis=-1, keepdims=True)
        assert (np.abs(g - w) <= bound).all(), f"{name}: {np.abs(g - w).max()} apart"
        differ = (_ulp_diff(got, want) > 0).mean()
        assert differ < 2e-3, f"{name}: {differ:.2e} of the elements differ"


def test_fused_equals_unfused_route_for_attention():
    # q', cache from the fused kernel feed the decode kernel exactly like norm -> rope -> append done on the host
    from nano_vllm_jax_b200.kernels import paged_kv as K
    c = _case(11, 16, 1, 128)
    pos = np.arange(100, 116, dtype=np.int32).reshape(16, 1)
    tables = np.arange(16 * 8, dtype=np.int32).reshape(16, 8)
    slots = R.compute_slot_mapping(pos, tables, BS)
    ref_q, ref_k, ref_v = N.qk_norm_rope_kv_append(c["qg"][..., :256], c["k"], c["v"], c["qw"], c["kw"], pos, slots, c["kc"], c["vc"])
    kc, vc = to_torch(c["kc"]), to_torch(c["vc"])
    q_out, _, _ = K.qk_norm_rope_kv_append(to_torch(c["qg"])[..., :256], to_torch(c["k"]), to_torch(c["v"]), to_torch(c["qw"]),
                                           to_torch(c["kw"]), to_torch(pos), to_torch(slots), kc[0], vc[0])
    lens = (pos[:, 0] + 1).astype(np.int32)
    out = K.paged_decode_attention(q_out[:, 0], kc[0], vc[0], to_torch(tables), to_torch(lens), 0.0625)
    want = R.paged_attention_decode(ref_q, ref_k, ref_v, tables, lens, BS, 0.0625, 4)
    torch.cuda.synchronize()
    assert np.abs(to_numpy(out).reshape(want.shape) - want).max() <= 2e-3


def test_masked_and_padded_tokens_write_nothing():
    from nano_vllm_jax_b200.kernels import paged_kv as K
    c = _case(5, 1, 40, 32)
    qsl = np.array([0, 17, 29], np.int32)  # tokens 29.. are padding
    valid = R.write_kv_valid_mask(c["slots"].shape, qsl, True)
    _, ref_k, ref_v = N.qk_norm_rope_kv_append(c["qg"][..., :256], c["k"], c["v"], c["qw"], c["kw"], c["pos"], c["slots"],
                                               c["kc"], c["vc"], valid_mask=valid)
    kc, vc = to_torch(c["kc"]), to_torch(c["vc"])
    K.qk_norm_rope_kv_append(to_torch(c["qg"])[..., :256], to_torch(c["k"]), to_torch(c["v"]), to_torch(c["qw"]), to_torch(c["kw"]),
                             to_torch(c["pos"]), to_torch(c["slots"]), kc[0], vc[0], query_start_loc=to_torch(qsl), packed=True)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(bits(to_numpy(vc)), bits(ref_v))
    assert (_ulp_diff(to_numpy(kc), ref_k) > 0).mean() < 2e-3


def test_unsupported_shapes_are_refused():
    from nano_vllm_jax_b200._lib import NvjError
    from nano_vllm_jax_b200.kernels import paged_kv as K
    c = _case(1, 2, 1, 8, d=256)
    kc = to_torch(c["kc"]).float()
    with pytest.raises(NvjError):  # fp32 cache
        K.qk_norm_rope_kv_append(to_torch(c["qg"])[..., :256], to_torch(c["k"]), to_torch(c["v"]), to_torch(c["qw"]), to_torch(c["kw"]),
                                 to_torch(c["pos"]), to_torch(c["slots"]), kc[0], kc[0].clone())


@pytest.mark.parametrize("rows,cols", [(23, 1), (1, 130)])
def test_multimodal_three_row_positions(rows, cols):
    """Temporal, height and width rows that differ: frequency i takes the row layers.py:79-139 gives it (sections
    11 / 11 / 10); three equal rows reproduce the text result bit for bit."""
    from nano_vllm_jax_b200.kernels import paged_kv as K
    c = _case(rows + cols, rows, cols, 64, max_pos=3000)
    rng = np.random.default_rng(99)
    pos3 = np.stack([c["pos"], rng.integers(0, 64, size=c["pos"].shape), rng.integers(0, 64, size=c["pos"].shape)]).astype(np.int32)
    q_view = c["qg"][..., :256]
    ref_q, ref_k, ref_v = N.qk_norm_rope_kv_append(q_view, c["k"], c["v"], c["qw"], c["kw"], pos3, c["slots"], c["kc"], c["vc"],
                                                   mrope_section=(11, 11, 10))
    text_q, _, _ = N.qk_norm_rope_kv_append(q_view, c["k"], c["v"], c["qw"], c["kw"], c["pos"], c["slots"], c["kc"], c["vc"])
    assert (_ulp_diff(ref_q, text_q) > 0).mean() > 0.05      # the rows really matter in this case
    kc, vc = to_torch(c["kc"]), to_torch(c["vc"])
    args = (to_torch(c["qg"])[..., :256], to_torch(c["k"]), to_torch(c["v"]), to_torch(c["qw"]), to_torch(c["kw"]))
    q_out, _, _ = K.qk_norm_rope_kv_append(*args, to_torch(pos3), to_torch(c["slots"]), kc[0], vc[0], mrope_section=(11, 11, 10))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(bits(to_numpy(vc)), bits(ref_v))
    for name, got, want in (("q", to_numpy(q_out), ref_q), ("k cache", to_numpy(kc), ref_k)):
        g, w = got.astype(np.float32), want.astype(np.float32)
        assert (np.abs(g - w) <= 2.0 ** -7 * np.abs(w).max(axis=-1, keepdims=True)).all(), name
        assert (_ulp_diff(got, want) > 0).mean() < 2e-3, name
    # three equal rows == one row
    kc1, vc1, kc3, vc3 = to_torch(c["kc"]), to_torch(c["vc"]), to_torch(c["kc"]), to_torch(c["vc"])
    q1, _, _ = K.qk_norm_rope_kv_append(*args, to_torch(c["pos"]), to_torch(c["slots"]), kc1[0], vc1[0])
    q3, _, _ = K.qk_norm_rope_kv_append(*args, to_torch(np.stack([c["pos"]] * 3)), to_torch(c["slots"]), kc3[0], vc3[0])
    torch.cuda.synchronize()
    assert torch.equal(q1, q3) and torch.equal(kc1, kc3) and torch.equal(vc1, vc3)
