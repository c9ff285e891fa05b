"""Device-resident decode metadata and the decode step replayed from a CUDA graph: equal to eager steps bit for bit,
and to the CPU oracle's append + paged attention step by step."""

import numpy as np
import pytest
import torch

from helpers import BS, SCALE, bits, decode_case, to_numpy, to_torch
from oracle import kv_cache_ref as R

pytestmark = pytest.mark.gpu


def test_advance_kernel_matches_the_scheduler_rule_and_flags_overflow():
    from nano_vllm_jax_b200.engine.resident_decode import ResidentDecodeMetadata
    from nano_vllm_jax_b200.kernels.paged_kv import DeviceStatusError
    meta = ResidentDecodeMetadata(rows=6, table_width=2, block_size=16)
    meta.load(np.zeros((5, 2), np.int32), np.array([0, 1, 15, 16, 30], np.int32))
    meta.advance()
    # active rows: position = old length, length + 1; inactive rows (0) untouched (scheduler.py:790-803, 864-870)
    assert meta.seq_lens.tolist() == [0, 2, 16, 17, 31, 0]
    assert meta.positions.view(-1).tolist() == [0, 1, 15, 16, 30, 0]
    meta.advance()
    meta.check()
    assert meta.seq_lens.tolist() == [0, 3, 17, 18, 32, 0]
    meta.advance()  # row 4 would need a 33rd token in a 32-token table
    assert meta.seq_lens.tolist() == [0, 4, 18, 19, 32, 0]
    with pytest.raises(DeviceStatusError):
        meta.check()


def test_graph_replayed_steps_equal_eager_steps():
    from nano_vllm_jax_b200.backends import B200Backend
    from nano_vllm_jax_b200.engine.resident_decode import DecodeStepGraph, ResidentDecodeMetadata
    from nano_vllm_jax_b200.kernels import paged_kv as K
    from nano_vllm_jax_b200.kv_cache import KVCacheStorage

    steps, rows = 6, 20
    c = decode_case(41, 2048, rows, 200, 700, empty_rows=(3,))  # tables cover the lengths of the LAST step
    lens0 = np.where(c["seq_lens"] > 0, c["seq_lens"] - steps, 0).astype(np.int32)  # lengths before the first step
    k_g, v_g = to_torch(c["k_cache"]), to_torch(c["v_cache"])
    k_e, v_e = k_g.clone(), v_g.clone()
    rng = np.random.default_rng(9)
    qs = [to_torch(rng.standard_normal((rows, 1, 8, 256), dtype=np.float32)).to(torch.bfloat16) for _ in range(steps)]
    ks = [to_torch(rng.standard_normal((rows, 1, 2, 256), dtype=np.float32)).to(torch.bfloat16) for _ in range(steps)]
    vs = [to_torch(rng.standard_normal((rows, 1, 2, 256), dtype=np.float32)).to(torch.bfloat16) for _ in range(steps)]

    meta = ResidentDecodeMetadata(rows, c["tables"].shape[1], BS)
    meta.load(c["tables"], lens0)
    g = DecodeStepGraph(meta, k_g, v_g, 0, SCALE, 4)
    got = []
    for s in range(steps):
        g.query.copy_(qs[s]); g.new_k.copy_(ks[s]); g.new_v.copy_(vs[s])
        out, tok = g.capture() if s == 0 else g.replay()
        got.append((out.clone(), tok.clone()))
    torch.cuda.synchronize()
    meta.check()
    assert meta.seq_lens.cpu().numpy().tolist() == np.where(lens0 > 0, lens0 + steps, 0).tolist()

    backend = B200Backend()
    cache = KVCacheStorage(k_e, v_e)
    tables = to_torch(c["tables"])
    for s in range(steps):
        lens = torch.from_numpy(np.where(lens0 > 0, lens0 + s + 1, 0).astype(np.int32)).cuda()
        pos = (lens - 1).clamp(min=0).view(rows, 1)
        md = backend.build_attention_metadata(pos, tables, lens, BS, False)
        _, ref = backend.write_kv_and_attention(0, qs[s], ks[s], vs[s], cache, md, BS, SCALE, 4, False)
        active = (lens > 0).cpu().numpy()
        assert torch.equal(got[s][0][active], ref[active]), f"step {s}: graph output differs from the eager step"
        assert torch.equal(got[s][1][active], K.row_argmax(ref.view(rows, -1))[active])
    np.testing.assert_array_equal(bits(to_numpy(k_g)), bits(to_numpy(k_e)))
    np.testing.assert_array_equal(bits(to_numpy(v_g)), bits(to_numpy(v_e)))

    # the same steps in the CPU oracle: slot mapping -> masked append -> paged attention (the reference's pure path)
    ok, ov = c["k_cache"], c["v_cache"]
    for s in range(steps):
        lens = np.where(lens0 > 0, lens0 + s + 1, 0).astype(np.int32)
        pos = np.maximum(lens - 1, 0)[:, None]
        slots = R.compute_slot_mapping(pos, c["tables"], BS)
        ok, ov = R.update_kv_cache(ok, ov, slots, to_numpy(ks[s]), to_numpy(vs[s]), 0, valid_mask=(lens > 0)[:, None])
        ref = R.paged_attention_decode(to_numpy(qs[s]), ok, ov, c["tables"], lens, BS, SCALE, 4)
        active = lens > 0
        err = np.abs(to_numpy(got[s][0])[active] - ref[active]).max()
        assert err <= 2e-3, f"step {s}: graph output vs oracle max-abs {err}"
        assert not to_numpy(got[s][0])[~active].any()
    np.testing.assert_array_equal(bits(to_numpy(k_g)), bits(ok))
    np.testing.assert_array_equal(bits(to_numpy(v_g)), bits(ov))


@pytest.mark.parametrize("variant,dtype", [(3, "bf16"), (2, "bf16"), (1, "bf16"), (1, "f32")])
def test_pre_append_form_equals_the_form_with_positions(variant, dtype):
    """positions=None: the token goes to position seq_lens[b] and seq_lens[b] + 1 keys are attended, bit for bit what
    the call with (positions = old length, seq_lens = old length + 1) does; inactive rows stay inactive."""
    from nano_vllm_jax_b200.kernels import paged_kv as K
    rows = 24
    c = decode_case(77, 2048, rows, 40, 600, empty_rows=(5,))
    td = torch.float32 if dtype == "f32" else torch.bfloat16
    after = c["seq_lens"].astype(np.int32)
    before = np.where(after > 0, after - 1, 0).astype(np.int32)
    rng = np.random.default_rng(3)
    q = to_torch(rng.standard_normal((rows, 1, 8, 256), dtype=np.float32)).to(td)
    nk = to_torch(rng.standard_normal((rows, 1, 2, 256), dtype=np.float32)).to(td)
    nv = to_torch(rng.standard_normal((rows, 1, 2, 256), dtype=np.float32)).to(td)
    tables = to_torch(c["tables"])
    k_a, v_a = to_torch(c["k_cache"]).to(td), to_torch(c["v_cache"]).to(td)
    k_b, v_b = k_a.clone(), v_a.clone()
    ref, _, _ = K.paged_decode_attention_with_kv_append(q, nk, nv, k_a, v_a, tables, torch.from_numpy(after).cuda(),
                                                        torch.from_numpy(before).cuda().view(rows, 1), 0, BS, SCALE, 4,
                                                        variant=variant)
    got, _, _ = K.paged_decode_attention_with_kv_append(q, nk, nv, k_b, v_b, tables, torch.from_numpy(before).cuda(),
                                                        None, 0, BS, SCALE, 4, variant=variant)
    torch.cuda.synchronize()
    assert torch.equal(got, ref)
    assert torch.equal(k_a.view(torch.uint8), k_b.view(torch.uint8)) and torch.equal(v_a.view(torch.uint8), v_b.view(torch.uint8))
    assert not got[5].any()


def test_pre_append_form_flags_a_row_without_room():
    from nano_vllm_jax_b200.kernels import paged_kv as K
    k = torch.zeros((1, 8, BS, 2, 256), dtype=torch.bfloat16, device="cuda")
    v = torch.zeros_like(k)
    q = torch.ones((2, 1, 8, 256), dtype=torch.bfloat16, device="cuda")
    n = torch.ones((2, 1, 2, 256), dtype=torch.bfloat16, device="cuda")
    tables = torch.tensor([[1, 2], [3, 4]], dtype=torch.int32, device="cuda")
    lens = torch.tensor([2 * BS, 5], dtype=torch.int32, device="cuda")  # row 0 is full: no place for a 33rd token
    with pytest.raises(K.DeviceStatusError):
        K.paged_decode_attention_with_kv_append(q, n, n, k, v, tables, lens, None, 0, BS, SCALE, 4)
    assert not k[0, 1:3].any() and k[0, 3, 5].any()  # the full row wrote nothing, the other row appended at 5


def test_token_pick_with_advance_is_pick_plus_advance():
    from nano_vllm_jax_b200.engine.resident_decode import ResidentDecodeMetadata
    from nano_vllm_jax_b200.kernels import paged_kv as K
    x = torch.randn((6, 2048), device="cuda")
    meta = ResidentDecodeMetadata(rows=6, table_width=2, block_size=16)
    meta.load(np.zeros((5, 2), np.int32), np.array([0, 1, 15, 16, 31], np.int32))
    tok = K.row_argmax(x, advance=(meta.seq_lens, meta.positions, 2, 16))
    assert torch.equal(tok, x.argmax(dim=1).to(torch.int32))
    assert meta.seq_lens.tolist() == [0, 2, 16, 17, 32, 0]
    assert meta.positions.view(-1).tolist() == [0, 1, 15, 16, 31, 0]
    with pytest.raises(K.DeviceStatusError):  # row 4 is full now
        K.row_argmax(x, advance=(meta.seq_lens, None, 2, 16))
    assert meta.seq_lens.tolist() == [0, 3, 17, 18, 32, 0]
