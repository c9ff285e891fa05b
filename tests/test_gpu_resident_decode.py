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
