"""The decode entry point that allocates nothing (workspace inside the library image).

Collected last on purpose: if it fails, a run that stops at the first failure has
already run every other test.  It must pass alone in a fresh process and after
the rest of the suite, so it makes no assumption about what ran before it.

Who needs this: a caller that cannot allocate device memory during a step, such
as a custom-call handler that is handed only its operands and results, or a
plugin living inside another runtime's memory pool, has no place to keep the
workspace `nvj_paged_decode` wants.  `nvj_paged_decode_static_scratch` takes that
workspace from a fixed array in the library, shared by all calls on a device.
"""

import numpy as np
import pytest
import torch

from helpers import BS, SCALE, decode_case, to_numpy, to_torch
from oracle import kv_cache_ref as R

pytestmark = pytest.mark.gpu

TIGHT = 2e-3  # the regression bound the other decode tests use (contract: 2e-2)


def _inputs(c):
    return (to_torch(c["q"][:, 0]).contiguous(), to_torch(c["k_cache"][0]), to_torch(c["v_cache"][0]),
            to_torch(c["tables"]), to_torch(c["seq_lens"]))


def test_no_alloc_decode_matches_the_workspace_entry_point_twice_in_a_row():
    from nano_vllm_jax_b200.kernels import paged_kv as K
    # rows short enough to live in one CTA, rows long enough to be merged across CTAs, one empty row
    cases = [decode_case(21, 1500, 24, 1, 900, empty_rows=(3,)), decode_case(22, 600, 3, 2500, 3000)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for c in cases:  # two different calls back to back share the one scratch array
        q, k, v, tables, lens = _inputs(c)
        want = K.paged_decode_attention(q, k, v, tables, lens, SCALE)            # existing entry point
        oracle = R.paged_attention_decode(c["q"], c["k_cache"], c["v_cache"], c["tables"], c["seq_lens"], BS, SCALE, 4)
        oracle = oracle.reshape(len(c["seq_lens"]), 8, 256)                       # and the CPU restatement of the reference
        active = c["seq_lens"] > 0
        for _ in range(2):                                                        # and the same call twice
            out = torch.full_like(want, float("nan"))
            got = K.paged_decode_attention_no_alloc(q, k, v, tables, lens, SCALE, out, status_out=status)
            torch.cuda.synchronize()
            assert got is out
            assert int(status.item()) == 0
            assert not torch.isnan(out).any()
            assert float((out - want).abs().max()) <= TIGHT
            assert np.abs(to_numpy(out)[active] - oracle[active]).max() <= TIGHT
            assert not out[lens == 0].any()


def test_no_alloc_decode_generic_shapes_and_flagged_call_leaves_scratch_usable():
    from nano_vllm_jax_b200.kernels import paged_kv as K
    rng = np.random.default_rng(23)
    k = to_torch(rng.standard_normal((6, 4, 2, 8)).astype(np.float32))
    v = to_torch(rng.standard_normal((6, 4, 2, 8)).astype(np.float32))
    q = to_torch(rng.standard_normal((2, 4, 8)).astype(np.float32))
    tables = to_torch(np.array([[3, 1, 5], [2, 4, 0]], np.int32))
    lens = to_torch(np.array([7, 10], np.int32))
    want = K.paged_decode_attention(q, k, v, tables, lens, 0.35)
    out = torch.empty_like(want)
    K.paged_decode_attention_no_alloc(q, k, v, tables, lens, 0.35, out)
    torch.cuda.synchronize()
    assert float((out - want).abs().max()) <= 1e-5
    ref = R.paged_attention_decode(to_numpy(q)[:, None], to_numpy(k)[None], to_numpy(v)[None], to_numpy(tables),
                                   to_numpy(lens), 4, 0.35, 2).reshape(2, 4, 8)
    assert np.abs(to_numpy(out) - ref).max() <= 1e-5
    # a block id outside the pool is skipped and reported through status_out; the next call is clean
    c = decode_case(24, 64, 2, 30, 60)
    qq, kk, vv, tt, ll = _inputs(c)
    bad = tt.clone()
    bad[1, 1] = 64
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o = torch.empty((2, 8, 256), dtype=torch.float32, device="cuda")
    K.paged_decode_attention_no_alloc(qq, kk, vv, bad, ll, SCALE, o, status_out=status)
    torch.cuda.synchronize()
    assert int(status.item()) & 2
    K.paged_decode_attention_no_alloc(qq, kk, vv, tt, ll, SCALE, o, status_out=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert float((o - K.paged_decode_attention(qq, kk, vv, tt, ll, SCALE)).abs().max()) <= TIGHT
    ref = R.paged_attention_decode(c["q"], c["k_cache"], c["v_cache"], c["tables"], c["seq_lens"], BS, SCALE, 4)
    assert np.abs(to_numpy(o).reshape(2, -1) - ref[:, 0]).max() <= TIGHT


def test_no_alloc_decode_rejects_batches_beyond_the_built_in_limit():
    from nano_vllm_jax_b200 import _lib
    from nano_vllm_jax_b200.kernels import paged_kv as K
    n = K.STATIC_SCRATCH_MAX_BATCH + 1
    q = torch.zeros((n, 8, 256), dtype=torch.bfloat16, device="cuda")
    k = torch.zeros((4, BS, 2, 256), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((n, 8, 256), dtype=torch.float32, device="cuda")
    tables = torch.zeros((n, 1), dtype=torch.int32, device="cuda")
    lens = torch.zeros(n, dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.NvjError, match="built-in limit"):
        K.paged_decode_attention_no_alloc(q, k, k.clone(), tables, lens, SCALE, out)


def test_no_alloc_decode_rejects_operands_it_would_have_to_copy_or_cannot_trust():
    """The wrapper converts nothing: an operand of the wrong dtype, shape, layout or device is an error, never a copy
    (and never an out-of-bounds access on the device)."""
    from nano_vllm_jax_b200.kernels import paged_kv as K
    c = decode_case(25, 64, 3, 30, 60)
    q, k, v, tables, lens = _inputs(c)
    out = torch.empty((3, 8, 256), dtype=torch.float32, device="cuda")
    ok_status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def call(**kw):
        a = dict(q=q, k=k, v=v, tables=tables, lens=lens, out=out, status=ok_status)
        a.update(kw)
        return K.paged_decode_attention_no_alloc(a["q"], a["k"], a["v"], a["tables"], a["lens"], SCALE, a["out"],
                                                 status_out=a["status"])

    call()  # the unmodified operands are accepted
    bad = [
        dict(q=q[:, :, :128].contiguous()),                        # head_dim differs from the cache's
        dict(lens=lens[:2]),                                       # seq_lens shorter than the batch
        dict(lens=lens.to(torch.int64)),                           # would need a conversion
        dict(tables=tables.to(torch.int64)),
        dict(tables=tables.t().contiguous().t()),                  # non-contiguous table
        dict(lens=torch.stack([lens, lens], 1)[:, 0]),             # non-contiguous lengths
        dict(status=torch.zeros(1, dtype=torch.int32)),            # status word on the host
        dict(status=torch.zeros(1, dtype=torch.int64, device="cuda")),
        dict(status=torch.zeros(0, dtype=torch.int32, device="cuda")),
        dict(q=q.to(torch.float64)),
        dict(out=out.to(torch.float16)),
        dict(q=q.transpose(0, 1).contiguous().transpose(0, 1)),    # non-contiguous q
    ]
    for kw in bad:
        with pytest.raises(ValueError):
            call(**kw)
    torch.cuda.synchronize()
    call()
    torch.cuda.synchronize()
    assert int(ok_status.item()) == 0
