"""Token all-gather by NVLink peer stores: one rank alone, and one process per GPU where the box has several."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_single_rank_gather_is_a_copy():
    from nano_vllm_jax_b200.parallel import P2PTokenGather
    g = P2PTokenGather(37)
    assert (g.rank, g.world) == (0, 1)
    for step in range(5):
        tok = torch.arange(37, dtype=torch.int32, device="cuda") * 3 + step
        assert torch.equal(g.gather(tok), tok)
    g.check()
    with pytest.raises(ValueError):
        g.gather(torch.zeros(36, dtype=torch.int32, device="cuda"))
    g.close()


def test_split_form_publishes_with_the_token_pick_and_collects_one_step_later():
    from nano_vllm_jax_b200.kernels import paged_kv as K
    from nano_vllm_jax_b200.parallel import P2PTokenGather
    n, row_len = 53, 2048
    g = P2PTokenGather(n)
    gen = torch.Generator(device="cuda").manual_seed(5)
    out = torch.full((n,), -7, dtype=torch.int32, device="cuda")
    g.collect(out=out)                                      # nothing published yet: a no-op
    torch.cuda.synchronize()
    assert int(out.min()) == -7 and int(out.max()) == -7
    prev = None
    for step in range(6):
        x = torch.randn((n, row_len), generator=gen, device="cuda")
        x[step, 100] = float("inf")                         # a known winner in one row
        g.collect(out=out)                                  # the step before (if any)
        torch.cuda.synchronize()
        if prev is not None:
            assert torch.equal(out, prev)
        tok = g.publish_argmax(x)
        assert torch.equal(tok, K.row_argmax(x)) and int(tok[step]) == 100
        assert torch.equal(tok.long(), x.argmax(dim=1))
        prev = tok.clone()
    g.collect(out=out)
    g.collect(out=out)                                      # a second collect of the same step changes nothing
    torch.cuda.synchronize()
    assert torch.equal(out, prev)
    # the fused form: one launch collects the step before and publishes this one
    for step in range(4):
        x = torch.randn((n, row_len), generator=gen, device="cuda")
        out.fill_(-7)
        tok = g.publish_argmax(x, collect_out=out)
        torch.cuda.synchronize()
        assert torch.equal(tok.long(), x.argmax(dim=1))
        if step == 0:
            assert int(out.max()) == -7                     # everything published before had been collected
        else:
            assert torch.equal(out, prev)
        prev = tok.clone()
    g.collect(out=out)
    torch.cuda.synchronize()
    assert torch.equal(out, prev)
    g.check()
    g.close()


def _two_rank_buffers_on_one_gpu(n):
    """Exchange buffers of a 2-rank gather that both live on this GPU (no peer process): what a rank sees when its
    peer never shows up."""
    import ctypes

    from nano_vllm_jax_b200 import _lib
    lib = _lib.load()
    nbytes = int(lib.nvj_p2p_gather_buffer_bytes(2, n))
    bufs = []
    for _ in range(2):
        ptr, handle = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
        _lib.check(lib.nvj_p2p_buffer_create(nbytes, ctypes.byref(ptr), handle), "nvj_p2p_buffer_create")
        bufs.append(ptr.value)
    return lib, bufs, (ctypes.c_void_p * 2)(*bufs)


def test_a_peer_that_never_publishes_runs_the_wait_out_and_the_gather_recovers():
    """Failure detection without a fault: rank 1 is simply never launched.  Rank 0's kernel gives up after the wait
    limit, flags NVJ_DEV_TIMEOUT and returns; the context stays usable and the same step succeeds once the peer has
    published.  Kernels that wait for one another are never in flight together here: each launch is synchronised
    before the next, and every wait but the first is already satisfied when its kernel starts."""
    from nano_vllm_jax_b200 import _lib
    n = 16
    lib, bufs, ptrs = _two_rank_buffers_on_one_gpu(n)
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tok0 = torch.arange(n, dtype=torch.int32, device="cuda") + 100
    tok1 = torch.arange(n, dtype=torch.int32, device="cuda") + 200
    out0 = torch.full((2 * n,), -1, dtype=torch.int32, device="cuda")
    out1 = torch.full((2 * n,), -1, dtype=torch.int32, device="cuda")
    assert lib.nvj_get_wait_limit_ns() == 1_000_000_000
    lib.nvj_set_wait_limit_ns(2_000_000)  # 2 ms
    try:
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        _lib.check(lib.nvj_p2p_allgather_i32(tok0.data_ptr(), n, 0, 2, ptrs, 1, out0.data_ptr(), status.data_ptr(), stream), "rank 0")
        t1.record()
        torch.cuda.synchronize()
        assert int(status.item()) == _lib.NVJ_DEV_TIMEOUT
        assert 1.5 <= t0.elapsed_time(t1) < 200.0           # it waited for the limit, not for the default second
        assert int(out0[n:].max()) == -1                     # nothing of the silent peer was delivered
        status.zero_()
        # the peer arrives: its own wait is satisfied at once (rank 0 has published epoch 1 already)
        _lib.check(lib.nvj_p2p_allgather_i32(tok1.data_ptr(), n, 1, 2, ptrs, 1, out1.data_ptr(), status.data_ptr(), stream), "rank 1")
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and torch.equal(out1, torch.cat([tok0, tok1]))
        # rank 0 issues the same step again and now completes
        _lib.check(lib.nvj_p2p_allgather_i32(tok0.data_ptr(), n, 0, 2, ptrs, 1, out0.data_ptr(), status.data_ptr(), stream), "rank 0 again")
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and torch.equal(out0, torch.cat([tok0, tok1]))
        # split form: rank 0 publishes, its collect runs out (rank 1 silent), nothing is consumed; after rank 1's
        # publish the same collect delivers
        lib2, bufs2, ptrs2 = _two_rank_buffers_on_one_gpu(n)
        x0 = torch.zeros((n, 8), device="cuda"); x0[:, 3] = 1.0
        x1 = torch.zeros((n, 8), device="cuda"); x1[:, 5] = 1.0
        t = torch.empty(n, dtype=torch.int32, device="cuda")
        got = torch.full((2 * n,), -1, dtype=torch.int32, device="cuda")
        _lib.check(lib.nvj_p2p_argmax_publish(x0.data_ptr(), n, 8, t.data_ptr(), 0, 2, ptrs2, None, None, None, 0, 1, status.data_ptr(), stream), "publish 0")
        _lib.check(lib.nvj_p2p_collect(bufs2[0], n, 2, got.data_ptr(), status.data_ptr(), stream), "collect 0")
        torch.cuda.synchronize()
        assert int(status.item()) == _lib.NVJ_DEV_TIMEOUT and int(got[n:].max()) == -1
        status.zero_()
        _lib.check(lib.nvj_p2p_argmax_publish(x1.data_ptr(), n, 8, t.data_ptr(), 1, 2, ptrs2, None, None, None, 0, 1, status.data_ptr(), stream), "publish 1")
        _lib.check(lib.nvj_p2p_collect(bufs2[0], n, 2, got.data_ptr(), status.data_ptr(), stream), "collect 0 again")
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(got, torch.cat([torch.full((n,), 3, dtype=torch.int32, device="cuda"),
                                           torch.full((n,), 5, dtype=torch.int32, device="cuda")]))
        for b in bufs + bufs2:
            lib.nvj_p2p_buffer_destroy(b)
    finally:
        lib.nvj_set_wait_limit_ns(0)
    assert lib.nvj_get_wait_limit_ns() == 1_000_000_000


def test_bounded_mbarrier_wait_runs_out_and_every_thread_returns():
    """The wait the pipelined kernels use on their copies, on a barrier nobody arrives on: after the limit the first
    waiter flags the status word, the others see the CTA's abort flag, all 64 threads return."""
    from nano_vllm_jax_b200 import _lib
    lib = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    returned = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.nvj_set_wait_limit_ns(3_000_000)
    try:
        _lib.check(lib.nvj_selftest_bounded_wait(status.data_ptr(), returned.data_ptr(), torch.cuda.current_stream().cuda_stream),
                   "nvj_selftest_bounded_wait")
        torch.cuda.synchronize()
    finally:
        lib.nvj_set_wait_limit_ns(0)
    assert int(status.item()) == _lib.NVJ_DEV_TIMEOUT and int(returned.item()) == 64
    # the context is intact: an ordinary kernel of the library runs afterwards
    from nano_vllm_jax_b200.kernels import paged_kv as K
    x = torch.eye(4, device="cuda")
    assert K.row_argmax(x).tolist() == [0, 1, 2, 3]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ranks_on_separate_gpus_agree_with_the_library_gather():
    n = min(torch.cuda.device_count(), 4)
    worker = os.path.join(os.path.dirname(__file__), "p2p_gather_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29531", worker],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "P2P_GATHER_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
    print("\n".join(line for line in r.stdout.splitlines() if line.startswith("TIMING")))
