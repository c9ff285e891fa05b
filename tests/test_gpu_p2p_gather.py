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


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ranks_on_separate_gpus_agree_with_the_library_gather():
    n = min(torch.cuda.device_count(), 4)
    worker = os.path.join(os.path.dirname(__file__), "p2p_gather_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29531", worker],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "P2P_GATHER_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
