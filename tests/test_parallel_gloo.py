"""Request partition + token gather with two CPU ranks on the gloo backend."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nano_vllm_jax_b200 import parallel


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, num_requests, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ids = parallel.local_request_ids(num_requests, rank, world)
    local = torch.tensor([1000 + i for i in ids], dtype=torch.int32)  # token of request i is 1000 + i
    for _ in range(3):  # several steps reuse the same fixed-size collective
        full = parallel.gather_tokens(local, num_requests)
    torch.save(full, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.destroy_process_group()


def test_partition_is_round_robin_and_complete():
    assert parallel.local_request_ids(7, 0, 2) == [0, 2, 4, 6]
    assert parallel.local_request_ids(7, 1, 2) == [1, 3, 5]
    assert parallel.max_local_rows(7, 2) == 4
    owned = sorted(i for r in range(8) for i in parallel.local_request_ids(2048, r, 8))
    assert owned == list(range(2048))
    assert all(parallel.owner_rank(i, 8) == i % 8 for i in range(64))


def test_two_rank_gather_restores_global_request_order(tmp_path):
    world, n = 2, 7  # uneven split: rank 1 pads its last row
    mp.spawn(_worker, args=(world, _free_port(), n, str(tmp_path)), nprocs=world, join=True)
    want = torch.tensor([1000 + i for i in range(n)], dtype=torch.int32)
    for r in range(world):
        assert torch.equal(torch.load(os.path.join(tmp_path, f"rank{r}.pt")), want)


def test_single_process_gather_is_identity():
    t = torch.arange(5, dtype=torch.int32)
    assert torch.equal(parallel.gather_tokens(t, 5), t)


def _leaver(rank, world, port, out_dir):
    """Rank 1 leaves between two steps (no collective in flight); rank 0's next gather must end with an error after
    the process group's timeout instead of waiting for ever."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    local = torch.tensor([rank], dtype=torch.int32)
    parallel.gather_tokens(local, world)  # one healthy step
    if rank == 1:
        os._exit(0)  # gone, without a goodbye
    try:
        parallel.gather_tokens(local, world)
        verdict = "no error"
    except parallel.TokenGatherError as exc:
        verdict = "TokenGatherError: " + str(exc)[:80]
    with open(os.path.join(out_dir, "verdict.txt"), "w") as f:
        f.write(verdict)
    os._exit(0)  # the group cannot be torn down collectively any more


def test_a_rank_that_leaves_between_steps_ends_the_next_gather_with_an_error(tmp_path):
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_leaver, args=(r, 2, port, str(tmp_path))) for port in [_free_port()] for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=60)
        assert not p.is_alive(), "a rank is still waiting: the gather did not time out"
    verdict = (tmp_path / "verdict.txt").read_text()
    assert verdict.startswith("TokenGatherError"), verdict
