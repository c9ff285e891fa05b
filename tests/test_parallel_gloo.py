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
