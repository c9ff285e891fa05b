"""Worker of tests/test_gpu_p2p_gather.py: one process per GPU under torch.distributed.run."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nano_vllm_jax_b200.parallel import P2PTokenGather  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    n, steps = 256, 60
    g = P2PTokenGather(n)
    ref = torch.empty(world * n, dtype=torch.int32, device=dev)
    base = torch.arange(n, dtype=torch.int32, device=dev)
    for s in range(steps):
        tok = base + (rank * 100_000 + s * 1000)
        if s % 7 == rank % 7:
            torch.cuda._sleep(2_000_000)  # ranks drift apart: a late peer must be waited for, an early one must not overwrite
        out = g.gather(tok)
        dist.all_gather_into_tensor(ref, tok)
        assert torch.equal(out, ref), f"rank {rank} step {s}: peer-store gather differs from the NCCL gather"
    g.check()
    # split form on a second set of buffers: the token pick publishes, the collect of step s - 1 runs one step later
    g2 = P2PTokenGather(n)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    got = torch.full((world * n,), -1, dtype=torch.int32, device=dev)
    prev_ref = None
    for s in range(steps):
        x = torch.randn((n, 512), generator=gen, device=dev)
        if s % 5 == rank % 5:
            torch.cuda._sleep(3_000_000)  # a late rank: the others' collect of its step waits, their publish does not
        if s % 2 == 0:   # the two-launch form and the fused form take turns
            g2.collect(out=got)
            tok = g2.publish_argmax(x)
        else:
            tok = g2.publish_argmax(x, collect_out=got)
        if prev_ref is not None:
            assert torch.equal(got, prev_ref), f"rank {rank} step {s}: collected tokens differ from the NCCL gather of step {s - 1}"
        assert torch.equal(tok.long(), x.argmax(dim=1))
        dist.all_gather_into_tensor(ref, tok)
        prev_ref = ref.clone()
    g2.collect(out=got)
    assert torch.equal(got, prev_ref)
    g2.check()
    g2.close()
    # timing, both ways, 200 steps each
    tok = base.clone()
    for fn, name in ((lambda: g.gather(tok, out=ref), "p2p"), (lambda: dist.all_gather_into_tensor(ref, tok), "nccl")):
        for _ in range(20):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(200):
            fn()
        e1.record(); torch.cuda.synchronize()
        if rank == 0:
            print(f"TIMING {name} {e0.elapsed_time(e1) / 200 * 1e3:.1f} us per gather of {n} int32 x {world} ranks", flush=True)
    g.check()
    g.close()
    if rank == 0:
        print("P2P_GATHER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
