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
    # timing, 200 steps each: the blocking gather, the library gather, and the pieces of the split form
    from nano_vllm_jax_b200.kernels import paged_kv as K
    tok = base.clone()
    x = torch.randn((n, 2048), device=dev)
    g3 = P2PTokenGather(n)
    tmp = torch.empty(n, dtype=torch.int32, device=dev)
    cases = ((lambda: g.gather(tok, out=ref), "p2p blocking gather"),
             (lambda: dist.all_gather_into_tensor(ref, tok), "nccl all-gather"),
             (lambda: K.row_argmax(x), "row_argmax alone"),
             (lambda: g3.publish_argmax(x, tmp, collect_out=ref), "argmax + publish + collect of the step before (one launch)"),
             (lambda: (g3.publish_argmax(x, tmp), g3.collect(out=ref)), "argmax + publish, then collect of the same step (two launches)"))
    side = torch.cuda.Stream(dev)
    for fn, name in cases:
        for _ in range(20):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        if "nccl" in name:  # eager launches: the host's launch rate is part of this figure
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(200):
                fn()
            e1.record(); torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / 200 * 1e3
        else:           # 20 launches per CUDA graph, 10 replays: device time per launch
            graph = torch.cuda.CUDAGraph()
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.graph(graph, stream=side):
                for _ in range(20):
                    fn()
            dist.barrier(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                graph.replay()
            e1.record(); torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / 200 * 1e3
        if rank == 0:
            print(f"TIMING {name}: {us:.1f} us per step, {n} int32 x {world} ranks", flush=True)
    g3.collect(out=ref)
    g3.check()
    g3.close()
    g.check()
    g.close()
    if rank == 0:
        print("P2P_GATHER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
