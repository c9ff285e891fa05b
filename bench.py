"""Benchmark of the paged KV-cache hot path: KV append + paged GQA decode attention.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload c2|c5]

One "step" = one decode step of one full-attention layer over one batch: append
each row's new K/V row, attend the whole context through the block table, turn
each row's output into a token (argmax stand-in for the sampler) and, with N > 1
ranks, all-gather the tokens over NCCL.  Rank r owns its own rows, block tables
and KV pool (request partition); nothing but the tokens crosses GPUs.

Workload c2 (default; per rank): 256 rows, contexts uniform in [1024, 4096],
400k-block bf16 pool, block tables a scattered permutation, N(0,1) values.
Workload c5: 2048 rows, contexts uniform in [8192, 32768], rows dealt round-robin
to the ranks (strong scaling).

Prints ONE JSON line (rank 0).  `value` = rows per second over all ranks with the
inputs resident in HBM; `e2e` = the same through the backend API from pinned host
buffers, copies inside the timed region; `roofline` = algorithmic bytes of the
fused append+decode kernel over its CUDA-event duration (events around every
launch of the timed region) against the measured HBM copy peak; `cpu_baseline` = the CPU restatement of the reference path on a
bounded sample of the same rows.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BS, HQ, HKV, D = 16, 8, 2, 256
SCALE = 1.0 / 16.0
TOKEN_BYTES = 2 * HKV * D * 2  # K + V row of one token, bf16
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of decode_wide_kernel over its algorithmic bytes, from the
# ncu capture of `--workload c2small` (profiles/decode_wide_c2small_ncu_full.md): 314.2-314.7 MB moved for
# 310.5 MB algorithmic.  K/V traffic grows in proportion to the tokens read, so the ratio carries over to c2.
DRAM_TRAFFIC_RATIO = 1.012

WORKLOADS = {
    # name: (total rows at N=1 or overall, ctx_lo, ctx_hi, pool blocks per rank or None = sized to fit, scaling)
    "c2": dict(rows=256, lo=1024, hi=4096, pool=400_000, scaling="weak", seed=2,
               desc="decode step, 256 rows/GPU, ctx U[1024,4096], 400k-block bf16 pool, 8q/2kv heads, head_dim 256, block 16"),
    # reduced c2 for profiler captures: a few GB on the device, still far larger than L2 per step
    "c2small": dict(rows=64, lo=1024, hi=4096, pool=40_000, scaling="weak", seed=2,
                    desc="decode step, 64 rows/GPU, ctx U[1024,4096], 40k-block bf16 pool (reduced c2 for profiling)"),
    "c5": dict(rows=2048, lo=8192, hi=32768, pool=None, scaling="strong", seed=5,
               desc="decode step, 2048 rows round-robin over the GPUs, ctx U[8192,32768], bf16 pool sized to the rows"),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-sample-rows", type=int, default=16)
    return ap.parse_args()


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def make_rows(w, rank, world, steps_total):
    """Context lengths and block tables of this rank's rows (NumPy, seeded)."""
    rng = np.random.default_rng(w["seed"])
    if w["scaling"] == "weak":
        rng = np.random.default_rng(w["seed"] * 1000 + rank)
        ctx = rng.integers(w["lo"], w["hi"] + 1, size=w["rows"])
    else:
        ctx_all = rng.integers(w["lo"], w["hi"] + 1, size=w["rows"])
        ctx = ctx_all[rank::world]  # request id i -> rank i % world
        rng = np.random.default_rng(w["seed"] * 1000 + rank)
    final_len = ctx + steps_total  # every step appends one token
    need = -(-final_len // BS)
    pool = int(w["pool"] or (need.sum() + 64))
    if need.sum() > pool:
        raise RuntimeError("pool too small for the rows")
    width = int(need.max())
    perm = rng.permutation(pool)
    tables = np.zeros((len(ctx), width), np.int32)
    o = 0
    for b in range(len(ctx)):
        tables[b, :need[b]] = perm[o:o + need[b]]
        o += need[b]
    return ctx.astype(np.int64), tables, pool


def algorithmic_bytes(ctx_after_append, rows):
    """Bytes one fused append+decode launch must move: K/V rows read once, the new rows read and
    written, q in (bf16), out (fp32), block-table entries, per-row scalars."""
    kv = int(ctx_after_append.sum()) * TOKEN_BYTES
    table = int((-(-ctx_after_append // BS)).sum()) * 4
    return kv + rows * TOKEN_BYTES * 2 + rows * HQ * D * 2 + rows * HQ * D * 4 + table + rows * 12


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "25"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU arm (oracle port)

def cpu_sample_case(w, sample_rows):
    """A bounded sample of the workload for the CPU restatement: the first rows of rank 0."""
    from ml_dtypes import bfloat16
    ctx, tables, _ = make_rows(w, 0, 1, 1)
    ctx, tables = ctx[:sample_rows], tables[:sample_rows]
    # compact the sampled rows' blocks into a small pool (same values per block, same table shape)
    used = np.unique(tables)
    remap = np.zeros(int(tables.max()) + 1, np.int32)
    remap[used] = np.arange(len(used), dtype=np.int32)
    tables = remap[tables]
    rng = np.random.default_rng(w["seed"] + 77)
    shape = (1, len(used), BS, HKV, D)
    k = rng.standard_normal(shape, dtype=np.float32).astype(bfloat16)
    v = rng.standard_normal(shape, dtype=np.float32).astype(bfloat16)
    q = rng.standard_normal((sample_rows, 1, HQ, D), dtype=np.float32).astype(bfloat16)
    nk = rng.standard_normal((sample_rows, 1, HKV, D), dtype=np.float32).astype(bfloat16)
    nv = rng.standard_normal((sample_rows, 1, HKV, D), dtype=np.float32).astype(bfloat16)
    return dict(k=k, v=v, q=q, nk=nk, nv=nv, tables=tables, ctx=ctx)


def cpu_step(case):
    """One decode step of the reference's pure path, restated on the CPU (append, then paged attention)."""
    from oracle import kv_cache_ref as R
    pos = case["ctx"].astype(np.int32)[:, None]
    slots = R.compute_slot_mapping(pos, case["tables"], BS)
    k, v = R.update_kv_cache(case["k"], case["v"], slots, case["nk"], case["nv"], 0)
    return R.paged_attention_decode(case["q"], k, v, case["tables"], (case["ctx"] + 1).astype(np.int32), BS, SCALE,
                                    HQ // HKV, mode="ref")


def time_cpu(w, sample_rows, steps, warmup, budget_s=25.0):
    case = cpu_sample_case(w, sample_rows)
    for _ in range(max(1, min(warmup, 2))):
        cpu_step(case)
    times = []
    t_start = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_step(case)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_start > budget_s:
            break
    med = statistics.median(times)
    cores = len(os.sched_getaffinity(0))
    return dict(value=sample_rows / med, unit="tok/s", cores=cores, kind="port",
                sample=f"{sample_rows} of the workload's rows per step (append + paged decode, NumPy/BLAS on "
                       f"{cores} host threads), median of {len(times)} steps"), med, len(times)


def run_reference_arm(args, w):
    """`--impl reference`: the reference's own CPU path.  JAX is not installed on this image, so the
    timed code is the NumPy restatement of that path (oracle/), on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, med, n = time_cpu(w, args.cpu_sample_rows, max(1, args.steps), args.warmup, budget_s=120.0)
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s_paged_attention_plus_kv_append", "value": base["value"],
        "unit": "tok/s", "n_gpus": args.gpus, "steps": n, "warmup": min(args.warmup, 2), "ms_per_step": med * 1e3,
        "higher_is_better": True, "scaling": w["scaling"], "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload + ": " + w["desc"], "note": "bounded sample: " + base["sample"]},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm

def fill_normal_bf16(t, seed, chunk_blocks=8192):
    """N(0,1) values into a big bf16 tensor without a float32 copy of the whole pool."""
    import torch
    g = torch.Generator(device=t.device).manual_seed(seed)
    flat = t.view(-1, t.shape[-3] * t.shape[-2] * t.shape[-1]) if t.ndim > 2 else t
    for i in range(0, flat.shape[0], chunk_blocks):
        part = flat[i:i + chunk_blocks]
        part.copy_(torch.randn(part.shape, generator=g, device=t.device, dtype=torch.float32))


def run_b200(args, w):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from nano_vllm_jax_b200.backends import B200Backend
    from nano_vllm_jax_b200.kernels import paged_kv as K
    from nano_vllm_jax_b200.kv_cache import KVCacheStorage

    K_steps, W_steps = args.steps, max(args.warmup, 3)
    n_passes = 4  # eager device-resident pass (times every kernel launch), CUDA-graph pass, serial and pipelined end-to-end passes
    total_steps = n_passes * (K_steps + W_steps) + 4
    ctx, tables_np, pool = make_rows(w, rank, world, total_steps)
    rows = len(ctx)

    k_cache = torch.empty((1, pool, BS, HKV, D), dtype=torch.bfloat16, device=dev)
    v_cache = torch.empty_like(k_cache)
    fill_normal_bf16(k_cache[0], 100 + rank)
    fill_normal_bf16(v_cache[0], 200 + rank)
    cache = KVCacheStorage(k_cache, v_cache)
    backend = B200Backend(device=dev)

    g = torch.Generator(device=dev).manual_seed(300 + rank)
    q = torch.randn((rows, 1, HQ, D), generator=g, device=dev).to(torch.bfloat16)
    nk = torch.randn((rows, 1, HKV, D), generator=g, device=dev).to(torch.bfloat16)
    nv = torch.randn((rows, 1, HKV, D), generator=g, device=dev).to(torch.bfloat16)
    tables = torch.from_numpy(tables_np).to(dev)
    # per-step metadata, built before any timed region: positions = current length, seq_lens = +1
    steps_idx = torch.arange(total_steps, device=dev, dtype=torch.int32)[:, None]
    ctx_t = torch.from_numpy(ctx.astype(np.int32)).to(dev)[None, :]
    all_pos = (ctx_t + steps_idx).contiguous()          # [steps, rows]
    all_len = (all_pos + 1).contiguous()
    gathered = torch.empty(rows * world, dtype=torch.int32, device=dev) if world > 1 else None
    step_no = [0]

    kernel_events = []  # (start, end) CUDA events around every fused append+decode launch of the timed passes

    def device_step():
        s = step_no[0]
        step_no[0] += 1
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out, _, _ = K.paged_decode_attention_with_kv_append(q, nk, nv, k_cache, v_cache, tables, all_len[s],
                                                            all_pos[s], 0, BS, SCALE, HQ // HKV)
        e1.record()
        kernel_events.append((s, e0, e1))
        tok = K.row_argmax(out.view(rows, HQ * D))
        if world > 1:
            dist.all_gather_into_tensor(gathered, tok)
        return tok

    # end-to-end: host (pinned) -> device inputs every step, result back to the host every step
    h_q, h_k, h_v = (t.cpu().pin_memory() for t in (q, nk, nv))
    h_tables = tables.cpu().pin_memory()
    h_pos = all_pos.cpu().pin_memory()
    h_len = all_len.cpu().pin_memory()
    h_out = torch.empty((rows, 1, HQ * D), dtype=torch.float32).pin_memory()
    d_q, d_k, d_v, d_tab = torch.empty_like(q), torch.empty_like(nk), torch.empty_like(nv), torch.empty_like(tables)
    d_pos = torch.empty((rows, 1), dtype=torch.int32, device=dev)
    d_len = torch.empty(rows, dtype=torch.int32, device=dev)
    h2d = sum(t.numel() * t.element_size() for t in (h_q, h_k, h_v, h_tables)) + rows * 8
    d2h = h_out.numel() * 4

    def e2e_step():
        s = step_no[0]
        step_no[0] += 1
        d_q.copy_(h_q, non_blocking=True); d_k.copy_(h_k, non_blocking=True); d_v.copy_(h_v, non_blocking=True)
        d_tab.copy_(h_tables, non_blocking=True)
        d_pos.copy_(h_pos[s].view(rows, 1), non_blocking=True); d_len.copy_(h_len[s], non_blocking=True)
        md = backend.build_attention_metadata(d_pos, d_tab, d_len, BS, False)
        _, out = backend.write_kv_and_attention(0, d_q, d_k, d_v, cache, md, BS, SCALE, HQ // HKV, False)
        h_out.copy_(out, non_blocking=True)
        if world > 1:
            dist.all_gather_into_tensor(gathered, K.row_argmax(out.view(rows, HQ * D)))

    token_gather = None
    if world > 1 and os.environ.get("NVJ_BENCH_NCCL_GATHER", "0") != "1":
        from nano_vllm_jax_b200.parallel import P2PTokenGather
        try:  # peer stores over NVLink inside the graph; all ranks succeed or all fall back to the NCCL gather
            token_gather = P2PTokenGather(rows)
        except Exception as exc:
            if rank == 0:
                print(f"[bench] NVLink token gather unavailable ({exc!r}); using the NCCL all-gather", file=sys.stderr, flush=True)
    from nano_vllm_jax_b200.host_pipeline import HostDecodePipeline
    # The compute stage of each pipeline slot (append + decode, token pick, NVLink token gather) is replayed from a CUDA
    # graph; with the NCCL gather in it (no peer access) it is launched eagerly.
    pipe_capture = (world == 1 or token_gather is not None) and os.environ.get("NVJ_BENCH_EAGER_PIPELINE", "0") != "1"
    pipe = HostDecodePipeline(backend, cache, rows, tables.shape[1], BS, SCALE, HQ // HKV, depth=2, capture=pipe_capture)
    gathered_p2p = torch.empty(world * rows, dtype=torch.int32, device=dev) if token_gather is not None else None

    def gather_tokens(out):
        if world > 1:
            tok = K.row_argmax(out.view(rows, HQ * D))
            if token_gather is not None:
                token_gather.gather(tok, out=gathered_p2p)
            else:
                dist.all_gather_into_tensor(gathered, tok)

    def e2e_pipelined_step():
        s = step_no[0]
        step_no[0] += 1
        pipe.submit(0, h_q, h_k, h_v, h_tables, h_pos[s], h_len[s], after_compute=gather_tokens)

    def timed(fn, finish=None):
        for _ in range(W_steps):
            fn()
        if finish is not None:
            finish()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K_steps):
            fn()
        if finish is not None:
            finish()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # The same step replayed from a CUDA graph over device-resident metadata: advance (positions, seq_lens) -> fused
    # append + decode -> token argmax, one graph launch per step; the token all-gather (N > 1) follows each replay.
    from nano_vllm_jax_b200.engine.resident_decode import DecodeStepGraph, ResidentDecodeMetadata
    meta = ResidentDecodeMetadata(rows, tables.shape[1], BS, device=dev)
    graph = DecodeStepGraph(meta, k_cache, v_cache, 0, SCALE, HQ // HKV, token_gather=token_gather)
    graph.query.copy_(q); graph.new_k.copy_(nk); graph.new_v.copy_(nv)
    graph_ready = [False]

    def graph_step():
        if not graph_ready[0]:  # first call: install the lengths reached so far and capture (runs one real step)
            meta.load(tables, all_len[step_no[0]] - 1)
            _, tok = graph.capture()
            graph_ready[0] = True
        else:
            _, tok = graph.replay()
        step_no[0] += 1
        if world > 1 and token_gather is None:
            dist.all_gather_into_tensor(gathered, tok)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_eager = timed(device_step)
    timed_events = kernel_events[-K_steps:]  # the launches of the timed region (warm-up launches come first)
    step_mode = "CUDA graph replay over device-resident metadata (advance -> append+decode -> argmax)"
    try:
        ms_dev = timed(graph_step)
        meta.check()
        if token_gather is not None:
            token_gather.check()
            step_mode += " -> token all-gather by NVLink peer stores, all in the graph"
            ok = torch.equal(graph.gathered.view(world, rows)[rank], graph.tokens)
            if not ok:
                raise SystemExit("token all-gather returned something else than this rank's own tokens")
    except Exception as exc:  # a capture problem must not cost the measurement: the eager pass is the same step
        if world > 1:
            raise
        print(f"[bench] graph pass failed ({exc!r}); reporting the eager pass", file=sys.stderr, flush=True)
        torch.cuda.synchronize()
        ms_dev, step_mode = ms_eager, "eager launches (graph capture failed)"
    ms_e2e_serial = timed(e2e_step)
    ms_e2e = timed(e2e_pipelined_step, finish=pipe.drain)
    clocks = sampler.stop() if rank == 0 else None
    K.check_device_status(dev)

    total_rows = rows * world if w["scaling"] == "weak" else w["rows"]
    if world > 1:
        cnt = torch.tensor([rows], device=dev)
        dist.all_reduce(cnt)
        total_rows = int(cnt.item())

    # roofline of the fused append+decode kernel: bytes of the timed launches over their duration
    kernel_ms = [e0.elapsed_time(e1) for _, e0, e1 in timed_events]
    ms_kernel = sum(kernel_ms)
    bytes_total = sum(algorithmic_bytes(ctx + s + 1, rows) for s, _, _ in timed_events)
    bytes_per_launch = bytes_total // K_steps
    peak, peak_kind = measured_hbm_peak()
    achieved = bytes_total / (ms_kernel * 1e-3) / 1e9

    cpu = None
    if rank == 0 and world == 1:
        cpu, _, _ = time_cpu(w, args.cpu_sample_rows, 20, 2)

    if rank == 0:
        line = {
            "metric": "decode_tokens_per_s_paged_attention_plus_kv_append",
            "value": total_rows / (ms_dev / K_steps * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K_steps,
            "warmup": W_steps, "ms_per_step": ms_dev / K_steps, "higher_is_better": True, "scaling": w["scaling"],
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload + ": " + w["desc"], "rows_total": total_rows, "rows_per_gpu": rows,
                       "layers": 1, "pool_blocks_per_gpu": pool, "cache_timing": "inputs exceed L2 (>= 1.3 GB of K/V read per step)",
                       "parallelism": (f"request-partitioned x{world}, all-gather of tokens (" +
                                       ("NVLink peer stores" if token_gather is not None else "NCCL") + ")") if world > 1 else "single GPU"},
            "e2e": {"value": total_rows / (ms_e2e / K_steps * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / K_steps,
                    "mode": "HostDecodePipeline: 2 steps in flight on copy/compute/copy streams; every step copies all operands "
                            "from pinned host memory and its whole result back; compute stage "
                            + ("replayed from a CUDA graph per slot" if pipe_capture else "launched eagerly"),
                    "serial_value": total_rows / (ms_e2e_serial / K_steps * 1e-3), "serial_ms_per_step": ms_e2e_serial / K_steps},
            # per step of the timed pass: metadata advance, fused append+decode, token argmax (+ the NVLink token gather)
            "gpu_launches": (4 if token_gather is not None else 3) * K_steps,
            "step_mode": step_mode,
            "eager_value": total_rows / (ms_eager / K_steps * 1e-3), "eager_ms_per_step": ms_eager / K_steps,
            "roofline": {"bound": "hbm", "kernel": "decode_wide_kernel at width 1 (fused append + paged GQA decode, TMA-staged, tensor-core tiles)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_kind + " HBM copy bandwidth", "frac_of_8TBs_nominal": achieved / 8000.0,
                         "bytes_per_launch": bytes_per_launch, "us_per_launch": ms_kernel / K_steps * 1e3,
                         "traffic": DRAM_TRAFFIC_RATIO * bytes_per_launch,
                         "traffic_source": "ncu dram bytes of the c2small capture scaled by algorithmic bytes (ratio 1.012)"},
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, w)
    else:
        run_b200(args, w)


if __name__ == "__main__":
    main()
