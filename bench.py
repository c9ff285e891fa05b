"""Benchmark of the paged KV-cache hot path: KV append + paged GQA decode attention.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload c2|c2small|c5]

One "step" = one decode step of one full-attention layer over one batch: append
each row's new K/V row, attend the whole context through the block table, turn
each row's output into a token (argmax stand-in for the sampler) and, with N > 1
ranks, all-gather the tokens.  Rank r owns its own rows, block tables and KV pool
(request partition); nothing but the tokens crosses GPUs.

Workload c2 (default; per rank): 256 rows, contexts uniform in [1024, 4096] (the same seeded
draw on every rank), 400k-block bf16 pool, block tables a scattered permutation and N(0,1)
values of the rank's own.
Workload c5: 2048 rows, contexts uniform in [8192, 32768], rows dealt round-robin
to the ranks (strong scaling), each rank's pool sized to min(150 GB, 0.9 x free
memory) with the block tables drawn over the whole pool.

Prints ONE JSON line (rank 0).  `value` = rows per second over all ranks with the
inputs resident in HBM, from the first timed block of exactly --steps steps; the
block is repeated until at least 100 steps are timed and `step_ms` gives median and
p10 / p90 over all of them.  `e2e` = the same through the backend API from pinned host
buffers, copies inside the timed region; `roofline` = algorithmic bytes of the
fused append+decode kernel over its CUDA-event duration (the launches of one timed
block replayed from a CUDA graph, events around the replay; events around every
single launch of the eager pass are reported beside it as `launch_us`) against the
measured HBM copy peak; every pass starts from the configured context lengths; `cpu_baseline` =
the CPU restatement of the reference path on the same rows; `parity_check` = the
last step's output of sampled rows and every appended cache row against that CPU
restatement, taken after the timed passes.
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
BLOCK_BYTES = BS * TOKEN_BYTES  # one block of K plus one block of V
FALLBACK_HBM_GBS = 6650.0
MIN_TIMED_STEPS = 100
# dram__bytes_read.sum + dram__bytes_write.sum of decode_wide_kernel in an ncu capture of `--workload c2small`
# (one launch) and the algorithmic bytes of that launch.  K/V traffic grows in proportion to the tokens
# read, so a launch of another workload is scaled by its own algorithmic bytes.
NCU_C2SMALL_DRAM_BYTES = 354.93e6
NCU_C2SMALL_ALGORITHMIC_BYTES = 356.35e6

WORKLOADS = {
    # rows: per rank (weak) or overall (strong); pool: blocks per rank, or None = sized from the free memory
    "c2": dict(rows=256, lo=1024, hi=4096, pool=400_000, scaling="weak", seed=2,
               desc="decode step, 256 rows/GPU, ctx U[1024,4096], 400k-block bf16 pool, 8q/2kv heads, head_dim 256, block 16"),
    # reduced c2 for profiler captures: a few GB on the device, still far larger than L2 per step
    "c2small": dict(rows=64, lo=1024, hi=4096, pool=40_000, scaling="weak", seed=2,
                    desc="decode step, 64 rows/GPU, ctx U[1024,4096], 40k-block bf16 pool (reduced c2 for profiling)"),
    "c5": dict(rows=2048, lo=8192, hi=32768, pool=None, pool_bytes=150e9, scaling="strong", seed=5,
               desc="decode step, 2048 rows round-robin over the GPUs, ctx U[8192,32768], bf16 pool of min(150 GB, 0.9 x free) per GPU"),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-sample-rows", type=int, default=0, help="rows of the CPU arm per step (0 = all, c5: 16)")
    ap.add_argument("--pool-gb", type=float, default=0.0, help="c5: cap of the per-GPU pool in GB (default 150)")
    return ap.parse_args()


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def row_lengths(w, rank, world):
    """Context lengths of this rank's rows (seeded).  Weak scaling: every rank runs the configuration itself, i.e. the
    SAME seeded lengths (its block tables and values are its own), so that the per-N figures compare the system and
    not the ranks' luck in the draw.  Strong scaling: one draw for all rows, dealt round-robin."""
    ctx_all = np.random.default_rng(w["seed"]).integers(w["lo"], w["hi"] + 1, size=w["rows"])
    if w["scaling"] == "weak":
        return ctx_all.astype(np.int64)
    return ctx_all[rank::world].astype(np.int64)  # request id i -> rank i % world


def make_rows(w, rank, world, steps_total, pool_blocks=None):
    """Context lengths and block tables of this rank's rows: consecutive slices of a permutation of the whole pool."""
    ctx = row_lengths(w, rank, world)
    rng = np.random.default_rng(w["seed"] * 1000 + rank + 500)
    final_len = ctx + steps_total  # every step appends one token
    need = -(-final_len // BS)
    pool = int(pool_blocks or w["pool"] or (need.sum() + 64))
    if need.sum() > pool:
        raise RuntimeError(f"pool of {pool} blocks too small for the rows ({int(need.sum())} needed)")
    width = int(need.max())
    perm = rng.permutation(pool)
    tables = np.zeros((len(ctx), width), np.int32)
    o = 0
    for b in range(len(ctx)):
        tables[b, :need[b]] = perm[o:o + need[b]]
        o += need[b]
    return ctx, tables, pool


def algorithmic_bytes(ctx_after_append, rows):
    """Bytes one fused append+decode launch must move: K/V rows read once, the new rows read and
    written, q in (bf16), out (fp32), block-table entries, per-row scalars."""
    kv = int(ctx_after_append.sum()) * TOKEN_BYTES
    table = int((-(-ctx_after_append // BS)).sum()) * 4
    return kv + rows * TOKEN_BYTES * 2 + rows * HQ * D * 2 + rows * HQ * D * 4 + table + rows * 12


def workload_config(args, w, world):
    """The `config` object of the JSON line: the same for both arms."""
    rows_total = w["rows"] * world if w["scaling"] == "weak" else w["rows"]
    return {"workload": args.workload + ": " + w["desc"], "rows_total": rows_total,
            "rows_per_gpu": w["rows"] if w["scaling"] == "weak" else -(-w["rows"] // world), "layers": 1,
            "cache_timing": "inputs exceed L2 (>= 1.3 GB of K/V read per step)",
            "parallelism": f"request-partitioned x{world}, all-gather of tokens" if world > 1 else "single GPU"}


def percentiles(xs):
    xs = sorted(xs)
    if not xs:
        return None
    pick = lambda f: xs[min(len(xs) - 1, int(round(f * (len(xs) - 1))))]
    return {"median": statistics.median(xs), "p10": pick(0.10), "p90": pick(0.90), "n": len(xs)}


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

def cpu_case(w, sample_rows):
    """The workload's rows (rank 0 of 1) for the CPU restatement; `sample_rows` > 0 keeps the first rows only.
    The rows' blocks are compacted into a pool that holds just them (same values per block, same table shape)."""
    from ml_dtypes import bfloat16
    ctx, tables, _ = make_rows(w, 0, 1, 1)
    if sample_rows > 0:
        ctx, tables = ctx[:sample_rows], tables[:sample_rows]
    used = np.unique(tables)
    remap = np.zeros(int(tables.max()) + 1, np.int32)
    remap[used] = np.arange(len(used), dtype=np.int32)
    tables = remap[tables]
    rng = np.random.default_rng(w["seed"] + 77)
    shape = (1, len(used), BS, HKV, D)
    k = rng.standard_normal(shape, dtype=np.float32).astype(bfloat16)
    v = rng.standard_normal(shape, dtype=np.float32).astype(bfloat16)
    n = len(ctx)
    q = rng.standard_normal((n, 1, HQ, D), dtype=np.float32).astype(bfloat16)
    nk = rng.standard_normal((n, 1, HKV, D), dtype=np.float32).astype(bfloat16)
    nv = rng.standard_normal((n, 1, HKV, D), dtype=np.float32).astype(bfloat16)
    return dict(k=k, v=v, q=q, nk=nk, nv=nv, tables=tables, ctx=ctx)


def cpu_step(case, chunk=32):
    """One decode step of the reference's pure path, restated on the CPU: append every row's token, then paged
    attention (in chunks of rows, which bounds the gathered window the path materialises)."""
    from oracle import kv_cache_ref as R
    pos = case["ctx"].astype(np.int32)[:, None]
    slots = R.compute_slot_mapping(pos, case["tables"], BS)
    k, v = R.update_kv_cache(case["k"], case["v"], slots, case["nk"], case["nv"], 0)
    lens = (case["ctx"] + 1).astype(np.int32)
    outs = []
    for i in range(0, len(lens), chunk):
        outs.append(R.paged_attention_decode(case["q"][i:i + chunk], k, v, case["tables"][i:i + chunk], lens[i:i + chunk],
                                             BS, SCALE, HQ // HKV, mode="ref"))
    return np.concatenate(outs)


def time_cpu(w, sample_rows, steps, warmup, budget_s):
    case = cpu_case(w, sample_rows)
    rows = len(case["ctx"])
    for _ in range(warmup):
        cpu_step(case)
    times = []
    t_start = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_step(case)
        times.append(time.perf_counter() - t0)
        if budget_s is not None and time.perf_counter() - t_start > budget_s:
            break
    med = statistics.median(times)
    cores = len(os.sched_getaffinity(0))
    what = "all" if sample_rows <= 0 else f"the first {rows}"
    return dict(value=rows / med, unit="tok/s", cores=cores, kind="port",
                sample=f"{what} of the workload's {w['rows']} rows per step (append + paged decode of the pure path restated in "
                       f"NumPy/BLAS, {cores} host threads), median of {len(times)} steps after {warmup} warm-up"), med, len(times)


def run_reference_arm(args, w):
    """`--impl reference`: the reference's own CPU path.  JAX is not installed on this image, so the
    timed code is the NumPy restatement of that path (oracle/), on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = args.cpu_sample_rows or (16 if args.workload == "c5" else 0)
    base, med, n = time_cpu(w, sample, max(1, args.steps), max(0, args.warmup), budget_s=None)
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s_paged_attention_plus_kv_append", "value": base["value"],
        "unit": "tok/s", "n_gpus": args.gpus, "steps": n, "warmup": max(0, args.warmup), "ms_per_step": med * 1e3,
        "higher_is_better": True, "scaling": w["scaling"], "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, w, args.gpus),
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


def parity_check(torch, k_cache, v_cache, tables_np, ctx0, appended_upto, lens_out, q, nk, nv, out, sample=8):
    """After the timed passes: (a) every row appended since the start (positions ctx0 .. appended_upto - 1 of each row)
    holds the new K/V row bit for bit; (b) `out`, the output of the step that stood at lengths `lens_out`, for `sample`
    rows against the CPU restatement of the reference path, fed those rows' blocks gathered to the host."""
    from ml_dtypes import bfloat16

    from oracle import kv_cache_ref as R
    rows = len(ctx0)
    dev = k_cache.device
    exact = True
    kf, vf = k_cache[0].view(-1, HKV, D), v_cache[0].view(-1, HKV, D)
    tab = torch.from_numpy(tables_np).to(dev).long()
    for b in range(rows):
        pos = torch.arange(int(ctx0[b]), int(appended_upto[b]), device=dev)
        slots = tab[b, pos // BS] * BS + pos % BS
        exact = exact and bool((kf[slots] == nk[b, 0]).all()) and bool((vf[slots] == nv[b, 0]).all())
    pick = np.unique(np.linspace(0, rows - 1, min(sample, rows)).astype(int))
    worst = 0.0
    for b in pick:
        nb = -(-int(lens_out[b]) // BS)
        blocks = torch.from_numpy(tables_np[b, :nb]).to(dev).long()
        k_np = k_cache[0][blocks].cpu().view(torch.int16).numpy().view(bfloat16)[None]
        v_np = v_cache[0][blocks].cpu().view(torch.int16).numpy().view(bfloat16)[None]
        q_np = q[b:b + 1].cpu().view(torch.int16).numpy().view(bfloat16)
        ref = R.paged_attention_decode(q_np, k_np, v_np, np.arange(nb, dtype=np.int32)[None],
                                       np.array([lens_out[b]], np.int32), BS, SCALE, HQ // HKV)
        worst = max(worst, float(np.abs(out[b].float().cpu().numpy().reshape(-1) - ref.reshape(-1)).max()))
    return {"rows": [int(b) for b in pick], "max_abs": worst, "tolerance": 2e-2, "cache_bit_exact": exact,
            "appended_rows_checked": int((np.asarray(appended_upto) - np.asarray(ctx0)).sum()),
            "against": "CPU restatement of the reference path (fp32 accumulate) on the rows' own blocks"}


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
    reps = max(1, -(-MIN_TIMED_STEPS // K_steps))  # timed blocks of K steps each, >= 100 steps in all
    long_pass = W_steps + reps * K_steps
    # Every pass (eager, graph, serial and pipelined end-to-end) starts again from the configured lengths and grows
    # every row by one token per step, so that all of them are timed on the same contexts: rows appended by an earlier
    # pass are written again with the same values.
    total_steps = long_pass + 4
    pool_blocks = None
    if w["pool"] is None:  # c5: the pool takes min(150 GB, 0.9 x free) and the tables are drawn over all of it
        free_b, _ = torch.cuda.mem_get_info(dev)
        cap = (args.pool_gb * 1e9) if args.pool_gb > 0 else w["pool_bytes"]
        pool_blocks = int(min(cap, 0.9 * free_b) // BLOCK_BYTES)
    ctx, tables_np, pool = make_rows(w, rank, world, total_steps, pool_blocks)
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
    launches = [0]      # kernels of this library launched by the pass being timed

    kernel_events = []  # (step, start, end) CUDA events around every fused append+decode launch of the eager pass

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
    # NVJ_BENCH_SELF_GATHER=1: on one GPU, run the step with the NVLink gather kernel gathering from itself (a
    # diagnostic that separates the kernel's own cost from waiting for other ranks)
    self_gather = world == 1 and os.environ.get("NVJ_BENCH_SELF_GATHER", "0") == "1"
    if (world > 1 and os.environ.get("NVJ_BENCH_NCCL_GATHER", "0") != "1") or self_gather:
        from nano_vllm_jax_b200.parallel import P2PTokenGather
        try:  # peer stores over NVLink inside the graph; all ranks succeed or all fall back to the NCCL gather
            token_gather = P2PTokenGather(rows)
        except Exception as exc:
            if rank == 0:
                print(f"[bench] NVLink token gather unavailable ({exc!r}); using the NCCL all-gather", file=sys.stderr, flush=True)
    from nano_vllm_jax_b200.host_pipeline import HostDecodePipeline
    # The compute stage of each pipeline slot (append + decode, token pick published over NVLink, collect of the step
    # before) is replayed from a CUDA graph; with the NCCL gather in it (no peer access) it is launched eagerly.
    pipe_capture = (world == 1 or token_gather is not None) and os.environ.get("NVJ_BENCH_EAGER_PIPELINE", "0") != "1"
    pipe = HostDecodePipeline(backend, cache, rows, tables.shape[1], BS, SCALE, HQ // HKV, depth=2, capture=pipe_capture)
    gathered_p2p = torch.empty(world * rows, dtype=torch.int32, device=dev) if token_gather is not None else None
    pipe_tokens = torch.empty(rows, dtype=torch.int32, device=dev)

    def gather_tokens(out):
        if world > 1:
            if token_gather is not None:  # the step before arrives (it has had a whole step to do so), then this one leaves
                token_gather.publish_argmax(out.view(rows, HQ * D), pipe_tokens, collect_out=gathered_p2p)
            else:
                dist.all_gather_into_tensor(gathered, K.row_argmax(out.view(rows, HQ * D)))

    def e2e_pipelined_step():
        s = step_no[0]
        step_no[0] += 1
        pipe.submit(0, h_q, h_k, h_v, h_tables, h_pos[s], h_len[s], after_compute=gather_tokens)

    def timed(fn, finish=None, blocks=1):
        """W warm-up steps, then `blocks` timed blocks of exactly K steps each.  Returns (ms of the first block as the
        max over ranks, this rank's ms per step of every timed step)."""
        for _ in range(W_steps):
            fn()
        if finish is not None:
            finish()
        block_ms, step_ms = [], []
        for _ in range(blocks):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(K_steps + 1)]
            ev[0].record()
            for i in range(K_steps):
                fn()
                if finish is None:
                    ev[i + 1].record()
            if finish is not None:
                finish()
                ev[K_steps].record()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            block_ms.append(ev[0].elapsed_time(ev[K_steps]))
            if finish is None:
                step_ms += [ev[i].elapsed_time(ev[i + 1]) for i in range(K_steps)]
        ms = torch.tensor([block_ms[0]], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), step_ms, block_ms

    # The same step replayed from a CUDA graph over device-resident metadata: fused append + decode (pre-append form:
    # the row's token goes to position seq_lens[b]) -> token argmax that also advances the lengths, one graph launch
    # of two kernels per step.  With N > 1 the argmax launch also publishes the tokens to every rank over NVLink and
    # collects the step before.
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
    steps_done = [0]

    def new_pass():
        steps_done[0] = max(steps_done[0], step_no[0])
        step_no[0] = 0

    ms_eager, _, _ = timed(device_step, blocks=reps)
    new_pass()
    # The kernel without the host's launch latency between the events: the K launches of one timed block (fused append +
    # decode only, one node per step, each at its own lengths) captured into one CUDA graph; events bracket a replay.
    block_kernel_ms = []
    try:
        from nano_vllm_jax_b200.engine.resident_decode import CapturedStep

        def kernel_block():
            for s in range(W_steps, W_steps + K_steps):
                K.paged_decode_attention_with_kv_append(q, nk, nv, k_cache, v_cache, tables, all_len[s], all_pos[s], 0, BS,
                                                        SCALE, HQ // HKV)

        kernel_graph = CapturedStep(kernel_block, dev)
        kernel_graph.capture()
        for i in range(1 + max(2, reps)):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); kernel_graph.replay(); e1.record()
            torch.cuda.synchronize()
            if i > 0:
                block_kernel_ms.append(e0.elapsed_time(e1))
        del kernel_graph
    except Exception as exc:  # the per-launch events of the eager pass remain
        print(f"[bench] kernel-only graph failed ({exc!r}); kernel time from the eager pass's events", file=sys.stderr, flush=True)
        torch.cuda.synchronize()
        block_kernel_ms = []
    timed_events = kernel_events[W_steps:]  # the launches of the timed blocks (warm-up launches come first)
    step_mode = "CUDA graph replay over device-resident metadata (append+decode -> argmax+advance)"
    graph_ok = True
    try:
        ms_dev, dev_step_ms, dev_block_ms = timed(graph_step, blocks=reps)
        meta.check()
        if token_gather is not None:
            graph.flush()
            token_gather.check()
            step_mode += "; the argmax launch collects the tokens of the step before and publishes this step's over NVLink peer stores, all in the graph"
            ok = torch.equal(graph.gathered.view(world, rows)[rank], graph.tokens)
            if not ok:
                raise SystemExit("token all-gather returned something else than this rank's own tokens")
    except Exception as exc:  # a capture problem must not cost the measurement: the eager pass is the same step
        if world > 1:
            raise
        print(f"[bench] graph pass failed ({exc!r}); reporting the eager pass", file=sys.stderr, flush=True)
        torch.cuda.synchronize()
        graph_ok = False
        ms_dev, step_mode = ms_eager, "eager launches (graph capture failed)"
        dev_step_ms, dev_block_ms = [], [ms_eager]
    new_pass()
    ms_e2e_serial, _, _ = timed(e2e_step)
    new_pass()
    ms_e2e, _, e2e_block_ms = timed(e2e_pipelined_step, finish=pipe.drain, blocks=reps)
    new_pass()
    if token_gather is not None:
        token_gather.collect(out=gathered_p2p)
        token_gather.check()
    clocks = sampler.stop() if rank == 0 else None
    K.check_device_status(dev)

    # The gather launch on its own (N > 1): token pick + publish + collect of the step before, 20 launches in a CUDA
    # graph, so that the figure is device time per launch and not the host's launch rate.  Back to back the collect has
    # to wait for the peers' publish of a moment ago, which it never does inside a decode step.
    gather_us = None
    if token_gather is not None:
        x = graph.out.view(rows, HQ * D) if graph_ok else torch.zeros((rows, HQ * D), device=dev)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        g_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_graph, stream=side):
            for _ in range(20):
                token_gather.publish_argmax(x, pipe_tokens, collect_out=gathered_p2p)
        for timing in (False, True):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                g_graph.replay()
            e1.record(); torch.cuda.synchronize()
            if timing:
                gather_us = e0.elapsed_time(e1) / 100 * 1e3
        token_gather.collect(out=gathered_p2p)
        token_gather.check()

    total_rows = rows
    rank_ms = rank_kernel_us = None
    if world > 1:
        cnt = torch.tensor([rows], device=dev)
        dist.all_reduce(cnt)
        total_rows = int(cnt.item())
        mine = torch.tensor([statistics.mean(dev_block_ms) / K_steps], device=dev)  # this rank's own mean step time
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        per_rank = sorted(float(t.item()) for t in every)
        rank_ms = {"min": per_rank[0], "median": statistics.median(per_rank), "max": per_rank[-1]}
        # the decode kernel alone (eager pass, events around the launch: no collective inside), per rank
        mine = torch.tensor([statistics.mean(e0.elapsed_time(e1) for _, e0, e1 in kernel_events[W_steps:]) * 1e3], device=dev)
        dist.all_gather(every, mine)
        per_rank = sorted(float(t.item()) for t in every)
        rank_kernel_us = {"min": per_rank[0], "median": statistics.median(per_rank), "max": per_rank[-1]}

    # roofline of the fused append+decode kernel: bytes of the timed launches over their duration
    kernel_ms = [e0.elapsed_time(e1) for _, e0, e1 in timed_events]
    ms_kernel = sum(kernel_ms)
    bytes_total = sum(algorithmic_bytes(ctx + s + 1, rows) for s, _, _ in timed_events)
    bytes_per_launch = bytes_total // len(timed_events)
    peak, peak_kind = measured_hbm_peak()
    achieved = bytes_total / (ms_kernel * 1e-3) / 1e9
    us_per_launch = ms_kernel / len(timed_events) * 1e3
    kernel_timing = "CUDA events around every launch of the eager pass (the host's launch latency lies inside the events)"
    if block_kernel_ms:
        block_bytes = sum(algorithmic_bytes(ctx + s + 1, rows) for s in range(W_steps, W_steps + K_steps))
        bytes_per_launch = block_bytes // K_steps
        us_per_launch = statistics.mean(block_kernel_ms) / K_steps * 1e3
        achieved = bytes_per_launch / (us_per_launch * 1e-6) / 1e9
        kernel_timing = (f"{K_steps} launches (one per step of a timed block, each at its own lengths) replayed from one CUDA graph, "
                         f"CUDA events around the replay, mean of {len(block_kernel_ms)} replays / {K_steps}: the gaps between the "
                         "launches are inside, the host's launch latency is not; launch_us = events around single eager launches")

    # parity of what was just timed: the last graph step's output and every appended row (rank 0's own rows)
    parity = None
    if rank == 0 and graph_ok:
        parity = parity_check(torch, k_cache, v_cache, tables_np, ctx, ctx + steps_done[0],
                              meta.seq_lens.cpu().numpy().astype(np.int64), q, nk, nv, graph.out.view(rows, HQ * D))

    cpu = None
    if rank == 0 and world == 1:
        sample = args.cpu_sample_rows or (16 if args.workload == "c5" else 0)
        cpu, _, _ = time_cpu(w, sample, 8, 1, budget_s=20.0)

    if rank == 0:
        cfg = workload_config(args, w, world)
        line = {
            "metric": "decode_tokens_per_s_paged_attention_plus_kv_append",
            "value": total_rows / (ms_dev / K_steps * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K_steps,
            "warmup": W_steps, "ms_per_step": ms_dev / K_steps, "higher_is_better": True, "scaling": w["scaling"],
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": cfg,
            "pool": {"blocks_per_gpu": pool, "gb_per_gpu": pool * BLOCK_BYTES / 1e9,
                     "live_gb_per_gpu": float((ctx + total_steps).sum()) * TOKEN_BYTES / 1e9},
            "token_gather": (("NVLink peer stores, split publish / collect" if token_gather is not None else "NCCL all-gather")
                             if world > 1 else None),
            "timed_blocks": {"blocks": reps, "steps_per_block": K_steps,
                             "note": "value and ms_per_step come from the first block of exactly --steps steps; "
                                     "step_ms covers every timed step of all blocks",
                             "contexts": "every pass (eager, graph, serial and pipelined end to end) starts from the configured "
                                         "lengths and adds one token per row and step, so all are timed on the same contexts"},
            "step_ms": percentiles(dev_step_ms),
            "e2e": {"value": total_rows / (ms_e2e / K_steps * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / K_steps,
                    "block_ms_per_step": percentiles([m / K_steps for m in e2e_block_ms]),
                    "mode": "HostDecodePipeline: 2 steps in flight on copy/compute/copy streams; every step copies all operands "
                            "from pinned host memory and its whole result back; compute stage "
                            + ("replayed from a CUDA graph per slot" if pipe_capture else "launched eagerly"),
                    "serial_value": total_rows / (ms_e2e_serial / K_steps * 1e-3), "serial_ms_per_step": ms_e2e_serial / K_steps},
            # per step of the timed pass: fused append+decode, token argmax with the metadata advance (N > 1: the same
            # launch also collects and publishes)
            "gpu_launches": 2 * K_steps,
            "step_mode": step_mode,
            "eager_value": total_rows / (ms_eager / K_steps * 1e-3), "eager_ms_per_step": ms_eager / K_steps,
            "roofline": {"bound": "hbm", "kernel": "decode_wide_kernel at width 1 (fused append + paged GQA decode, TMA-staged, tensor-core tiles)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_kind + " HBM copy bandwidth", "frac_of_8TBs_nominal": achieved / 8000.0,
                         "bytes_per_launch": bytes_per_launch, "us_per_launch": us_per_launch, "kernel_timing": kernel_timing,
                         "launch_us": percentiles([m * 1e3 for m in kernel_ms]),
                         "traffic": NCU_C2SMALL_DRAM_BYTES / NCU_C2SMALL_ALGORITHMIC_BYTES * bytes_per_launch,
                         "traffic_source": "dram bytes of one ncu-captured launch of --workload c2small (354.93 MB for 356.35 MB "
                                           "algorithmic) scaled to this launch by algorithmic bytes"},
            "rank_ms": rank_ms, "rank_kernel_us": rank_kernel_us, "gather_us": gather_us,
            "parity_check": parity,
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if token_gather is not None:
        token_gather.close()
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
