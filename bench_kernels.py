"""Per-kernel timings of the path on one GPU (one JSON line per kernel).

    python bench_kernels.py [--iters N] [--only decode|prefill|...]

Every case uses seeded synthetic inputs with the shapes of the baseline
configurations (append and decode: 256 rows, contexts U[1024, 4096]; prefill and
block copy: 8 prompts U[64, 2048] in 512-token chunks with a shared 512-token
prefix; GDN state: 18 layers x [16, 128, 128] fp32 + conv [6144, 4] bf16).
Timing: CUDA events around each launch, an L2 flush (a 256 MiB write) before
every timed launch of the small kernels, median over the iterations.  Bytes are
the algorithmic minimum each kernel must move (stated per case).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from nano_vllm_jax_b200.engine.prefix_state import HybridStateTable, PrefixStateCache  # noqa: E402
from nano_vllm_jax_b200.kernels import paged_kv as K  # noqa: E402

BS, HQ, HKV, D = 16, 8, 2, 256
SCALE = 1.0 / 16.0
TOKEN_BYTES = 2 * HKV * D * 2
NOMINAL_GBS, MEASURED_GBS = 8000.0, 6555.5


def _randn_bf16(shape, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    out = torch.empty(shape, dtype=torch.bfloat16, device=dev)
    flat = out.view(-1)
    step = 1 << 26
    for i in range(0, flat.numel(), step):
        part = flat[i:i + step]
        part.copy_(torch.randn(part.shape, generator=g, device=dev))
    return out


class Timer:
    def __init__(self, dev, iters, flush=True):
        self.iters = iters
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if flush else None

    def run(self, fn, setup=None):
        times = []
        for i in range(self.iters + 3):
            if setup is not None:
                setup()
            if self.flush is not None:
                self.flush.zero_()
            torch.cuda._sleep(300_000)  # keep the GPU busy while the host enqueues: the events then bracket only the kernel
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                times.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(times)


def report(name, us, nbytes, extra=None):
    gbs = nbytes / us / 1e3
    line = {"kernel": name, "us": round(us, 2), "algorithmic_bytes": int(nbytes), "GB/s": round(gbs, 1),
            "pct_of_8TBs": round(100 * gbs / NOMINAL_GBS, 1), "pct_of_measured_copy": round(100 * gbs / MEASURED_GBS, 1)}
    if extra:
        line.update(extra)
    print(json.dumps(line), flush=True)


def tables_for(lens, pool, rng):
    need = -(-lens // BS)
    perm = rng.permutation(pool)
    t = np.zeros((len(lens), int(need.max())), np.int32)
    o = 0
    for b in range(len(lens)):
        t[b, :need[b]] = perm[o:o + need[b]]
        o += need[b]
    return t


def decode_cases(dev, iters, small=False):
    rng = np.random.default_rng(2)
    rows, pool = (64, 40_000) if small else (256, 400_000)  # small: what a profiler capture may hold (2.6 GB of cache)
    ctx = rng.integers(1024, 4097, size=rows)
    lens = (ctx + 1).astype(np.int32)
    tables = torch.from_numpy(tables_for(lens, pool, rng)).to(dev)
    k = _randn_bf16((1, pool, BS, HKV, D), 1, dev)
    v = _randn_bf16((1, pool, BS, HKV, D), 2, dev)
    q = _randn_bf16((rows, 1, HQ, D), 3, dev)
    nk = _randn_bf16((rows, 1, HKV, D), 4, dev)
    nv = _randn_bf16((rows, 1, HKV, D), 5, dev)
    t_lens = torch.from_numpy(lens).to(dev)
    pos = (t_lens - 1).view(rows, 1).contiguous()
    slots = K.compute_slot_mapping(pos, tables, BS)
    kv_bytes = int(lens.sum()) * TOKEN_BYTES
    table_bytes = int((-(-lens // BS)).sum()) * 4
    io = rows * HQ * D * 2 + rows * HQ * D * 4 + table_bytes + rows * 12
    small = Timer(dev, iters)
    big = Timer(dev, iters, flush=False)  # 1.3 GB of K/V per launch: far beyond L2
    report("kv_append (decode step, 256 tokens)", small.run(lambda: K.kv_append_slots(nk, nv, slots, k[0], v[0])),
           2 * rows * TOKEN_BYTES + rows * 4, {"workload": "c2"})
    report("compute_slot_mapping (256 tokens)", small.run(lambda: K.compute_slot_mapping(pos, tables, BS)),
           rows * 12, {"workload": "c2"})
    report("paged_decode (tensor-core streaming kernel, variant 3: the default for bf16 queries)", big.run(lambda: K.paged_decode_attention(q[:, 0], k[0], v[0], tables, t_lens, SCALE, variant=3)),
           kv_bytes + io, {"workload": "c2", "tok/s": None})
    report("paged_decode + fused append (tensor-core streaming kernel)",
           big.run(lambda: K.paged_decode_attention_with_kv_append(q, nk, nv, k, v, tables, t_lens, pos, 0, BS, SCALE, 4, variant=3)),
           kv_bytes + io + 2 * rows * TOKEN_BYTES, {"workload": "c2"})
    report("paged_decode (CUDA-core pipelined kernel, variant 2)", big.run(lambda: K.paged_decode_attention(q[:, 0], k[0], v[0], tables, t_lens, SCALE, variant=2)),
           kv_bytes + io, {"workload": "c2", "tok/s": None})
    report("paged_decode + fused append (CUDA-core pipelined kernel)",
           big.run(lambda: K.paged_decode_attention_with_kv_append(q, nk, nv, k, v, tables, t_lens, pos, 0, BS, SCALE, 4, variant=2)),
           kv_bytes + io + 2 * rows * TOKEN_BYTES, {"workload": "c2"})
    sub = 16  # the generic kernel re-reads K/V once per query head: time a 16-row slice
    report("paged_decode (generic kernel, 16 rows)",
           Timer(dev, max(3, iters // 4), flush=False).run(
               lambda: K.paged_decode_attention(q[:sub, 0], k[0], v[0], tables[:sub], t_lens[:sub], SCALE, variant=1)),
           int(lens[:sub].sum()) * TOKEN_BYTES, {"workload": "c2, first 16 rows"})
    # speculative-verify decode: `width` query tokens per row at the row's last positions (rows already appended)
    from nano_vllm_jax_b200 import kv_cache as kvc
    for width in (2, 4, 5, 8, 9, 16):
        qw = _randn_bf16((rows, width, HQ, D), 6, dev)
        wpos = (t_lens[:, None] - width + torch.arange(width, device=dev, dtype=torch.int32)[None, :]).contiguous()
        wbytes = kv_bytes + table_bytes + rows * width * (HQ * D * 2 + HQ * D * 4)
        report("wide decode, %d query tokens per row (automatic: mma.sync tiles up to width 4, tcgen05 beyond)" % width,
               big.run(lambda: kvc.paged_attention_decode(qw, k, v, tables, t_lens, BS, SCALE, 4, positions=wpos, out_dtype=torch.float32)),
               wbytes, {"workload": "c2, width %d" % width})
        if width > 8:  # the mma.sync form ends at 8
            continue
        other, name = (1, "mma.sync tiles, two row tiles per warp pair") if width > 4 else (2, "tcgen05, query rows in a 128-row tile")
        report("wide decode, %d query tokens per row (%s)" % (width, name),
               big.run(lambda: K.paged_decode_attention_wide(qw, k[0], v[0], tables, t_lens, wpos, SCALE, form=other)),
               wbytes, {"workload": "c2, width %d" % width})
    width = 4
    qw = _randn_bf16((rows, width, HQ, D), 6, dev)
    wpos = (t_lens[:, None] - width + torch.arange(width, device=dev, dtype=torch.int32)[None, :]).contiguous()
    wbytes = kv_bytes + table_bytes + rows * width * (HQ * D * 2 + HQ * D * 4)
    qsl_w = torch.arange(rows + 1, dtype=torch.int32, device=dev) * width
    report("wide decode as a packed batch of equal-width rows (tcgen05 prefill tiles; what widths above 8 take)",
           big.run(lambda: K.packed_paged_prefill_attention(qw.reshape(1, rows * width, HQ, D), k[0], v[0], tables, t_lens,
                                                            wpos.reshape(1, -1), qsl_w, BS, SCALE, 4, num_decode_rows=0)),
           wbytes, {"workload": "c2, width 4"})
    rep_tables = tables.repeat_interleave(width, dim=0)
    rep_lens = torch.minimum(t_lens[:, None], wpos + 1).reshape(-1).contiguous()
    report("wide decode as 4 width-1 rows per sequence (decode kernel)",
           big.run(lambda: K.paged_decode_attention(qw.reshape(rows * width, HQ, D), k[0], v[0], rep_tables, rep_lens, SCALE)),
           wbytes, {"workload": "c2, width 4", "note": "K/V read once per query token"})
    K.check_device_status(dev)
    del k, v


def prefill_and_copy_cases(dev, iters, small=False):
    rng = np.random.default_rng(3)
    pool, chunk, layers = (4096, 512, 1) if small else (65_536, 512, 6)
    prompts = rng.integers(64, 2049, size=8)
    prompts[:4] = np.maximum(prompts[:4], 513)  # rows 0-3 share a 512-token prefix
    k = _randn_bf16((layers, pool, BS, HKV, D), 11, dev)
    v = _randn_bf16((layers, pool, BS, HKV, D), 12, dev)
    tables_np = tables_for(prompts.astype(np.int32), pool, rng)
    tables = torch.from_numpy(tables_np).to(dev)
    # one representative packed chunk: 512 tokens over the rows that still have work after 512 tokens each
    done = np.minimum(prompts, 512)
    take, left = [], chunk
    for r in range(8):
        t = int(min(prompts[r] - done[r], left))
        take.append(t)
        left -= t
    rows = [r for r in range(8) if take[r] > 0]
    qsl = np.concatenate([[0], np.cumsum([take[r] for r in rows])]).astype(np.int32)
    total = int(qsl[-1])
    pos = np.zeros((1, chunk), np.int32)
    rid = np.zeros((1, chunk), np.int32)
    pos[0, :total] = np.concatenate([np.arange(done[r], done[r] + take[r]) for r in rows])
    rid[0, :total] = np.repeat(np.arange(len(rows)), [take[r] for r in rows])
    kv_lens = np.array([done[r] + take[r] for r in rows], np.int32)
    t_tab = tables[torch.tensor(rows, device=dev)].contiguous()
    t_pos, t_rid = torch.from_numpy(pos).to(dev), torch.from_numpy(rid).to(dev)
    t_qsl, t_len = torch.from_numpy(qsl).to(dev), torch.from_numpy(kv_lens).to(dev)
    q = _randn_bf16((1, chunk, HQ, D), 13, dev)
    nk = _randn_bf16((1, chunk, HKV, D), 14, dev)
    nv = _randn_bf16((1, chunk, HKV, D), 15, dev)
    slots = K.compute_slot_mapping(t_pos, t_tab, BS, t_rid)
    tm = Timer(dev, iters)
    report("kv_append (packed prefill chunk, %d valid of 512 tokens)" % total,
           tm.run(lambda: K.kv_append_slots(nk, nv, slots, k[0], v[0], query_start_loc=t_qsl, packed=True)),
           2 * total * TOKEN_BYTES + chunk * 4, {"workload": "c3 chunk"})
    visible = int(sum(int(pos[0, i]) + 1 for i in range(total)))
    flops = 4 * HQ * D * visible
    nbytes = total * TOKEN_BYTES * 2 + int(kv_lens.sum()) * TOKEN_BYTES + total * (HQ * D * 2 + HQ * D * 4)
    for variant, name in ((2, "mma.sync tiles"), (3, "tcgen05 tiles"), (4, "tcgen05 CTA pairs"), (5, "tcgen05 CTA pairs, bf16 P")):
        us = tm.run(lambda: K.packed_paged_prefill_attention(q, k[0], v[0], t_tab, t_len, t_pos, t_qsl, BS, SCALE, 4,
                                                             variant=variant, num_decode_rows=0))
        report("packed prefill attention, %s (%d tokens, %d rows)" % (name, total, len(rows)), us, nbytes,
               {"workload": "c3 chunk", "TFLOP/s": round(flops / us / 1e6, 2), "flops": flops})
    # one 512-token chunk behind a long cached prefix: few query tiles, long key ranges (what the key-range splits are for)
    for prefix in (512, 1536, 3584):
        if (prefix + chunk) // BS > pool:
            continue
        c_tab = torch.from_numpy(rng.permutation(pool)[:(prefix + chunk) // BS].astype(np.int32).reshape(1, -1)).to(dev)
        c_pos = (prefix + torch.arange(chunk, dtype=torch.int32, device=dev))[None].contiguous()
        c_qsl = torch.tensor([0, chunk], dtype=torch.int32, device=dev)
        c_len = torch.tensor([prefix + chunk], dtype=torch.int32, device=dev)
        c_flops = 4 * HQ * D * sum(prefix + i + 1 for i in range(chunk))
        c_bytes = (prefix + chunk) * TOKEN_BYTES + chunk * (HQ * D * 2 + HQ * D * 4)
        for splits in ("1", "0"):
            os.environ["NVJ_PREFILL_KEY_SPLITS"] = splits
            us = tm.run(lambda: K.packed_paged_prefill_attention(q, k[0], v[0], c_tab, c_len, c_pos, c_qsl, BS, SCALE, 4,
                                                                 variant=4, num_decode_rows=0))
            report("packed prefill attention, tcgen05 CTA pairs, key ranges %s (512-token chunk behind %d cached tokens)"
                   % ("split" if splits == "1" else "unsplit", prefix), us, c_bytes,
                   {"workload": "chunk behind a prefix", "TFLOP/s": round(c_flops / us / 1e6, 2), "flops": c_flops})
        os.environ.pop("NVJ_PREFILL_KEY_SPLITS", None)
    # long prompts in a single chunk, nothing cached
    for n_long in (4096, 16384):
        if n_long // BS > pool:
            continue
        l_tab = torch.from_numpy(rng.permutation(pool)[:n_long // BS].astype(np.int32).reshape(1, -1)).to(dev)
        l_pos = torch.arange(n_long, dtype=torch.int32, device=dev)[None]
        l_qsl = torch.tensor([0, n_long], dtype=torch.int32, device=dev)
        l_len = torch.tensor([n_long], dtype=torch.int32, device=dev)
        lq = _randn_bf16((1, n_long, HQ, D), 16, dev)
        l_flops = 4 * HQ * D * (n_long * (n_long + 1) // 2)
        l_bytes = n_long * TOKEN_BYTES + n_long * (HQ * D * 2 + HQ * D * 4)
        for variant, name in ((2, "mma.sync tiles"), (3, "tcgen05 tiles"), (4, "tcgen05 CTA pairs"), (5, "tcgen05 CTA pairs, bf16 P")):
            if variant == 2 and n_long > 4096:
                continue
            us = tm.run(lambda: K.packed_paged_prefill_attention(lq, k[0], v[0], l_tab, l_len, l_pos, l_qsl, BS, SCALE, 4,
                                                                 variant=variant, num_decode_rows=0))
            report("packed prefill attention, %s (one row of %d tokens)" % (name, n_long), us, l_bytes,
                   {"workload": "long prompt", "TFLOP/s": round(l_flops / us / 1e6, 2), "flops": l_flops})
        del lq
    src = torch.from_numpy(tables_np[0, :32].copy()).to(dev)
    used = set(tables_np.reshape(-1).tolist())
    dst = torch.tensor([b for b in range(pool) if b not in used][:32], dtype=torch.int32, device=dev)
    report("copy_blocks (32-block prefix, %d layers, K and V)" % layers, tm.run(lambda: K.copy_blocks(k, v, src, dst)),
           2 * 32 * 2 * BS * HKV * D * 2 * layers, {"workload": "c3 prefix"})
    K.check_device_status(dev)
    del k, v


def norm_rope_append_cases(dev, iters):
    """RMSNorm(q, k) + partial RoPE + append in one launch: a 256-row decode step and a 512-token prefill chunk."""
    rng = np.random.default_rng(6)
    pool = 65_536
    k = _randn_bf16((1, pool, BS, HKV, D), 31, dev)
    v = _randn_bf16((1, pool, BS, HKV, D), 32, dev)
    qw, kw = _randn_bf16((D,), 33, dev) * 0.1, _randn_bf16((D,), 34, dev) * 0.1
    tm = Timer(dev, iters)
    for rows, cols, name in ((256, 1, "256 decode rows"), (1, 512, "512-token packed chunk")):
        n = rows * cols
        qg = _randn_bf16((rows, cols, HQ, 2 * D), 35, dev)  # query|gate projection: q is its strided first half
        nk, nv = _randn_bf16((rows, cols, HKV, D), 36, dev), _randn_bf16((rows, cols, HKV, D), 37, dev)
        pos = torch.from_numpy(rng.integers(0, 4096, size=(rows, cols)).astype(np.int32)).to(dev)
        slots = torch.from_numpy(rng.permutation(pool * BS)[:n].reshape(rows, cols).astype(np.int32)).to(dev)
        nbytes = n * (2 * HQ * D * 2 + 2 * 2 * HKV * D * 2 + 8)
        us = tm.run(lambda: K.qk_norm_rope_kv_append(qg[..., :D], nk, nv, qw, kw, pos, slots, k[0], v[0]))
        report("qk_norm + rope + kv_append fused (%s)" % name, us, nbytes, {"workload": "front of the path"})
    K.check_device_status(dev)
    del k, v


def comparator_case(dev, iters):
    """External yard-stick, not a dependency of the product: FlashInfer's batch decode over the same paged cache
    (the reference's promoted decode route is this library, nanovllm_jax/kernels/flashinfer_ffi.py:991-1086),
    timed on the C2 rows beside this library's decode kernel.  Skipped with a line saying so when FlashInfer
    cannot be imported or cannot build its kernel offline."""
    try:
        import flashinfer
    except Exception as exc:  # pragma: no cover
        print(json.dumps({"kernel": "flashinfer BatchDecodeWithPagedKVCacheWrapper", "unavailable": repr(exc)}), flush=True)
        return
    rng = np.random.default_rng(2)
    rows, pool = 256, 400_000
    ctx = rng.integers(1024, 4097, size=rows)
    lens = (ctx + 1).astype(np.int32)
    tables_np = tables_for(lens, pool, rng)
    need = -(-lens // BS)
    indptr = np.concatenate([[0], np.cumsum(need)]).astype(np.int32)
    indices = np.concatenate([tables_np[r, :need[r]] for r in range(rows)]).astype(np.int32)
    last = ((lens - 1) % BS + 1).astype(np.int32)
    k = _randn_bf16((pool, BS, HKV, D), 1, dev)
    v = _randn_bf16((pool, BS, HKV, D), 2, dev)
    q = _randn_bf16((rows, HQ, D), 3, dev)
    tables, t_lens = torch.from_numpy(tables_np).to(dev), torch.from_numpy(lens).to(dev)
    nbytes = int(lens.sum()) * TOKEN_BYTES + int(need.sum()) * 4 + rows * HQ * D * (2 + 4) + rows * 12
    big = Timer(dev, iters, flush=False)
    mine = K.paged_decode_attention(q, k, v, tables, t_lens, SCALE)
    report("paged_decode (this library)", big.run(lambda: K.paged_decode_attention(q, k, v, tables, t_lens, SCALE)), nbytes,
           {"workload": "c2"})
    ws = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for tc in (False, True):
        name = "flashinfer %s BatchDecodeWithPagedKVCacheWrapper (use_tensor_cores=%s)" % (flashinfer.__version__, tc)
        try:
            w = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD", use_tensor_cores=tc)
            w.plan(torch.from_numpy(indptr).to(dev), torch.from_numpy(indices).to(dev), torch.from_numpy(last).to(dev),
                   HQ, HKV, D, BS, pos_encoding_mode="NONE", q_data_type=torch.bfloat16, kv_data_type=torch.bfloat16,
                   sm_scale=SCALE)
            theirs = w.run(q, (k, v))
            us = big.run(lambda: w.run(q, (k, v)))
        except Exception as exc:
            print(json.dumps({"kernel": name, "unavailable": repr(exc)[:200]}), flush=True)
            continue
        report(name, us, nbytes, {"workload": "c2", "max_abs_diff_vs_this_library": float((mine - theirs.float()).abs().max()),
                                  "note": "bf16 output; plan() outside the timed region"})
    del k, v
    # ---- paged prefill: one prompt in one chunk, and a 512-token chunk behind a 512-token cached prefix
    pool2 = 4096
    k = _randn_bf16((pool2, BS, HKV, D), 11, dev)
    v = _randn_bf16((pool2, BS, HKV, D), 12, dev)
    tm = Timer(dev, iters)
    ws2 = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    for n_ctx, chunk in ((1024, 512), (4096, 4096), (16384, 16384)):
        nblk = n_ctx // BS
        idx = rng.permutation(pool2)[:nblk].astype(np.int32)
        q = _randn_bf16((chunk, HQ, D), 13, dev)
        tab = torch.from_numpy(idx.reshape(1, -1)).to(dev)
        pos = torch.arange(n_ctx - chunk, n_ctx, dtype=torch.int32, device=dev)[None]
        qsl = torch.tensor([0, chunk], dtype=torch.int32, device=dev)
        lens1 = torch.tensor([n_ctx], dtype=torch.int32, device=dev)
        flops = 4 * HQ * D * (n_ctx * (n_ctx + 1) // 2 - (n_ctx - chunk) * (n_ctx - chunk + 1) // 2)
        nb2 = chunk * (HQ * D * 2 + HQ * D * 4) + n_ctx * TOKEN_BYTES
        mine = K.packed_paged_prefill_attention(q[None], k, v, tab, lens1, pos, qsl, BS, SCALE, 4, num_decode_rows=0)
        us = tm.run(lambda: K.packed_paged_prefill_attention(q[None], k, v, tab, lens1, pos, qsl, BS, SCALE, 4, num_decode_rows=0))
        report("packed prefill (this library), %d tokens at context %d" % (chunk, n_ctx), us, nb2,
               {"workload": "prefill", "TFLOP/s": round(flops / us / 1e6, 1)})
        name = "flashinfer %s BatchPrefillWithPagedKVCacheWrapper, %d tokens at context %d" % (flashinfer.__version__, chunk, n_ctx)
        try:
            w = flashinfer.BatchPrefillWithPagedKVCacheWrapper(ws2, "NHD")
            w.plan(torch.tensor([0, chunk], dtype=torch.int32, device=dev), torch.tensor([0, nblk], dtype=torch.int32, device=dev),
                   torch.from_numpy(idx).to(dev), torch.tensor([BS], dtype=torch.int32, device=dev), HQ, HKV, D, BS, causal=True,
                   sm_scale=SCALE, q_data_type=torch.bfloat16, kv_data_type=torch.bfloat16)
            theirs = w.run(q, (k, v))
            us = tm.run(lambda: w.run(q, (k, v)))
        except Exception as exc:
            print(json.dumps({"kernel": name, "unavailable": repr(exc)[:200]}), flush=True)
            continue
        report(name, us, nb2, {"workload": "prefill", "TFLOP/s": round(flops / us / 1e6, 1),
                               "max_abs_diff_vs_this_library": float((mine.reshape(chunk, HQ, D) - theirs.float()).abs().max()),
                               "note": "bf16 output; plan() outside the timed region"})
    del k, v


def mixed_step_case(dev, iters):
    """The KV path of one mixed continuous-batching step over 6 layers: 32 decode rows (contexts in
    [128, 2048]) plus 2 prefill chunks of 256 tokens, packed; per layer one append and one attention."""
    from nano_vllm_jax_b200.backends import B200Backend
    from nano_vllm_jax_b200.kv_cache import KVCacheStorage
    rng = np.random.default_rng(4)
    layers, pool = 6, 8192
    ctx = rng.integers(128, 2049, size=32)
    starts = np.concatenate([ctx - 1, [256, 0]])          # first position each row runs this step
    qlens = np.array([1] * 32 + [256, 256])
    kv_lens = (starts + qlens).astype(np.int32)
    tables = torch.from_numpy(tables_for(kv_lens, pool, rng)).to(dev)
    total = int(qlens.sum())
    pos = torch.from_numpy(np.concatenate([np.arange(s, s + n) for s, n in zip(starts, qlens)]).astype(np.int32)[None]).to(dev)
    rid = torch.from_numpy(np.repeat(np.arange(34), qlens).astype(np.int32)[None]).to(dev)
    qsl = torch.from_numpy(np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)).to(dev)
    t_len = torch.from_numpy(kv_lens).to(dev)
    k = _randn_bf16((layers, pool, BS, HKV, D), 21, dev)
    v = _randn_bf16((layers, pool, BS, HKV, D), 22, dev)
    q = _randn_bf16((1, total, HQ, D), 23, dev)
    nk = _randn_bf16((1, total, HKV, D), 24, dev)
    nv = _randn_bf16((1, total, HKV, D), 25, dev)
    be = B200Backend(device=dev)
    cache = KVCacheStorage(k, v)
    md = be.build_attention_metadata(pos, tables, t_len, BS, True, query_start_loc=qsl, token_row_ids=rid,
                                     query_lens_host=tuple(int(n) for n in qlens))

    def step():
        for layer in range(layers):
            be.write_kv_and_attention(layer, q, nk, nv, cache, md, BS, SCALE, 4, True)

    visible = int(sum(int(x) + 1 for x in pos[0].tolist()))
    nbytes = layers * (2 * total * TOKEN_BYTES + int(kv_lens.sum()) * TOKEN_BYTES + total * (HQ * D * 2 + HQ * D * 4))
    us = Timer(dev, iters).run(step)
    report("mixed step KV path, 6 layers (32 decode rows + 2 x 256 prefill tokens, packed), eager launches", us, nbytes,
           {"workload": "c4", "TFLOP/s": round(layers * 4 * HQ * D * visible / us / 1e6, 2)})
    # the same step replayed from one CUDA graph: the host's launch rate is out of the figure
    from nano_vllm_jax_b200.engine.resident_decode import CapturedStep
    captured = CapturedStep(step, dev)
    captured.capture()
    us = Timer(dev, iters).run(captured.replay)
    report("mixed step KV path, 6 layers (32 decode rows + 2 x 256 prefill tokens, packed), one CUDA graph", us, nbytes,
           {"workload": "c4", "TFLOP/s": round(layers * 4 * HQ * D * visible / us / 1e6, 2)})
    K.check_device_status(dev)


def hybrid_cases(dev, iters):
    for n in (1, 8):
        table = HybridStateTable((18, 6144, 4), (18, 16, 128, 128), max_slots=16, conv_dtype=torch.bfloat16, device=dev)
        cache = PrefixStateCache(table, capacity=16)
        ids = list(range(n))
        for i in ids:
            table.state(i).recurrent_state.normal_()
        row = 18 * 16 * 128 * 128 * 4 + 18 * 6144 * 4 * 2
        tm = Timer(dev, iters)
        report("hybrid snapshot (%d sequences)" % n, tm.run(lambda: cache.snapshot(ids, [100 + i for i in ids])),
               2 * n * row, {"workload": "c4 state", "note": "includes the host-side index upload"})
        report("hybrid restore (%d sequences)" % n, tm.run(lambda: cache.restore(ids, [100 + i for i in ids])),
               2 * n * row, {"workload": "c4 state", "note": "includes the host-side index upload"})
        slots = torch.tensor([table.slot(i) for i in ids], dtype=torch.int32, device=dev)
        rows = torch.arange(n, dtype=torch.int32, device=dev)
        report("hybrid state copy kernel alone (%d sequences)" % n,
               tm.run(lambda: K.hybrid_copy(table.conv, table.rec, cache.conv_pool, cache.rec_pool, slots, rows, restore=False)),
               2 * n * row, {"workload": "c4 state", "note": "indices already on the device"})
        del table, cache
    K.check_device_status(dev)


def _use_phase_timing_library():
    """Build the library once more with -DNVJ_PHASE_TIMING (under the package's build/ folder, beside the normal one)
    and make it the one this process loads: the streaming decode kernel then stamps the global timer at its phase
    boundaries and `nvj_debug_phase_ns` copies the stamps out."""
    from pathlib import Path

    from nano_vllm_jax_b200 import build as B
    B.NVCC_FLAGS = B.NVCC_FLAGS + ["-DNVJ_PHASE_TIMING"]
    B.OBJ_DIR = B.PKG_DIR / "build" / "phase"
    B.OBJ_DIR.mkdir(parents=True, exist_ok=True)
    B.LIB_PATH = Path(B.OBJ_DIR) / "libnvj_b200_phase.so"
    B.build()


def decode_phase_cases(dev, iters):
    """Where the time of a SHORT decode batch goes: per case, the kernel's phase boundaries relative to the first
    CTA's entry (min / median / max over the CTAs of the last launch), next to the CUDA-event time of the call."""
    import ctypes

    from nano_vllm_jax_b200 import _lib
    lib = _lib.load()
    lib.nvj_debug_phase_ns.argtypes = [ctypes.c_void_p]
    lib.nvj_debug_phase_ns.restype = ctypes.c_int
    pool = 48_000
    k = _randn_bf16((1, pool, BS, HKV, D), 1, dev)
    v = _randn_bf16((1, pool, BS, HKV, D), 2, dev)
    timer = Timer(dev, iters)
    names = ["entry", "lengths scanned", "start located, barriers up", "block ids staged, first copies issued",
             "first block landed", "last block done", "segment finished (folds included)", "partial counted in"]
    rng = np.random.default_rng(2)
    c2_lens = (rng.integers(1024, 4097, size=256) + 1).astype(np.int32)  # the benchmark's batch, for comparison
    for rows, ctx in ((1, 32768), (16, 4096), (32, 1500), (8, 1040), (256, 0)):
        if ctx:
            nb = -(-ctx // BS)
            tables = torch.randperm(pool, device=dev)[: rows * nb].to(torch.int32).view(rows, nb).contiguous()
            lens = torch.full((rows,), ctx, dtype=torch.int32, device=dev)
        else:  # 256 rows of U[1024, 4096] tokens over the same pool (blocks drawn without replacement)
            tables = torch.from_numpy(tables_for(c2_lens, pool, rng)).to(dev)
            lens = torch.from_numpy(c2_lens).to(dev)
        q = _randn_bf16((rows, HQ, D), 3, dev)
        us = timer.run(lambda: K.paged_decode_attention(q, k[0], v[0], tables, lens, SCALE, variant=3))
        host = np.zeros((256, 12), np.uint64)
        if lib.nvj_debug_phase_ns(host.ctypes.data) != 0:
            raise RuntimeError("nvj_debug_phase_ns failed")
        if os.environ.get("NVJ_PHASE_DUMP"):  # per CTA: index, SM, blocks, first block landed, last block done (us)
            base_ns = int(host[:, 0].max()) - 400_000
            t_first = int(host[host[:, 0] >= base_ns][:, 0].min())
            np.savetxt(os.environ["NVJ_PHASE_DUMP"] + "_%dx%d.txt" % (rows, ctx),
                       np.array([[i, int(host[i, 8]), int(host[i, 9]), (int(host[i, 4]) - t_first) / 1e3, (int(host[i, 5]) - t_first) / 1e3,
                                  int(host[i, 10]) / 1e3, int(host[i, 11])]
                                 for i in range(256) if host[i, 0] >= base_ns]), fmt="%.2f")
        t0 = host[:, 0].astype(np.int64)
        live = t0 >= t0.max() - 200_000  # CTAs of the last launch
        rel = (host[live].astype(np.int64) - t0[live].min()) / 1e3
        phases = {}
        for i, name in enumerate(names):
            col = rel[:, i]
            col = col[col >= 0]  # a CTA that left early keeps an older launch's stamp
            if len(col):
                phases[name] = {"min": round(float(col.min()), 2), "median": round(float(np.median(col)), 2),
                                "max": round(float(col.max()), 2), "ctas": int(len(col))}
        report("paged_decode, %d rows x %s tokens: phases in us after the first CTA's entry" % (rows, ctx or "U[1024, 4096]"), us,
               int(lens.sum().item()) * TOKEN_BYTES, {"workload": "short batch" if ctx else "c2 lengths", "ctas": int(live.sum()), "phases": phases})
    K.check_device_status(dev)
    del k, v

    # the CTA-pair prefill kernel on a 512-token chunk behind a 512-token prefix: per CTA, phases and key tiles
    lib.nvj_debug_prefill_phase_ns.argtypes = [ctypes.c_void_p]
    lib.nvj_debug_prefill_phase_ns.restype = ctypes.c_int
    pool, chunk, prefix = 4096, 512, 512
    k = _randn_bf16((1, pool, BS, HKV, D), 11, dev)
    v = _randn_bf16((1, pool, BS, HKV, D), 12, dev)
    tab = torch.randperm(pool, device=dev)[: (prefix + chunk) // BS].to(torch.int32).view(1, -1).contiguous()
    pos = (prefix + torch.arange(chunk, dtype=torch.int32, device=dev))[None].contiguous()
    qsl = torch.tensor([0, chunk], dtype=torch.int32, device=dev)
    kvl = torch.tensor([prefix + chunk], dtype=torch.int32, device=dev)
    q = _randn_bf16((1, chunk, HQ, D), 13, dev)
    us = timer.run(lambda: K.packed_paged_prefill_attention(q, k[0], v[0], tab, kvl, pos, qsl, BS, SCALE, 4, variant=4,
                                                            num_decode_rows=0))
    host = np.zeros((512, 8), np.uint64)
    if lib.nvj_debug_prefill_phase_ns(host.ctypes.data) != 0:
        raise RuntimeError("nvj_debug_prefill_phase_ns failed")
    t0 = host[:, 0].astype(np.int64)
    live = (t0 >= t0.max() - 200_000) & (host[:, 7] > 0)  # CTAs of the last launch that had key tiles
    rel = (host[live, :7].astype(np.int64) - t0[t0 >= t0.max() - 200_000].min()) / 1e3
    names = ["entry", "set up (tensor memory, barriers, cluster barrier)", "query rows staged", "first scores ready",
             "last tile's weights written", "output written", "pair released"]
    per_cta = [{"tiles": int(host[i, 7]), **{names[j]: round(float((int(host[i, j]) - int(t0[t0 >= t0.max() - 200_000].min())) / 1e3), 2)
                                               for j in range(7)}} for i in np.nonzero(live)[0]]
    per_cta.sort(key=lambda d: d["tiles"])
    flops = 4 * HQ * D * int(sum(prefix + i + 1 for i in range(chunk)))
    report("packed prefill, tcgen05 CTA pairs, %d-token chunk behind a %d-token prefix: phases in us after the first CTA's entry"
           % (chunk, prefix), us, (prefix + chunk) * TOKEN_BYTES + chunk * HQ * D * 6,
           {"workload": "c3 chunk", "TFLOP/s": round(flops / us / 1e6, 2), "ctas": int(live.sum()),
            "fewest_tiles": per_cta[0], "most_tiles": per_cta[-1], "kernel_end": round(float(rel[:, 6].max()), 2)})
    K.check_device_status(dev)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill", "hybrid", "mixed", "front", "comparator", "phases"])
    ap.add_argument("--small", action="store_true",
                    help="prefill cases on a 1-layer, 4096-block cache (128 MiB), decode cases on 64 rows over a 40 000-block cache (2.6 GB): the sizes to run under a profiler")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.only == "phases":  # its own library build: not part of "all"
        _use_phase_timing_library()
        decode_phase_cases(dev, args.iters)
        return
    if args.only in ("all", "decode"):
        decode_cases(dev, args.iters, small=args.small)
    if args.only in ("all", "prefill"):
        prefill_and_copy_cases(dev, args.iters, small=args.small)
    if args.only in ("all", "hybrid"):
        hybrid_cases(dev, args.iters)
    if args.only in ("all", "mixed"):
        mixed_step_case(dev, args.iters)
    if args.only in ("all", "front"):
        norm_rope_append_cases(dev, args.iters)
    if args.only == "comparator":
        comparator_case(dev, args.iters)


if __name__ == "__main__":
    main()
