"""bench.py on the CPU: the workloads' row partition and block tables, the byte count behind the roofline
figure, and the line the reference arm prints (a small sample of rows through the CPU restatement)."""

import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_algorithmic_bytes_counts_every_operand_once():
    lens = np.array([1, 16, 17, 4096], np.int64)
    rows = len(lens)
    kv = int(lens.sum()) * 2048                       # K and V rows of every attended token, bf16
    new_rows = rows * 2048 * 2                        # the new K/V row read and written
    q_out = rows * 8 * 256 * (2 + 4)                  # query bf16 in, output fp32 out
    tables = (1 + 1 + 2 + 256) * 4                    # one block id per started block
    assert bench.algorithmic_bytes(lens, rows) == kv + new_rows + q_out + tables + rows * 12


def test_weak_scaling_ranks_draw_the_same_lengths_and_their_own_tables():
    w = bench.WORKLOADS["c2"]
    ctx0, tab0, pool0 = bench.make_rows(w, 0, 8, 109)
    ctx1, tab1, pool1 = bench.make_rows(w, 5, 8, 109)
    assert pool0 == pool1 == 400_000 and len(ctx0) == 256
    assert ctx0.min() >= 1024 and ctx0.max() <= 4096
    np.testing.assert_array_equal(ctx0, ctx1)
    assert not np.array_equal(tab0, tab1)
    need = -(-(ctx0 + 109) // 16)
    used = np.concatenate([tab0[b, :need[b]] for b in range(256)])
    assert len(np.unique(used)) == len(used) and used.min() >= 0 and used.max() < pool0  # no block serves two rows
    assert tab0.shape[1] == need.max()
    assert used.max() > 2 ** 18  # byte offsets beyond 4 GiB are part of the workload


def test_strong_scaling_deals_every_row_to_exactly_one_rank():
    w = bench.WORKLOADS["c5"]
    whole = bench.row_lengths(w, 0, 1)
    assert len(whole) == 2048 and whole.min() >= 8192 and whole.max() <= 32768
    for world in (2, 4, 8):
        parts = [bench.row_lengths(w, r, world) for r in range(world)]
        assert sum(len(p) for p in parts) == 2048
        dealt = np.empty(2048, np.int64)
        for r, p in enumerate(parts):
            dealt[r::world] = p
        np.testing.assert_array_equal(dealt, whole)


def test_pool_too_small_is_refused():
    w = dict(bench.WORKLOADS["c2small"])
    try:
        bench.make_rows(w, 0, 1, 10, pool_blocks=100)
    except RuntimeError as exc:
        assert "too small" in str(exc)
    else:
        raise AssertionError("a pool that cannot hold the rows was accepted")


def test_percentiles():
    p = bench.percentiles([5.0, 1.0, 3.0, 2.0, 4.0])
    assert p == {"median": 3.0, "p10": 1.0, "p90": 5.0, "n": 5}
    assert bench.percentiles([]) is None


def test_reference_arm_prints_the_contract_line():
    # 4 of the 64 rows of the reduced workload, one warm-up and one timed step: a few seconds of NumPy
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "c2small",
                          "--cpu-sample-rows", "4", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tok/s" and line["higher_is_better"] is True
    assert line["metric"] == "decode_tokens_per_s_paged_attention_plus_kv_append"
    assert line["value"] > 0 and line["steps"] == 1 and line["n_gpus"] == 1
    assert line["e2e"] == {"value": line["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["config"]["workload"].startswith("c2small")
    assert line["gpu_launches"] == 0
