"""Generate tests/golden/decode_step_small.npz and tests/golden/prefill_chunk_small.npz from the CPU oracle.

The reference cannot be imported where this was written (it needs JAX, which is
not installed), so these vectors come from the NumPy restatement in oracle/ and
pin IT: a later change to the oracle, or a kernel that drifts, shows up against
stored bytes.  Run from the repository root:  python tests/golden/make_golden.py
"""

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import BS, SCALE, decode_case  # noqa: E402
from oracle import kv_cache_ref as R  # noqa: E402
from oracle import norm_rope_ref as N  # noqa: E402


def main():
    c = decode_case(1234, 12, 3, 5, 50)  # 3 rows, contexts in [5, 50], 12-block bf16 pool, model head shape
    slots = R.compute_slot_mapping(c["positions"], c["tables"], BS)
    ek, ev = R.update_kv_cache(c["k_cache"], c["v_cache"], slots, c["new_k"], c["new_v"], 0)
    out32 = R.paged_attention_decode(c["q"], ek, ev, c["tables"], c["seq_lens"], BS, SCALE, 4, mode="fp32")
    outref = R.paged_attention_decode(c["q"], ek, ev, c["tables"], c["seq_lens"], BS, SCALE, 4, mode="ref")
    u16 = lambda a: np.ascontiguousarray(a).view(np.uint16)
    np.savez_compressed(
        os.path.join(ROOT, "tests", "golden", "decode_step_small.npz"),
        k_cache=u16(c["k_cache"]), v_cache=u16(c["v_cache"]), q=u16(c["q"]), new_k=u16(c["new_k"]),
        new_v=u16(c["new_v"]), tables=c["tables"], seq_lens=c["seq_lens"], positions=c["positions"], slots=slots,
        k_after=u16(ek), v_after=u16(ev), out_fp32=out32, out_ref_bf16=u16(outref))


def prefill_chunk():
    """A packed chunk step: rows of 21 (cached prefix 48), 1 (decode row, 70 cached) and 12 tokens plus 6 pad tokens,
    through q/k RMSNorm + partial RoPE + append and packed prefill attention; 12-block pool.  Only the cache rows the
    step writes are stored for the "after" state."""
    from ml_dtypes import bfloat16
    rng = np.random.default_rng(4321)
    d, hq, hkv, nb, bucket = 256, 8, 2, 12, 40
    cached, chunk = [48, 70, 0], [21, 1, 12]
    ends = [c + n for c, n in zip(cached, chunk)]
    need = [-(-e // BS) for e in ends]
    perm = rng.permutation(nb)
    tables = np.zeros((3, max(need)), np.int32)
    o = 0
    for r in range(3):
        tables[r, :need[r]] = perm[o:o + need[r]]
        o += need[r]
    total = sum(chunk)
    pos = np.zeros((1, bucket), np.int32)
    rid = np.zeros((1, bucket), np.int32)
    pos[0, :total] = np.concatenate([np.arange(c, e) for c, e in zip(cached, ends)])
    rid[0, :total] = np.repeat(np.arange(3), chunk)
    qsl = np.concatenate([[0], np.cumsum(chunk)]).astype(np.int32)
    kc = rng.standard_normal((1, nb, BS, hkv, d), dtype=np.float32).astype(bfloat16)
    vc = rng.standard_normal((1, nb, BS, hkv, d), dtype=np.float32).astype(bfloat16)
    q_raw = (rng.standard_normal((1, bucket, hq, d), dtype=np.float32) * 1.5).astype(bfloat16)
    k_raw = (rng.standard_normal((1, bucket, hkv, d), dtype=np.float32) * 0.7).astype(bfloat16)
    v_raw = rng.standard_normal((1, bucket, hkv, d), dtype=np.float32).astype(bfloat16)
    qw = (rng.standard_normal(d, dtype=np.float32) * 0.2).astype(bfloat16)
    kw = (rng.standard_normal(d, dtype=np.float32) * 0.2).astype(bfloat16)
    slots = R.compute_packed_slot_mapping(pos, tables, rid, BS)
    valid = R.write_kv_valid_mask(slots.shape, qsl, True)
    q, ek, ev = N.qk_norm_rope_kv_append(q_raw, k_raw, v_raw, qw, kw, pos, slots, kc, vc, valid_mask=valid)
    out = R.paged_attention_prefill_packed(q, ek, ev, tables, np.array(ends, np.int32), pos, rid, qsl, BS, SCALE, 4)
    u16 = lambda a: np.ascontiguousarray(a).view(np.uint16)
    np.savez_compressed(
        os.path.join(ROOT, "tests", "golden", "prefill_chunk_small.npz"),
        k_cache=u16(kc), v_cache=u16(vc), q_raw=u16(q_raw), k_raw=u16(k_raw), v_raw=u16(v_raw), q_norm=u16(qw), k_norm=u16(kw),
        tables=tables, kv_lens=np.array(ends, np.int32), positions=pos, row_ids=rid, query_start_loc=qsl, slots=slots,
        q_after=u16(q), k_rows_after=u16(ek.reshape(-1, hkv, d)[slots[0, :total]]),
        v_rows_after=u16(ev.reshape(-1, hkv, d)[slots[0, :total]]), out_fp32=out.astype(np.float32))


if __name__ == "__main__":
    main()
    prefill_chunk()
