"""Generate tests/golden/decode_step_small.npz from the CPU oracle.

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


if __name__ == "__main__":
    main()
