"""Independent dense attention in float64.  TEST INFRASTRUCTURE ONLY.

Used to cross-check the paged oracle the way the reference's own tests do
(paged == dense, tests/test_backend_boundaries.py:315-378 in the reference):
keys and values are handed over as plain per-sequence arrays, no block table,
no slot arithmetic, and every (sequence, head) is one explicit softmax.
"""

from __future__ import annotations

import numpy as np


def dense_gqa_attention(q, keys, values, scale, groups, query_positions=None):
    """q [T, Hq, D]; keys/values [S, Hkv, D] (only the attended keys) -> [T, Hq, D] float64.

    query_positions[t], when given, limits query t to keys p <= query_positions[t].
    """
    q = np.asarray(q, np.float64)
    keys = np.asarray(keys, np.float64)
    values = np.asarray(values, np.float64)
    T, Hq, D = q.shape
    S = keys.shape[0]
    out = np.zeros((T, Hq, D))
    for t in range(T):
        n = S if query_positions is None else min(S, int(query_positions[t]) + 1)
        if n <= 0:
            continue
        for h in range(Hq):
            kv = h // groups
            s = keys[:n, kv] @ q[t, h] * scale
            w = np.exp(s - s.max())
            w /= w.sum()
            out[t, h] = w @ values[:n, kv]
    return out
