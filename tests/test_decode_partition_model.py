"""The index arithmetic behind the decode kernels' cross-CTA merge, restated in Python and checked on random batches.

The kernels (csrc/decode_parts.cuh) cut the sequence of all blocks of all rows into one contiguous range per CTA;
behind the blocks of every non-empty row the sequence holds ROW_END_COST phantom blocks that nobody reads, so that a
range with more row ends gets fewer real blocks.
A CTA parks the partial result of a row it shares with other CTAs in slot 2c (the row began elsewhere) or 2c + 1
(the row begins here); a row cut into more than 32 partials is merged per group of 13 consecutive CTA ids first,
with counter and slot 2g (+ 1 if the row begins in group g).  These tests check what the kernels rely on: no two
partials share a slot, no two rows share a group counter, and the arrival counts add up.
"""

import numpy as np
import pytest

MIN_BLOCKS_PER_CTA, GROUP, TREE_MIN, ROW_END_COST = 6, 13, 32, 6


def in_sequence(nb):
    return nb + ROW_END_COST if nb > 0 else 0


def partition(total, grid):
    cap = -(-total // MIN_BLOCKS_PER_CTA)
    return min(cap, grid)


def start(c, total, n):
    return c * total // n


def cta_of(g, total, n):
    return ((g + 1) * n - 1) // total


def segments(blocks_per_row, grid):
    """(cta, row, j0, j1) for every row segment with real blocks, the way next_seg walks them; the positions of the
    rows in the sequence; the sequence's length; the number of ranges."""
    seq = [in_sequence(int(nb)) for nb in blocks_per_row]
    total = int(sum(seq))
    n = partition(total, grid)
    row_start = np.concatenate([[0], np.cumsum(seq)])
    out = []
    for c in range(n):
        g0, g1 = start(c, total, n), start(c + 1, total, n)
        b = int(np.searchsorted(row_start, g0, side="right") - 1)
        g = g0
        while g < g1:
            while seq[b] == 0 or g >= row_start[b + 1]:
                b += 1
            j0 = g - row_start[b]
            take = min(seq[b] - j0, g1 - g)
            j1 = min(j0 + take, int(blocks_per_row[b]))
            if j1 > j0:  # a range may hold only phantom blocks of a row
                out.append((c, b, int(j0), int(j1)))
            g += take
    return out, row_start, total, n


@pytest.mark.parametrize("grid", [148, 296, 416])
@pytest.mark.parametrize("seed", range(6))
def test_slots_and_counters_are_private(grid, seed):
    rng = np.random.default_rng(seed)
    shape = [(1, 2001), (5, 900), (40, 300), (300, 40), (3, 1)][seed % 5]
    rows = int(rng.integers(1, shape[0] + 1))
    blocks = rng.integers(0, shape[1] + 1, size=rows)
    if blocks.sum() == 0:
        blocks[0] = 7
    segs, row_start, total, n = segments(blocks, grid)
    assert sum(j1 - j0 for _, _, j0, j1 in segs) == int(blocks.sum())  # every block is read exactly once
    seen = {}
    for c, b, j0, j1 in segs:
        assert seen.setdefault((b, j0), c) == c and j0 == sum(y - x for cc, bb, x, y in segs if bb == b and x < j0)  # in order, no gaps
    slots, group_keys, arrivals, group_arrivals = set(), {}, {}, {}
    for c, b, j0, j1 in segs:
        nb = int(blocks[b])
        if j0 == 0 and j1 == nb:
            continue  # the CTA holds the whole row: no partial
        c_lo, c_hi = cta_of(int(row_start[b]), total, n), cta_of(int(row_start[b]) + nb - 1, total, n)
        assert c_lo <= c <= c_hi and (j0 == 0) == (c == c_lo)
        slot = 2 * c + (1 if j0 == 0 else 0)
        assert slot not in slots, "two partials in one slot"
        slots.add(slot)
        arrivals[b] = arrivals.get(b, 0) + 1
        if c_hi - c_lo + 1 > TREE_MIN:
            g, g_lo = c // GROUP, c_lo // GROUP
            key = (g, g == g_lo)
            assert group_keys.setdefault(key, b) == b, "two rows on one group counter"
            group_arrivals[(b, g)] = group_arrivals.get((b, g), 0) + 1
    for b, count in arrivals.items():
        nb = int(blocks[b])
        c_lo, c_hi = cta_of(int(row_start[b]), total, n), cta_of(int(row_start[b]) + nb - 1, total, n)
        assert count == c_hi - c_lo + 1  # every CTA id inside the row's span delivers one partial
        if c_hi - c_lo + 1 > TREE_MIN:
            for g in range(c_lo // GROUP, c_hi // GROUP + 1):
                first, last = max(c_lo, g * GROUP), min(c_hi, g * GROUP + GROUP - 1)
                assert group_arrivals[(b, g)] == last - first + 1
            assert c_hi // GROUP - c_lo // GROUP + 1 <= 32  # what one fold takes
        else:
            assert count <= 32
    assert 2 * (-(-n // GROUP)) <= 64  # group counters in the workspace header
