"""The baseline configurations at their stated sizes, against the CPU oracle.

  config 2   256 rows, contexts U[1024, 4096], block tables a scattered permutation over a 400 000-block pool
             (6.55 GB per array): the shape the benchmark times.  Fused append + decode.
  config 5   (shape of its rows) 8 rows of 30-32k tokens scattered over the same pool: byte offsets beyond 4 GiB,
             block ids beyond 2^18, rows cut over every CTA and merged in two levels.
  config 3   8 prompts U[64, 2048], rows 0-3 sharing a 512-token prefix, a 65 536-block pool, chunks of 512 tokens
             through the packed builder; the prefix served once by block sharing (reference count 4 on 32 blocks)
             and once by the block-copy kernel.

The oracle cannot hold pools of this size in host memory per call, so it works on the blocks the rows use, gathered
to the host and renumbered; values, table shapes and lengths are those of the device run.  Cache contents are
compared bit for bit, attention within 2e-3 (contract 2e-2).  Reference semantics: nanovllm_jax/kv_cache.py:476-564,
721-998; the reference's own paged-vs-dense checks are tests/test_backend_boundaries.py:4178-4313.
"""

import numpy as np
import pytest
import torch
from ml_dtypes import bfloat16

from helpers import BS, SCALE, bits, to_numpy, to_torch
from oracle import kv_cache_ref as R

pytestmark = pytest.mark.gpu

TIGHT = 2e-3
POOL = 400_000


def _K():
    from nano_vllm_jax_b200.kernels import paged_kv as K
    return K


def _fill(t, seed, chunk=8192):
    g = torch.Generator(device=t.device).manual_seed(seed)
    flat = t.view(t.shape[0], -1)
    for i in range(0, flat.shape[0], chunk):
        part = flat[i:i + chunk]
        part.copy_(torch.randn(part.shape, generator=g, device=t.device, dtype=torch.float32))


@pytest.fixture(scope="module")
def big_pool():
    free_b, _ = torch.cuda.mem_get_info()
    if free_b < 20e9:
        pytest.skip("needs 20 GB of free device memory")
    k = torch.empty((1, POOL, BS, 2, 256), dtype=torch.bfloat16, device="cuda")
    v = torch.empty_like(k)
    _fill(k[0], 11)
    _fill(v[0], 12)
    yield k, v
    del k, v
    torch.cuda.empty_cache()


def _tables(rng, lens, pool):
    need = -(-lens // BS)
    perm = rng.permutation(pool)
    tables = np.zeros((len(lens), int(need.max())), np.int32)
    o = 0
    for b in range(len(lens)):
        tables[b, :need[b]] = perm[o:o + need[b]]
        o += need[b]
    return tables, need


def _host_blocks(cache_layer, ids):
    return to_numpy(cache_layer[to_torch(np.asarray(ids, np.int64))])


def _oracle_row(k_layer, v_layer, table_row, length, q_row):
    """Oracle decode of one row on its own blocks, gathered to the host and renumbered 0..n-1."""
    nb = -(-int(length) // BS)
    k_np = _host_blocks(k_layer, table_row[:nb])[None]
    v_np = _host_blocks(v_layer, table_row[:nb])[None]
    return R.paged_attention_decode(q_row[None, None], k_np, v_np, np.arange(nb, dtype=np.int32)[None],
                                    np.array([length], np.int32), BS, SCALE, 4)[0, 0]


@pytest.mark.parametrize("variant", [3, 2])
def test_config2_fused_append_and_decode_at_the_benchmarked_size(big_pool, variant):
    K = _K()
    k_cache, v_cache = big_pool
    rng = np.random.default_rng(2)
    rows = 256
    ctx = rng.integers(1024, 4097, size=rows)
    lens = (ctx + 1).astype(np.int32)
    tables, need = _tables(rng, lens.astype(np.int64), POOL)
    assert tables.max() >= 1 << 18                      # rows reach beyond the first 4 GiB of each array
    q = rng.standard_normal((rows, 1, 8, 256), dtype=np.float32).astype(bfloat16)
    nk = rng.standard_normal((rows, 1, 2, 256), dtype=np.float32).astype(bfloat16)
    nv = rng.standard_normal((rows, 1, 2, 256), dtype=np.float32).astype(bfloat16)
    positions = ctx.astype(np.int32)[:, None]

    # the blocks the append touches, before: the oracle updates a host copy of exactly those
    touched = tables[np.arange(rows), ctx // BS]
    k_before, v_before = _host_blocks(k_cache[0], touched)[None], _host_blocks(v_cache[0], touched)[None]
    local_tables = np.arange(rows, dtype=np.int32)[:, None]             # row b's touched block is local block b
    local_slots = R.compute_slot_mapping(positions % BS, local_tables, BS)
    ek, ev = R.update_kv_cache(k_before, v_before, local_slots, nk, nv, 0)
    bystanders = np.setdiff1d(rng.integers(0, POOL, size=64), touched)   # blocks nobody may write
    by_before = _host_blocks(k_cache[0], bystanders)

    t_tables, t_lens = to_torch(tables), to_torch(lens)
    out, rk, rv = K.paged_decode_attention_with_kv_append(to_torch(q), to_torch(nk), to_torch(nv), k_cache, v_cache, t_tables,
                                                          t_lens, to_torch(positions), 0, BS, SCALE, 4, variant=variant)
    torch.cuda.synchronize()
    assert rk is k_cache and rv is v_cache
    np.testing.assert_array_equal(bits(_host_blocks(k_cache[0], touched)), bits(ek[0]))
    np.testing.assert_array_equal(bits(_host_blocks(v_cache[0], touched)), bits(ev[0]))
    np.testing.assert_array_equal(bits(_host_blocks(k_cache[0], bystanders)), bits(by_before))

    out = out.reshape(rows, 2048)
    generic = K.paged_decode_attention(to_torch(q[:, 0]), k_cache[0], v_cache[0], t_tables, t_lens, SCALE, variant=1)
    generic = generic.reshape(rows, 2048)
    err = float((out - generic).abs().max())
    if not err <= TIGHT:  # say which kernel left which rows unwritten (outputs start as NaN in the tests)
        for name, t in (("fused", out), ("generic", generic)):
            bad = torch.isnan(t).any(dim=1).nonzero().view(-1).tolist()
            assert not bad, f"{name} kernel left rows {bad[:8]} unwritten (lens {[int(lens[b]) for b in bad[:8]]}, cols {torch.isnan(t[bad[0]]).nonzero().view(-1).tolist()[:6]})"
    assert err <= TIGHT
    out_np = to_numpy(out)
    for b in np.linspace(0, rows - 1, 8).astype(int):
        ref = _oracle_row(k_cache[0], v_cache[0], tables[b], lens[b], q[b, 0])
        assert np.abs(out_np[b] - ref).max() <= TIGHT, f"row {b}"

    # put the touched blocks back so that the next variant appends into the same state
    k_cache[0][to_torch(touched.astype(np.int64))] = to_torch(k_before[0])
    v_cache[0][to_torch(touched.astype(np.int64))] = to_torch(v_before[0])


@pytest.mark.parametrize("variant", [3, 2])
def test_config5_shaped_rows_of_32k_tokens_over_the_large_pool(big_pool, variant):
    K = _K()
    k_cache, v_cache = big_pool
    rng = np.random.default_rng(5)
    rows = 8
    lens = rng.integers(30_000, 32_769, size=rows).astype(np.int32)
    tables, need = _tables(rng, lens.astype(np.int64), POOL)
    assert tables.max() >= 1 << 18 and tables.shape[1] >= 1875
    q = rng.standard_normal((rows, 8, 256), dtype=np.float32).astype(bfloat16)
    t_tables, t_lens = to_torch(tables), to_torch(lens)
    out = K.paged_decode_attention(to_torch(q), k_cache[0], v_cache[0], t_tables, t_lens, SCALE, variant=variant)
    generic = K.paged_decode_attention(to_torch(q), k_cache[0], v_cache[0], t_tables, t_lens, SCALE, variant=1)
    torch.cuda.synchronize()
    assert float((out - generic).abs().max()) <= TIGHT
    out_np = to_numpy(out).reshape(rows, -1)
    for b in (0, 3, 7):
        ref = _oracle_row(k_cache[0], v_cache[0], tables[b], lens[b], q[b])
        assert np.abs(out_np[b] - ref).max() <= TIGHT, f"row {b}"
    again = K.paged_decode_attention(to_torch(q), k_cache[0], v_cache[0], t_tables, t_lens, SCALE, variant=variant)
    assert torch.equal(out, again)                                      # counters of the two-level merge were left clean


class _Config3:
    """Host-side driver of config 3: sequences, block manager, the oracle's renumbered pool."""

    NB, WIDTH, BUCKET = 65_536, 128, 512

    def __init__(self):
        from nano_vllm_jax_b200.backends import B200Backend
        from nano_vllm_jax_b200.engine.block_manager import BlockManager
        from nano_vllm_jax_b200.engine.sequence import Sequence
        from nano_vllm_jax_b200.kv_cache import KVCacheStorage
        rng = np.random.default_rng(3)
        lens = rng.integers(64, 2049, size=8)
        lens[:4] = np.maximum(lens[:4], 513)
        shared = rng.integers(0, 248_320, size=512)
        self.seqs, self.q, self.k, self.v = [], [], [], []
        k_shared = rng.standard_normal((512, 2, 256), dtype=np.float32).astype(bfloat16)
        v_shared = rng.standard_normal((512, 2, 256), dtype=np.float32).astype(bfloat16)
        for r in range(8):
            ids = rng.integers(0, 248_320, size=int(lens[r]))
            kr = rng.standard_normal((int(lens[r]), 2, 256), dtype=np.float32).astype(bfloat16)
            vr = rng.standard_normal((int(lens[r]), 2, 256), dtype=np.float32).astype(bfloat16)
            if r < 4:  # a causal model gives equal K/V rows to equal prefixes
                ids[:512], kr[:512], vr[:512] = shared, k_shared, v_shared
            self.seqs.append(Sequence(ids.tolist(), seq_id=r))
            self.q.append(rng.standard_normal((int(lens[r]), 8, 256), dtype=np.float32).astype(bfloat16))
            self.k.append(kr); self.v.append(vr)
        self.bm = BlockManager(self.NB, BS)
        # scatter the free list over the pool through the public interface: fill it, free it in shuffled order
        fillers = [Sequence([0] * (16 * BS), seq_id=1000 + i) for i in range(self.NB // 16)]
        for s in fillers:
            self.bm.allocate(s, use_prefix_cache=False)
        for i in rng.permutation(len(fillers)):
            self.bm.deallocate(fillers[i])
        self.backend = B200Backend()
        kc = torch.empty((1, self.NB, BS, 2, 256), dtype=torch.bfloat16, device="cuda")
        vc = torch.empty_like(kc)
        _fill(kc[0], 31); _fill(vc[0], 32)
        self.k0, self.v0 = kc.clone(), vc.clone()
        self.cache = KVCacheStorage(kc, vc)
        self.local = {}                                   # device block id -> block id in the oracle's pool
        self.ok = np.zeros((1, 1400, BS, 2, 256), bfloat16)
        self.ov = np.zeros((1, 1400, BS, 2, 256), bfloat16)
        self.chunks_run = 0

    def local_ids(self, ids):
        fresh = [b for b in ids if b not in self.local]
        if fresh:
            base = len(self.local)
            for i, b in enumerate(fresh):
                self.local[b] = base + i
            self.ok[0, base:base + len(fresh)] = _host_blocks(self.k0[0], fresh)
            self.ov[0, base:base + len(fresh)] = _host_blocks(self.v0[0], fresh)
        return np.array([self.local[b] for b in ids], np.int32)

    def run_prefill(self, active):
        """Chunks of at most 512 tokens per step over `active` until their prompts are computed; every step's cache
        and attention are checked against the oracle."""
        from nano_vllm_jax_b200.engine.scheduled_batch import build_packed_prefill_batch
        while any(s.num_cached_tokens < s.num_tokens for s in active):
            budget, seqs, chunks = self.BUCKET, [], []
            for s in active:
                rem = s.num_tokens - s.num_cached_tokens
                if rem > 0 and budget > 0:
                    seqs.append(s); chunks.append(min(rem, budget)); budget -= chunks[-1]
            batch = build_packed_prefill_batch(seqs, chunks, max_blocks_per_seq=self.WIDTH, token_bucket=self.BUCKET)
            q = np.zeros((1, self.BUCKET, 8, 256), bfloat16)
            nk = np.zeros((1, self.BUCKET, 2, 256), bfloat16)
            nv = np.zeros((1, self.BUCKET, 2, 256), bfloat16)
            o = 0
            for s, c in zip(seqs, chunks):
                a = s.num_cached_tokens
                q[0, o:o + c], nk[0, o:o + c], nv[0, o:o + c] = self.q[s.seq_id][a:a + c], self.k[s.seq_id][a:a + c], self.v[s.seq_id][a:a + c]
                o += c
            md = self.backend.build_attention_metadata(batch.positions, batch.block_tables, batch.seq_lens, BS, True,
                                                       query_start_loc=batch.query_start_loc, token_row_ids=batch.token_row_ids,
                                                       query_lens_host=batch.query_lens_host)
            assert md.single_token_rows == sum(1 for c in chunks if c == 1)
            assert md.query_tile_pairs == sum(-(-c // 64) for c in chunks if c > 1)
            self.cache, out = self.backend.write_kv_and_attention(0, to_torch(q), to_torch(nk), to_torch(nv), self.cache, md,
                                                                  BS, SCALE, 4, True)
            torch.cuda.synchronize()
            # the same step in the oracle, on its renumbered pool
            tab = np.zeros((len(seqs), self.WIDTH), np.int32)
            for r, s in enumerate(seqs):
                tab[r, :len(s.block_table)] = self.local_ids(s.block_table)
            pos, rid, qsl = to_numpy(batch.positions), to_numpy(batch.token_row_ids), to_numpy(batch.query_start_loc)
            kv_lens = to_numpy(batch.seq_lens)
            slots = R.compute_packed_slot_mapping(pos, tab, rid, BS)
            self.ok, self.ov = R.update_kv_cache(self.ok, self.ov, slots, nk, nv, 0,
                                                 valid_mask=R.write_kv_valid_mask(slots.shape, qsl, True))
            ref = R.paged_attention_prefill_packed(q, self.ok, self.ov, tab, kv_lens, pos, rid, qsl, BS, SCALE, 4)
            err = np.abs(to_numpy(out) - ref).max()
            assert err <= TIGHT, f"chunk {self.chunks_run}: attention max-abs {err}"
            self.check_cache()
            for s, c in zip(seqs, chunks):
                self.bm.record_computed_prefix(s, s.num_cached_tokens + c, publish=True)
                s.num_cached_tokens += c
            self.chunks_run += 1

    def check_cache(self):
        ids = list(self.local)
        n = len(ids)
        np.testing.assert_array_equal(bits(_host_blocks(self.cache.k_cache[0], ids)), bits(self.ok[0, :n]))
        np.testing.assert_array_equal(bits(_host_blocks(self.cache.v_cache[0], ids)), bits(self.ov[0, :n]))

    def check_untouched_blocks(self):
        used = torch.zeros(self.NB, dtype=torch.bool, device="cuda")
        used[to_torch(np.array(list(self.local), np.int64))] = True
        assert torch.equal(self.cache.k_cache[0][~used], self.k0[0][~used])
        assert torch.equal(self.cache.v_cache[0][~used], self.v0[0][~used])


@pytest.mark.parametrize("mode", ["share", "copy"])
def test_config3_chunked_prefill_with_a_shared_prefix(mode):
    K = _K()
    c = _Config3()
    first, late = [c.seqs[0]] + c.seqs[4:], c.seqs[1:4]
    for s in first:
        c.bm.allocate(s)
        assert s.num_cached_tokens == 0
    assert max(max(s.block_table) for s in first) > 40_000 and min(min(s.block_table) for s in first) < 25_000  # scattered
    c.run_prefill(first)
    donor = c.seqs[0]
    if mode == "share":   # prefix reuse as the reference does it: the three late rows share row 0's 32 blocks
        for s in late:
            c.bm.allocate(s)
            assert s.num_cached_tokens == 512 and s.block_table[:32] == donor.block_table[:32]
        assert all(c.bm.blocks[b].ref_count == 4 for b in donor.block_table[:32])
        assert all(c.bm.blocks[b].ref_count == 1 for b in donor.block_table[32:])
    else:                 # prefix reuse by copy: private blocks filled by the block-copy kernel
        for s in late:
            c.bm.allocate(s, use_prefix_cache=False)
            assert s.num_cached_tokens == 0 and not set(s.block_table) & set(donor.block_table)
            src, dst = np.array(donor.block_table[:32], np.int32), np.array(s.block_table[:32], np.int32)
            lsrc, ldst = c.local_ids(list(src)), c.local_ids(list(dst))
            K.copy_blocks(c.cache.k_cache, c.cache.v_cache, to_torch(src), to_torch(dst))
            c.ok, c.ov = R.copy_blocks(c.ok, c.ov, lsrc, ldst)
            s.num_cached_tokens = 512
        torch.cuda.synchronize()
        c.check_cache()
    c.run_prefill(late)
    assert all(s.num_cached_tokens == s.num_tokens for s in c.seqs)
    assert c.chunks_run >= 10
    c.check_cache()
    c.check_untouched_blocks()
