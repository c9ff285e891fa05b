"""Mixed continuous-batching steps over a 6-layer stand-in stack: greedy tokens with the B200
kernels equal those with the CPU oracle as the attention backend, caches stay bit-identical, and
GDN state snapshots/restores keyed by prefix hash are bit-exact.

Shape of the scenario (the baseline's mixed-step configuration): 32 decode rows with contexts in
[128, 2048] plus 2 prefill chunks of 256 tokens per step, hidden 1024, 8 q / 2 kv heads, head_dim
256, random bf16 weights, GDN state [18, 16, 128, 128] fp32 + conv [18, 6144, 4] bf16 per
sequence, every second new request hits the prefix cache.  Order of an engine step as in the
reference (nanovllm_jax/engine/llm_engine.py:432-457): install cached prefix states, run, record
computed prefix states, append tokens.
"""

import numpy as np
import pytest
import torch

from helpers import bits, to_numpy
from standin_stack import LAYERS, VOCAB, OracleAttention, forward, make_weights

pytestmark = pytest.mark.gpu

BS = 16


def _fake_gdn_state(table, seq_id, computed_tokens):
    """Stand-in for what the GDN layers leave in a sequence's slot after `computed_tokens` tokens."""
    g = torch.Generator(device="cuda").manual_seed(1_000_003 * seq_id + computed_tokens)
    st = table.state(seq_id)
    st.recurrent_state.copy_(torch.randn(st.recurrent_state.shape, generator=g, device="cuda"))
    st.conv_state.copy_(torch.randn(st.conv_state.shape, generator=g, device="cuda").to(st.conv_state.dtype))
    table.mark_written([seq_id])


def test_mixed_steps_tokens_caches_and_state_reuse():
    from nano_vllm_jax_b200.backends import B200Backend
    from nano_vllm_jax_b200.engine.block_manager import BlockManager
    from nano_vllm_jax_b200.engine.prefix_state import HybridStateTable, PrefixStateCache
    from nano_vllm_jax_b200.engine.scheduled_batch import build_decode_batch, build_mixed_prefill_decode_batch, build_packed_prefill_batch
    from nano_vllm_jax_b200.engine.sequence import Sequence
    from nano_vllm_jax_b200.kv_cache import KVCacheSpec

    rng = np.random.default_rng(4)
    pool = 6144
    backend = B200Backend()
    cache = backend.allocate_kv_cache(KVCacheSpec(LAYERS, pool, BS, 2, 256, torch.bfloat16), 64, 160)
    weights = make_weights(4)
    bm = BlockManager(pool, BS)
    table = HybridStateTable((18, 6144, 4), (18, 16, 128, 128), max_slots=40, conv_dtype=torch.bfloat16)
    states = PrefixStateCache(table, capacity=8)

    # 32 running sequences whose contexts are already in the cache (random K/V stands in for their prefill)
    decode = []
    for i in range(32):
        s = Sequence(rng.integers(0, VOCAB, size=int(rng.integers(128, 2049))).tolist(), seq_id=i)
        bm.allocate(s, use_prefix_cache=False)
        table.slot(s.seq_id)
        decode.append(s)
    g = torch.Generator(device="cuda").manual_seed(44)
    used = torch.tensor(sorted({b for s in decode for b in s.block_table}), device="cuda")
    for c in (cache.k_cache, cache.v_cache):
        c[:, used] = torch.randn((LAYERS, len(used), BS, 2, 256), generator=g, device="cuda").to(torch.bfloat16)
    oracle = OracleAttention(cache.k_cache, cache.v_cache)   # a reference system of its own (its k/v drift by bf16 flips)
    shadow = OracleAttention(cache.k_cache, cache.v_cache)   # fed the kernels' own q/k/v: caches comparable bit for bit

    def step(batch):
        tok_gpu, log_gpu = forward(weights, backend, backend, cache, batch, shadow=shadow)
        tok_ref, log_ref = forward(weights, oracle, backend, cache, batch)
        torch.cuda.synchronize()
        print("attention max-abs vs oracle per layer:", " ".join(f"{e:.1e}" for e in shadow.errors[-LAYERS:]))
        rows = len([i for i in batch.seq_ids_host if i >= 0])
        tg, tr = tok_gpu[:rows].cpu().numpy(), tok_ref[:rows].cpu().numpy()
        diff = float((log_gpu[:rows] - log_ref[:rows]).abs().max())
        for r in np.nonzero(tg != tr)[0]:  # a flip is only acceptable between numerically tied logits
            top2 = torch.topk(log_ref[r], 2).values
            assert float(top2[0] - top2[1]) <= 4 * diff, f"row {r}: tokens differ beyond a numerical tie"
        assert (tg != tr).sum() == 0, f"{(tg != tr).sum()} greedy tokens differ (max logit diff {diff:.3e})"
        return tr, diff

    # ---- step 0: a donor request prefills a 256-token prompt; its block-aligned prefix and state get published
    prefix = rng.integers(0, VOCAB, size=256).tolist()
    donor = Sequence(prefix, seq_id=100)
    bm.allocate(donor, cacheable_hashes=states.cacheable_hashes)
    assert donor.num_cached_tokens == 0
    tok, _ = step(build_packed_prefill_batch([donor], token_bucket=256))
    _fake_gdn_state(table, donor.seq_id, 256)
    donor_state = (table.state(100).conv_state.clone(), table.state(100).recurrent_state.clone())
    states.record_computed_prefix_states(bm, [donor], [256])
    assert len(states) == 1

    # ---- step 1: 32 decode rows + 2 prefill chunks of 256 tokens: one prefix hit (restore), one miss
    hit = Sequence(prefix + rng.integers(0, VOCAB, size=256).tolist(), seq_id=101)
    miss = Sequence(rng.integers(0, VOCAB, size=512).tolist(), seq_id=102)
    for s in (hit, miss):
        assert bm.can_allocate(s, cacheable_hashes=states.cacheable_hashes)
        bm.allocate(s, cacheable_hashes=states.cacheable_hashes)
    assert hit.num_cached_tokens == 256 and hit.block_table[:16] == donor.block_table and miss.num_cached_tokens == 0
    states.install_cached_prefix_hybrid_states(decode + [hit, miss])
    assert torch.equal(table.state(101).conv_state, donor_state[0]) and torch.equal(table.state(101).recurrent_state, donor_state[1])
    for s in decode:
        bm.may_append_slots(s, 1)
    batch = build_mixed_prefill_decode_batch(decode_seqs=decode, prefill_seqs=[hit, miss], prefill_chunk_lens=[256, 256],
                                             token_bucket=32 + 512)
    assert batch.query_lens_host[:32] == (1,) * 32 and batch.query_lens_host[32:] == (256, 256)
    tok, d1 = step(batch)
    _fake_gdn_state(table, 101, 512)
    _fake_gdn_state(table, 102, 256)
    states.record_computed_prefix_states(bm, [hit, miss], [256, 256])
    miss.num_cached_tokens = 256  # the scheduler advances a chunked prompt (postprocess)
    for s, t in zip(decode, tok[:32]):
        s.append_token(int(t))
    hit.append_token(int(tok[32]))  # its prompt is complete: it joins the decode set
    assert len(states) == 3

    # ---- step 2: decode rows (now 33) + the miss's second chunk + a new request that hits the miss's first chunk
    hit2 = Sequence(miss.token_ids[:256] + rng.integers(0, VOCAB, size=256).tolist(), seq_id=103)
    bm.allocate(hit2, cacheable_hashes=states.cacheable_hashes)
    assert hit2.num_cached_tokens == 256 and hit2.block_table[:16] == miss.block_table[:16]
    miss_state = (table.state(102).conv_state.clone(), table.state(102).recurrent_state.clone())
    _fake_gdn_state(table, 102, 257)  # the live slot moves on; the snapshot must not
    states.install_cached_prefix_hybrid_states([hit2])
    assert torch.equal(table.state(103).recurrent_state, miss_state[1]) and torch.equal(table.state(103).conv_state, miss_state[0])
    decode2 = decode + [hit]
    for s in decode2:
        bm.may_append_slots(s, 1)
    batch = build_mixed_prefill_decode_batch(decode_seqs=decode2, prefill_seqs=[miss, hit2], prefill_chunk_lens=[256, 256],
                                             token_bucket=33 + 512)
    tok, d2 = step(batch)
    for s, t in zip(decode2, tok[:33]):
        s.append_token(int(t))

    # ---- step 3: a plain decode batch (fused append + decode kernel), padded to a 40-row bucket
    for s in decode2:
        bm.may_append_slots(s, 1)
    tok, d3 = step(build_decode_batch(decode2, batch_size_bucket=40))

    # ---- caches written by the kernels equal the oracle's, bit for bit, in every layer
    np.testing.assert_array_equal(bits(to_numpy(cache.k_cache)), bits(shadow.k))
    np.testing.assert_array_equal(bits(to_numpy(cache.v_cache)), bits(shadow.v))
    print(f"max logit differences per step: {d1:.2e} {d2:.2e} {d3:.2e}")
