"""Host-side block allocator with hash-chained prefix reuse.

Behaviour and public names follow nanovllm_jax/engine/block_manager.py:12-387 so
the reference scheduler can drive it unchanged: reference-counted blocks, one
xxh64 digest per *full* block chained on the previous block's digest, a
`hash_to_block_id` map that only holds blocks whose KV rows were actually
computed (publish after compute), and look-ahead slot reservation for decode.
Prefix reuse is sharing by reference count; nothing is copied on the device.

The hash must be bit-identical to the reference's
(block_manager.py:49-56): xxh64 over `prefix.to_bytes(8, "little")` (when a
prefix exists) followed by the token ids as native int64 bytes.
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Dict, Iterable, List, Optional, Set

import numpy as np
import xxhash

from ..kv_cache import BlockTables

NO_HASH = -1


class Block:
    """One physical cache block: owner count, content digest, the tokens it holds."""

    __slots__ = ("block_id", "ref_count", "hash", "token_ids")

    def __init__(self, block_id: int):
        self.block_id = block_id
        self.ref_count = 0
        self.hash = NO_HASH
        self.token_ids: List[int] = []

    def update(self, hash_val: int, token_ids: List[int]) -> None:
        self.hash = hash_val
        self.token_ids = token_ids

    def reset(self) -> None:
        self.ref_count = 1
        self.hash = NO_HASH
        self.token_ids = []


class _FreeList:
    """FIFO of free block ids with O(1) removal of an arbitrary id (deque.remove is O(n))."""

    def __init__(self, ids: Iterable[int]):
        self._d: "OrderedDict[int, None]" = OrderedDict((i, None) for i in ids)

    def __len__(self) -> int:
        return len(self._d)

    def __contains__(self, block_id: int) -> bool:
        return block_id in self._d

    def __iter__(self):
        return iter(self._d)

    def __getitem__(self, index: int) -> int:
        if index != 0:
            raise IndexError("only the head of the free list is addressable")
        return next(iter(self._d))

    def remove(self, block_id: int) -> None:
        del self._d[block_id]

    def append(self, block_id: int) -> None:
        self._d[block_id] = None


class BlockManager:
    def __init__(self, num_blocks: int, block_size: int):
        self.block_size = block_size
        self.blocks: List[Block] = [Block(i) for i in range(num_blocks)]
        self.hash_to_block_id: Dict[int, int] = {}
        self.free_block_ids = _FreeList(range(num_blocks))
        self.used_block_ids: Set[int] = set()

    # ------------------------------------------------------------------ hashing
    @classmethod
    def compute_hash(cls, token_ids: List[int], prefix: int = NO_HASH) -> int:
        h = xxhash.xxh64()
        if prefix != NO_HASH:
            h.update(int(prefix).to_bytes(8, "little"))
        h.update(np.asarray(token_ids, dtype=np.int64).tobytes())
        return h.intdigest()

    def _chain(self, seq):
        """Yield (block_idx, tokens, digest-or-NO_HASH) for every block the sequence needs."""
        h = NO_HASH
        bs = self.block_size
        for idx in range(self._num_blocks(seq)):
            toks = seq.token_ids[idx * bs:(idx + 1) * bs]
            if len(toks) == bs:
                h = self.compute_hash(toks, h)
                yield idx, toks, h
            else:
                yield idx, toks, NO_HASH

    def _num_blocks(self, seq) -> int:
        return -(-seq.num_tokens // self.block_size)

    def _lookup(self, h: int, token_ids: List[int]) -> int:
        """Published block holding exactly these tokens under this digest, else -1."""
        bid = self.hash_to_block_id.get(h, -1)
        if bid == -1:
            return -1
        blk = self.blocks[bid]
        return bid if (blk.hash == h and blk.token_ids == token_ids) else -1

    # ------------------------------------------------------------------ block state changes
    def _take_fresh(self, block_id: int) -> Block:
        blk = self.blocks[block_id]
        assert blk.ref_count == 0
        if blk.hash != NO_HASH and self.hash_to_block_id.get(blk.hash) == block_id:
            del self.hash_to_block_id[blk.hash]  # its old content is about to be overwritten
        blk.reset()
        self.free_block_ids.remove(block_id)
        self.used_block_ids.add(block_id)
        return blk

    def _take_cached(self, block_id: int) -> Block:
        blk = self.blocks[block_id]
        assert blk.ref_count == 0
        blk.ref_count = 1  # content and digest stay: the rows are still valid
        self.free_block_ids.remove(block_id)
        self.used_block_ids.add(block_id)
        return blk

    def _release(self, block_id: int) -> None:
        assert self.blocks[block_id].ref_count == 0
        self.used_block_ids.remove(block_id)
        self.free_block_ids.append(block_id)

    # aliases under the reference's private names, which its tests reach for
    _allocate_block = _take_fresh
    _reuse_cached_block = _take_cached
    _deallocate_block = _release
    _cached_block_id = _lookup

    # ------------------------------------------------------------------ prefix queries
    def cached_prefix_info(self, seq, *, cacheable_hashes: Optional[Set[int]] = None):
        """(reusable tokens, digest of that prefix): longest run of published full blocks.

        With `cacheable_hashes` the run is cut back to the longest prefix whose own
        chained digest is in the set (hybrid models need the GDN state of exactly
        that prefix).
        """
        best_blocks, best_hash = 0, None
        for idx, toks, h in self._chain(seq):
            if h == NO_HASH or self._lookup(h, toks) == -1:
                break
            if cacheable_hashes is None or h in cacheable_hashes:
                best_blocks, best_hash = idx + 1, h
        return best_blocks * self.block_size, best_hash

    def _num_required_blocks(self, seq, *, use_prefix_cache=True, cacheable_hashes=None) -> int:
        if not use_prefix_cache:
            return self._num_blocks(seq)
        cached_tokens, _ = self.cached_prefix_info(seq, cacheable_hashes=cacheable_hashes)
        cached_blocks = cached_tokens // self.block_size
        need = 0
        for idx, toks, h in self._chain(seq):
            if idx < cached_blocks and self._lookup(h, toks) in self.used_block_ids:
                continue  # shared with a live sequence: costs no free block
            need += 1
        return need

    def can_allocate(self, seq, *, use_prefix_cache=True, cacheable_hashes=None) -> bool:
        return len(self.free_block_ids) >= self._num_required_blocks(
            seq, use_prefix_cache=use_prefix_cache, cacheable_hashes=cacheable_hashes)

    # ------------------------------------------------------------------ allocate / free
    def allocate(self, seq, *, use_prefix_cache=True, cacheable_hashes=None) -> None:
        assert not seq.block_table
        seq.block_size = self.block_size
        seq.num_cached_tokens = 0
        seq.cached_prefix_hash = None
        seq.cached_prefix_hybrid_seeded = False
        seq.prefix_cache_enabled = bool(use_prefix_cache)
        cached_tokens, cached_hash = (self.cached_prefix_info(seq, cacheable_hashes=cacheable_hashes)
                                      if use_prefix_cache else (0, None))
        cached_blocks = cached_tokens // self.block_size
        for idx, toks, h in self._chain(seq):
            hit = -1
            if h != NO_HASH and idx < cached_blocks:
                hit = self._lookup(h, toks)
                if hit == -1:
                    raise AssertionError("cached prefix disappeared during allocation")
            if hit == -1:
                blk = self._take_fresh(self.free_block_ids[0])
            else:
                seq.num_cached_tokens += self.block_size
                if hit in self.used_block_ids:
                    blk = self.blocks[hit]
                    blk.ref_count += 1
                else:
                    blk = self._take_cached(hit)
            if h != NO_HASH:
                blk.update(h, toks)  # recorded, but published only after compute
            seq.block_table.append(blk.block_id)
        seq.cached_prefix_hash = cached_hash if seq.num_cached_tokens > 0 else None

    def deallocate(self, seq) -> None:
        for bid in reversed(seq.block_table):
            blk = self.blocks[bid]
            blk.ref_count -= 1
            if blk.ref_count == 0:
                self._release(bid)
        seq.num_cached_tokens = 0
        seq.cached_prefix_hash = None
        seq.cached_prefix_hybrid_seeded = False
        seq.prefix_cache_enabled = False
        seq.block_table.clear()

    # ------------------------------------------------------------------ decode growth
    def _blocks_for(self, tokens: int) -> int:
        return -(-tokens // self.block_size)

    def can_append(self, seq) -> bool:
        return self.can_append_slots(seq, 1)

    def can_append_slots(self, seq, num_slots: int) -> bool:
        target = len(seq) + max(0, int(num_slots) - 1)
        return len(self.free_block_ids) >= max(0, self._blocks_for(target) - len(seq.block_table))

    def may_append(self, seq) -> None:
        self.may_append_slots(seq, 1)

    def may_append_slots(self, seq, num_slots: int) -> None:
        table = seq.block_table
        if self._blocks_for(len(seq)) > len(table):
            last = len(table) - 1
            self._record_completed_block_hash(seq, last)
            if self.blocks[table[-1]].hash == NO_HASH and not seq.block_has_unmaterialized_device_tokens(last):
                raise AssertionError("completed block hash was not recorded")
            table.append(self._take_fresh(self.free_block_ids[0]).block_id)
        if len(seq) % self.block_size == 0:
            self._record_completed_block_hash(seq, len(seq) // self.block_size - 1)
        want = self._blocks_for(len(seq) + max(0, int(num_slots) - 1))
        while len(table) < want:
            table.append(self._take_fresh(self.free_block_ids[0]).block_id)

    def trim_append_slots(self, seq, num_slots: int) -> None:
        table = seq.block_table
        want = self._blocks_for(len(seq) + max(0, int(num_slots) - 1))
        while len(table) > want:
            blk = self.blocks[table.pop()]
            if blk.hash != NO_HASH or blk.token_ids:
                raise AssertionError("cannot trim a materialized KV block")
            blk.ref_count -= 1
            self._release(blk.block_id)

    def commit_processed_token(self, seq) -> None:
        if len(seq) % self.block_size == 0:
            self._record_completed_block_hash(seq, len(seq) // self.block_size - 1)

    # ------------------------------------------------------------------ publish after compute
    def _record_completed_block_hash(self, seq, block_idx: int, *, publish: Optional[bool] = None):
        if not 0 <= block_idx < len(seq.block_table):
            return None
        if seq.block_has_unmaterialized_device_tokens(block_idx):
            return None
        bs = self.block_size
        toks = seq.token_ids[block_idx * bs:(block_idx + 1) * bs]
        if len(toks) != bs:
            return None
        blk = self.blocks[seq.block_table[block_idx]]
        do_publish = seq.prefix_cache_enabled if publish is None else bool(publish)
        if blk.hash == NO_HASH:
            prev = self.blocks[seq.block_table[block_idx - 1]].hash if block_idx > 0 else NO_HASH
            blk.update(self.compute_hash(toks, prev), toks)
        if do_publish:
            self.hash_to_block_id[blk.hash] = blk.block_id
        return blk.hash

    def record_computed_prefix(self, seq, upto_tokens: int, *, publish: bool):
        """Record digests of the full prompt blocks below `upto_tokens`; return the last one's
        digest when `upto_tokens` is a positive multiple of the block size, else None."""
        upto = max(0, min(int(upto_tokens), int(seq.num_prompt_tokens)))
        full = upto // self.block_size
        last = None
        for idx in range(full):
            last = self._record_completed_block_hash(seq, idx, publish=publish)
        return last if (upto > 0 and upto % self.block_size == 0) else None

    def publish_computed_prefix(self, seq, upto_tokens: int):
        return self.record_computed_prefix(seq, upto_tokens, publish=True)

    # ------------------------------------------------------------------ diagnostics
    def stats(self) -> dict:
        return {"total_blocks": len(self.blocks), "free_blocks": len(self.free_block_ids),
                "used_blocks": len(self.used_block_ids)}

    def snapshot(self, seqs=None) -> BlockTables:
        return BlockTables(tables=[list(s.block_table) for s in seqs] if seqs is not None else [],
                           ref_counts=[b.ref_count for b in self.blocks],
                           hashes=[b.hash for b in self.blocks])
