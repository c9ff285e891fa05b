"""GDN hybrid-state slot table with snapshot / restore keyed by prefix hash.

What the reference does (nanovllm_jax/engine/model_runner.py:3755-3905,
nanovllm_jax/engine/scheduler.py:67-69, 218-279):

* every resident sequence owns one slot of two device tables, `conv_state
  [S, L_lin, conv_dim, K]` (model dtype) and `recurrent_state [S, L_lin, Hv, Dv,
  Dk]` fp32; a slot is zeroed when it is first assigned;
* after a prefill chunk that ends on a block boundary, the sequence's state is
  read out (`_get_hybrid_state`) and stored in `prefix_cache_hybrid_states`
  under the chained hash of that prefix, and only then is the prefix published
  to the block manager's map (`record_computed_prefix_states`);
* a later sequence that reuses that prefix gets the stored state written into
  its own slot before it runs (`install_cached_prefix_hybrid_states`); a missing
  state is a RuntimeError.

Here the stored states live in a preallocated device pool (the reference keeps
an unbounded dict of arrays); snapshot and restore are index-list copy kernels
(nvj_hybrid_snapshot / nvj_hybrid_restore), batched over all sequences of a
step.  When the pool is full the least recently used entry is dropped and its
hash leaves `cacheable_hashes`, so the block manager stops offering that prefix
to hybrid models.  Two kinds of entry are never dropped: one that was assigned
earlier in the same `snapshot()` batch (its pool row is a destination of the
copy kernel about to be launched), and one that a sequence has been allocated
against but not yet seeded from (`pin` / `install_cached_prefix_hybrid_states`).
When nothing can be dropped the snapshot of that sequence is skipped and its
prefix is not published: a later request recomputes it, as it would after an
eviction.
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Dict, Iterable, List, Optional, Sequence as Seq

import torch

from ..kernels import paged_kv as _k
from ..kv_cache import HybridLayerState


class HybridStateTable:
    """Slot table of GDN state for resident sequences (model_runner.py:3758-3867)."""

    def __init__(self, conv_shape: Optional[tuple], rec_shape: Optional[tuple], max_slots: int,
                 conv_dtype=torch.bfloat16, device="cuda"):
        self.max_slots = int(max_slots)
        self.conv = None if conv_shape is None else torch.zeros((max_slots, *conv_shape), dtype=conv_dtype, device=device)
        self.rec = None if rec_shape is None else torch.zeros((max_slots, *rec_shape), dtype=torch.float32, device=device)
        self.device = torch.device(device)
        self._slot_of: Dict[int, int] = {}
        self._free: List[int] = list(range(max_slots - 1, -1, -1))
        self._clean = set(range(max_slots))  # slots known to hold zeros

    # ---- slot bookkeeping
    def slot(self, seq_id: int) -> int:
        """Slot of `seq_id`, assigning (and zeroing) one on first use."""
        if seq_id < 0:
            return -1
        s = self._slot_of.get(seq_id)
        if s is not None:
            return s
        if not self._free:
            raise RuntimeError("No free hybrid-state slots; max_num_resident_seqs is exhausted")
        if seq_id < self.max_slots and seq_id in self._free:
            self._free.remove(seq_id)
            s = seq_id
        else:
            s = self._free.pop()
        self._slot_of[seq_id] = s
        if s not in self._clean:
            for t in (self.conv, self.rec):
                if t is not None:
                    t[s].zero_()
            self._clean.add(s)
        return s

    def has(self, seq_id: int) -> bool:
        return seq_id in self._slot_of

    def mark_written(self, seq_ids: Iterable[int]) -> None:
        for i in seq_ids:
            s = self._slot_of.get(i)
            if s is not None:
                self._clean.discard(s)

    def release(self, seq_ids: Iterable[int]) -> None:
        for i in seq_ids:
            s = self._slot_of.pop(i, None)
            if s is not None:
                self._free.append(s)

    def state(self, seq_id: int) -> HybridLayerState:
        """View of one sequence's state rows (the forward pass updates them in place)."""
        s = self.slot(seq_id)
        return HybridLayerState(None if self.conv is None else self.conv[s:s + 1],
                                None if self.rec is None else self.rec[s:s + 1])

    # ---- a step's batch (model_runner.py:4181-4305)
    def batch_slot_ids(self, seq_ids: Seq[int]) -> List[int]:
        """Slots of a scheduled batch, assigning (and zeroing) new ones; -1 for padding rows (seq id < 0).  A forward
        pass that indexes the table by these ids needs no gather (model_runner.py:4307-4330)."""
        return [self.slot(int(i)) if int(i) >= 0 else -1 for i in seq_ids]

    def _pairs(self, slots: Seq[int], rows: Seq[int]):
        if self.device.type == "cuda" and len(slots) <= _k.HYBRID_HOST_SLOTS:
            return list(slots), list(rows)
        t = torch.tensor(list(slots) + list(rows), dtype=torch.int32)
        if self.device.type == "cuda":
            t = t.pin_memory().to(self.device, non_blocking=True)
        return t[:len(slots)], t[len(slots):]

    def gather_batch(self, seq_ids: Seq[int], out: Optional[HybridLayerState] = None) -> HybridLayerState:
        """The batch's state rows as one `[B, ...]` pair, row r = the slot of seq_ids[r] (`_batch_hybrid_state`): zeros
        for padding rows and for sequences seen for the first time.  When the batch is the whole table in slot order
        the table itself is returned, as the reference does; otherwise one index-list copy launch into `out`
        (allocated when not given)."""
        slots = self.batch_slot_ids(seq_ids)
        n = len(slots)
        if n == self.max_slots and slots == list(range(n)):
            return HybridLayerState(self.conv, self.rec)
        if out is None:
            out = HybridLayerState(None if self.conv is None else torch.empty((n, *self.conv.shape[1:]), dtype=self.conv.dtype, device=self.device),
                                   None if self.rec is None else torch.empty((n, *self.rec.shape[1:]), dtype=self.rec.dtype, device=self.device))
        live = [(s, r) for r, s in enumerate(slots) if s >= 0]
        for r, s in enumerate(slots):
            if s < 0:
                for t in (out.conv_state, out.recurrent_state):
                    if t is not None:
                        t[r].zero_()
        if live:
            t_slots, t_rows = self._pairs([s for s, _ in live], [r for _, r in live])
            _k.hybrid_copy(self.conv, self.rec, out.conv_state, out.recurrent_state, t_slots, t_rows, restore=False)
        return out

    def store_batch(self, seq_ids: Seq[int], state: Optional[HybridLayerState], query_lens: Optional[Seq[int]] = None,
                    is_prefill: bool = True) -> None:
        """table[slot(seq_ids[r])] <- state[r] for the rows that ran (`_store_batch_hybrid_state`): padding rows, and in
        a decode batch rows whose query length is 0, are left alone.  Nothing to do when `state` is the table."""
        if state is None or (state.conv_state is self.conv and state.recurrent_state is self.rec):
            if state is not None:
                self.mark_written([int(i) for i in seq_ids if int(i) >= 0])
            return
        rows, slots, ids = [], [], []
        for r, i in enumerate(seq_ids):
            i = int(i)
            if i < 0 or (not is_prefill and query_lens is not None and int(query_lens[r]) <= 0):
                continue
            rows.append(r)
            slots.append(self.slot(i))
            ids.append(i)
        if not rows:
            return
        t_slots, t_rows = self._pairs(slots, rows)
        _k.hybrid_copy(self.conv, self.rec, state.conv_state, state.recurrent_state, t_slots, t_rows, restore=True)
        self.mark_written(ids)


class PrefixStateCache:
    """Pool of state snapshots keyed by prefix hash (scheduler.py:67-69, 239-279)."""

    def __init__(self, table: HybridStateTable, capacity: int):
        self.table = table
        self.capacity = int(capacity)
        dev = table.device
        self.conv_pool = None if table.conv is None else torch.zeros((capacity, *table.conv.shape[1:]), dtype=table.conv.dtype, device=dev)
        self.rec_pool = None if table.rec is None else torch.zeros((capacity, *table.rec.shape[1:]), dtype=torch.float32, device=dev)
        self._entry: "OrderedDict[int, int]" = OrderedDict()  # hash -> pool row, LRU order
        self._free = list(range(capacity - 1, -1, -1))
        self._pins: Dict[int, int] = {}  # hash -> sequences allocated against it and not yet seeded

    def __contains__(self, prefix_hash: int) -> bool:
        return int(prefix_hash) in self._entry

    def __len__(self) -> int:
        return len(self._entry)

    @property
    def cacheable_hashes(self) -> set:
        """Hashes a hybrid model may reuse (`Scheduler._prefix_cacheable_hashes`)."""
        return set(self._entry)

    # ---- pins: a hash a sequence was allocated against stays until that sequence has been seeded
    def pin(self, prefix_hash: int) -> None:
        h = int(prefix_hash)
        self._pins[h] = self._pins.get(h, 0) + 1

    def unpin(self, prefix_hash: int) -> None:
        h = int(prefix_hash)
        n = self._pins.get(h, 0) - 1
        if n > 0:
            self._pins[h] = n
        else:
            self._pins.pop(h, None)

    def pin_for(self, seqs) -> None:
        """Call after `BlockManager.allocate`: protects the state of every prefix a new sequence will start from."""
        for seq in seqs:
            h = getattr(seq, "cached_prefix_hash", None)
            if (h is not None and int(getattr(seq, "num_cached_tokens", 0)) > 0
                    and not getattr(seq, "cached_prefix_hybrid_seeded", False)
                    and not getattr(seq, "_prefix_state_pinned", False)):
                self.pin(h)
                seq._prefix_state_pinned = True

    def _row_for(self, prefix_hash: int, in_batch: set) -> Optional[int]:
        """Pool row for a new snapshot of `prefix_hash`; None when the pool is full of rows that must stay."""
        row = self._entry.pop(prefix_hash, None)
        if row is None:
            if self._free:
                row = self._free.pop()
            else:
                victim = next((h for h in self._entry if h not in in_batch and h not in self._pins), None)
                if victim is None:
                    return None
                row = self._entry.pop(victim)  # the least recently used snapshot that may go
        self._entry[prefix_hash] = row
        return row

    def _idx_pair(self, first: List[int], second: List[int]):
        """The two index lists of one copy: as they are when few enough to ride in the kernel's parameters, else on
        the device, uploaded with a single host-to-device copy."""
        n = len(first)
        if self.table.device.type == "cuda" and n <= _k.HYBRID_HOST_SLOTS:
            return list(first), list(second)
        t = torch.tensor(list(first) + list(second), dtype=torch.int32)
        if self.table.device.type == "cuda":
            t = t.pin_memory().to(self.table.device, non_blocking=True)
        return t[:n], t[n:]

    def snapshot(self, seq_ids: Seq[int], prefix_hashes: Seq[int]) -> List[bool]:
        """pool[hash] <- table[slot(seq)] for every pair, one batched copy.  Returns, per pair, whether the state is
        stored now (False: the pool had no row that could be given up)."""
        stored: List[bool] = []
        slots, rows, in_batch = [], [], set()
        for s, h in zip(seq_ids, prefix_hashes):
            h = int(h)
            if h in in_batch:  # the same prefix twice in one step: one copy is enough (the states are identical)
                stored.append(True)
                continue
            row = self._row_for(h, in_batch)
            if row is None:
                stored.append(False)
                continue
            in_batch.add(h)
            slots.append(self.table.slot(int(s)))
            rows.append(row)
            stored.append(True)
        if rows:
            t_slots, t_rows = self._idx_pair(slots, rows)
            _k.hybrid_copy(self.table.conv, self.table.rec, self.conv_pool, self.rec_pool, t_slots, t_rows, restore=False)
        return stored

    def restore(self, seq_ids: Seq[int], prefix_hashes: Seq[int]) -> None:
        """table[slot(seq)] <- pool[hash]; a hash without a snapshot is a RuntimeError."""
        if not seq_ids:
            return
        rows = []
        for h in prefix_hashes:
            row = self._entry.get(int(h))
            if row is None:
                raise RuntimeError(f"missing hybrid prefix state for cached prefix hash {int(h)}")
            self._entry.move_to_end(int(h))
            rows.append(row)
        slots = [self.table.slot(int(s)) for s in seq_ids]
        t_slots, t_rows = self._idx_pair(slots, rows)
        _k.hybrid_copy(self.table.conv, self.table.rec, self.conv_pool, self.rec_pool, t_slots, t_rows, restore=True)
        self.table.mark_written(seq_ids)

    # ---- the two engine-step hooks (llm_engine.py:432-457)
    def install_cached_prefix_hybrid_states(self, seqs) -> None:
        """Seed the slot of every sequence that starts from a cached prefix (model_runner.py:3886-3905)."""
        ids, hashes, todo = [], [], []
        for seq in seqs:
            h = getattr(seq, "cached_prefix_hash", None)
            if h is None or int(getattr(seq, "num_cached_tokens", 0)) <= 0:
                continue
            if getattr(seq, "cached_prefix_hybrid_seeded", False):
                continue
            ids.append(int(seq.seq_id)); hashes.append(int(h)); todo.append(seq)
        self.restore(ids, hashes)
        for seq in todo:
            seq.cached_prefix_hybrid_seeded = True
            if getattr(seq, "_prefix_state_pinned", False):
                self.unpin(seq.cached_prefix_hash)
                seq._prefix_state_pinned = False

    def record_computed_prefix_states(self, block_manager, seqs, prefill_chunk_lengths) -> None:
        """After a prefill step: snapshot block-aligned prefixes, then publish them (scheduler.py:239-279)."""
        if len(prefill_chunk_lengths) != len(seqs):
            return
        ids, hashes, publish = [], [], []
        for seq, chunk in zip(seqs, prefill_chunk_lengths):
            chunk = int(chunk)
            if chunk <= 0:
                continue
            computed = min(seq.num_prompt_tokens, seq.num_cached_tokens + chunk)
            if computed <= 0:
                continue
            h = block_manager.record_computed_prefix(seq, computed, publish=False)
            if h is None or not self.table.has(int(seq.seq_id)):
                continue
            ids.append(int(seq.seq_id)); hashes.append(int(h)); publish.append((seq, computed))
        stored = self.snapshot(ids, hashes)
        for (seq, computed), ok in zip(publish, stored):
            if ok:  # a prefix without a stored state must not be offered to later requests
                block_manager.publish_computed_prefix(seq, computed)
