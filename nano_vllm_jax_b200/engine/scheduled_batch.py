"""Scheduler -> executor batch contract and its builders.

`ScheduledBatch` carries the fields of the reference's dataclass that this path
reads (nanovllm_jax/engine/scheduled_batch.py:11-49).  The three builders restate
the layouts `Scheduler.build_scheduled_batch`, `_build_packed_prefill_batch` and
`build_mixed_prefill_decode_batch` produce (nanovllm_jax/engine/scheduler.py:
734-1098): decode rows carry `tokens=[last]`, `positions=[num_tokens-1]`,
`seq_lens=num_tokens`; packed batches hold every query token in one row of
`token_bucket` entries with `token_row_ids`, padded with (token 0, position 0,
row 0); padded rows have an all-zero table, `seq_len 0` and `seq_id -1`.
Host lists are built with NumPy and moved to the device in one copy each.
"""

from __future__ import annotations

from dataclasses import dataclass, replace
from typing import List, Optional, Sequence as Seq

import numpy as np
import torch


@dataclass
class ScheduledBatch:
    tokens: torch.Tensor
    positions: torch.Tensor
    seq_ids: torch.Tensor
    query_start_loc: torch.Tensor
    is_prefill: bool
    num_prefill_tokens: int
    num_decode_tokens: int
    block_tables: torch.Tensor
    seq_lens: torch.Tensor
    prefill_is_final: Optional[List[bool]] = None
    seq_ids_host: Optional[tuple] = None
    query_lens_host: Optional[tuple] = None
    seq_lens_host: Optional[tuple] = None
    block_tables_host: Optional[tuple] = None
    packed_prefill: bool = False
    token_row_ids: Optional[torch.Tensor] = None
    mixed_prefill_decode: bool = False

    @property
    def batch_size(self) -> int:
        return int(self.block_tables.shape[0] if self.packed_prefill else self.tokens.shape[0])

    @property
    def query_lens(self) -> torch.Tensor:
        return torch.diff(self.query_start_loc).to(torch.int32)


def _dev(a, device) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32))
    if torch.device(device).type == "cuda":
        t = t.pin_memory().to(device, non_blocking=True)
    return t


def _table_rows(seqs, width: int, pad_rows: int) -> np.ndarray:
    tab = np.zeros((len(seqs) + pad_rows, width), np.int32)
    for r, s in enumerate(seqs):
        if len(s.block_table) > width:
            raise ValueError(f"scheduled block table needs {len(s.block_table)} blocks but bucket has {width}")
        tab[r, :len(s.block_table)] = s.block_table
    return tab


def build_decode_batch(seqs, *, max_blocks_per_seq: Optional[int] = None,
                       batch_size_bucket: Optional[int] = None, device="cuda") -> ScheduledBatch:
    """Width-1 decode batch (scheduler.py:790-803, 850-870)."""
    n = len(seqs)
    bucket = n if batch_size_bucket is None else batch_size_bucket
    if n > bucket:
        raise ValueError(f"scheduled batch has {n} seqs but bucket has {bucket}")
    width = max_blocks_per_seq or max(1, max(len(s.block_table) for s in seqs))
    pad = bucket - n
    tokens = np.array([[s.last_token] for s in seqs] + [[0]] * pad, np.int32)
    positions = np.array([[s.num_tokens - 1] for s in seqs] + [[0]] * pad, np.int32)
    seq_lens = np.array([s.num_tokens for s in seqs] + [0] * pad, np.int32)
    qsl = np.concatenate([[0], np.cumsum([1] * n + [0] * pad)]).astype(np.int32)
    seq_ids = tuple([s.seq_id for s in seqs] + [-1] * pad)
    tab = _table_rows(seqs, width, pad)
    return ScheduledBatch(
        tokens=_dev(tokens, device), positions=_dev(positions, device), seq_ids=_dev(seq_ids, device),
        query_start_loc=_dev(qsl, device), is_prefill=False, num_prefill_tokens=0, num_decode_tokens=n,
        block_tables=_dev(tab, device), seq_lens=_dev(seq_lens, device), seq_ids_host=seq_ids,
        query_lens_host=tuple([1] * n + [0] * pad), seq_lens_host=tuple(int(x) for x in seq_lens),
        block_tables_host=tuple(tuple(int(x) for x in row) for row in tab))


def _pack(rows_tokens, rows_positions, seqs, seq_lens, finals, *, width, bucket_rows, token_bucket,
          device) -> ScheduledBatch:
    qlens = [len(t) for t in rows_tokens]
    actual = sum(qlens)
    if actual <= 0:
        raise ValueError("packed prefill requires at least one executable token")
    token_bucket = actual if token_bucket is None else token_bucket
    if actual > token_bucket:
        raise ValueError(f"scheduled prefill needs {actual} tokens but bucket has {token_bucket}")
    pad_rows = bucket_rows - len(seqs)
    pad = token_bucket - actual
    toks = np.zeros((1, token_bucket), np.int32)
    pos = np.zeros((1, token_bucket), np.int32)
    rid = np.zeros((1, token_bucket), np.int32)
    toks[0, :actual] = np.concatenate([np.asarray(t, np.int32) for t in rows_tokens])
    pos[0, :actual] = np.concatenate([np.asarray(p, np.int32) for p in rows_positions])
    rid[0, :actual] = np.repeat(np.arange(len(seqs), dtype=np.int32), qlens)
    qsl = np.concatenate([[0], np.cumsum(qlens + [0] * pad_rows)]).astype(np.int32)
    lens = np.array(list(seq_lens) + [0] * pad_rows, np.int32)
    seq_ids = tuple([s.seq_id for s in seqs] + [-1] * pad_rows)
    tab = _table_rows(seqs, width, pad_rows)
    return ScheduledBatch(
        tokens=_dev(toks, device), positions=_dev(pos, device), seq_ids=_dev(seq_ids, device),
        query_start_loc=_dev(qsl, device), is_prefill=True, num_prefill_tokens=actual, num_decode_tokens=0,
        block_tables=_dev(tab, device), seq_lens=_dev(lens, device), prefill_is_final=list(finals),
        seq_ids_host=seq_ids, query_lens_host=tuple(qlens + [0] * pad_rows),
        seq_lens_host=tuple(int(x) for x in lens),
        block_tables_host=tuple(tuple(int(x) for x in row) for row in tab),
        packed_prefill=True, token_row_ids=_dev(rid, device))


def build_packed_prefill_batch(seqs, prefill_chunk_lens: Optional[Seq[int]] = None, *,
                               max_blocks_per_seq: Optional[int] = None, batch_size_bucket: Optional[int] = None,
                               token_bucket: Optional[int] = None, device="cuda") -> ScheduledBatch:
    """Packed prefill: each row runs tokens [num_cached_tokens, +chunk) (scheduler.py:774-789, 1034-1098)."""
    toks, poss, lens, finals = [], [], [], []
    for i, s in enumerate(seqs):
        start = s.num_cached_tokens
        chunk = s.num_tokens - start if prefill_chunk_lens is None else int(prefill_chunk_lens[i])
        if chunk <= 0:
            raise ValueError(f"Scheduled sequence {s.seq_id} has no executable tokens")
        end = start + chunk
        toks.append(s.token_ids[start:end]); poss.append(list(range(start, end)))
        lens.append(end); finals.append(end >= s.num_tokens)
    width = max_blocks_per_seq or max(1, max(len(s.block_table) for s in seqs))
    return _pack(toks, poss, seqs, lens, finals, width=width,
                 bucket_rows=len(seqs) if batch_size_bucket is None else batch_size_bucket,
                 token_bucket=token_bucket, device=device)


def build_mixed_prefill_decode_batch(*, decode_seqs, prefill_seqs, prefill_chunk_lens,
                                     max_blocks_per_seq: Optional[int] = None,
                                     batch_size_bucket: Optional[int] = None,
                                     token_bucket: Optional[int] = None, device="cuda") -> ScheduledBatch:
    """Decode rows (one token each) first, then prefill chunks, in the packed form (scheduler.py:956-1032)."""
    if not decode_seqs:
        raise ValueError("mixed prefill/decode batch requires at least one decode row")
    if not prefill_seqs:
        raise ValueError("mixed prefill/decode batch requires at least one prefill row")
    if len(prefill_seqs) != len(prefill_chunk_lens):
        raise ValueError("prefill_chunk_lens length must match prefill_seqs")
    toks = [[s.last_token] for s in decode_seqs]
    poss = [[s.num_tokens - 1] for s in decode_seqs]
    lens = [s.num_tokens for s in decode_seqs]
    finals = [True] * len(decode_seqs)
    for s, c in zip(prefill_seqs, prefill_chunk_lens):
        start = s.num_cached_tokens
        chunk = min(int(c), s.num_prompt_tokens - start)
        if chunk <= 0:
            raise ValueError(f"Scheduled sequence {s.seq_id} has no executable prefill tokens")
        end = start + chunk
        toks.append(s.token_ids[start:end]); poss.append(list(range(start, end)))
        lens.append(end); finals.append(end >= s.num_tokens)
    seqs = list(decode_seqs) + list(prefill_seqs)
    width = max_blocks_per_seq or max(1, max(len(s.block_table) for s in seqs))
    batch = _pack(toks, poss, seqs, lens, finals, width=width,
                  bucket_rows=len(seqs) if batch_size_bucket is None else batch_size_bucket,
                  token_bucket=token_bucket, device=device)
    return replace(batch, mixed_prefill_decode=True)
