"""Per-request host state used by the block manager and the batch builders.

The fields are the ones the reference's `Sequence` exposes to this path
(nanovllm_jax/engine/sequence.py:43-140): token ids, block table, prefix-cache
bookkeeping.  Sampling, speculative decoding and deferred device tokens belong to
the serving loop and are not modelled; `block_has_unmaterialized_device_tokens`
therefore always answers False.
"""

from __future__ import annotations

from dataclasses import dataclass
from itertools import count
from typing import List, Optional


@dataclass
class SamplingParams:
    temperature: float = 1.0
    max_tokens: int = 256
    ignore_eos: bool = False
    top_p: float = 1.0
    top_k: int = -1


class Sequence:
    block_size: int = 16
    counter = count()

    def __init__(self, token_ids: List[int], sampling_params: Optional[SamplingParams] = None,
                 seq_id: Optional[int] = None):
        self.seq_id = next(Sequence.counter) if seq_id is None else seq_id
        self.token_ids = list(token_ids)
        self.last_token = self.token_ids[-1]
        self.num_tokens = len(self.token_ids)
        self.num_prompt_tokens = len(self.token_ids)
        self.num_cached_tokens = 0
        self.cached_prefix_hash: Optional[int] = None
        self.cached_prefix_hybrid_seeded = False
        self.prefix_cache_enabled = False
        self.block_table: List[int] = []
        sp = sampling_params or SamplingParams()
        self.temperature, self.max_tokens, self.ignore_eos = sp.temperature, sp.max_tokens, sp.ignore_eos

    def __len__(self) -> int:
        return self.num_tokens

    def __getitem__(self, key):
        return self.token_ids[key]

    @property
    def num_completion_tokens(self) -> int:
        return self.num_tokens - self.num_prompt_tokens

    @property
    def num_cached_blocks(self) -> int:
        return self.num_cached_tokens // self.block_size

    @property
    def num_blocks(self) -> int:
        return -(-self.num_tokens // self.block_size)

    def block_has_unmaterialized_device_tokens(self, block_idx: int) -> bool:
        return False

    def append_token(self, token_id: int) -> None:
        self.token_ids.append(int(token_id))
        self.last_token = int(token_id)
        self.num_tokens += 1
