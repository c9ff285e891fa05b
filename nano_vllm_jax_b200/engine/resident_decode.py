"""Decode metadata that lives on the device, and a decode step replayed from a CUDA graph.

The reference keeps the block tables and sequence lengths of a steady decode batch on the
device between steps ("static" / "resident" decode metadata,
nanovllm_jax/engine/scheduler.py:1100-1219) and lets the compiled executor derive the width-1
positions from the lengths (nanovllm_jax/engine/model_executor.py:560-562), so that a step
costs no host-to-device traffic for metadata.  Here the same arrays are torch CUDA tensors:

  ResidentDecodeMetadata   block_tables [rows, W], seq_lens [rows], positions [rows, 1];
                           `advance()` grows every active row by one token on the device,
                           `set_block()` pushes a newly allocated block id from the host
                           (the only per-step host work, and only when a row crosses a block
                           boundary), `load()` (re)installs a batch.
  DecodeStepGraph          captures  fused append + paged decode -> token pick + advance
                           once and replays it: one graph launch per step, two kernels back to
                           back, and nothing is allocated or copied per step.  The decode pass
                           runs in its pre-append form (a row's token goes to position
                           seq_lens[b], seq_lens[b] + 1 keys are attended) and the token pick
                           advances the lengths for the next step in the same launch.  On
                           several GPUs the token pick also publishes the tokens to every
                           peer over NVLink and, in the same launch, collects the PREVIOUS
                           step's tokens, which have had a whole step to arrive: the wait for
                           the slowest rank never sits between two steps (`gathered` lags one
                           step; `flush()` fetches the last one).

The query and the new K/V rows are static buffers the caller fills before `replay()` (in a
model they are produced by the projections that run in front of this path).
"""

from __future__ import annotations

import os
from typing import Optional

import torch

from .. import _lib
from ..kernels import paged_kv as _k


class CapturedStep:
    """A step function over static device buffers, run once and then replayed from a CUDA graph.

    `fn` must launch on the current stream only, allocate nothing it keeps using after the call except through
    torch's allocator (the graph's private pool keeps such tensors alive), and never synchronise with the host.
    `capture()` runs `fn` once for real on a side stream (kernels, workspaces and tensor maps are then warm; this
    run is the step's first execution) and records a second run; `replay()` launches the recording.  Reading the
    device status word back after every call (`NVJ_CHECK_STATUS=1`, what the tests do) is a host synchronisation,
    so it is switched off while `fn` runs here; call `paged_kv.check_device_status()` afterwards instead.
    """

    def __init__(self, fn, device="cuda"):
        self.fn = fn
        self.device = torch.device(device)
        self._stream = torch.cuda.Stream(self.device)
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self.result = None

    def capture(self):
        strict = os.environ.get("NVJ_CHECK_STATUS")
        os.environ["NVJ_CHECK_STATUS"] = "0"
        try:
            self._stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._stream):
                first = self.fn()
            self._stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self._stream):
                self.result = self.fn()
            self._graph = graph
        finally:
            if strict is None:
                os.environ.pop("NVJ_CHECK_STATUS", None)
            else:
                os.environ["NVJ_CHECK_STATUS"] = strict
        torch.cuda.current_stream(self.device).wait_stream(self._stream)
        return first

    def replay(self):
        if self._graph is None:
            raise RuntimeError("capture() has not been called")
        self._graph.replay()
        return self.result


class ResidentDecodeMetadata:
    def __init__(self, rows: int, table_width: int, block_size: int, device="cuda"):
        self.device = torch.device(device)
        self.rows, self.table_width, self.block_size = int(rows), int(table_width), int(block_size)
        self.block_tables = torch.zeros((rows, table_width), dtype=torch.int32, device=self.device)
        self.seq_lens = torch.zeros((rows,), dtype=torch.int32, device=self.device)
        self.positions = torch.zeros((rows, 1), dtype=torch.int32, device=self.device)
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)

    def load(self, block_tables, seq_lens) -> None:
        """Install a batch: `seq_lens` are the lengths BEFORE the next step's token (0 = inactive row)."""
        bt = torch.as_tensor(block_tables, dtype=torch.int32)
        sl = torch.as_tensor(seq_lens, dtype=torch.int32)
        if bt.ndim != 2 or bt.shape[0] > self.rows or bt.shape[1] > self.table_width or sl.shape != (bt.shape[0],):
            raise ValueError("block_tables [rows, W] and seq_lens [rows] must fit the resident arrays")
        if int(sl.max()) >= self.table_width * self.block_size:
            raise ValueError("a row has no room left in its block table")
        self.block_tables.zero_()
        self.seq_lens.zero_()
        self.block_tables[: bt.shape[0], : bt.shape[1]].copy_(bt, non_blocking=True)
        self.seq_lens[: sl.shape[0]].copy_(sl, non_blocking=True)
        self.positions.copy_((self.seq_lens - 1).clamp_(min=0).view(-1, 1))

    def set_block(self, row: int, index: int, block_id: int) -> None:
        """The host allocated block `block_id` as block `index` of `row` (do this before the row's length reaches it)."""
        if not (0 <= row < self.rows and 0 <= index < self.table_width):
            raise ValueError("row or block index outside the resident block table")
        self.block_tables[row, index] = int(block_id)

    def advance(self) -> None:
        """positions <- seq_lens, seq_lens += 1 for every active row; no host involvement."""
        lib = _lib.load()
        _lib.check(lib.nvj_advance_decode_metadata(self.seq_lens.data_ptr(), self.positions.data_ptr(), self.rows,
                                                   self.table_width, self.block_size, self._status.data_ptr(),
                                                   torch.cuda.current_stream(self.device).cuda_stream),
                   "nvj_advance_decode_metadata")

    def check(self) -> None:
        """Synchronise and raise if a row ran out of block-table room."""
        word = int(self._status.item())
        if word:
            self._status.zero_()
            raise _k.DeviceStatusError(f"resident decode metadata: device status {word} (a row outgrew its block table)")


class DecodeStepGraph:
    """append + decode -> argmax + metadata advance of one layer, captured once, replayed per step."""

    def __init__(self, meta: ResidentDecodeMetadata, k_cache: torch.Tensor, v_cache: torch.Tensor, layer_id: int,
                 scale: float, num_key_value_groups: int, query_dtype=torch.bfloat16, token_gather=None):
        """`token_gather` (a `parallel.P2PTokenGather` over `meta.rows` tokens) makes the token pick publish the step's
        tokens to every rank over NVLink; `gathered` holds every rank's tokens of the step BEFORE the one just replayed
        (each step's launch collects the step before), and `flush()` brings it up to date."""
        if k_cache.ndim != 5:
            raise ValueError("k_cache must be the 5-D cache [L, NB, bs, Hkv, D]")
        self.meta, self.k_cache, self.v_cache = meta, k_cache, v_cache
        self.layer_id, self.scale, self.groups = int(layer_id), float(scale), int(num_key_value_groups)
        _, _, bs, hkv, d = k_cache.shape
        if bs != meta.block_size:
            raise ValueError("cache block size differs from the metadata's")
        dev = meta.device
        self.query = torch.zeros((meta.rows, 1, hkv * self.groups, d), dtype=query_dtype, device=dev)
        self.new_k = torch.zeros((meta.rows, 1, hkv, d), dtype=k_cache.dtype, device=dev)
        self.new_v = torch.zeros((meta.rows, 1, hkv, d), dtype=v_cache.dtype, device=dev)
        self.out: Optional[torch.Tensor] = None
        self.tokens: Optional[torch.Tensor] = None
        self.token_gather = token_gather
        self.gathered = (torch.empty(token_gather.world * meta.rows, dtype=torch.int32, device=dev)
                         if token_gather is not None else None)
        self._captured: Optional[CapturedStep] = None
        self._tokens = torch.empty(meta.rows, dtype=torch.int32, device=dev)

    def _step(self):
        m = self.meta
        out, _, _ = _k.paged_decode_attention_with_kv_append(self.query, self.new_k, self.new_v, self.k_cache, self.v_cache,
                                                             m.block_tables, m.seq_lens, None, self.layer_id, m.block_size,
                                                             self.scale, self.groups)
        advance = (m.seq_lens, m.positions, m.table_width, m.block_size)
        if self.token_gather is None:
            return out, _k.row_argmax(out.view(m.rows, -1), self._tokens, advance=advance)
        # one launch: collect the step before, pick this step's tokens, publish them, advance the lengths
        return out, self.token_gather.publish_argmax(out.view(m.rows, -1), self._tokens, collect_out=self.gathered,
                                                     advance=advance)

    def flush(self) -> Optional[torch.Tensor]:
        """Collect the tokens of the last replayed step into `gathered` (several GPUs only)."""
        if self.token_gather is not None:
            self.token_gather.collect(out=self.gathered)
        return self.gathered

    def capture(self):
        """Run one real step from the current `query`, `new_k`, `new_v` (on a side stream: capture needs warm kernels
        and workspaces) and then capture the step for `replay()`.  Returns that first step's (out, tokens)."""
        self._captured = CapturedStep(self._step, self.meta.device)
        first = self._captured.capture()
        self.out, self.tokens = self._captured.result
        return first

    def replay(self):
        """One decode step from the current contents of `query`, `new_k`, `new_v`; returns (out, tokens) views that
        the next replay overwrites."""
        if self._captured is None:
            raise RuntimeError("capture() has not been called")
        return self._captured.replay()
