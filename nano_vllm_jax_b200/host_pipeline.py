"""Decode steps whose operands live in host memory, with the copies taken off the critical path.

A caller that keeps queries, new K/V rows and batch metadata in (pinned) host
memory pays a host-to-device copy before every `write_kv_and_attention` and a
device-to-host copy after it.  On one stream these serialise with the kernel
(C2: ~0.4 ms per step against 0.25 ms of kernel time).  `HostDecodePipeline`
keeps `depth` steps in flight on three streams, so the two copy engines move
step i + 1's operands and step i - 1's result while step i computes:

    h2d stream      copy(i+1)            copy(i+2)
    compute stream  append+decode(i)     append+decode(i+1)
    d2h stream      result(i-1)          result(i)

Every step still copies all of its operands from the host and its whole result
back; steps are issued in order and the cache is only touched by the compute
stream, so the cache contents are those of the serial execution.  The
attention call itself is `B200Backend.write_kv_and_attention`
(the reference's boundary, nanovllm_jax/backends.py:1252-1461).

With `capture=True` the compute part of a slot (metadata, fused append +
decode, `after_compute`) is captured into a CUDA graph the first time the slot
is used for a layer and replayed afterwards.  The per-step host work of the
attention call (argument checks, pointer marshalling, the launch itself: a few
hundred microseconds of Python, more than the kernel takes) shrinks to one
graph launch, and the pipeline becomes device-bound.  `after_compute` must then
be capturable (no host synchronisation) and the same callable on every step.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch

from .backends import B200Backend
from .kernels import paged_kv as _k
from .kv_cache import KVCacheStorage


@dataclass
class _Slot:
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    tables: torch.Tensor
    positions: torch.Tensor
    seq_lens: torch.Tensor
    host_out: torch.Tensor
    in_done: torch.cuda.Event
    compute_done: torch.cuda.Event
    out_done: torch.cuda.Event
    busy: bool = False
    graphs: Dict[int, torch.cuda.CUDAGraph] = field(default_factory=dict)  # per layer, with capture=True
    graph_out: Dict[int, torch.Tensor] = field(default_factory=dict)
    inputs: tuple = ()           # (q, k, v, tables, positions, seq_lens): the targets of the step's operand copies
    h2d_list: object = None      # paged_kv.CopyList over `inputs`; the sources are set per step
    d2h_lists: Dict[int, object] = field(default_factory=dict)  # per layer: host_out <- that layer's graph output
    sources: list = field(default_factory=list)
    last_out: Optional[torch.Tensor] = None


class HostDecodePipeline:
    """`depth` decode steps in flight; operands from host tensors, results into pinned host tensors."""

    def __init__(self, backend: B200Backend, cache: KVCacheStorage, rows: int, table_width: int, block_size: int,
                 scale: float, num_key_value_groups: int, depth: int = 2, query_dtype=torch.bfloat16,
                 capture: bool = False):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        if not isinstance(backend, B200Backend):
            raise TypeError("backend must be a B200Backend")
        dev = cache.k_cache.device
        _, _, _, hkv, d = cache.k_cache.shape
        hq = hkv * num_key_value_groups
        self.backend, self.cache, self.capture = backend, cache, bool(capture)
        self.rows, self.block_size, self.scale, self.groups = rows, block_size, scale, num_key_value_groups
        self.h2d, self.compute, self.d2h = (torch.cuda.Stream(dev) for _ in range(3))
        self.slots = []
        for _ in range(depth):
            self.slots.append(_Slot(
                q=torch.empty((rows, 1, hq, d), dtype=query_dtype, device=dev),
                k=torch.empty((rows, 1, hkv, d), dtype=cache.k_cache.dtype, device=dev),
                v=torch.empty((rows, 1, hkv, d), dtype=cache.v_cache.dtype, device=dev),
                tables=torch.empty((rows, table_width), dtype=torch.int32, device=dev),
                positions=torch.empty((rows, 1), dtype=torch.int32, device=dev),
                seq_lens=torch.empty((rows,), dtype=torch.int32, device=dev),
                host_out=torch.empty((rows, 1, hq * d), dtype=torch.float32).pin_memory(),
                in_done=torch.cuda.Event(), compute_done=torch.cuda.Event(), out_done=torch.cuda.Event()))
        for slot in self.slots:
            slot.inputs = (slot.q, slot.k, slot.v, slot.tables, slot.positions, slot.seq_lens)
            slot.h2d_list = _k.CopyList(slot.inputs, slot.inputs)  # sources replaced by every submit
        self.compute.wait_stream(torch.cuda.current_stream(dev))  # whatever prepared the cache comes first
        self.submitted = 0
        self.h2d_bytes_per_step = sum(t.numel() * t.element_size() for t in
                                      (self.slots[0].q, self.slots[0].k, self.slots[0].v, self.slots[0].tables,
                                       self.slots[0].positions, self.slots[0].seq_lens))
        self.d2h_bytes_per_step = self.slots[0].host_out.numel() * 4

    def submit(self, layer_id: int, query, k, v, block_tables, positions, seq_lens,
               after_compute=None) -> int:
        """Queue one step from host tensors (pinned for the copies to be asynchronous); returns its ticket.

        Blocks the host only while the slot's previous step (`depth` steps ago) is still in flight.
        `after_compute(out)` runs on the compute stream right after the attention call (token pick, collectives).
        """
        ticket = self.submitted
        slot = self.slots[ticket % len(self.slots)]
        if slot.busy:
            slot.out_done.synchronize()  # its operands were consumed and its result has left the device
        # the step's operands: six copies in one library call (a framework copy per operand costs the host ~8 us each)
        srcs = []
        for i, (t, dst) in enumerate(zip((query, k, v, block_tables, positions, seq_lens), slot.inputs)):
            if t.dtype != dst.dtype or not t.is_contiguous():
                t = t.to(dst.dtype).contiguous()
            if t.numel() != dst.numel():
                raise ValueError(f"operand {i} has {t.numel()} elements, the slot holds {dst.numel()}")
            slot.h2d_list.set_source(i, t)
            srcs.append(t)
        slot.sources = srcs  # alive until the slot comes round again
        slot.h2d_list.issue(self.h2d)
        slot.in_done.record(self.h2d)
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(slot.in_done)
            if not self.capture:
                out = self._compute(slot, layer_id, after_compute)
            elif layer_id in slot.graphs:
                slot.graphs[layer_id].replay()
                out = slot.graph_out[layer_id]
            else:
                out = self._capture(slot, layer_id, after_compute)
            slot.compute_done.record(self.compute)
        self.d2h.wait_event(slot.compute_done)
        back = slot.d2h_lists.get(layer_id) if out is slot.graph_out.get(layer_id) else None
        if back is None:
            back = _k.CopyList([slot.host_out], [out.reshape(slot.host_out.shape)])
            if out is slot.graph_out.get(layer_id):
                slot.d2h_lists[layer_id] = back  # a graph's output lives in the graph's own pool: same address every step
            else:
                out.record_stream(self.d2h)
                slot.last_out = out
        back.issue(self.d2h)
        slot.out_done.record(self.d2h)
        slot.busy = True
        self.submitted += 1
        return ticket

    def _compute(self, slot: _Slot, layer_id: int, after_compute):
        md = self.backend.build_attention_metadata(slot.positions, slot.tables, slot.seq_lens, self.block_size, False)
        _, out = self.backend.write_kv_and_attention(layer_id, slot.q, slot.k, slot.v, self.cache, md, self.block_size,
                                                     self.scale, self.groups, False)
        if after_compute is not None:
            after_compute(out)
        return out

    def _capture(self, slot: _Slot, layer_id: int, after_compute):
        """First use of (slot, layer): run the step once (this is the step's execution; it also warms kernels and
        workspaces), then record the same calls for the replays.  Runs on the compute stream."""
        first = self._compute(slot, layer_id, after_compute)
        strict = os.environ.get("NVJ_CHECK_STATUS")
        os.environ["NVJ_CHECK_STATUS"] = "0"  # reading the status word back is a host sync: not capturable
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self.compute, capture_error_mode="thread_local"):
                slot.graph_out[layer_id] = self._compute(slot, layer_id, after_compute)
            slot.graphs[layer_id] = graph
        finally:
            if strict is None:
                os.environ.pop("NVJ_CHECK_STATUS", None)
            else:
                os.environ["NVJ_CHECK_STATUS"] = strict
        return first

    def result(self, ticket: int) -> torch.Tensor:
        """The step's attention output `[rows, 1, Hq*D]` fp32 in pinned host memory (valid until the slot is reused)."""
        if not self.submitted - len(self.slots) <= ticket < self.submitted:
            raise ValueError("ticket is not in flight any more (or not submitted yet)")
        slot = self.slots[ticket % len(self.slots)]
        slot.out_done.synchronize()
        return slot.host_out

    def drain(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        """Make `stream` (default: the current one) wait for every step submitted so far, without blocking the host."""
        stream = torch.cuda.current_stream(self.cache.k_cache.device) if stream is None else stream
        for slot in self.slots:
            if slot.busy:
                stream.wait_event(slot.out_done)
