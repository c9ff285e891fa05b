"""Request partition across GPUs and the per-step token gather.

The path shards by request: request id i lives on rank i % world, which owns that
request's KV blocks, block-table rows and GDN state; appends and attention never
touch another rank's memory.  The only exchange is the gather of each step's
output tokens (int32 per row): `gather_tokens` does it with `torch.distributed`
(NCCL on GPUs; the same code runs on the gloo backend in CPU tests), and
`P2PTokenGather` with one small kernel per rank that stores the tokens straight
into its peers' memory over NVLink (one node, one process per GPU), which takes
a few microseconds where the library call takes 7-20.  Its split form
(`publish_argmax` / `collect`) fuses the publish with the step's token pick and
collects a step's tokens one step later, so that a rank which is late by less
than one step delays nobody.  The reference is
single-device and has no counterpart of this module.

Failures.  A rank that dies or never joins shows up here in one of two ways:
the library collective raises when the process group's timeout runs out
(`gather_tokens` re-raises it as `TokenGatherError` naming the rank), or a
device-side wait of the peer-store gather runs out (`nvj_set_wait_limit_ns`),
the kernel returns, and `P2PTokenGather.check()` raises `DeviceStatusError`.
Nothing waits without a limit.

Prefix reuse and GDN snapshots stay rank-local: a request can only hit a prefix
that an earlier request of the same rank computed.
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def owner_rank(request_id: int, world: int) -> int:
    return int(request_id) % int(world)


def local_request_ids(num_requests: int, rank: int, world: int) -> List[int]:
    """Global ids of the requests rank `rank` owns, in local row order."""
    return list(range(rank, num_requests, world))


def max_local_rows(num_requests: int, world: int) -> int:
    return -(-num_requests // world)


class TokenGatherError(RuntimeError):
    """The per-step token all-gather failed (a peer left, or the process group's timeout ran out)."""


def set_wait_limit(seconds: float) -> None:
    """Limit of every device-side wait on another GPU (default 1 s)."""
    from . import _lib
    _lib.load().nvj_set_wait_limit_ns(int(max(0.0, float(seconds)) * 1e9))


def gather_tokens(local_tokens: torch.Tensor, num_requests: int, group: Optional[dist.ProcessGroup] = None,
                  pad_value: int = -1) -> torch.Tensor:
    """All-gather one int32 token per local row and return them in global request order.

    Every rank contributes `max_local_rows` entries (short ranks pad), so one
    fixed-size all-gather serves every step.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return local_tokens[:num_requests].clone()
    rows = max_local_rows(num_requests, world)
    send = torch.full((rows,), pad_value, dtype=torch.int32, device=local_tokens.device)
    send[: local_tokens.numel()] = local_tokens.to(torch.int32)
    recv = torch.empty(world * rows, dtype=torch.int32, device=local_tokens.device)
    try:
        dist.all_gather_into_tensor(recv, send, group=group)
    except (RuntimeError, dist.DistBackendError) as exc:  # a peer that left, or the group's timeout
        raise TokenGatherError(f"rank {dist.get_rank(group)} of {world}: token all-gather failed: {exc}") from exc
    # rank r's row j is request j * world + r: transpose [world, rows] -> [rows, world]
    return recv.view(world, rows).t().reshape(-1)[:num_requests].contiguous()


class P2PTokenGather:
    """All-gather of `n` int32 per rank by NVLink peer stores (nvj_p2p_allgather_i32).

    Every rank allocates an exchange buffer, the ranks swap its CUDA IPC handle through the process
    group once, and each step is then a single kernel launch per rank with no library collective.
    All ranks must call `gather` the same number of times.  Raises `NvjError` at construction when the
    buffers cannot be shared (ranks on different nodes, IPC disabled): fall back to `gather_tokens`.
    """

    def __init__(self, n: int, group: Optional[dist.ProcessGroup] = None, device=None):
        import ctypes

        from . import _lib
        self._lib = _lib.load()
        self._check = _lib.check
        self.n = int(n)
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._peers = []
        with torch.cuda.device(self.device):
            nbytes = int(self._lib.nvj_p2p_gather_buffer_bytes(self.world, self.n))
            if nbytes <= 0:
                raise ValueError("world size or row count outside the supported range")
            own = ctypes.c_void_p()
            handle = (ctypes.c_ubyte * 64)()
            rc = self._lib.nvj_p2p_buffer_create(nbytes, ctypes.byref(own), handle)
            self._own = own.value if rc == 0 else None
            if self.world == 1:
                self._check(rc, "nvj_p2p_buffer_create")
            # from here to the all_reduce below every rank takes every collective, whatever failed locally
            handles = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, bytes(handle) if rc == 0 else None, group=group)
            ptrs, failure = [], (rc if rc != 0 else None)
            for r in range(self.world):
                if failure is not None:
                    break
                if r == self.rank:
                    ptrs.append(self._own)
                    continue
                if handles[r] is None:
                    failure = -2
                    break
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(handles[r])
                peer = ctypes.c_void_p()
                rc = self._lib.nvj_p2p_buffer_open(buf, ctypes.byref(peer))
                if rc != 0:
                    failure = rc
                    break
                self._peers.append(peer.value)
                ptrs.append(peer.value)
            self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
            if self.world > 1:
                # every buffer is mapped everywhere before the first store; and either all ranks go on or none does
                ok = torch.tensor([0 if failure is not None else 1], dtype=torch.int32, device=self.device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
                if int(ok.item()) == 0:
                    self.close(group=None, _collective=False)
                    self._check(failure if failure is not None else -2, "nvj_p2p_buffer_open (on some rank)")  # -2 = NVJ_ERR_UNSUPPORTED
            self._ptr_array = (ctypes.c_void_p * self.world)(*ptrs)

    def gather(self, local_tokens: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Returns `[world * n]` int32: rank r's tokens at `[r * n, (r + 1) * n)`; launches on the current stream."""
        if local_tokens.dtype != torch.int32 or local_tokens.numel() != self.n or not local_tokens.is_cuda:
            raise ValueError("local_tokens must be a CUDA int32 tensor of n elements")
        local_tokens = local_tokens.contiguous()
        if out is None:
            out = torch.empty(self.world * self.n, dtype=torch.int32, device=self.device)
        # epoch 0: the step count lives in the exchange buffer and the kernel advances it, so the same launch can be
        # captured into a CUDA graph and replayed
        rc = self._lib.nvj_p2p_allgather_i32(local_tokens.data_ptr(), self.n, self.rank, self.world, self._ptr_array,
                                             0, out.data_ptr(), self._status.data_ptr(),
                                             torch.cuda.current_stream(self.device).cuda_stream)
        self._check(rc, "nvj_p2p_allgather_i32")
        return out

    def publish_argmax(self, x: torch.Tensor, tokens: Optional[torch.Tensor] = None,
                       collect_out: Optional[torch.Tensor] = None, advance=None) -> torch.Tensor:
        """tokens[r] = argmax of row r of the float32 `[n, row_len]` tensor, and the same tokens stored into every peer's
        buffer and published as this rank's next epoch.  The publish waits for nobody.  With `collect_out` (`[world * n]`
        int32) the same launch first collects the step before into it, as `collect` would: one launch per step, and the
        gathered tokens lag the step by one.  `advance=(seq_lens, positions or None, table_width, block_size)` also
        advances the rows' resident decode metadata in that launch (see `paged_kv.row_argmax`).  Returns the local
        tokens."""
        if x.dtype != torch.float32 or x.ndim != 2 or x.shape[0] != self.n or not x.is_cuda or not x.is_contiguous():
            raise ValueError("x must be a contiguous CUDA float32 tensor [n, row_len]")
        if tokens is None:
            tokens = torch.empty(self.n, dtype=torch.int32, device=self.device)
        if collect_out is not None and (collect_out.dtype != torch.int32 or collect_out.numel() != self.world * self.n
                                        or not collect_out.is_cuda or not collect_out.is_contiguous()):
            raise ValueError("collect_out must be a contiguous CUDA int32 tensor of world * n elements")
        seq_lens = positions = None
        table_width, block_size = 0, 1
        if advance is not None:
            from .kernels.paged_kv import _advance_args
            seq_lens, positions, table_width, block_size = _advance_args(advance, self.n)
        rc = self._lib.nvj_p2p_argmax_publish(x.data_ptr(), self.n, int(x.shape[1]), tokens.data_ptr(), self.rank, self.world,
                                              self._ptr_array, None if collect_out is None else collect_out.data_ptr(),
                                              None if seq_lens is None else seq_lens.data_ptr(),
                                              None if positions is None else positions.data_ptr(), table_width, block_size,
                                              self._status.data_ptr(), torch.cuda.current_stream(self.device).cuda_stream)
        self._check(rc, "nvj_p2p_argmax_publish")
        return tokens

    def collect(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Fetch the oldest published step that has not been collected: `[world * n]` int32, rank r's tokens at
        `[r * n, (r + 1) * n)`.  Leaves `out` untouched when every published step has been collected already."""
        if out is None:
            out = torch.empty(self.world * self.n, dtype=torch.int32, device=self.device)
        rc = self._lib.nvj_p2p_collect(self._own, self.n, self.world, out.data_ptr(), self._status.data_ptr(),
                                       torch.cuda.current_stream(self.device).cuda_stream)
        self._check(rc, "nvj_p2p_collect")
        return out

    def check(self) -> None:
        """Synchronise and raise if a wait for the peers ran out."""
        if int(self._status.item()):
            self._status.zero_()
            from .kernels.paged_kv import DeviceStatusError
            raise DeviceStatusError("token all-gather: a peer did not publish its tokens within the limit")

    def close(self, group: Optional[dist.ProcessGroup] = None, _collective: bool = True) -> None:
        """Unmap the peers' buffers, wait for every rank to have done so, free the own buffer."""
        torch.cuda.synchronize(self.device)
        for p in self._peers:
            self._lib.nvj_p2p_buffer_close(p)
        self._peers = []
        if _collective and self.world > 1 and dist.is_initialized():
            dist.barrier(group=group)
        if self._own:
            self._lib.nvj_p2p_buffer_destroy(self._own)
            self._own = None
