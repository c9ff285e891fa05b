"""Request partition across GPUs and the per-step token gather.

The path shards by request: request id i lives on rank i % world, which owns that
request's KV blocks, block-table rows and GDN state; appends and attention never
touch another rank's memory.  The only exchange is the gather of each step's
output tokens (int32 per row), done with `torch.distributed` (NCCL on GPUs; the
same code runs on the gloo backend in CPU tests).  The reference is
single-device and has no counterpart of this module.

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
    dist.all_gather_into_tensor(recv, send, group=group)
    # rank r's row j is request j * world + r: transpose [world, rows] -> [rows, world]
    return recv.view(world, rows).t().reshape(-1)[:num_requests].contiguous()
