"""Sharding of the path across the GPUs of one node (one process per GPU, torch.distributed).

Two schemes, both taken from the reference:

* request sharding - every data-parallel group owns its requests and its own page pool and no tensor
  crosses GPUs (runtime/src/model/resource.rs:83-87 per-group pools, :118-126 round-robin placement,
  pie/src/pie/manager.py:473-488 one worker process per GPU);
* KV-head sharding - rank g holds KV heads [g*Hkv/G, (g+1)*Hkv/G) and their query heads of EVERY request,
  with identical page tables (pie/src/pie_worker/model/llama3.py:607-610,963-965).  The reference then
  all-reduces after the row-parallel o_proj (llama3.py:698-706); on a path that ends at the attention
  output the equivalent exchange is an all-gather of the per-rank head slices.

The collective is NCCL's (gloo on CPU for the tests); nothing here touches peer memory directly.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_requests(num_requests: int, world: int, rank: int) -> List[int]:
    """Requests of rank `rank`: r -> GPU r mod G (round-robin, resource.rs:118-126)."""
    return list(range(rank, num_requests, world))


def shard_heads(num_qo_heads: int, num_kv_heads: int, world: int, rank: int) -> Tuple[slice, slice]:
    """(query-head slice, kv-head slice) of rank `rank`; heads of one GQA group stay together."""
    if num_kv_heads % world != 0 or num_qo_heads % num_kv_heads != 0:
        raise ValueError(f"{num_kv_heads} KV heads cannot be split over {world} ranks")
    kl = num_kv_heads // world
    group = num_qo_heads // num_kv_heads
    return slice(rank * kl * group, (rank + 1) * kl * group), slice(rank * kl, (rank + 1) * kl)


def allgather_heads(out_local: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                    gather_buffer: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[n, Hq/G, D] on every rank -> [n, Hq, D] on every rank (rank order = head order).

    One all-gather (4 MiB at 256 requests x 64 heads x 128 x bf16: latency bound on NVLink) and one
    strided copy that interleaves the rank-major result back into head order."""
    world = dist.get_world_size(group)
    n, hl, d = out_local.shape
    if world == 1:
        return out_local
    buf = gather_buffer
    if buf is None or tuple(buf.shape) != (world, n, hl, d) or buf.dtype != out_local.dtype:
        buf = torch.empty((world, n, hl, d), dtype=out_local.dtype, device=out_local.device)
    src = out_local.contiguous()
    try:
        dist.all_gather_into_tensor(buf.view(world * n, hl, d), src, group=group)
    except (RuntimeError, NotImplementedError):
        dist.all_gather([buf[g] for g in range(world)], src, group=group)
    return buf.permute(1, 0, 2, 3).reshape(n, world * hl, d)
