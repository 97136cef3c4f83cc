"""Sharding of the path across the GPUs of one node (one process per GPU, torch.distributed).

Two schemes, both taken from the reference:

* request sharding - every data-parallel group owns its requests and its own page pool and no tensor
  crosses GPUs (runtime/src/model/resource.rs:83-87 per-group pools, :118-126 round-robin placement,
  pie/src/pie/manager.py:473-488 one worker process per GPU);
* KV-head sharding - rank g holds KV heads [g*Hkv/G, (g+1)*Hkv/G) and their query heads of EVERY request,
  with identical page tables (pie/src/pie_worker/model/llama3.py:607-610,963-965).  The reference then
  all-reduces after the row-parallel o_proj (llama3.py:698-706); on a path that ends at the attention
  output the equivalent exchange is an all-gather of the per-rank head slices.

`allgather_heads` uses NCCL's collective (gloo on CPU for the tests).  `PeerOutputs` is the other way
to join head-sharded ranks: output buffers mapped into every process of the node, which the decode
kernel itself fills on all GPUs with plain peer stores, so no collective follows the attention.
"""
from __future__ import annotations

import ctypes as C
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


class _RawCuda:
    """Lets torch view device memory that the library allocated (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def peer_layout(batch_max: int, row_heads: int, head_dim: int, elem_size: int) -> Tuple[int, int, int]:
    """(offset of output buffer 0, offset of output buffer 1, total bytes) inside a rank's shared
    allocation; the flag words sit at offset 0."""
    buf = (batch_max * row_heads * head_dim * elem_size + 255) // 256 * 256
    return 256, 256 + buf, 256 + 2 * buf


class PeerOutputs:
    """Head-sharded decode without a collective: every rank's decode kernel writes its heads into the
    output rows of ALL ranks (NVLink peer stores) and raises a flag; `wait()` queues a bounded wait for
    all flags on the stream, after which `full(batch)` is the [batch, row_heads, head_dim] result on
    this rank.  Two output buffers alternate from step to step.

    One process per GPU on one node.  Collective constructor and `close()` (every rank must call them
    together): the IPC handles travel through `torch.distributed.all_gather_object`."""

    def __init__(self, batch_max: int, row_heads: int, head_dim: int, dtype: torch.dtype, device,
                 group: Optional[dist.ProcessGroup] = None) -> None:
        from . import _lib
        self._lib = _lib
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > _lib.MAX_PEERS:
            raise ValueError(f"{self.world} ranks: at most {_lib.MAX_PEERS} GPUs of one node")
        self.device = torch.device(device)
        self.batch_max, self.row_heads, self.head_dim, self.dtype = int(batch_max), int(row_heads), int(head_dim), dtype
        es = torch.empty((), dtype=dtype).element_size()
        self._off0, self._off1, self.nbytes = peer_layout(batch_max, row_heads, head_dim, es)
        ptr = C.c_void_p()
        handle = C.create_string_buffer(_lib.PEER_HANDLE_BYTES)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib.piekv_peer_alloc(self.nbytes, C.byref(ptr), handle), "peer_alloc")
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            self._own = int(ptr.value)
            self._base: List[int] = []
            for r in range(self.world):
                if r == self.rank:
                    self._base.append(self._own)
                    continue
                q = C.c_void_p()
                _lib.check(_lib.lib.piekv_peer_open(handles[r], C.byref(q)), f"peer_open(rank {r})")
                self._base.append(int(q.value))
        self._local = torch.as_tensor(_RawCuda(self._own, self.nbytes), device=self.device)
        self.step = 0
        self._counter_off = 128  # device-side step counter (graph replays), after the flag words
        self._local[self._counter_off: self._counter_off + 4].view(torch.int32).fill_(1)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)  # every rank has mapped every buffer before anyone stores

    def begin_step(self):
        """Descriptor (ctypes struct) of the next step's destinations."""
        self.step += 1
        off = self._off0 if (self.step & 1) else self._off1
        d = self._lib.PeerOutputsC()
        for r in range(self.world):
            d.out[r] = self._base[r] + off
            d.flags[r] = self._base[r]
        d.world, d.rank, d.row_heads, d.step = self.world, self.rank, self.row_heads, self.step
        return d

    def counted_descriptor(self):
        """Descriptor for launches that take the step number from the device-side counter (odd steps use
        the first output buffer, even steps the second), i.e. for launches captured in a CUDA graph.
        Every captured or eager use must be followed by `wait_counted()` and `advance()`."""
        d = self._lib.PeerOutputsC()
        for r in range(self.world):
            d.out[r] = self._base[r] + self._off0
            d.out_alt[r] = self._base[r] + self._off1
            d.flags[r] = self._base[r]
        d.world, d.rank, d.row_heads, d.step = self.world, self.rank, self.row_heads, 0
        d.step_counter = self._own + self._counter_off
        return d

    def wait_counted(self) -> None:
        """Queue the wait for the step the device counter names; it increments the counter afterwards."""
        from .ops import _err_word, _stream
        self._lib.check(self._lib.lib.piekv_peer_wait_counted(self._own, self.world, self._own + self._counter_off,
                                                              _err_word(self.device).data_ptr(),
                                                              _stream(self.device)), "peer_wait_counted")

    def advance(self, steps: int = 1) -> None:
        """Tell the host mirror that `steps` counted steps have been queued (once per graph replay of that
        many steps), so that `full()` names the buffer of the latest one."""
        self.step += int(steps)

    def wait(self) -> None:
        """Queue, on the current stream, the wait for every rank's flag of the current step."""
        from .ops import _err_word, _stream
        self._lib.check(self._lib.lib.piekv_peer_wait(self._own, self.world, self.step,
                                                      _err_word(self.device).data_ptr(), _stream(self.device)),
                        "peer_wait")

    def full(self, batch: int) -> torch.Tensor:
        """[batch, row_heads, head_dim] rows of the current step on this rank (valid after `wait()`)."""
        off = self._off0 if (self.step & 1) else self._off1
        n = batch * self.row_heads * self.head_dim
        return self._local[off:].view(self.dtype)[:n].view(batch, self.row_heads, self.head_dim)

    def close(self) -> None:
        if self._base is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # nobody is still storing into a buffer about to go away
        with torch.cuda.device(self.device):
            for r, b in enumerate(self._base):
                if r != self.rank:
                    self._lib.lib.piekv_peer_close(b)
            self._local = None
            dist.barrier(group=self.group)  # everyone has unmapped before the owners free
            self._lib.lib.piekv_peer_free(self._own)
        self._base = None
