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
`PeerReduce` is the same idea one step further down the layer: the row-parallel o_proj whose epilogue
sums the ranks' partial results over NVLink, in place of the reference's linear + all_reduce + residual.
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


def reduce_layout(n_max: int, hidden: int, world: int, elem_size: int) -> dict:
    """Offsets inside a rank's shared allocation for `PeerReduce`: arrival flags, completion flags,
    staging, two output buffers; sizes from the library (`piekv_oproj_allreduce_sizes`)."""
    from . import _lib
    sizes = (C.c_int64 * 3)()
    _lib.check(_lib.lib.piekv_oproj_allreduce_sizes(n_max, hidden, world, sizes), "oproj_allreduce_sizes")
    stage_bytes, arrive_words, done_words = int(sizes[0]), int(sizes[1]), int(sizes[2])
    up = lambda x: (x + 255) // 256 * 256
    lay = {"stage_bytes": stage_bytes, "arrive_words": arrive_words, "done_words": done_words}
    lay["arrive"] = 0
    lay["done"] = up(4 * arrive_words)
    lay["stage"] = lay["done"] + up(4 * done_words)
    lay["out0"] = lay["stage"] + up(stage_bytes)
    out_bytes = up(n_max * hidden * elem_size)
    lay["out1"] = lay["out0"] + out_bytes
    lay["nbytes"] = lay["out1"] + out_bytes
    return lay


class PeerReduce:
    """Row-parallel output projection without a collective: `oproj(a, w_o, residual)` launches one kernel
    per rank that computes this rank's partial product, sends it as fp32 to the rank that owns each tile,
    sums the ranks there in rank order, adds the residual, rounds once and stores the rows into EVERY
    rank's output buffer (pie/src/pie_worker/model/llama3.py:693-709: linear, all_reduce, residual add).
    The returned [n, hidden] tensor is complete on this rank when the kernel ends, and holds the same
    bits on every rank.  Two output buffers alternate from step to step: a result stays valid until the
    call after the next.  Consume it on the stream the next call is queued on.
    `partial_sums="storage"` sends the partial sums rounded to the 16-bit dtype, as an all-reduce of 16-bit
    tensors does (half the NVLink bytes; for prefill-sized batches on four or more ranks, where the link is
    the limit); the default sends fp32 and rounds once.

    One process per GPU on one node; every rank makes the same calls with the same sizes.  Collective
    constructor and `close()`."""

    def __init__(self, n_max: int, hidden: int, dtype: torch.dtype, device,
                 group: Optional[dist.ProcessGroup] = None, partial_sums: str = "fp32") -> None:
        from . import _lib
        self._lib = _lib
        self.group = group
        if partial_sums not in ("fp32", "storage"):
            raise ValueError("partial_sums: 'fp32', or 'storage' to send them rounded to the 16-bit dtype")
        self.partial_sums = partial_sums
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > _lib.MAX_PEERS:
            raise ValueError(f"{self.world} ranks: at most {_lib.MAX_PEERS} GPUs of one node")
        self.device = torch.device(device)
        self.n_max, self.hidden, self.dtype = int(n_max), int(hidden), dtype
        es = torch.empty((), dtype=dtype).element_size()
        self._lay = reduce_layout(self.n_max, self.hidden, self.world, es)
        self.nbytes = self._lay["nbytes"]
        ptr = C.c_void_p()
        handle = C.create_string_buffer(_lib.PEER_HANDLE_BYTES)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib.piekv_peer_alloc(self.nbytes, C.byref(ptr), handle), "peer_alloc")
            self._own = int(ptr.value)
            self._base: Optional[List[int]] = [self._own] * self.world
            if self.world > 1:
                handles: List[Optional[bytes]] = [None] * self.world
                dist.all_gather_object(handles, handle.raw, group=group)
                for r in range(self.world):
                    if r == self.rank:
                        continue
                    q = C.c_void_p()
                    _lib.check(_lib.lib.piekv_peer_open(handles[r], C.byref(q)), f"peer_open(rank {r})")
                    self._base[r] = int(q.value)
        self._local = torch.as_tensor(_RawCuda(self._own, self.nbytes), device=self.device)
        self.step = 0
        self._desc = None
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=group)  # every rank has mapped every buffer before anyone stores

    def _descriptor(self):
        """The library's description of this step: one prebuilt struct per output buffer, the step number set."""
        if self._desc is None:
            lay = self._lay
            self._desc = []
            for off in (lay["out1"], lay["out0"]):   # index = step & 1
                d = self._lib.PeerReduceC()
                for r in range(self.world):
                    d.out[r] = self._base[r] + off
                    d.stage[r] = self._base[r] + lay["stage"]
                    d.arrive[r] = self._base[r] + lay["arrive"]
                    d.done[r] = self._base[r] + lay["done"]
                d.stage_bytes, d.arrive_words, d.done_words = lay["stage_bytes"], lay["arrive_words"], lay["done_words"]
                d.world, d.rank = self.world, self.rank
                d.flags = self._lib.REDUCE_PARTIALS_16BIT if self.partial_sums == "storage" else 0
                self._desc.append(d)
        d = self._desc[self.step & 1]
        d.step = self.step
        return d

    def oproj(self, a: torch.Tensor, w_o: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """a: [n, k_local] (or [n, local heads, head_dim]) this rank's attention rows; w_o: [hidden, k_local]
        this rank's columns of the projection weight; residual: None or [n, hidden] (the same on every rank).
        Returns residual + sum over ranks of a @ w_o.T as [n, hidden], a view of this step's buffer."""
        from .ops import _dtype_code, _err_word, _require_cuda, _stream
        _require_cuda(a, "a")
        _require_cuda(w_o, "w_o")
        if a.dim() == 3:
            a = a.reshape(a.shape[0], -1)
        if a.dim() != 2 or w_o.dim() != 2 or a.stride(1) != 1 or w_o.stride(1) != 1:
            raise ValueError("a and w_o must be 2-D with contiguous rows")
        n, k = a.shape
        if tuple(w_o.shape) != (self.hidden, k):
            raise ValueError(f"w_o shape {tuple(w_o.shape)} differs from ({self.hidden}, {k})")
        if n > self.n_max:
            raise ValueError(f"{n} rows: the buffers were sized for {self.n_max}")
        if a.dtype != self.dtype or w_o.dtype != self.dtype:
            raise ValueError("a and w_o must have the dtype the buffers were made for")
        if residual is not None:
            _require_cuda(residual, "residual")
            if tuple(residual.shape) != (n, self.hidden) or residual.dtype != self.dtype or residual.stride(1) != 1:
                raise ValueError("residual must be [n, hidden] with contiguous rows, of the same dtype")
        if n == 0:
            return torch.empty((0, self.hidden), dtype=self.dtype, device=self.device)
        self.step += 1
        d = self._descriptor()
        try:
            self._lib.check(self._lib.lib.piekv_oproj_allreduce(
                a.data_ptr(), a.stride(0), w_o.data_ptr(), w_o.stride(0),
                residual.data_ptr() if residual is not None else None,
                residual.stride(0) if residual is not None else 0, n, k, self.hidden,
                _dtype_code(self.dtype, "oproj_allreduce"), C.byref(d), _err_word(self.device).data_ptr(),
                _stream(self.device)), "oproj_allreduce")
        except Exception:
            self.step -= 1   # nothing was launched: the step number is not used up
            raise
        return self.result(n)

    def result(self, n: int) -> torch.Tensor:
        """[n, hidden] rows of the latest step on this rank."""
        off = self._lay["out0"] if (self.step & 1) else self._lay["out1"]
        return self._local[off:].view(self.dtype)[: n * self.hidden].view(n, self.hidden)

    def close(self) -> None:
        if self._base is None:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)  # nobody is still storing into a buffer about to go away
        with torch.cuda.device(self.device):
            for r, b in enumerate(self._base):
                if r != self.rank:
                    self._lib.lib.piekv_peer_close(b)
            self._local = None
            if self.world > 1:
                dist.barrier(group=self.group)  # everyone has unmapped before the owners free
            self._lib.lib.piekv_peer_free(self._own)
        self._base = None
