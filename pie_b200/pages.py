"""Host-side page bookkeeping: which physical page ids each request presents to the kernels.

Semantics follow the reference:
  * `IdPool`  - smallest-free-id allocator with tail compaction
                (runtime/src/utils.rs:42-158).
  * `PagePool` - reference counts on top of the id pool; a page returns to the pool when its last
                owner lets go (sdk/rust/inferlet/src/forward.rs:28-55 `KvPage` drop ->
                runtime/src/model/resource.rs:225-254 deallocate).  Recycled pages are NOT cleared.
  * `KvPageList` - one context's page list and last-page fill: grow / shrink / fork / adopt
                (sdk/javascript/src/kv-page-manager.ts, sdk/rust/inferlet/src/context.rs:147-225,356-399).
                `fork()` is the reference behaviour (share full pages, drop the partial one and report
                the tokens to recompute); `fork_cow()` is this library's extension: the partial page is
                duplicated with `ops.copy_kv_pages` instead of being recomputed.
  * `build_csr` - the kv_page_indices / kv_page_indptr / kv_last_page_lens arrays of a batch
                (wire layout runtime/src/model/request.rs:332-409).
"""
from __future__ import annotations

import heapq
from typing import Iterable, List, Optional, Sequence, Tuple

import numpy as np


class PoolExhausted(RuntimeError):
    """No free page id is left ("ID pool exhausted", runtime/src/utils.rs:86-93)."""


class IdPool:
    """Bounded pool that always hands out the smallest available id."""

    TAIL_COMPACTION_THRESHOLD = 1000  # runtime/src/utils.rs:119,133

    def __init__(self, max_capacity: int) -> None:
        self._next = 0
        self._free: set = set()
        self._heap: List[int] = []
        self._cap = int(max_capacity)

    @property
    def capacity(self) -> int:
        return self._cap

    def set_capacity(self, capacity: int) -> None:
        if capacity < self._next:
            raise ValueError("Cannot set capacity lower than the next ID")
        self._cap = int(capacity)

    def available(self) -> int:
        return len(self._free) + (self._cap - self._next)

    def acquire(self) -> int:
        while self._heap:
            i = heapq.heappop(self._heap)
            if i in self._free:  # lazy deletion: ids removed by tail compaction stay in the heap
                self._free.discard(i)
                return i
        if self._next < self._cap:
            i = self._next
            self._next += 1
            return i
        raise PoolExhausted("ID pool exhausted")

    def acquire_many(self, count: int) -> List[int]:
        if self.available() < count:
            raise PoolExhausted("ID pool exhausted")
        return [self.acquire() for _ in range(count)]

    def release(self, i: int) -> None:
        self.release_many([i])

    def release_many(self, ids: Iterable[int]) -> None:
        for i in ids:
            if i >= self._next or i < 0:
                raise ValueError("ID was never allocated")
            if i not in self._free:
                self._free.add(i)
                heapq.heappush(self._heap, i)
        if len(self._free) > self.TAIL_COMPACTION_THRESHOLD:
            self._tail_compaction()

    def _tail_compaction(self) -> None:
        while self._next > 0 and (self._next - 1) in self._free:
            self._free.discard(self._next - 1)
            self._next -= 1
        if len(self._heap) > 4 * (len(self._free) + 16):
            self._heap = list(self._free)
            heapq.heapify(self._heap)


class PagePool:
    """Reference-counted physical pages of one GPU's pool."""

    def __init__(self, num_pages: int) -> None:
        self.ids = IdPool(num_pages)
        self.refs = np.zeros(num_pages, dtype=np.int32)

    def alloc(self, count: int) -> List[int]:
        pages = self.ids.acquire_many(count)
        self.refs[pages] = 1
        return pages

    def ref(self, pages: Sequence[int]) -> None:
        for p in pages:
            if self.refs[p] <= 0:
                raise ValueError(f"page {p} is not allocated")
            self.refs[p] += 1

    def release(self, pages: Sequence[int]) -> List[int]:
        """Drop one reference per page; returns the pages that went back to the free list."""
        freed = []
        for p in pages:
            if self.refs[p] <= 0:
                raise ValueError(f"page {p} is not allocated")
            self.refs[p] -= 1
            if self.refs[p] == 0:
                freed.append(p)
        if freed:
            self.ids.release_many(freed)
        return freed

    def available(self) -> int:
        return self.ids.available()


class KvPageList:
    """Pages and last-page fill of one context."""

    def __init__(self, pool: PagePool, page_size: int) -> None:
        self.pool = pool
        self.page_size = int(page_size)
        self.pages: List[int] = []
        self.last_page_len = 0

    # -- kv-page-manager.ts:19-31
    @property
    def page_count(self) -> int:
        return len(self.pages)

    @property
    def total_tokens(self) -> int:
        if not self.pages:
            return self.last_page_len
        return (len(self.pages) - 1) * self.page_size + self.last_page_len

    def _set_last(self, total: int) -> None:
        r = total % self.page_size
        self.last_page_len = self.page_size if (r == 0 and total > 0) else r

    # -- kv-page-manager.ts:150-181 (adjust)
    def grow(self, num_tokens: int) -> List[int]:
        """Make room for `num_tokens` more tokens; returns the newly allocated pages."""
        return self._adjust(num_tokens)

    def shrink(self, num_tokens: int) -> None:
        self._adjust(-num_tokens)

    def _adjust(self, delta: int) -> List[int]:
        if delta == 0:
            return []
        new_total = self.total_tokens + delta
        if new_total < 0:
            raise ValueError("Token count adjustment resulted in underflow")
        required = -(-new_total // self.page_size)
        new_pages: List[int] = []
        if required > len(self.pages):
            new_pages = self.pool.alloc(required - len(self.pages))
            self.pages.extend(new_pages)
        elif required < len(self.pages):
            drop = self.pages[required:]
            del self.pages[required:]
            self.pool.release(drop)
        self._set_last(new_total)
        return new_pages

    # -- kv-page-manager.ts:57-86 (fork shares FULL pages only)
    def fork(self) -> Tuple["KvPageList", int]:
        """Reference fork: the child shares every page but the last one; returns (child, number of
        tokens of the dropped last page that the caller has to recompute)."""
        kept = max(0, len(self.pages) - 1)
        child = KvPageList(self.pool, self.page_size)
        child.pages = self.pages[:kept]
        child.last_page_len = self.page_size if kept > 0 else 0
        self.pool.ref(child.pages)
        return child, self.total_tokens - kept * self.page_size

    def fork_cow(self) -> Tuple["KvPageList", Optional[Tuple[int, int, int]]]:
        """Copy-on-write fork: full pages are shared, a partially filled last page is given a private
        copy.  Returns (child, (src_page, dst_page, valid_len)) - the copy to run with
        `ops.copy_kv_pages` - or (child, None) when the last page is full (it is then shared: nobody
        writes into a full page again)."""
        child = KvPageList(self.pool, self.page_size)
        child.last_page_len = self.last_page_len
        if not self.pages:
            return child, None
        if self.last_page_len == self.page_size:
            child.pages = list(self.pages)
            self.pool.ref(child.pages)
            return child, None
        shared = self.pages[:-1]
        self.pool.ref(shared)
        (fresh,) = self.pool.alloc(1)
        child.pages = shared + [fresh]
        return child, (self.pages[-1], fresh, self.last_page_len)

    def release(self) -> List[int]:
        freed = self.pool.release(self.pages)
        self.pages = []
        self.last_page_len = 0
        return freed

    def adopt(self, other: "KvPageList") -> None:
        """Become a co-owner of `other`'s pages (beam-search winner, kv-page-manager.ts:103-112)."""
        self.release()
        self.pages = list(other.pages)
        self.last_page_len = other.last_page_len
        self.pool.ref(self.pages)

    def remove_page_at(self, index: int) -> None:
        """Drop one fully masked page (kv-page-manager.ts:127-140)."""
        if index < 0 or index >= len(self.pages):
            raise IndexError(f"Page index {index} out of bounds")
        removed = self.pages.pop(index)
        self.pool.release([removed])
        self._set_last(self.total_tokens)

    def drop_masked_kv_pages(self, masked: Sequence[bool]) -> List[int]:
        """Drop every FULL page all of whose tokens are masked (`masked[t]` true = token t is hidden from every
        later query), newest first, and return the indices (positions in the page list) that were dropped, in
        the order they were dropped - the caller removes the same token ranges from its token / position /
        mask lists.  The last page is only a candidate when it is full.  The physical pages go back to the pool
        (sdk/rust/inferlet/src/context.rs:298-345; used for attention-sink style windows)."""
        if len(masked) < self.total_tokens:
            raise ValueError(f"mask covers {len(masked)} tokens, the context holds {self.total_tokens}")
        total = self.total_tokens
        committed = total // self.page_size
        flags = np.asarray(masked[: committed * self.page_size], dtype=bool).reshape(committed, self.page_size)
        dropped: List[int] = []
        for i in range(committed - 1, -1, -1):
            if flags[i].all():
                self.pool.release([self.pages.pop(i)])
                dropped.append(i)
        self._set_last(total - len(dropped) * self.page_size)
        return dropped


def eval_max_num_kv_pages(free_bytes: int, gpu_mem_utilization: float, page_size: int, num_kv_heads: int,
                          head_dim: int, num_layers: int, dtype, tensor_parallel_size: int = 1,
                          group=None, device=None) -> int:
    """How many KV pages fit: `free_bytes * gpu_mem_utilization` over the bytes of one page across all layers,
    with the KV heads split over the tensor-parallel ranks (pie/src/pie_worker/model/llama3.py:177-202).  With
    a process group the free-memory figure is first reduced to the MINIMUM over its ranks, so every rank sizes
    the same pool (pie/src/pie_worker/utils.py:108-119)."""
    import torch

    if group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()
                             and tensor_parallel_size > 1):
        t = torch.tensor(int(free_bytes), dtype=torch.int64, device=device if device is not None else "cpu")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN, group=group)
        free_bytes = int(t.item())
    es = torch.empty((), dtype=dtype).element_size()
    local_kv_heads = num_kv_heads // tensor_parallel_size
    per_page = es * 2 * page_size * local_kv_heads * head_dim * num_layers
    return int((free_bytes * gpu_mem_utilization) // per_page)


def build_csr(contexts: Sequence[KvPageList]) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """(kv_page_indices, kv_page_indptr, kv_last_page_lens) int32 of a batch of contexts."""
    counts = np.fromiter((len(c.pages) for c in contexts), dtype=np.int64, count=len(contexts))
    indptr = np.zeros(len(contexts) + 1, dtype=np.int32)
    np.cumsum(counts, out=indptr[1:])
    indices = np.empty(int(indptr[-1]), dtype=np.int32)
    for c, s in zip(contexts, indptr[:-1]):
        indices[s: s + len(c.pages)] = c.pages
    last = np.fromiter((c.last_page_len for c in contexts), dtype=np.int32, count=len(contexts))
    return indices, indptr, last


class NativePageManager:
    """The library's native (C++) page manager: id pool, reference counts, per-instance ownership, the
    reference's out-of-memory policy (instances that started after the requester are terminated, newest
    first; runtime/src/model/resource.rs:112-319) and export / import by name (resource.rs:356-451).
    `IdPool` / `PagePool` above are the same id and reference-count rules in Python; this class is what a
    runtime embeds."""

    def __init__(self, num_pages: int) -> None:
        import ctypes as C

        from . import _lib
        self._C, self._lib = C, _lib
        self._h = _lib.lib.piekv_pages_create(int(num_pages))
        if not self._h:
            raise ValueError("piekv_pages_create failed")
        self.num_pages = int(num_pages)

    def close(self) -> None:
        if self._h:
            self._lib.lib.piekv_pages_destroy(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    def _arr(self, pages: Sequence[int]):
        return (self._C.c_int32 * len(pages))(*[int(p) for p in pages])

    def available(self) -> int:
        return int(self._lib.lib.piekv_pages_available(self._h))

    def refcount(self, page: int) -> int:
        return int(self._lib.lib.piekv_pages_refcount(self._h, int(page)))

    def owned(self, instance: int) -> int:
        return int(self._lib.lib.piekv_pages_owned(self._h, int(instance)))

    def alloc(self, instance: int, count: int) -> Tuple[List[int], List[int]]:
        """(pages, instances terminated to make room).  Raises PoolExhausted when even that is not enough."""
        out = (self._C.c_int32 * max(count, 1))()
        rc = self._lib.lib.piekv_pages_alloc(self._h, int(instance), int(count), out)
        if rc == self._lib.STATUS_OUT_OF_PAGES:
            raise PoolExhausted(self._lib.lib.piekv_last_error_string().decode())
        self._lib.check(rc, "pages_alloc")
        vbuf = (self._C.c_uint64 * 64)()
        nv = int(self._lib.lib.piekv_pages_last_victims(self._h, vbuf, 64))
        return [int(out[i]) for i in range(count)], [int(vbuf[i]) for i in range(min(nv, 64))]

    def free(self, instance: int, pages: Sequence[int]) -> None:
        self._lib.check(self._lib.lib.piekv_pages_free(self._h, int(instance), self._arr(pages), len(pages)),
                        "pages_free")

    def share(self, instance: int, pages: Sequence[int]) -> None:
        self._lib.check(self._lib.lib.piekv_pages_share(self._h, int(instance), self._arr(pages), len(pages)),
                        "pages_share")

    def cleanup(self, instance: int) -> None:
        self._lib.check(self._lib.lib.piekv_pages_cleanup(self._h, int(instance)), "pages_cleanup")

    def export(self, instance: int, pages: Sequence[int], name: str) -> None:
        self._lib.check(self._lib.lib.piekv_pages_export(self._h, int(instance), self._arr(pages), len(pages),
                                                         name.encode()), "pages_export")

    def import_(self, name: str) -> List[int]:
        out = (self._C.c_int32 * self.num_pages)()
        n = int(self._lib.lib.piekv_pages_import(self._h, name.encode(), out, self.num_pages))
        if n < 0:
            raise KeyError(name)
        return [int(out[i]) for i in range(n)]

    def release_exported(self, name: str) -> None:
        self._lib.check(self._lib.lib.piekv_pages_release_exported(self._h, name.encode()), "pages_release_exported")


class DevicePageTable:
    """Page tables, reference counts and the free list of one pool kept in DEVICE memory
    (`piekv_pagestate_*`): the same rules as `IdPool` / `PagePool` / `KvPageList` above - smallest free id
    first, pages = ceil(tokens / page_size), forks share full pages and copy a partial one, a page goes back
    to the free list with its last holder - advanced by small stream-ordered kernels.  A decode loop, or a
    beam search that forks and drops contexts, then runs without the host building or uploading a page
    table, and the whole step can sit in a CUDA graph.

    Requests live in numbered slots.  Slot lists are int32 device tensors (a slot at most once per call);
    requests are served in list order, exactly like a host loop over the same list."""

    def __init__(self, num_pages: int, max_requests: int, pages_per_request: int, page_size: int = 16,
                 device="cuda", max_batch: Optional[int] = None) -> None:
        import torch

        from . import _lib, ops
        self._torch, self._lib, self._ops = torch, _lib, ops
        self.num_pages, self.max_requests = int(num_pages), int(max_requests)
        self.pages_per_request, self.page_size = int(pages_per_request), int(page_size)
        self.device = torch.device(device)
        nbytes = int(_lib.lib.piekv_pagestate_bytes(self.num_pages, self.max_requests, self.pages_per_request))
        self.state = torch.empty(nbytes // 4, dtype=torch.int32, device=self.device)
        mb = int(max_batch or min(self.max_requests, 1024))
        self.max_batch = mb
        i32 = dict(dtype=torch.int32, device=self.device)
        self.kv_indptr = torch.zeros(mb + 1, **i32)
        self.kv_indices = torch.zeros(mb * self.pages_per_request, **i32)
        self.kv_last_page_len = torch.zeros(mb, **i32)
        self.pos_ids = torch.zeros(mb, **i32)
        self.copy_src = torch.zeros(mb, **i32)
        self.copy_dst = torch.zeros(mb, **i32)
        self.copy_valid = torch.zeros(mb, **i32)
        _lib.check(_lib.lib.piekv_pagestate_init(self.state.data_ptr(), nbytes, *self._dims(), self._stream()),
                   "pagestate_init")

    def _dims(self):
        return self.num_pages, self.max_requests, self.pages_per_request, self.page_size

    def _stream(self):
        return self._ops._stream(self.device)

    def _err(self):
        return self._ops._err_word(self.device).data_ptr()

    def _slots(self, slots, name="slots"):
        self._ops._require_i32(slots, name)
        if slots.shape[0] > self.max_batch:
            raise ValueError(f"{name}: {slots.shape[0]} entries, this table was built for {self.max_batch}")
        return slots

    def grow(self, slots, delta=1, csr: bool = True):
        """Make room for `delta` more tokens (an int for all, or an int32 device tensor per request; negative
        values shrink) in the listed requests - `adjust_kv_pages` of the reference
        (sdk/rust/inferlet/src/context.rs:356-399).  With `csr`, the page table of exactly this batch is
        written to this object's buffers and returned as views:
        (kv_indptr, kv_indices, kv_last_page_len, pos_ids); pos_ids = tokens held before the call."""
        slots = self._slots(slots)
        n = slots.shape[0]
        torch = self._torch
        deltas_ptr, delta_all = None, 0
        if isinstance(delta, torch.Tensor):
            self._ops._require_i32(delta, "delta")
            if delta.shape[0] != n:
                raise ValueError("delta: one entry per slot")
            deltas_ptr = delta.data_ptr()
        else:
            delta_all = int(delta)
        self._lib.check(self._lib.lib.piekv_pagestate_adjust(
            self.state.data_ptr(), *self._dims(), slots.data_ptr(), deltas_ptr, delta_all, n,
            self.kv_indptr.data_ptr() if csr else None, self.kv_indices.data_ptr() if csr else None,
            self.kv_last_page_len.data_ptr() if csr else None, self.pos_ids.data_ptr() if csr else None,
            self._err(), self._stream()), "pagestate_adjust")
        if not csr:
            return None
        return self.kv_indptr[: n + 1], self.kv_indices, self.kv_last_page_len[:n], self.pos_ids[:n]

    def table_of(self, slots):
        """The CSR page table of a batch without changing it."""
        return self.grow(slots, 0, csr=True)

    def release(self, slots) -> None:
        """The listed requests let go of all their pages (`KvPageList.release`)."""
        slots = self._slots(slots)
        self._lib.check(self._lib.lib.piekv_pagestate_release(self.state.data_ptr(), *self._dims(), slots.data_ptr(),
                                                              slots.shape[0], self._err(), self._stream()),
                        "pagestate_release")

    def fork(self, parents, children):
        """children[i] becomes a copy-on-write fork of parents[i] (`KvPageList.fork_cow`).  Returns the device
        tensors (src_pages, dst_pages, valid_len) for `ops.copy_kv_pages`, one entry per fork (valid 0 where the
        parent's last page was full and is shared)."""
        parents, children = self._slots(parents, "parents"), self._slots(children, "children")
        n = parents.shape[0]
        if children.shape[0] != n:
            raise ValueError("parents and children differ in length")
        self._lib.check(self._lib.lib.piekv_pagestate_fork(
            self.state.data_ptr(), *self._dims(), parents.data_ptr(), children.data_ptr(), n,
            self.copy_src.data_ptr(), self.copy_dst.data_ptr(), self.copy_valid.data_ptr(), self._err(),
            self._stream()), "pagestate_fork")
        return self.copy_src[:n], self.copy_dst[:n], self.copy_valid[:n]

    def snapshot(self) -> dict:
        """Host copy of the whole state (synchronises): free page count, per-slot page lists and last-page
        fill, reference counts, and the set of free ids."""
        w = self.state.cpu().numpy()
        r, c, p = self.max_requests, self.pages_per_request, self.num_pages
        npages = w[16: 16 + r].copy()
        last = w[16 + r: 16 + 2 * r].copy()
        table = w[16 + 2 * r: 16 + 2 * r + r * c].reshape(r, c)
        refs = w[16 + 2 * r + r * c: 16 + 2 * r + r * c + p].copy()
        bits = w[16 + 2 * r + r * c + p:].view(np.uint32)
        free = np.unpackbits(bits.view(np.uint8), bitorder="little")[:p].astype(bool)
        return {"free_pages": int(w[0]), "npages": npages, "last_page_len": last,
                "pages": [table[i, : npages[i]].tolist() for i in range(r)], "refs": refs, "free": free}
