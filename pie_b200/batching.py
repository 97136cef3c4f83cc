"""Host feeder of the path: wire fields of a batched forward-pass request -> index arrays and the
flat boolean attention mask.

Mirror of the part of `Batch.__init__` / `get_model_inputs` that feeds the paged-KV operators
(pie/src/pie_worker/batching.py:28-135,196-239; wire layout runtime/src/model/request.rs:250-298):
the fields arrive as little-endian uint32 byte strings (lists are accepted too), are decoded to int32
arrays, and the per-token BRLE masks are expanded to one row of kv_len booleans per query token.
BRLE = alternating run lengths starting with an ATTEND run (sdk/rust/inferlet/src/brle.rs:4-21);
only the first `position + 1` bits of a row can be set, where position = context_len + index of the token
in its request (pie/src/pie_worker/batching.py:113-122,367-387).

The expansion is vectorised numpy (the reference uses a Numba loop); the result is the tensor that
`BatchPrefillWithPagedKVCacheWrapper.plan(custom_mask=...)` takes, which the library then bit-packs
on the device.
"""
from __future__ import annotations

from typing import Any, Dict

import numpy as np
import torch


def _u32(data) -> np.ndarray:
    if isinstance(data, (bytes, bytearray, memoryview)):
        return np.frombuffer(data, dtype=np.uint32)
    return np.asarray(data, dtype=np.uint32)


def decode_brle_batch(flattened_masks: np.ndarray, mask_indptr: np.ndarray, position_ids: np.ndarray,
                      token_acc_seq_lens: np.ndarray) -> np.ndarray:
    """Flat boolean mask from per-token BRLE runs (semantics of pie/src/pie_worker/batching.py:337-389).

    Vectorised: every run becomes a [start, end) interval inside its token's row, clipped to the row's
    valid length; attend-runs (even index within the token) add +1 / -1 to a difference array whose
    prefix sum is the mask."""
    runs = np.asarray(flattened_masks, dtype=np.int64)
    ptr = np.asarray(mask_indptr, dtype=np.int64)
    valid = np.asarray(position_ids, dtype=np.int64) + 1
    acc = np.asarray(token_acc_seq_lens, dtype=np.int64)
    total = int(acc[-1])
    if total == 0 or len(runs) == 0:
        return np.zeros(total, dtype=np.bool_)
    ntok = len(valid)
    counts = np.diff(ptr)
    tok = np.repeat(np.arange(ntok), counts)
    # exclusive prefix of the run lengths inside each token
    csum = np.cumsum(runs)
    base = np.concatenate([[0], csum])[ptr[:-1]]
    start = csum - runs - np.repeat(base, counts)
    end = start + runs
    v = valid[tok]
    start = np.minimum(start, v)
    end = np.minimum(end, v)
    idx_in_tok = np.arange(len(runs)) - np.repeat(ptr[:-1], counts)
    attend = (idx_in_tok % 2 == 0) & (end > start)
    row0 = acc[:-1][tok]
    diff = np.zeros(total + 1, dtype=np.int32)
    np.add.at(diff, (row0 + start)[attend], 1)
    np.add.at(diff, (row0 + end)[attend], -1)
    return np.cumsum(diff[:-1]) > 0


class Batch:
    """The index arrays and mask of one batched forward pass."""

    def __init__(self, args: Dict[str, Any], kv_page_size: int) -> None:
        self.token_ids = _u32(args["token_ids"]).astype(np.int64)
        self.position_ids = _u32(args["position_ids"]).astype(np.int32)
        self.kv_page_indices = _u32(args["kv_page_indices"]).astype(np.int32)
        self.kv_page_indptr = _u32(args["kv_page_indptr"]).astype(np.int32)
        self.kv_last_page_lens = _u32(args["kv_last_page_lens"]).astype(np.int32)
        self.qo_indptr = _u32(args["qo_indptr"]).astype(np.int32)
        self.single_token_mode = bool(args.get("single_token_mode", False))
        self.total_tokens = int(len(self.token_ids))

        self.flattened_masks = _u32(args["flattened_masks"]).astype(np.uint32)
        self.mask_indptr = _u32(args["mask_indptr"]).astype(np.int32)
        runs = self.flattened_masks.astype(np.int64)
        mask_indptr = self.mask_indptr.astype(np.int64)
        counts = np.diff(self.qo_indptr).astype(np.int64)
        npages = np.diff(self.kv_page_indptr).astype(np.int64)
        last = self.kv_last_page_lens.astype(np.int64)
        # a request without pages keeps last_len as its length (pie/src/pie_worker/batching.py:104-111)
        self.seq_lens = np.where(npages > 0, (npages - 1) * kv_page_size + last, last)
        all_seq = np.repeat(self.seq_lens, counts)
        ctx = self.seq_lens - counts
        pos = np.arange(self.total_tokens, dtype=np.int64) - np.repeat(self.qo_indptr[:-1].astype(np.int64), counts) \
            + np.repeat(ctx, counts)
        acc = np.zeros(self.total_tokens + 1, dtype=np.int64)
        np.cumsum(all_seq, out=acc[1:])
        self.mask_bits = int(acc[-1])
        self.attention_masks = decode_brle_batch(runs, mask_indptr, pos, acc)

    def brle_inputs(self, device):
        """The mask in its wire form for `BatchPrefillWithPagedKVCacheWrapper.plan(brle_mask=...)`:
        (run lengths, per-token offsets into them, number of (query, key) pairs).  A few bytes per query
        token instead of one byte per pair; the library expands it to bits on the device."""
        dev = torch.device(device)
        # int32 view of the unsigned words: the kernel reads them as unsigned again
        runs = torch.from_numpy(np.ascontiguousarray(self.flattened_masks).view(np.int32).copy())
        return (runs.to(dev), torch.as_tensor(self.mask_indptr, dtype=torch.int32, device=dev), self.mask_bits)

    def get_model_inputs(self, device) -> Dict[str, Any]:
        """Device tensors in the form the operators take (pie/src/pie_worker/batching.py:196-239)."""
        dev = torch.device(device)

        def t(a, dt):
            return torch.as_tensor(a, device=dev, dtype=dt)

        return {
            "token_ids": t(self.token_ids, torch.long),
            "position_ids": t(self.position_ids, torch.int32),
            "qo_indptr": t(self.qo_indptr, torch.int32),
            "kv_page_indices": t(self.kv_page_indices, torch.int32),
            "kv_page_indptr": t(self.kv_page_indptr, torch.int32),
            "kv_last_page_lens": t(self.kv_last_page_lens, torch.int32),
            "custom_mask": t(self.attention_masks, torch.bool),
            "single_token_inference_mode": self.single_token_mode,
            "total_pages_cpu": self.kv_page_indptr[-1] if len(self.kv_page_indptr) else 0,
        }


WIRE_FIELDS = ("token_ids", "position_ids", "kv_page_indices", "kv_page_indptr", "kv_last_page_lens", "qo_indptr",
               "flattened_masks", "mask_indptr")


class DeviceBatch:
    """A batched forward-pass request taken to the device in its wire form.

    The eight uint32 arrays of `BatchedForwardPassRequest` (runtime/src/model/request.rs:250-298) are
    concatenated into one pinned host buffer and uploaded with ONE copy; what `Batch.__init__` derives on the
    host per token or per (query, key) pair (pie/src/pie_worker/batching.py:96-135) is derived on the device:
    `seq_lens`, `batch_indices`, `positions` (kv slot of every token = the position the mask rows are cut at),
    int64 `token_ids`, optionally `token_acc_seq_lens`, and - through
    `BatchPrefillWithPagedKVCacheWrapper.plan(brle_mask=batch.brle_inputs())` - the attention mask, bit-packed
    straight from the run lengths.  The index tensors (`kv_page_indptr`, `kv_page_indices`, `kv_last_page_lens`,
    `qo_indptr`, `position_ids`) are int32 VIEWS of the uploaded buffer: no conversion, no second copy.
    The only host work is O(requests): the field lengths and the number of mask entries."""

    def __init__(self, args: Dict[str, Any], kv_page_size: int, device="cuda", acc_seq_lens: bool = False) -> None:
        import ctypes as C

        from . import _lib, ops
        dev = torch.device(device)
        fields = {k: np.ascontiguousarray(_u32(args[k])) for k in WIRE_FIELDS}
        lay = _lib.WireBatch()
        off = 0
        for k in WIRE_FIELDS:
            setattr(lay, k, off)
            off += int(fields[k].size)
        lay.nnz = int(fields["token_ids"].size)
        lay.batch = max(int(fields["qo_indptr"].size) - 1, 0)
        lay.total_pages = int(fields["kv_page_indices"].size)
        lay.num_runs = int(fields["flattened_masks"].size)
        if fields["kv_page_indptr"].size != lay.batch + 1 or fields["kv_last_page_lens"].size != lay.batch:
            raise ValueError("kv_page_indptr / kv_last_page_lens / qo_indptr describe different batch sizes")
        if fields["position_ids"].size != lay.nnz or fields["mask_indptr"].size not in (0, lay.nnz + 1):
            raise ValueError("position_ids / mask_indptr do not match the number of tokens")
        host = torch.empty(max(off, 1), dtype=torch.int32).pin_memory()
        hv = host.numpy().view(np.uint32)
        for k in WIRE_FIELDS:
            o = getattr(lay, k)
            hv[o: o + fields[k].size] = fields[k]
        self.wire = host.to(dev, non_blocking=True)  # the one upload
        self.layout = lay
        self.page_size = int(kv_page_size)
        self.single_token_mode = bool(args.get("single_token_mode", False))
        self.total_tokens, self.batch = lay.nnz, lay.batch
        self.total_pages_cpu = lay.total_pages

        def view(name, n):
            o = getattr(lay, name)
            return self.wire[o: o + n]

        self.position_ids = view("position_ids", lay.nnz)
        self.kv_page_indices = view("kv_page_indices", lay.total_pages)
        self.kv_page_indptr = view("kv_page_indptr", lay.batch + 1)
        self.kv_last_page_lens = view("kv_last_page_lens", lay.batch)
        self.qo_indptr = view("qo_indptr", lay.batch + 1)
        self._runs = view("flattened_masks", lay.num_runs)
        self._run_indptr = view("mask_indptr", int(fields["mask_indptr"].size))
        # O(requests) on the host: how many (query, key) pairs the mask has (sizes the packed mask)
        counts = np.diff(fields["qo_indptr"].astype(np.int64))
        npages = np.diff(fields["kv_page_indptr"].astype(np.int64))
        last = fields["kv_last_page_lens"].astype(np.int64)
        self.mask_bits = int(np.sum(counts * np.where(npages > 0, (npages - 1) * kv_page_size + last, last)))
        i32 = dict(dtype=torch.int32, device=dev)
        self.token_ids = torch.empty(lay.nnz, dtype=torch.int64, device=dev)
        self.seq_lens = torch.empty(lay.batch, **i32)
        self.batch_indices = torch.empty(lay.nnz, **i32)
        self.positions = torch.empty(lay.nnz, **i32)
        self.token_acc_seq_lens = torch.empty(lay.nnz + 1, dtype=torch.int64, device=dev) if acc_seq_lens else None
        _lib.check(_lib.lib.piekv_batch_from_wire(
            self.wire.data_ptr(), C.byref(lay), self.page_size, self.token_ids.data_ptr(), self.seq_lens.data_ptr(),
            self.batch_indices.data_ptr(), self.positions.data_ptr(),
            self.token_acc_seq_lens.data_ptr() if acc_seq_lens else None, ops._stream(dev)), "batch_from_wire")

    def brle_inputs(self):
        """(run lengths, per-token offsets, mask entries) as views of the uploaded buffer, for
        `BatchPrefillWithPagedKVCacheWrapper.plan(brle_mask=...)`."""
        return self._runs, self._run_indptr, self.mask_bits

    def get_model_inputs(self) -> Dict[str, Any]:
        """The reference's `get_model_inputs` dictionary (pie/src/pie_worker/batching.py:196-239) with the mask in
        its wire form under `brle_mask` instead of the expanded `custom_mask`."""
        return {
            "token_ids": self.token_ids, "position_ids": self.position_ids, "qo_indptr": self.qo_indptr,
            "kv_page_indices": self.kv_page_indices, "kv_page_indptr": self.kv_page_indptr,
            "kv_last_page_lens": self.kv_last_page_lens, "brle_mask": self.brle_inputs(),
            "single_token_inference_mode": self.single_token_mode, "total_pages_cpu": self.total_pages_cpu,
        }
