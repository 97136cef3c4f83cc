"""CUDA-graph decode step with batch-size bins and padding.

Mirror of the reference's graphed decode path for the part that touches the paged-KV operators
(pie/src/pie_worker/model/llama3.py: bins 241-249, capture 315-414, replay 866-956): one graph per
batch-size bin is captured over static buffers; a step copies its metadata into those buffers, pads
the batch up to the bin with rows that own one scratch page holding one token, replays the graph and
returns a copy of the real rows.  Batches larger than the largest bin fall back to an eager plan + run.

What is captured per layer is the single fused launch of this library (RoPE + append + attention,
`BatchDecodeWithPagedKVCacheWrapper.run_fused`); the wrapper reads the page tables on the device at run
time, so replaying with new table contents needs no re-plan.  With several layer pools the graph holds the
whole layer loop over ONE set of step metadata, as the reference's does (llama3.py:915-956): either the
default loop (layer l reads q/k/v[l] and writes out[l]) or a caller's `body`, which may put its own work
(projections, norms) between the `attend` calls so that one replay is one whole decode step.

Two deliberate differences from the reference's replay code: the padded rows' page ids are written
every step (the reference leaves whatever the shared index buffer held beyond the real pages), and
the padded rows append into the scratch page (the reference sends them to request 0, position 0).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from . import ops


def graph_bins(limit: int) -> List[int]:
    """Batch sizes that get a graph: powers of two up to 16, then every 16 from 24, then the limit
    itself (llama3.py:241-249)."""
    limit = int(limit) if limit else 512
    bins = [b for b in (1, 2, 4, 8, 16) if b <= limit]
    if limit > 16:
        bins.extend(range(24, limit + 1, 16))
        if bins[-1] < limit:
            bins.append(limit)
    return sorted(set(bins))


def pick_bin(bins: List[int], batch: int) -> Optional[int]:
    """Smallest bin that holds `batch` requests, None when none does."""
    for b in bins:
        if b >= batch:
            return b
    return None


class GraphedDecodeStep:
    """One captured decode step per bin over shared static buffers: a fused launch per layer.

    `pool` is one layer's pool or a list of them (all of one shape).  `body(runner, b)`, if given, is what
    gets captured for bin `b` instead of the default layer loop; it calls `runner.attend(layer, q, k, v)` once
    per layer on tensors of `b` rows that live in static memory of its own."""

    def __init__(self, pool, num_qo_heads: int, num_kv_heads: int, max_batch: int,
                 max_total_pages: int, rope: Optional[ops.RopeConfig] = None,
                 workspace: Optional[torch.Tensor] = None, body=None) -> None:
        self.pools = list(pool) if isinstance(pool, (list, tuple)) else [pool]
        self._single = not isinstance(pool, (list, tuple))
        self.body = body
        shapes = {tuple(p.shape) for p in self.pools}
        if len(shapes) != 1 or len({p.dtype for p in self.pools}) != 1:
            raise ValueError("layer pools differ in shape or dtype")
        pool = self.pools[0]
        num_pages, page_size, hkv, d = ops._check_pool(pool)
        if hkv != num_kv_heads:
            raise ValueError("pool kv heads differ from num_kv_heads")
        self.pool = pool
        self.scratch_page = num_pages - 1  # the reference allocates P + 1 pages, the last one for padding
        self.hq, self.hkv, self.d, self.page_size = int(num_qo_heads), int(num_kv_heads), int(d), int(page_size)
        self.rope = rope if rope is not None else ops.RopeConfig()
        self.bins = graph_bins(max_batch)
        self.max_bin = self.bins[-1]
        dev, dt = pool.device, pool.dtype
        L = len(self.pools)
        self.num_layers = L
        self.q = torch.zeros((L, self.max_bin, self.hq, d), dtype=dt, device=dev)
        self.k = torch.zeros((L, self.max_bin, self.hkv, d), dtype=dt, device=dev)
        self.v = torch.zeros((L, self.max_bin, self.hkv, d), dtype=dt, device=dev)
        self.out = torch.zeros((L, self.max_bin, self.hq, d), dtype=dt, device=dev)
        self.pos = torch.zeros(self.max_bin, dtype=torch.int32, device=dev)
        self.indices = torch.full((int(max_total_pages) + self.max_bin,), self.scratch_page, dtype=torch.int32,
                                  device=dev)
        # per bin: (indptr, last_page_len) of exactly the bin's size, as in the reference
        self.aux: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {
            b: (torch.zeros(b + 1, dtype=torch.int32, device=dev), torch.ones(b, dtype=torch.int32, device=dev))
            for b in self.bins}
        self.workspace = workspace if workspace is not None else torch.zeros(128 << 20, dtype=torch.uint8, device=dev)
        self.wrappers = {b: ops.BatchDecodeWithPagedKVCacheWrapper(self.workspace, "NHD") for b in self.bins}
        self.fallback = ops.BatchDecodeWithPagedKVCacheWrapper(self.workspace, "NHD")
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self._pad_ramp = torch.arange(1, self.max_bin + 1, dtype=torch.int32, device=dev)

    def attend(self, layer: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The fused RoPE + append + attention launch of `layer` on the current step metadata (for `body`).
        `q` decides the bin: it must have as many rows as the bin being captured."""
        b = q.shape[0]
        return self.wrappers[b].run_fused(q, k, v, self.pos[:b], self.pools[layer], self.rope,
                                          out=out if out is not None else self.out[layer, :b])

    def _launch(self, b: int) -> None:
        if self.body is not None:
            self.body(self, b)
            return
        for l in range(self.num_layers):
            self.attend(l, self.q[l, :b], self.k[l, :b], self.v[l, :b], out=self.out[l, :b])

    def capture(self) -> None:
        """Capture every bin (the reference's warm-up, llama3.py:315-414)."""
        for b in self.bins:
            indptr, last = self.aux[b]
            indptr.copy_(torch.arange(b + 1, dtype=torch.int32, device=indptr.device))  # one page per row
            last.fill_(1)
            self.indices[:b].fill_(self.scratch_page)
            self.pos[:b].zero_()
            self.wrappers[b].plan(indptr, self.indices, last, self.hq, self.hkv, self.d, self.page_size,
                                  pos_encoding_mode="NONE", q_data_type=self.pool.dtype)
            self._launch(b)  # once outside the capture
            torch.cuda.synchronize(self.pool.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._launch(b)
            self.graphs[b] = g
        torch.cuda.synchronize(self.pool.device)

    def run(self, q: Optional[torch.Tensor], k: Optional[torch.Tensor], v: Optional[torch.Tensor],
            position_ids: torch.Tensor, kv_page_indices: torch.Tensor, kv_page_indptr: torch.Tensor,
            kv_last_page_lens: torch.Tensor, total_pages_cpu: int) -> torch.Tensor:
        """One decode step (the page lists already hold the new token's slot).  q / k / v are [batch, H, D]
        for a single pool, [layers, batch, H, D] for a list of pools, or None with a `body` (which owns its
        inputs).  Returns [batch, Hq, D] or [layers, batch, Hq, D]."""
        batch = kv_page_indptr.shape[0] - 1
        if q is not None and self._single:
            q, k, v = q[None], k[None], v[None]
        if q is not None and (q.shape[0] != self.num_layers or q.shape[1] != batch):
            raise ValueError(f"q must be [{self.num_layers}, {batch}, heads, head_dim]")
        b = pick_bin(self.bins, batch)
        if b is None or b not in self.graphs:
            if q is None:
                raise ValueError("a batch beyond the largest bin needs q / k / v (the body is only captured)")
            self.fallback.plan(kv_page_indptr, kv_page_indices, kv_last_page_lens, self.hq, self.hkv, self.d,
                               self.page_size, pos_encoding_mode="NONE", q_data_type=q.dtype)
            outs = [self.fallback.run_fused(q[l], k[l], v[l], position_ids, self.pools[l], self.rope)
                    for l in range(self.num_layers)]
            return outs[0] if self._single else torch.stack(outs)
        total = int(total_pages_cpu)
        if total + (b - batch) > self.indices.numel():
            raise ValueError("more pages than the static index buffer holds")
        indptr, last = self.aux[b]
        if q is not None:
            self.q[:, :batch].copy_(q)
            self.k[:, :batch].copy_(k)
            self.v[:, :batch].copy_(v)
        self.pos[:batch].copy_(position_ids[:batch])
        indptr[: batch + 1].copy_(kv_page_indptr)
        last[:batch].copy_(kv_last_page_lens)
        self.indices[:total].copy_(kv_page_indices[:total])
        if batch < b:
            rem = b - batch
            indptr[batch + 1:].copy_(self._pad_ramp[:rem] + total)  # one more page per padded row
            self.indices[total: total + rem].fill_(self.scratch_page)
            last[batch:].fill_(1)
            self.pos[batch:b].zero_()
        self.graphs[b].replay()
        res = self.out[:, :batch].clone()
        return res[0] if self._single else res
