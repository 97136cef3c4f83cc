"""Seeded synthetic workloads with the shapes of the benchmark configurations.

Everything here is host-side index bookkeeping (numpy) plus seeded tensor generation; the
configurations are the five cases the benchmarks and parity tests are quoted on:

  1  plumbing      4 q / 2 kv heads, D 64, fp32, 64 pages, contexts {37, 64, 100, 5}, one decode step
  2  8B decode     32 / 8 heads, D 128, bf16, 32768 pages (fragmented), 64 requests, ctx U[512, 4096]
  3  chunked mix   8 prompts of 2048 + 8 chunks of 512 on 6144 cached tokens, causal
  4  beam sharing  16 prefixes x 4 beams sharing prefix pages (see pie_b200.pages)
  5  70B decode    64 / 8 heads, 256 requests, lognormal contexts, eviction churn, KV heads sharded

No public dataset is involved: the reference measures none on this path, so the inputs are
synthetic with the stated shapes and N(0,1)-scaled values.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

PAGE_SIZE = 16


def seeded_perm(n: int, seed: int) -> np.ndarray:
    g = torch.Generator().manual_seed(seed)
    return torch.randperm(n, generator=g).numpy().astype(np.int32)


def randn(shape, seed: int, dtype: torch.dtype, scale: float = 1.0, device="cpu") -> torch.Tensor:
    """Seeded N(0,1)*scale.  On CPU the values are reproducible everywhere; on a CUDA device a device
    generator is used (fast for multi-GiB pools) and values are reproducible per device type only."""
    device = torch.device(device)
    g = torch.Generator(device=device).manual_seed(seed)
    shape = tuple(shape)
    out = torch.empty(shape, dtype=dtype, device=device)
    if device.type == "cpu" or out.numel() <= (1 << 26) or len(shape) < 2:
        x = torch.randn(shape, generator=g, dtype=torch.float32, device=device)
        out.copy_(x.mul_(scale) if scale != 1.0 else x)
        return out
    # big device tensors: generate in slabs so the fp32 staging buffer stays small
    rows = max(1, (1 << 26) // max(1, out[0].numel()))
    for s in range(0, shape[0], rows):
        e = min(shape[0], s + rows)
        x = torch.randn((e - s,) + shape[1:], generator=g, dtype=torch.float32, device=device)
        out[s:e].copy_(x.mul_(scale) if scale != 1.0 else x)
    return out


def pages_needed(tokens: int, page_size: int = PAGE_SIZE) -> int:
    return -(-tokens // page_size)


def last_len_of(tokens: int, page_size: int = PAGE_SIZE) -> int:
    r = tokens % page_size
    return page_size if (r == 0 and tokens > 0) else r


@dataclass
class StepMeta:
    """CSR page table of one step, AFTER room for the step's new tokens has been made
    (the reference grows the page list before the forward pass, sdk/rust/inferlet/src/context.rs:489)."""

    kv_indices: np.ndarray      # int32 [total pages]
    kv_indptr: np.ndarray       # int32 [B+1]
    kv_last_page_len: np.ndarray  # int32 [B]
    qo_indptr: np.ndarray       # int32 [B+1]
    pos_ids: np.ndarray         # int32 [n]  RoPE positions of the new tokens

    @property
    def batch(self) -> int:
        return len(self.kv_indptr) - 1

    @property
    def nnz(self) -> int:
        return int(self.qo_indptr[-1])

    @property
    def seq_lens(self) -> np.ndarray:
        npg = np.diff(self.kv_indptr)
        return np.where(npg > 0, (npg - 1) * PAGE_SIZE + self.kv_last_page_len, 0).astype(np.int32)


class PagedRequests:
    """Page lists of a set of requests dealt from a fixed permutation of the pool
    (the "fragmented page table" of the benchmark configs), with a free list for recycling."""

    def __init__(self, perm: Sequence[int], page_size: int = PAGE_SIZE) -> None:
        self.page_size = page_size
        self._perm = np.asarray(perm, dtype=np.int32)
        self._cursor = 0
        self._free: List[int] = []
        self.pages: List[List[int]] = []
        self.tokens: List[int] = []

    def _take(self, n: int) -> List[int]:
        out: List[int] = []
        while n > 0 and self._free:
            out.append(self._free.pop())
            n -= 1
        if n > 0:
            if self._cursor + n > len(self._perm):
                raise RuntimeError("page pool exhausted")
            out.extend(int(x) for x in self._perm[self._cursor: self._cursor + n])
            self._cursor += n
        return out

    def add(self, tokens: int, reserve: int = 0) -> int:
        """New request holding `tokens` cached tokens, with pages for `reserve` more dealt up front."""
        self.pages.append(self._take(pages_needed(tokens + reserve, self.page_size)))
        self.tokens.append(int(tokens))
        return len(self.pages) - 1

    def grow(self, r: int, n: int = 1) -> None:
        new_total = self.tokens[r] + n
        need = pages_needed(new_total, self.page_size) - len(self.pages[r])
        if need > 0:
            self.pages[r].extend(self._take(need))
        self.tokens[r] = new_total

    def evict(self, r: int, new_tokens: int) -> None:
        """Recycle request r's pages and refill the slot with a fresh context."""
        self._free.extend(self.pages[r])
        self.pages[r] = self._take(pages_needed(new_tokens, self.page_size))
        self.tokens[r] = int(new_tokens)

    def csr(self):
        counts = np.fromiter((len(p) for p in self.pages), dtype=np.int64, count=len(self.pages))
        indptr = np.zeros(len(self.pages) + 1, dtype=np.int32)
        np.cumsum(counts, out=indptr[1:])
        indices = np.fromiter((x for p in self.pages for x in p), dtype=np.int32, count=int(indptr[-1]))
        last = np.array([last_len_of(t, self.page_size) for t in self.tokens], dtype=np.int32)
        return indices, indptr, last


def decode_steps(reqs: PagedRequests, steps: int) -> List[StepMeta]:
    """Metadata of `steps` consecutive decode steps, one new token per request per step."""
    out = []
    b = len(reqs.pages)
    qo = np.arange(b + 1, dtype=np.int32)
    for _ in range(steps):
        pos = np.array(reqs.tokens, dtype=np.int32)  # position of the new token = old length
        for r in range(b):
            reqs.grow(r, 1)
        idx, ptr, last = reqs.csr()
        out.append(StepMeta(idx, ptr, last, qo, pos))
    return out


@dataclass
class HeadConfig:
    num_qo_heads: int
    num_kv_heads: int
    head_dim: int
    dtype: torch.dtype
    num_pages: int
    page_size: int = PAGE_SIZE
    rope_theta: float = 500000.0
    rope_mode: str = "llama31"
    rope_scale: float = 8.0
    value_scale: float = 0.5

    def pool_shape(self):
        return (self.num_pages, 2, self.page_size, self.num_kv_heads, self.head_dim)

    def page_bytes(self) -> int:
        es = 4 if self.dtype == torch.float32 else 2
        return 2 * self.page_size * self.num_kv_heads * self.head_dim * es


# ---- config 1 ---------------------------------------------------------------------------
CONFIG1 = HeadConfig(4, 2, 64, torch.float32, 64, rope_theta=10000.0, rope_mode="plain", rope_scale=1.0,
                     value_scale=1.0)
CONFIG1_CONTEXTS = (37, 64, 100, 5)


def config1_requests() -> PagedRequests:
    reqs = PagedRequests(seeded_perm(CONFIG1.num_pages, 0))
    for c in CONFIG1_CONTEXTS:
        reqs.add(c, reserve=1)  # pages {3, 5, 7, 1} dealt in order, as after the decode step
    return reqs


# ---- config 2 ---------------------------------------------------------------------------
CONFIG2 = HeadConfig(32, 8, 128, torch.bfloat16, 32768)


def config2_requests(batch: int = 64, lo: int = 512, hi: int = 4096, seed: int = 1,
                     num_pages: int = 32768, perm_seed: Optional[int] = None) -> PagedRequests:
    """Context lengths U{lo..hi} drawn with `seed`; pages dealt from a permutation seeded with
    `perm_seed` (default: the same seed)."""
    g = torch.Generator().manual_seed(seed)
    ctx = torch.randint(lo, hi + 1, (batch,), generator=g).tolist()
    reqs = PagedRequests(seeded_perm(num_pages, seed if perm_seed is None else perm_seed))
    for c in ctx:
        reqs.add(c)
    return reqs


# ---- config 3 ---------------------------------------------------------------------------
CONFIG3 = HeadConfig(32, 8, 128, torch.bfloat16, 4352 + 64)


def config3_meta(num_prompts: int = 8, prompt_len: int = 2048, num_chunks: int = 8, chunk_len: int = 512,
                 chunk_ctx: int = 6144, seed: int = 3, num_pages: Optional[int] = None) -> StepMeta:
    """8 new prompts of 2048 tokens + 8 chunks of 512 tokens on 6144 cached tokens, packed by qo_indptr."""
    total_pages = num_prompts * pages_needed(prompt_len) + num_chunks * pages_needed(chunk_ctx + chunk_len)
    reqs = PagedRequests(seeded_perm(num_pages or max(total_pages, CONFIG3.num_pages), seed))
    qo = [0]
    pos = []
    for _ in range(num_prompts):
        reqs.add(prompt_len)
        qo.append(qo[-1] + prompt_len)
        pos.extend(range(prompt_len))
    for _ in range(num_chunks):
        reqs.add(chunk_ctx + chunk_len)
        qo.append(qo[-1] + chunk_len)
        pos.extend(range(chunk_ctx, chunk_ctx + chunk_len))
    idx, ptr, last = reqs.csr()
    return StepMeta(idx, ptr, last, np.array(qo, dtype=np.int32), np.array(pos, dtype=np.int32))


def causal_pairs(meta: StepMeta) -> int:
    """Number of (query, key) pairs a causal-with-offset mask allows, summed over requests."""
    qo = np.diff(meta.qo_indptr).astype(np.int64)
    kv = meta.seq_lens.astype(np.int64)
    return int(np.sum(qo * (qo + 1) // 2 + qo * (kv - qo)))


# ---- config 5 ---------------------------------------------------------------------------
CONFIG5 = HeadConfig(64, 8, 128, torch.bfloat16, 98304)


def config5_contexts(batch: int = 256, seed: int = 5) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(batch, generator=g, dtype=torch.float64)
    l = torch.exp(math.log(2048.0) + z).clamp(128, 32768)
    return [int(x) for x in l.tolist()]


def config5_requests(batch: int = 256, seed: int = 5, num_pages: int = CONFIG5.num_pages) -> PagedRequests:
    reqs = PagedRequests(seeded_perm(num_pages, seed))
    for c in config5_contexts(batch, seed):
        reqs.add(c)
    return reqs


def eviction_victims(batch: int, step: int, seed: int = 5, fraction: float = 0.2) -> List[int]:
    g = torch.Generator().manual_seed(seed * 1000003 + step)
    k = int(round(batch * fraction))
    return torch.randperm(batch, generator=g)[:k].tolist()


# ---- byte accounting (the roofline numerator) -------------------------------------------
def decode_step_bytes(meta: StepMeta, cfg: HeadConfig, kv_heads: Optional[int] = None,
                      qo_heads: Optional[int] = None) -> int:
    """Algorithmic HBM bytes of one fused RoPE + append + decode-attention step:
    every cached token's K and V once, q read + out written, the new k/v read and written to
    their page, and the int32 metadata."""
    es = 4 if cfg.dtype == torch.float32 else 2
    hkv = kv_heads or cfg.num_kv_heads
    hq = qo_heads or cfg.num_qo_heads
    d = cfg.head_dim
    tokens = int(meta.seq_lens.astype(np.int64).sum())
    b = meta.batch
    kv_read = tokens * 2 * hkv * d * es
    q_o = b * 2 * hq * d * es
    new_kv = b * 2 * 2 * hkv * d * es
    metadata = 4 * (len(meta.kv_indices) + 3 * b)
    return kv_read + q_o + new_kv + metadata
