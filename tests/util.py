"""Shared scenario builder for the parity tests: the same seeded inputs go to the CPU oracle and,
moved to the GPU, through pie_b200.ops (which calls the C ABI)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from pie_b200 import workloads as W


@dataclass
class Scenario:
    hq: int
    hkv: int
    d: int
    dtype: torch.dtype
    page_size: int
    num_pages: int
    meta: W.StepMeta
    pool: torch.Tensor      # CPU, [P, 2, ps, Hkv, D], prior contents everywhere (stale rows included)
    q: torch.Tensor         # CPU [n, Hq, D]
    k: torch.Tensor         # CPU [n, Hkv, D]
    v: torch.Tensor         # CPU [n, Hkv, D]

    @property
    def n(self) -> int:
        return self.meta.nnz


def make_scenario(hq: int, hkv: int, d: int, dtype: torch.dtype, ctx_and_new: Sequence[Tuple[int, int]],
                  seed: int = 0, page_size: int = 16, num_pages: Optional[int] = None, scale: float = 1.0,
                  perm_seed: Optional[int] = None) -> Scenario:
    """Requests given as (existing context length, new tokens).  The page table is a seeded permutation
    dealt in order; the pool is filled with seeded noise everywhere so stale rows are not zero."""
    need = sum(W.pages_needed(c + m, page_size) for c, m in ctx_and_new)
    num_pages = num_pages or max(need + 3, 8)
    reqs = W.PagedRequests(W.seeded_perm(num_pages, seed if perm_seed is None else perm_seed), page_size)
    qo = [0]
    pos: List[int] = []
    for c, m in ctx_and_new:
        r = reqs.add(c, reserve=m)
        reqs.tokens[r] = c + m
        qo.append(qo[-1] + m)
        pos.extend(range(c, c + m))
    idx, ptr, last = reqs.csr()
    # requests with zero tokens and zero pages keep last_len 0
    meta = W.StepMeta(idx, ptr, last, np.array(qo, dtype=np.int32), np.array(pos, dtype=np.int32))
    n = qo[-1]
    pool = W.randn((num_pages, 2, page_size, hkv, d), seed + 11, dtype, scale)
    q = W.randn((n, hq, d), seed + 12, dtype, scale)
    k = W.randn((n, hkv, d), seed + 13, dtype, scale)
    v = W.randn((n, hkv, d), seed + 14, dtype, scale)
    return Scenario(hq, hkv, d, dtype, page_size, num_pages, meta, pool, q, k, v)


def dev(x, device="cuda"):
    if isinstance(x, np.ndarray):
        return torch.from_numpy(np.ascontiguousarray(x)).to(device)
    return x.to(device)


def ulp_diff_bf16(a: torch.Tensor, b: torch.Tensor) -> int:
    """Largest distance in units of bf16 representable steps (sign-magnitude ordering)."""
    def key(t):
        i = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(i < 0, -(i & 0x7FFF), i)
    return int((key(a) - key(b)).abs().max().item()) if a.numel() else 0


def oracle_decode_after_append(q, pos_ids, pool_after, indptr, indices, last, rope_mode="llama31", theta=500000.0,
                               scale=8.0):
    """CPU-oracle decode attention for a fused step whose append has already happened: rotate q on the CPU
    (on-the-fly sin / cos, within one rounding step of the device's) and attend over `pool_after`, the pool
    as the device left it.  All arguments may be device tensors or numpy arrays."""
    from oracle import paged_kv_ref as R

    def host(x):
        return x.cpu().numpy() if isinstance(x, torch.Tensor) else np.asarray(x)

    qc = q.detach().cpu()
    inv = R.rope_inv_freq(qc.shape[-1], theta, rope_mode, scale)
    c, s = R.rope_cos_sin(host(pos_ids), inv)
    return R.decode_attention(R.apply_rope(qc, c, s), pool_after.detach().cpu(), host(indptr), host(indices),
                              host(last))
