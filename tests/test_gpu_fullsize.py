"""Config 2 at its full size (64 requests, 32768-page pool of 2 GiB): properties that need no CPU oracle.

* re-paging invariance: moving every request's pages to other physical pages (page copy) and permuting the
  request order leaves every attention output bit-identical;
* the tuned kernel agrees with the general kernel (an independent implementation) on the same inputs;
* append -> gather round trip: the fused step's new K/V rows are found where the page table says.
"""
import numpy as np
import pytest
import torch

from pie_b200 import ops
from pie_b200 import workloads as W
from tests.util import dev

pytestmark = pytest.mark.gpu


def test_config2_full_size_properties():
    cfg = W.CONFIG2
    HQ, HKV, D, B = cfg.num_qo_heads, cfg.num_kv_heads, cfg.head_dim, 64
    reqs = W.config2_requests()
    used = sum(len(p) for p in reqs.pages)
    meta = W.decode_steps(reqs, 1)[0]
    pool = W.randn(cfg.pool_shape(), 7, cfg.dtype, 0.5, device="cuda")
    q = W.randn((B, HQ, D), 8, cfg.dtype, 0.5, device="cuda")
    k = W.randn((B, HKV, D), 9, cfg.dtype, 0.5, device="cuda")
    v = W.randn((B, HKV, D), 10, cfg.dtype, 0.5, device="cuda")
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
    w = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    indptr, indices, last = dev(meta.kv_indptr), dev(meta.kv_indices), dev(meta.kv_last_page_len)
    w.plan(indptr, indices, last, HQ, HKV, D, 16, q_data_type=cfg.dtype)
    rope = ops.RopeConfig()
    out = w.run_fused(q, k, v, dev(meta.pos_ids), pool, rope)
    assert ops.device_error("cuda") is None and torch.isfinite(out).all()

    # round trip: V rows are copied bit-exactly into slot last_len-1 of each request's last page
    last_pages = torch.from_numpy(meta.kv_indices[meta.kv_indptr[1:] - 1].astype(np.int64)).cuda()
    slots = torch.from_numpy((meta.kv_last_page_len - 1).astype(np.int64)).cuda()
    assert torch.equal(pool[last_pages, 1, slots], v)
    # and K holds the rotated k: same norm per head as the input (rotation), not the raw rows
    kk = pool[last_pages, 0, slots].float()
    assert torch.allclose(kk.norm(dim=-1), k.float().norm(dim=-1), rtol=2e-2)

    # the general kernel on the same (already appended) pool, q rotated by the separate op
    q_rot, k_rot = q.clone(), k.clone()
    ops.apply_llama31_rope_pos_ids_inplace(q_rot, k_rot, dev(meta.pos_ids))
    tuned = w.run(q_rot, pool)
    assert (tuned.float() - out.float()).abs().max().item() <= 4e-3
    p = ops.BatchPrefillWithPagedKVCacheWrapper(ws, "NHD")
    total = int(meta.seq_lens.astype(np.int64).sum())
    p.plan(dev(meta.qo_indptr), indptr, indices, last, HQ, HKV, D, 16,
           custom_mask=torch.ones(total, dtype=torch.bool, device="cuda"), q_data_type=cfg.dtype)
    masked = p.run(q_rot, pool)  # prefill kernel with an all-true mask, one token per request
    assert (masked.float() - tuned.float()).abs().max().item() <= 1e-2

    # re-paging: copy all used pages to the free tail of the pool in a new order, permute the requests
    rng = np.random.default_rng(0)
    free = np.setdiff1d(np.arange(cfg.num_pages, dtype=np.int32), meta.kv_indices)
    new_ids = rng.permutation(free)[: len(meta.kv_indices)].astype(np.int32)
    ops.copy_kv_pages(pool, dev(meta.kv_indices), dev(new_ids))
    order = rng.permutation(B)
    ptr2 = np.concatenate([[0], np.cumsum(np.diff(meta.kv_indptr)[order])]).astype(np.int32)
    idx2 = np.concatenate([new_ids[meta.kv_indptr[b]: meta.kv_indptr[b + 1]] for b in order]).astype(np.int32)
    w.plan(dev(ptr2), dev(idx2), dev(meta.kv_last_page_len[order]), HQ, HKV, D, 16, q_data_type=cfg.dtype)
    moved = w.run(q_rot[torch.from_numpy(order).cuda()], pool)
    # the partition of the flat page list differs, so the merge order may differ: values agree to rounding,
    # and requests that were not split anywhere agree exactly
    assert (moved.float() - tuned[torch.from_numpy(order).cuda()].float()).abs().max().item() <= 4e-3
    assert ops.device_error("cuda") is None
    assert used > 8000  # the workload really is the full-size one
