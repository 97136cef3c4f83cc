"""Small-scale versions of the beam-sharing and eviction workloads: the page bookkeeping runs on the host
(pie_b200.pages / workloads), every device step is mirrored on the CPU oracle, and pools and attention
outputs must agree step by step."""
import numpy as np
import pytest
import torch

from oracle import paged_kv_ref as R
from pie_b200 import ops, pages
from pie_b200 import workloads as W
from tests.util import dev

pytestmark = pytest.mark.gpu

HQ, HKV, D = 32, 8, 128


def _oracle_step(pool, q, k, v, pos_ids, indices, indptr, last, table):
    c, s = table[pos_ids, : D // 2], table[pos_ids, D // 2:]
    q_r, k_r = R.apply_rope(q, c, s), R.apply_rope(k, c, s)
    b = len(pos_ids)
    seq = R.get_seq_lens(indptr, last, 16)
    bi, kp = R.get_batch_indices_positions(np.arange(b + 1), seq, b)
    R.append_paged_kv_cache(k_r, v, bi, kp, pool, indices, indptr)
    return R.decode_attention(q_r, pool, indptr, indices, last)


def test_beam_search_page_sharing_with_copy_on_write():
    """Groups of 4 beams share their prefix pages; every few steps the 2 best beams of a group survive and
    fork again: full pages are shared by reference count, a partial last page is copied, losers' private
    pages go back to the free list and are reused."""
    num_pages, groups, beams, prefix = 256, 3, 4, 40  # 40 tokens = 2 full pages + 8 tokens
    rng = np.random.default_rng(0)
    pool_cpu = W.randn((num_pages, 2, 16, HKV, D), 1, torch.bfloat16, 0.5)
    pool_gpu = pool_cpu.cuda()
    table = R.make_cos_sin_table(256, R.rope_inv_freq(D, 500000.0, "llama31", 8.0))
    rope = ops.RopeConfig(mode="table", cos_sin_table=dev(table))
    pp = pages.PagePool(num_pages)
    ctxs = []
    copies = []
    for g in range(groups):
        root = pages.KvPageList(pp, 16)
        root.grow(prefix)
        members = [root]
        for _ in range(beams - 1):
            child, cp = root.fork_cow()
            assert cp is not None and cp[2] == prefix % 16
            copies.append(cp)
            members.append(child)
        ctxs.append(members)

    def run_copies(cps):
        if not cps:
            return
        src, dst, val = (np.array(x, np.int32) for x in zip(*cps))
        ops.copy_kv_pages(pool_gpu, dev(src), dev(dst), dev(val))
        R.copy_pages([pool_cpu], src, dst, val)

    run_copies(copies)
    w = ops.BatchDecodeWithPagedKVCacheWrapper(torch.zeros(32 << 20, dtype=torch.uint8, device="cuda"), "NHD")
    freed_total = 0
    for step in range(20):
        flat = [c for grp in ctxs for c in grp]
        pos_ids = np.array([c.total_tokens for c in flat], np.int32)
        for c in flat:
            c.grow(1)
        indices, indptr, last = pages.build_csr(flat)
        b = len(flat)
        q = W.randn((b, HQ, D), 100 + step, torch.bfloat16, 0.5)
        k = W.randn((b, HKV, D), 200 + step, torch.bfloat16, 0.5)
        v = W.randn((b, HKV, D), 300 + step, torch.bfloat16, 0.5)
        ref = _oracle_step(pool_cpu, q, k, v, pos_ids, indices, indptr, last, table)
        w.plan(dev(indptr), dev(indices), dev(last), HQ, HKV, D, 16, q_data_type=torch.bfloat16)
        out = w.run_fused(q.cuda(), k.cuda(), v.cuda(), dev(pos_ids), pool_gpu, rope)
        assert (out.cpu().float() - ref.float()).abs().max().item() <= 2e-2, step
        assert torch.equal(pool_gpu.cpu().view(torch.uint8), pool_cpu.view(torch.uint8)), step
        if step % 4 == 3:  # keep the 2 best beams of every group, fork each once
            cps = []
            for gi, grp in enumerate(ctxs):
                order = rng.permutation(beams)
                keep = [grp[i] for i in order[:2]]
                for i in order[2:]:
                    freed_total += len(grp[i].release())
                new = []
                for c in keep:
                    child, cp = c.fork_cow()
                    if cp is not None:
                        cps.append(cp)
                    new += [c, child]
                ctxs[gi] = new
            run_copies(cps)
    assert ops.device_error("cuda") is None
    assert freed_total > 0  # losers' private pages were recycled
    # shared prefix pages are referenced by every beam of their group
    for grp in ctxs:
        first = grp[0].pages[0]
        assert all(c.pages[0] == first for c in grp) and pp.refs[first] == beams


def test_eviction_churn_and_kv_head_sharding_on_one_gpu():
    """70B-shaped heads (64 q / 8 kv).  Every few steps a quarter of the requests is evicted, their pages
    recycled and the slots refilled with fresh contexts written through the append path.  The same steps
    run once with all heads and once as two KV-head shards (4 kv heads each) whose outputs are
    concatenated: both must match the oracle."""
    hq, hkv = 64, 8
    num_pages, B = 512, 8
    reqs = W.PagedRequests(W.seeded_perm(num_pages, 5))
    for c in (130, 700, 40, 2000, 16, 333, 90, 1024):
        reqs.add(c)
    pool_cpu = W.randn((num_pages, 2, 16, hkv, D), 2, torch.bfloat16, 0.5)
    pool_gpu = pool_cpu.cuda()
    shard_pools = [pool_cpu[:, :, :, :4].contiguous().cuda(), pool_cpu[:, :, :, 4:].contiguous().cuda()]
    table = R.make_cos_sin_table(4096, R.rope_inv_freq(D, 500000.0, "llama31", 8.0))
    rope = ops.RopeConfig(mode="table", cos_sin_table=dev(table))
    ws = torch.zeros(32 << 20, dtype=torch.uint8, device="cuda")
    w_full = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    w_shard = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    for step in range(12):
        if step % 4 == 3:
            victims = W.eviction_victims(B, step, fraction=0.25)
            for r in victims:
                reqs.evict(r, 40)
            # refill: 40 tokens per victim, RoPE + append only
            idx, ptr, last = reqs.csr()
            qo = np.zeros(B + 1, np.int32)
            for r in victims:
                qo[r + 1] = 40
            qo = np.cumsum(qo).astype(np.int32)
            n = int(qo[-1])
            pos = np.concatenate([np.arange(40) for _ in victims]).astype(np.int32)
            k = W.randn((n, hkv, D), 400 + step, torch.bfloat16, 0.5)
            v = W.randn((n, hkv, D), 500 + step, torch.bfloat16, 0.5)
            seq = R.get_seq_lens(ptr, last, 16)
            bi, kp = R.get_batch_indices_positions(qo, seq, n)
            k_r = R.apply_rope(k, table[pos, : D // 2], table[pos, D // 2:])
            R.append_paged_kv_cache(k_r, v, bi, kp, pool_cpu, idx, ptr)
            dseq = ops.get_seq_lens(dev(ptr), dev(last), 16)
            dbi, dkp = ops.get_batch_indices_positions(dev(qo), dseq, n)
            assert np.array_equal(dbi.cpu().numpy(), bi) and np.array_equal(dkp.cpu().numpy(), kp)
            ops.rope_append_paged_kv_cache(None, k.cuda(), v.cuda(), dev(pos), dbi, dkp, pool_gpu, dev(idx), dev(ptr),
                                           dev(last), rope)
            for sidx, sp in enumerate(shard_pools):
                hs = slice(4 * sidx, 4 * sidx + 4)
                ops.rope_append_paged_kv_cache(None, k[:, hs].contiguous().cuda(), v[:, hs].contiguous().cuda(),
                                               dev(pos), dbi, dkp, sp, dev(idx), dev(ptr), dev(last), rope)
        meta = W.decode_steps(reqs, 1)[0]
        q = W.randn((B, hq, D), 100 + step, torch.bfloat16, 0.5)
        k = W.randn((B, hkv, D), 200 + step, torch.bfloat16, 0.5)
        v = W.randn((B, hkv, D), 300 + step, torch.bfloat16, 0.5)
        ref = _oracle_step(pool_cpu, q, k, v, meta.pos_ids, meta.kv_indices, meta.kv_indptr, meta.kv_last_page_len,
                           table)
        indptr, indices, last = dev(meta.kv_indptr), dev(meta.kv_indices), dev(meta.kv_last_page_len)
        w_full.plan(indptr, indices, last, hq, hkv, D, 16, q_data_type=torch.bfloat16)
        out = w_full.run_fused(q.cuda(), k.cuda(), v.cuda(), dev(meta.pos_ids), pool_gpu, rope)
        assert (out.cpu().float() - ref.float()).abs().max().item() <= 2e-2, step
        assert torch.equal(pool_gpu.cpu().view(torch.uint8), pool_cpu.view(torch.uint8)), step
        # two KV-head shards with identical page tables; concatenation = the all-gather of their outputs
        w_shard.plan(indptr, indices, last, hq // 2, hkv // 2, D, 16, q_data_type=torch.bfloat16)
        parts = []
        for sidx, sp in enumerate(shard_pools):
            qs, ks = slice(32 * sidx, 32 * sidx + 32), slice(4 * sidx, 4 * sidx + 4)
            parts.append(w_shard.run_fused(q[:, qs].contiguous().cuda(), k[:, ks].contiguous().cuda(),
                                           v[:, ks].contiguous().cuda(), dev(meta.pos_ids), sp, rope))
        sharded = torch.cat(parts, dim=1)  # a different split of the work: same values up to rounding
        assert (sharded.float() - out.float()).abs().max().item() <= 4e-3
        assert (sharded.cpu().float() - ref.float()).abs().max().item() <= 2e-2
    assert ops.device_error("cuda") is None
