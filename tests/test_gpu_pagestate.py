"""Device-resident page tables (pie_b200.pages.DevicePageTable / piekv_pagestate_*) against the host
bookkeeping (`PagePool` / `KvPageList`, themselves pinned to the reference's rules in tests/test_pages.py):
the same operations in the same order must leave identical page lists, reference counts and free sets.
The beam-search workload (config 4 at its full size) then runs for 64 steps with every page table produced
on the device - no per-step host-to-device copy - and must end with a pool that is bit-identical to the run
whose page tables the host built and uploaded."""
import numpy as np
import pytest
import torch

from pie_b200 import ops, pages
from pie_b200 import workloads as W
from tests.util import dev, oracle_decode_after_append

pytestmark = pytest.mark.gpu


def _i32(x):
    return torch.tensor(list(x), dtype=torch.int32, device="cuda")


def _same(dpt: pages.DevicePageTable, pool: pages.PagePool, ctxs):
    """Device state == host state for the given {slot: KvPageList}."""
    s = dpt.snapshot()
    assert ops.device_error("cuda") is None
    for slot in range(dpt.max_requests):
        c = ctxs.get(slot)
        want = c.pages if c is not None else []
        assert s["pages"][slot] == want, slot
        assert int(s["last_page_len"][slot]) == (c.last_page_len if c is not None and c.pages else 0), slot
    assert np.array_equal(s["refs"], pool.refs)
    assert s["free_pages"] == pool.available() == int(s["free"].sum())
    host_free = np.ones(dpt.num_pages, dtype=bool)
    host_free[: pool.ids._next] = False
    host_free[list(pool.ids._free)] = True
    assert np.array_equal(s["free"], host_free)


def test_grow_shrink_release_and_id_reuse_follow_the_host_pool():
    P, R, C = 200, 12, 40
    dpt = pages.DevicePageTable(P, R, C)
    pool = pages.PagePool(P)
    ctxs = {}
    rng = np.random.default_rng(1)
    # requests 0..7 start with assorted lengths (page boundaries included)
    lens = [1, 16, 17, 100, 0, 33, 48, 5]
    for slot, n in enumerate(lens):
        ctxs[slot] = pages.KvPageList(pool, 16)
        ctxs[slot].grow(n)
    indptr, indices, last, pos = dpt.grow(_i32(range(8)), _i32(lens))
    assert pos.tolist() == [0] * 8
    want_idx, want_ptr, want_last = pages.build_csr([ctxs[s] for s in range(8)])
    assert indptr.tolist() == want_ptr.tolist()
    assert indices[: want_ptr[-1]].tolist() == want_idx.tolist()
    assert last.tolist() == [x if lens[i] else 0 for i, x in enumerate(want_last.tolist())]
    _same(dpt, pool, ctxs)
    for step in range(40):
        kind = step % 4
        if kind == 0:      # a few decode steps for a shuffled subset
            order = [int(x) for x in rng.permutation(8)[: 5]]
            for s_ in order:
                ctxs[s_].grow(1)
            indptr, indices, last, pos = dpt.grow(_i32(order), 1)
            want_idx, want_ptr, want_last = pages.build_csr([ctxs[s] for s in order])
            assert indptr.tolist() == want_ptr.tolist() and indices[: want_ptr[-1]].tolist() == want_idx.tolist()
            assert last.tolist() == want_last.tolist()
            assert pos.tolist() == [ctxs[s].total_tokens - 1 for s in order]
        elif kind == 1:    # release two requests, start them again with new lengths
            victims = [int(x) for x in rng.permutation(8)[:2]]
            for v in victims:
                ctxs[v].release()
            dpt.release(_i32(victims))
            _same(dpt, pool, ctxs)
            news = [int(x) for x in rng.integers(1, 90, size=2)]
            for v, n in zip(victims, news):
                ctxs[v].grow(n)
            dpt.grow(_i32(victims), _i32(news), csr=False)
        elif kind == 2:    # shrink one, grow another in one call (shrinks first)
            a, b = (int(x) for x in rng.permutation(8)[:2])
            cut = min(ctxs[a].total_tokens, int(rng.integers(1, 40)))
            ctxs[a].shrink(cut)
            ctxs[b].grow(23)
            dpt.grow(_i32([a, b]), _i32([-cut, 23]), csr=False)
        else:              # forks into the spare slots, then drop them again
            parents = [int(x) for x in rng.permutation(8)[:3]]
            kids = [8, 9, 10]
            copies = []
            for p_, k_ in zip(parents, kids):
                ctxs[k_], cp = ctxs[p_].fork_cow()
                copies.append(cp if cp is not None else (0, 0, 0))
            src, dst, val = dpt.fork(_i32(parents), _i32(kids))
            got = list(zip(src.tolist(), dst.tolist(), val.tolist()))
            assert [g if g[2] else (0, 0, 0) for g in got] == copies
            _same(dpt, pool, ctxs)
            for k_ in kids:
                ctxs[k_].release()
                del ctxs[k_]
            dpt.release(_i32(kids))
        _same(dpt, pool, ctxs)


def test_problems_are_reported_not_faulted():
    dpt = pages.DevicePageTable(8, 4, 4)
    dpt.grow(_i32([0]), 16 * 5, csr=False)            # 5 pages in a row of 4
    e = ops.device_error("cuda")
    assert e is not None and e["code"] == 9
    dpt.grow(_i32([0, 1, 2]), 16 * 3, csr=False)      # 9 pages from a pool of 8
    e = ops.device_error("cuda")
    assert e is not None and e["code"] == 8
    assert dpt.snapshot()["free_pages"] == 8          # nothing was taken
    dpt.grow(_i32([7]), 1, csr=False)                 # no such slot
    e = ops.device_error("cuda")
    assert e is not None and e["code"] == 10
    dpt.grow(_i32([0, 1]), 20, csr=False)
    dpt.fork(_i32([0]), _i32([1]))                    # child slot in use
    e = ops.device_error("cuda")
    assert e is not None and e["code"] == 10
    with pytest.raises(ValueError):
        dpt.grow(torch.zeros(5000, dtype=torch.int32, device="cuda"), 1)


def _beam_schedule(groups, beams, steps, every, seed):
    """Which beams of every group survive at the fork steps (a seeded random score), as slot lists:
    per fork step (losers, parents, children); children reuse the losers' slots."""
    rng = np.random.default_rng(seed)
    plan = {}
    for i in range(steps):
        if i % every == every - 1:
            losers, parents, children = [], [], []
            for g in range(groups):
                order = rng.permutation(beams)
                keep = [g * beams + int(j) for j in order[:2]]
                lose = [g * beams + int(j) for j in order[2:]]
                losers += lose
                parents += keep
                children += lose[: len(keep)]
            plan[i] = (losers, parents, children)
    return plan


def test_beam_search_on_device_page_tables_equals_the_host_run(deterministic_decode):
    """Config 4 at full size: 16 prefixes of 1024 tokens x 4 beams, 64 decode steps, top-2 of each group kept
    and forked every 8 steps."""
    groups, beams, prefix, steps, every = 16, 4, 1024, 64, 8
    HQ, HKV, D = 32, 8, 128
    P, B = 8192, groups * beams
    dt = torch.bfloat16
    pool0 = W.randn((P, 2, 16, HKV, D), 400, dt, 0.5, device="cuda")
    qkv = W.randn((4, B, (HQ + 2 * HKV) * D), 401, dt, 0.5, device="cuda")
    rope = ops.RopeConfig()
    plan = _beam_schedule(groups, beams, steps, every, seed=4)

    def split(x):
        return (x[:, : HQ * D].view(B, HQ, D), x[:, HQ * D: (HQ + HKV) * D].view(B, HKV, D),
                x[:, (HQ + HKV) * D:].view(B, HKV, D))

    # ---- host run: KvPageList bookkeeping, tables uploaded every step
    pool_h = pool0.clone()
    pp = pages.PagePool(P)
    ctxs = {}
    for g in range(groups):
        root = pages.KvPageList(pp, 16)
        root.grow(prefix)
        ctxs[g * beams] = root
    for g in range(groups):
        for j in range(1, beams):
            ctxs[g * beams + j], cp = ctxs[g * beams].fork_cow()
            assert cp is None
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
    w = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    outs_h = []
    for i in range(steps):
        flat = [ctxs[s] for s in range(B)]
        pos = np.array([c.total_tokens for c in flat], np.int32)
        for c in flat:
            c.grow(1)
        idx, ptr, last = pages.build_csr(flat)
        q, k, v = split(qkv[i % 4])
        w.plan(dev(ptr), dev(idx), dev(last), HQ, HKV, D, 16, q_data_type=dt)
        outs_h.append(w.run_fused(q, k, v, dev(pos), pool_h, rope).clone())
        if i in plan:
            losers, parents, children = plan[i]
            for s in losers:
                ctxs[s].release()
            cps = []
            for p_, c_ in zip(parents, children):
                ctxs[c_], cp = ctxs[p_].fork_cow()
                cps.append(cp if cp is not None else (0, 0, 0))
            src, dst, val = (np.array(x, np.int32) for x in zip(*cps))
            ops.copy_kv_pages(pool_h, dev(src), dev(dst), dev(val))
    torch.cuda.synchronize()

    # ---- device run: everything the steps need is on the device before the first step
    pool_d = pool0.clone()
    dpt = pages.DevicePageTable(P, B, 256, max_batch=B)
    roots = _i32(g * beams for g in range(groups))
    dpt.grow(roots, prefix, csr=False)
    dpt.fork(_i32(g * beams for g in range(groups) for _ in range(beams - 1)),
             _i32(g * beams + j for g in range(groups) for j in range(1, beams)))
    all_slots = _i32(range(B))
    dplan = {i: tuple(_i32(x) for x in v) for i, v in plan.items()}
    w2 = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    torch.cuda.synchronize()
    outs_d = []
    for i in range(steps):
        indptr, indices, last, pos = dpt.grow(all_slots, 1)
        q, k, v = split(qkv[i % 4])
        w2.plan(indptr, indices, last, HQ, HKV, D, 16, q_data_type=dt)
        outs_d.append(w2.run_fused(q, k, v, pos, pool_d, rope).clone())
        if i in dplan:
            losers, parents, children = dplan[i]
            dpt.release(losers)
            src, dst, val = dpt.fork(parents, children)
            ops.copy_kv_pages(pool_d, src, dst, val)
    torch.cuda.synchronize()
    assert ops.device_error("cuda") is None
    _same(dpt, pp, ctxs)
    assert torch.equal(pool_d.view(torch.int16), pool_h.view(torch.int16))
    for i in range(steps):
        assert torch.equal(outs_d[i], outs_h[i]), i
    # one more step on the device tables alone, against the CPU oracle
    indptr, indices, last, pos = dpt.grow(all_slots, 1)
    q, k, v = split(qkv[0])
    w2.plan(indptr, indices, last, HQ, HKV, D, 16, q_data_type=dt)
    out = w2.run_fused(q, k, v, pos, pool_d, rope)
    assert pos.tolist() == [ctxs[s].total_tokens for s in range(B)]
    ref = oracle_decode_after_append(q, pos, pool_d, indptr, indices[: int(indptr[-1].item())], last)
    assert (out.cpu().float() - ref.float()).abs().max().item() <= 2e-2
    assert ops.device_error("cuda") is None
    assert sum(len(v_[0]) for v_ in plan.values()) > 0 and pp.available() < P


def test_device_page_tables_inside_a_cuda_graph(deterministic_decode):
    """One decode step - page-table advance, CSR gather and the fused attention launch - captured once and
    replayed: the page tables move on by themselves from replay to replay."""
    HQ, HKV, D, B, P = 32, 8, 128, 24, 2048
    dt = torch.bfloat16
    pool = W.randn((P, 2, 16, HKV, D), 7, dt, 0.5, device="cuda")
    pool_ref = pool.clone()
    q = W.randn((B, HQ, D), 8, dt, 0.5, device="cuda")
    k = W.randn((B, HKV, D), 9, dt, 0.5, device="cuda")
    v = W.randn((B, HKV, D), 10, dt, 0.5, device="cuda")
    rope = ops.RopeConfig()
    lens = [int(x) for x in np.random.default_rng(3).integers(1, 700, size=B)]
    slots = _i32(range(B))
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")

    def fresh():
        t = pages.DevicePageTable(P, B, 64, max_batch=B)
        t.grow(slots, _i32(lens), csr=False)
        return t

    # eager reference: 6 steps
    t0 = fresh()
    w0 = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    want = []
    for _ in range(6):
        indptr, indices, last, pos = t0.grow(slots, 1)
        w0.plan(indptr, indices, last, HQ, HKV, D, 16, q_data_type=dt)
        want.append(w0.run_fused(q, k, v, pos, pool_ref, rope).clone())
    # graph: warm up on a scratch table, capture one step on a fresh one, replay it 6 times
    t1 = fresh()
    out = torch.empty_like(q)
    w1 = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD", use_cuda_graph=True, paged_kv_indptr_buffer=t1.kv_indptr[: B + 1],
                                                paged_kv_indices_buffer=t1.kv_indices,
                                                paged_kv_last_page_len_buffer=t1.kv_last_page_len[:B])
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        indptr, indices, last, pos = t1.grow(slots, 1)
        w1.plan(indptr, indices, last, HQ, HKV, D, 16, q_data_type=dt)
        w1.run_fused(q, k, v, pos, pool, rope, out=out)
    for i in range(6):
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want[i]), i
    assert ops.device_error("cuda") is None
    assert torch.equal(pool.view(torch.int16), pool_ref.view(torch.int16))
    a, b = t0.snapshot(), t1.snapshot()
    assert a["pages"] == b["pages"] and np.array_equal(a["refs"], b["refs"])
