"""Graph-bin decode runner (pie_b200.graphed): bin arithmetic on the CPU, replay-vs-eager parity on the GPU."""
import numpy as np
import pytest
import torch

from pie_b200.graphed import graph_bins, pick_bin


def test_bins_follow_the_reference_rule():
    # pie/src/pie_worker/model/llama3.py:241-249: powers of two to 16, then steps of 16 from 24, then the limit
    assert graph_bins(512)[:8] == [1, 2, 4, 8, 16, 24, 40, 56]
    assert graph_bins(512)[-1] == 512 and len(graph_bins(512)) == 5 + 31 + 1
    assert graph_bins(20) == [1, 2, 4, 8, 16, 20]
    assert graph_bins(16) == [1, 2, 4, 8, 16]
    assert graph_bins(6) == [1, 2, 4]
    assert graph_bins(40) == [1, 2, 4, 8, 16, 24, 40]
    assert graph_bins(0) == graph_bins(512)          # `max_batch_size or 512`


def test_pick_bin():
    bins = graph_bins(40)
    assert [pick_bin(bins, n) for n in (1, 3, 16, 17, 25, 40, 41)] == [1, 4, 16, 24, 40, 40, None]


@pytest.mark.gpu
def test_graphed_step_matches_eager_step():
    from pie_b200 import ops
    from pie_b200 import workloads as W
    from pie_b200.graphed import GraphedDecodeStep
    from tests.util import oracle_decode_after_append

    hq, hkv, pages = 32, 8, 2048
    dt = torch.bfloat16
    pool = W.randn((pages + 1, 2, 16, hkv, 128), 1, dt, 0.5, device="cuda")  # + the scratch page
    runner = GraphedDecodeStep(pool, hq, hkv, max_batch=40, max_total_pages=pages)
    runner.capture()
    assert sorted(runner.graphs) == [1, 2, 4, 8, 16, 24, 40]
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
    eager = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    rng = np.random.default_rng(2)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    for step, batch in enumerate([1, 3, 17, 24, 40, 47, 5]):   # 47 exceeds the largest bin: eager fallback
        ctx = rng.integers(1, 600, size=batch)
        pr = W.PagedRequests(W.seeded_perm(pages, 10 + step))
        for c in ctx:
            pr.add(int(c) + 1)
        idx, ptr, last = pr.csr()
        q = W.randn((batch, hq, 128), 100 + step, dt, 0.5, device="cuda")
        k = W.randn((batch, hkv, 128), 200 + step, dt, 0.5, device="cuda")
        v = W.randn((batch, hkv, 128), 300 + step, dt, 0.5, device="cuda")
        pos = t(ctx.astype(np.int32))
        ref_pool = pool.clone()
        eager.plan(t(ptr), t(idx), t(last), hq, hkv, 128, 16, q_data_type=dt)
        want = eager.run_fused(q, k, v, pos, ref_pool, rope=runner.rope)
        got = runner.run(q, k, v, pos, t(idx), t(ptr), t(last), int(ptr[-1]))
        torch.cuda.synchronize()
        assert ops.device_error("cuda") is None
        # padding changes how the page list is cut over the CTAs, hence the order of the merges: rounding only
        assert (got.float() - want.float()).abs().max().item() <= 4e-3, (step, batch)
        # every real page received exactly the bytes of the eager step; only the scratch page may differ
        assert torch.equal(pool[:pages], ref_pool[:pages]), (step, batch)
        # and the CPU oracle on the pool the replay left behind
        ref = oracle_decode_after_append(q, pos, pool, ptr, idx, last)
        assert (got.cpu().float() - ref.float()).abs().max().item() <= 2e-2, (step, batch)


@pytest.mark.gpu
def test_graphed_multi_layer_step_with_and_without_a_body():
    """Three layer pools over one set of step metadata: the default layer loop, and a caller's body that puts
    its own work between the layers (here: the next layer's q depends on this layer's output), each captured
    once per bin and replayed with changing page tables."""
    from pie_b200 import ops
    from pie_b200 import workloads as W
    from pie_b200.graphed import GraphedDecodeStep
    from tests.util import oracle_decode_after_append

    L, hq, hkv, pages = 3, 32, 8, 1024
    dt = torch.bfloat16
    pools = [W.randn((pages + 1, 2, 16, hkv, 128), 10 + l, dt, 0.5, device="cuda") for l in range(L)]
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
    eager = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    rng = np.random.default_rng(5)

    # ---- default loop: layer l reads q/k/v[l]
    runner = GraphedDecodeStep([p.clone() for p in pools], hq, hkv, max_batch=16, max_total_pages=pages)
    runner.capture()
    ref_pools = [p.clone() for p in pools]
    for step, batch in enumerate([3, 16, 9]):
        ctx = rng.integers(1, 500, size=batch)
        pr = W.PagedRequests(W.seeded_perm(pages, 20 + step))
        for c in ctx:
            pr.add(int(c) + 1)
        idx, ptr, last = pr.csr()
        q = W.randn((L, batch, hq, 128), 100 + step, dt, 0.5, device="cuda")
        k = W.randn((L, batch, hkv, 128), 200 + step, dt, 0.5, device="cuda")
        v = W.randn((L, batch, hkv, 128), 300 + step, dt, 0.5, device="cuda")
        pos = t(ctx.astype(np.int32))
        got = runner.run(q, k, v, pos, t(idx), t(ptr), t(last), int(ptr[-1]))
        eager.plan(t(ptr), t(idx), t(last), hq, hkv, 128, 16, q_data_type=dt)
        for l in range(L):
            want = eager.run_fused(q[l], k[l], v[l], pos, ref_pools[l], rope=runner.rope)
            assert (got[l].float() - want.float()).abs().max().item() <= 4e-3, (step, l)
            assert torch.equal(runner.pools[l][:pages], ref_pools[l][:pages]), (step, l)
        ref = oracle_decode_after_append(q[1], pos, runner.pools[1], ptr, idx, last)
        assert (got[1].cpu().float() - ref.float()).abs().max().item() <= 2e-2
    assert ops.device_error("cuda") is None

    # ---- a body: q of layer l + 1 is made from the output of layer l inside the captured step
    state = {}

    def body(r, b):
        x = state["x"][:b]
        for l in range(L):
            out = r.attend(l, x, state["k"][l, :b], state["v"][l, :b])
            x = (x.float() * 0.5 + out.float() * 0.5).to(dt)   # stands in for o_proj + MLP + the next qkv_proj
        state["y"][:b].copy_(x)

    state["x"] = torch.zeros((16, hq, 128), dtype=dt, device="cuda")
    state["k"] = torch.zeros((L, 16, hkv, 128), dtype=dt, device="cuda")
    state["v"] = torch.zeros((L, 16, hkv, 128), dtype=dt, device="cuda")
    state["y"] = torch.zeros((16, hq, 128), dtype=dt, device="cuda")
    runner2 = GraphedDecodeStep([p.clone() for p in pools], hq, hkv, max_batch=16, max_total_pages=pages, body=body)
    runner2.capture()
    ref_pools = [p.clone() for p in pools]
    for step, batch in enumerate([5, 16]):
        ctx = rng.integers(1, 500, size=batch)
        pr = W.PagedRequests(W.seeded_perm(pages, 40 + step))
        for c in ctx:
            pr.add(int(c) + 1)
        idx, ptr, last = pr.csr()
        x0 = W.randn((batch, hq, 128), 400 + step, dt, 0.5, device="cuda")
        kk = W.randn((L, batch, hkv, 128), 500 + step, dt, 0.5, device="cuda")
        vv = W.randn((L, batch, hkv, 128), 600 + step, dt, 0.5, device="cuda")
        state["x"][:batch].copy_(x0)
        state["k"][:, :batch].copy_(kk)
        state["v"][:, :batch].copy_(vv)
        pos = t(ctx.astype(np.int32))
        runner2.run(None, None, None, pos, t(idx), t(ptr), t(last), int(ptr[-1]))
        eager.plan(t(ptr), t(idx), t(last), hq, hkv, 128, 16, q_data_type=dt)
        x = x0
        for l in range(L):
            o = eager.run_fused(x, kk[l], vv[l], pos, ref_pools[l], rope=runner2.rope)
            x = (x.float() * 0.5 + o.float() * 0.5).to(dt)
        torch.cuda.synchronize()
        assert (state["y"][:batch].float() - x.float()).abs().max().item() <= 8e-3, step
        for l in range(L):
            assert torch.equal(runner2.pools[l][:pages], ref_pools[l][:pages]), (step, l)
    assert ops.device_error("cuda") is None
