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
