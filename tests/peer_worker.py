"""Child process of tests/test_gpu_peer.py::test_peer_stores_between_real_gpus: one rank per GPU,
head-sharded fused decode steps whose results every rank stores into every rank's buffer; each rank
checks its gathered rows against an unsharded run of the same step on its own GPU."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from pie_b200 import ops  # noqa: E402
from pie_b200 import workloads as W  # noqa: E402
from pie_b200.parallel import PeerOutputs, shard_heads  # noqa: E402
from tests.util import oracle_decode_after_append  # noqa: E402


def main() -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("gloo")  # host-side exchange of the handles and barriers only
    batch, hq, hkv, pages = 53, 32, 8, 4096
    rng = np.random.default_rng(7)
    ctx = rng.integers(1, 900, size=batch)
    pr = W.PagedRequests(W.seeded_perm(pages, 7))
    for c in ctx:
        pr.add(int(c) + 1)
    idx, ptr, last = pr.csr()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    ptr, idx, last = t(ptr), t(idx), t(last)
    pos = t(ctx.astype(np.int32))
    dt = torch.bfloat16
    pool = W.randn((pages, 2, 16, hkv, 128), 1, dt, 0.5, device=dev)
    rope = ops.RopeConfig()
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device=dev)
    qs, ks = shard_heads(hq, hkv, world, rank)
    pool_r = pool[:, :, :, ks, :].contiguous()
    pool_full = pool.clone()
    peers = PeerOutputs(batch, hq, 128, dt, dev)
    peers_counted = PeerOutputs(batch, hq, 128, dt, dev)   # a second set: counted and uncounted steps do not mix
    w_full = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    w_full.plan(ptr, idx, last, hq, hkv, 128, 16, q_data_type=dt)
    ws_r = torch.zeros(64 << 20, dtype=torch.uint8, device=dev)
    w_r = ops.BatchDecodeWithPagedKVCacheWrapper(ws_r, "NHD")
    w_r.plan(ptr, idx, last, hq // world, hkv // world, 128, 16, q_data_type=dt)
    for step in range(6):   # same page table each step: the new token's slot is rewritten, which is fine here
        q = W.randn((batch, hq, 128), 10 + step, dt, 0.5, device=dev)
        k = W.randn((batch, hkv, 128), 20 + step, dt, 0.5, device=dev)
        v = W.randn((batch, hkv, 128), 30 + step, dt, 0.5, device=dev)
        want = w_full.run_fused(q, k, v, pos, pool_full, rope=rope)
        got = w_r.run_fused_peer(q[:, qs].contiguous(), k[:, ks].contiguous(), v[:, ks].contiguous(), pos, pool_r,
                                 peers, rope=rope)
        torch.cuda.synchronize(dev)
        assert ops.device_error(dev) is None
        diff = (got.float() - want.float()).abs().max().item()
        assert diff <= 4e-3, f"rank {rank} step {step}: max diff {diff}"
        if step == 0:  # the gathered rows against the CPU oracle, once (it takes a second per rank)
            ref = oracle_decode_after_append(q, pos, pool_full, ptr, idx, last)
            odiff = (got.cpu().float() - ref.float()).abs().max().item()
            assert odiff <= 2e-2, f"rank {rank}: max diff to the oracle {odiff}"
        # every rank holds the same bits: compare a checksum of the gathered rows across ranks
        sums = [None] * world
        dist.all_gather_object(sums, int(got.view(torch.int16).to(torch.int64).sum().item()))
        assert len(set(sums)) == 1, sums
    # the same two launches captured once and replayed: the step number then lives in device memory
    pc = peers_counted
    q = W.randn((batch, hq, 128), 99, dt, 0.5, device=dev)
    k = W.randn((batch, hkv, 128), 98, dt, 0.5, device=dev)
    v = W.randn((batch, hkv, 128), 97, dt, 0.5, device=dev)
    q_r, k_r, v_r = q[:, qs].contiguous(), k[:, ks].contiguous(), v[:, ks].contiguous()
    want = w_full.run_fused(q, k, v, pos, pool_full, rope=rope).clone()
    side = torch.cuda.Stream(device=dev)
    torch.cuda.synchronize(dev)
    with torch.cuda.stream(side):
        w_r.run_fused_peer(q_r, k_r, v_r, pos, pool_r, pc, rope=rope, counted=True)  # eager: advances by itself
    side.synchronize()
    assert pc.step == 1
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for _ in range(3):
            w_r.run_fused_peer(q_r, k_r, v_r, pos, pool_r, pc, rope=rope, counted=True)
    for rep in range(4):
        g.replay()
        pc.advance(3)
        torch.cuda.synchronize(dev)
        assert ops.device_error(dev) is None
        got = pc.full(batch)
        diff = (got.float() - want.float()).abs().max().item()
        assert diff <= 4e-3, f"rank {rank} graph replay {rep}: max diff {diff}"
    assert pc.step == 1 + 12
    dist.barrier()
    flags = pc._local[: 4 * world].view(torch.int32).tolist()
    assert flags == [pc.step] * world, flags
    pc.close()
    peers.close()
    print("PEER-OK", rank, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
