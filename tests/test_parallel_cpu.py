"""The N > 1 paths on CPU: two gloo ranks run the oracle on their shard and must reproduce the
single-process result (KV-head sharding + all-gather), and request sharding must partition the batch."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pie_b200 import parallel
from tests.util import make_scenario


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import paged_kv_ref as R

        sc = make_scenario(8, 4, 32, torch.float32, [(c - 1, 1) for c in (37, 5, 64, 100, 17)], seed=3)
        m = sc.meta
        full = R.decode_attention(sc.q, sc.pool, m.kv_indptr, m.kv_indices, m.kv_last_page_len)
        # KV-head sharding: this rank's slice of the pool and of q, identical page tables
        qs, ks = parallel.shard_heads(sc.hq, sc.hkv, world, rank)
        local = R.decode_attention(sc.q[:, qs].contiguous(), sc.pool[:, :, :, ks].contiguous(), m.kv_indptr,
                                   m.kv_indices, m.kv_last_page_len)
        gathered = parallel.allgather_heads(local)
        ok_tp = torch.equal(gathered, full)
        # request sharding: each rank attends over its own requests only; together they cover the batch
        mine = parallel.shard_requests(m.batch, world, rank)
        ptr = np.concatenate([[0], np.cumsum(np.diff(m.kv_indptr)[mine])]).astype(np.int32)
        idx = np.concatenate([m.kv_indices[m.kv_indptr[b]: m.kv_indptr[b + 1]] for b in mine]).astype(np.int32)
        part = R.decode_attention(sc.q[mine], sc.pool, ptr, idx, m.kv_last_page_len[mine])
        ok_dp = torch.equal(part, full[mine])
        counts = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(counts, torch.tensor([len(mine)]))
        ok_cover = int(sum(c.item() for c in counts)) == m.batch
        # pool sizing: every rank ends with the pool that fits the rank with the least free memory
        from pie_b200.pages import eval_max_num_kv_pages
        free = (100 if rank == 0 else 60) * 2 ** 30
        pages = eval_max_num_kv_pages(free, 0.9, 16, 8, 128, 32, torch.bfloat16, tensor_parallel_size=world,
                                      group=dist.group.WORLD)
        ok_pages = pages == int(60 * 2 ** 30 * 0.9 // (2 * 2 * 16 * (8 // world) * 128 * 32))
        ret[rank] = (ok_tp, ok_dp, ok_cover and ok_pages)
    finally:
        dist.destroy_process_group()


def test_head_and_request_sharding_two_gloo_ranks():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert len(ret) == world
    for r in range(world):
        assert ret[r] == (True, True, True), (r, ret[r])


def test_shard_arithmetic():
    assert parallel.shard_requests(7, 4, 1) == [1, 5]
    q, k = parallel.shard_heads(64, 8, 4, 2)
    assert (q.start, q.stop, k.start, k.stop) == (32, 48, 4, 6)
    try:
        parallel.shard_heads(32, 8, 3, 0)
    except ValueError:
        pass
    else:
        raise AssertionError("expected ValueError")


def test_peer_layout_is_aligned_and_disjoint():
    from pie_b200.parallel import peer_layout
    for batch, heads, d, es in ((1, 8, 128, 2), (256, 64, 128, 2), (37, 16, 128, 2)):
        off0, off1, total = peer_layout(batch, heads, d, es)
        need = batch * heads * d * es
        assert off0 >= 8 * 4                      # the flag words of up to 8 ranks come first
        assert off0 % 256 == 0 and off1 % 256 == 0 and total % 256 == 0
        assert off1 - off0 >= need and total - off1 >= need


def test_oproj_reduce_layout_sizes():
    """Staging and flag sizes of the o_proj exchange (host arithmetic of the library, no GPU)."""
    from pie_b200.parallel import reduce_layout
    lay = reduce_layout(128, 4096, 2, 2)
    # 64 narrow tiles: 32 per owner, one staged copy per sender
    assert lay["stage_bytes"] == 2 * 32 * 128 * 64 * 4
    assert lay["arrive_words"] == 32 * 2 * 8 and lay["done_words"] == 64 * 8
    assert reduce_layout(128, 4096, 1, 2)["stage_bytes"] == 0
    wide = reduce_layout(20480, 4096, 8, 2)
    assert wide["stage_bytes"] >= 20480 * 4096 * 4
    # regions do not overlap and are 256-byte aligned
    order = ["arrive", "done", "stage", "out0", "out1", "nbytes"]
    offs = [lay[k] for k in order]
    assert offs == sorted(offs) and all(o % 256 == 0 for o in offs)
    assert lay["done"] - lay["arrive"] >= 4 * lay["arrive_words"]
    assert lay["stage"] - lay["done"] >= 4 * lay["done_words"]
    assert lay["out0"] - lay["stage"] >= lay["stage_bytes"]
    assert lay["out1"] - lay["out0"] >= 128 * 4096 * 2


def test_oproj_staging_holds_every_tiling():
    """The index arithmetic of the o_proj exchange, redone on the host: for every shape the tile width the
    launcher picks, each tile's (owner, slot) is unique, and the staging and flag arrays that
    `piekv_oproj_allreduce_sizes` asks for hold every tile of every row count up to the maximum."""
    from pie_b200 import _lib
    from pie_b200.parallel import reduce_layout
    for hidden in (64, 1024, 4096, 8192):
        for world in (1, 2, 4, 8):
            for n_max in (1, 128, 300, 5000):
                lay = reduce_layout(n_max, hidden, world, 2)
                for n in sorted({1, n_max // 2 + 1, n_max}):
                    nt = _lib.lib.piekv_oproj_tile_cols(n, hidden)
                    assert nt in (64, 128, 256) and hidden % nt == 0
                    tiles = -(-n // 128) * (hidden // nt)
                    slots = -(-tiles // world)
                    seen = set()
                    for t in range(tiles):
                        key = (t % world, t // world)
                        assert key not in seen and key[1] < slots
                        seen.add(key)
                    if world > 1:
                        assert lay["stage_bytes"] >= world * slots * 128 * nt * 4
                    assert lay["arrive_words"] >= slots * world * 8
                    assert lay["done_words"] >= tiles * 8
    assert _lib.lib.piekv_oproj_tile_cols(8192, 8192) == 256      # enough wide tiles for every SM
    assert _lib.lib.piekv_oproj_tile_cols(256, 8192) == 128       # a decode step: 128 tiles
    assert _lib.lib.piekv_oproj_tile_cols(64, 4096) == 64
    assert _lib.lib.piekv_oproj_tile_cols(64, 96) == 0

