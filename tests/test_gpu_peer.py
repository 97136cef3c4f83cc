"""Head-sharded decode with results stored straight into every rank's output buffer
(piekv_decode_step_fused_peer / piekv_peer_wait).

On one GPU the two ranks are emulated as two launches, one after the other, whose "peer" buffers are
two local allocations: nothing waits on a kernel that is not running, and the stores, the completion
flags and the wait are the code that runs between real GPUs.  Every rank must end up with the same
bits; against the unsharded fused step the rows agree to rounding only (with fewer kv heads per launch
the kernel packs more pages per stage, which changes the order of the online-softmax merges), while the
appended pages are bit-exact.  With two or more GPUs a second test runs real ranks as child processes."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from pie_b200 import _lib, ops
from pie_b200 import workloads as W
from pie_b200.parallel import peer_layout, shard_heads
from tests.util import dev, oracle_decode_after_append

pytestmark = pytest.mark.gpu


def _scenario(batch, hq, hkv, seed):
    rng = np.random.default_rng(seed)
    ctx = rng.integers(1, 700, size=batch)
    pr = W.PagedRequests(W.seeded_perm(4096, seed))
    for c in ctx:
        pr.add(int(c) + 1)  # the page lists already hold the new token's slot
    idx, ptr, last = pr.csr()
    dtype = torch.bfloat16
    pool = W.randn((4096, 2, 16, hkv, 128), seed, dtype, 0.5, device="cuda")
    q = W.randn((batch, hq, 128), seed + 1, dtype, 0.5, device="cuda")
    k = W.randn((batch, hkv, 128), seed + 2, dtype, 0.5, device="cuda")
    v = W.randn((batch, hkv, 128), seed + 3, dtype, 0.5, device="cuda")
    pos = torch.from_numpy(ctx.astype(np.int32)).cuda()
    return dev(ptr), dev(idx), dev(last), pool, q, k, v, pos


@pytest.mark.parametrize("world", [2, 4])
def test_peer_stores_emulated_ranks_equal_unsharded_step(world):
    batch, hq, hkv = 37, 16, 8
    ptr, idx, last, pool, q, k, v, pos = _scenario(batch, hq, hkv, seed=3)
    rope = ops.RopeConfig()
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")

    # unsharded reference run (its own copy of the pool: the step appends)
    pool_ref = pool.clone()
    w = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    w.plan(ptr, idx, last, hq, hkv, 128, 16, q_data_type=torch.bfloat16)
    want = w.run_fused(q, k, v, pos, pool_ref, rope=rope).clone()
    ref = oracle_decode_after_append(q, pos, pool_ref, ptr, idx, last)   # the CPU oracle on the same step
    assert (want.cpu().float() - ref.float()).abs().max().item() <= 2e-2

    off0, off1, nbytes = peer_layout(batch, hq, 128, 2)
    mem = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    pools = []
    for step, off in ((1, off0), (2, off1), (3, off0)):   # both buffers, and a buffer reused
        for r in range(world):
            qs, ks = shard_heads(hq, hkv, world, r)
            if step == 1:
                pools.append(pool[:, :, :, ks, :].contiguous())
            q_r, k_r, v_r = q[:, qs].contiguous(), k[:, ks].contiguous(), v[:, ks].contiguous()
            d = _lib.PeerOutputsC()
            for t in range(world):
                d.out[t] = mem[t].data_ptr() + off
                d.flags[t] = mem[t].data_ptr()
            d.world, d.rank, d.row_heads, d.step = world, r, hq, step
            rp = rope.to_c(128)
            hq_r, hkv_r = hq // world, hkv // world
            _lib.check(_lib.lib.piekv_decode_step_fused_peer(
                q_r.data_ptr(), k_r.data_ptr(), v_r.data_ptr(), q_r.stride(0), q_r.stride(1), k_r.stride(0),
                k_r.stride(1), v_r.stride(0), v_r.stride(1), pos.data_ptr(), pools[r].data_ptr(), C.byref(d),
                ptr.data_ptr(), idx.data_ptr(), last.data_ptr(), batch, hq_r, hkv_r, 128, 16, 4096, _lib.PIEKV_BF16,
                C.byref(rp), 1.0 / np.sqrt(128.0), ws.data_ptr(), ws.numel(), err.data_ptr(), st), "fused_peer")
        for t in range(world):
            _lib.check(_lib.lib.piekv_peer_wait(mem[t].data_ptr(), world, step, err.data_ptr(), st), "peer_wait")
        torch.cuda.synchronize()
        assert err.tolist() == [0, 0, 0, 0]
        for t in range(world):
            flags = mem[t][: 4 * world].view(torch.int32).tolist()
            assert flags == [step] * world
            got = mem[t][off: off + batch * hq * 128 * 2].view(torch.bfloat16).view(batch, hq, 128)
            assert (got.float() - want.float()).abs().max().item() <= 4e-3, (step, t)
            assert (got.cpu().float() - ref.float()).abs().max().item() <= 2e-2, (step, t)
            assert torch.equal(mem[t][off: off + batch * hq * 128 * 2], mem[0][off: off + batch * hq * 128 * 2])
    # the sharded pools received the same appended rows as the unsharded one
    for r in range(world):
        _, ks = shard_heads(hq, hkv, world, r)
        assert torch.equal(pools[r], pool_ref[:, :, :, ks, :])


def test_peer_wait_reports_a_flag_that_never_comes():
    """The wait is bounded: a flag nobody raises ends in PIEKV_ERR_WAIT_TIMEOUT after 2 s, the context
    stays usable."""
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags[0] = 5
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    _lib.check(_lib.lib.piekv_peer_wait(flags.data_ptr(), 2, 5, err.data_ptr(), torch.cuda.current_stream().cuda_stream),
               "peer_wait")
    torch.cuda.synchronize()
    e = err.tolist()
    assert e[0] == _lib.PIEKV_ERR_WAIT_TIMEOUT and e[2] == 1   # rank 1's flag
    assert int((flags + 1).sum().item()) == 64 + 5            # the device still answers


def test_empty_batch_raises_no_flag_and_the_wrapper_skips_the_wait():
    """batch == 0: nothing is launched and no flag is raised, so the Python wrapper must neither take a step
    number nor queue a wait (which would spin to its time limit on every rank)."""
    class NoStep:  # stands in for PeerOutputs: any call that would consume a step fails the test
        dtype, batch_max, head_dim, world, row_heads = torch.bfloat16, 8, 128, 2, 16

        def begin_step(self):
            raise AssertionError("an empty batch must not take a step number")

        counted_descriptor = wait = wait_counted = advance = begin_step

        def full(self, batch):
            return torch.empty((batch, self.row_heads, self.head_dim), dtype=self.dtype, device="cuda")

    ws = torch.zeros(8 << 20, dtype=torch.uint8, device="cuda")
    w = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    z = lambda *shape: torch.zeros(shape, dtype=torch.int32, device="cuda")
    w.plan(z(1), z(1), z(1), 8, 4, 128, 16, q_data_type=torch.bfloat16)
    pool = torch.zeros((4, 2, 16, 4, 128), dtype=torch.bfloat16, device="cuda")
    e = lambda h: torch.empty((0, h, 128), dtype=torch.bfloat16, device="cuda")
    for counted in (False, True):
        out = w.run_fused_peer(e(8), e(4), e(4), z(1), pool, NoStep(), counted=counted)
        assert tuple(out.shape) == (0, 16, 128)
    # the C entry point itself: status 0, flags untouched
    mem = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    d = _lib.PeerOutputsC()
    for t in range(2):
        d.out[t] = mem.data_ptr() + 256
        d.flags[t] = mem.data_ptr()
    d.world, d.rank, d.row_heads, d.step = 2, 0, 16, 1
    rp = ops.RopeConfig().to_c(128)
    rc = _lib.lib.piekv_decode_step_fused_peer(None, None, None, 1024, 128, 512, 128, 512, 128, None, pool.data_ptr(),
                                               C.byref(d), None, None, None, 0, 8, 4, 128, 16, 4, _lib.PIEKV_BF16,
                                               C.byref(rp), 0.1, ws.data_ptr(), ws.numel(), None,
                                               torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(mem.view(torch.int32)[:2].abs().sum().item()) == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_stores_between_real_gpus():
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(root, "tests", "peer_worker.py")]
    r = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("PEER-OK") == n


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_oproj_sum_between_real_gpus():
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", "29534", os.path.join(root, "tests", "oproj_worker.py")]
    r = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("OPROJ-OK") == n
