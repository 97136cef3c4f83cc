"""Output projection with the sum over the ranks in its epilogue (piekv_oproj_allreduce), on one GPU:
the product itself (a world of one rank), the argument checks, and the bounded wait for a rank that never
comes.  The exchange between real GPUs is tests/test_gpu_peer.py::test_oproj_sum_between_real_gpus."""
import ctypes as C

import pytest
import torch

from pie_b200 import _lib, ops
from pie_b200 import workloads as W
from pie_b200.parallel import PeerReduce, reduce_layout

pytestmark = pytest.mark.gpu

STEP = 2.0 ** -7   # one rounding to bf16 is at most 2^-9 relative; fp32 sums in another order add a little


def reference(a, w, residual):
    """fp32 product of the 16-bit operands (+ residual), as the reference's linear would give before rounding."""
    out = a.float() @ w.float().t()
    if residual is not None:
        out = out + residual.float()
    return out


def close_enough(got, want, floor):
    err = (got.float() - want).abs()
    return bool((err <= STEP * want.abs().clamp_min(floor)).all()), err.max().item()


@pytest.mark.parametrize("n,k,hidden,with_res", [(53, 256, 512, True), (128, 2048, 4096, False), (1, 64, 64, True),
                                                 (300, 128, 1024, True), (1300, 192, 4096, True)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_single_rank_product(n, k, hidden, with_res, dtype):
    dev = torch.device("cuda")
    if dtype == torch.float16 and n == 1300:
        pytest.skip("one wide-tile case is enough for fp16")
    a = W.randn((n, k), 1, dtype, 0.5, device=dev)
    w = W.randn((hidden, k), 2, dtype, 0.5, device=dev)
    res = W.randn((n, hidden), 3, dtype, 1.0, device=dev) if with_res else None
    pr = PeerReduce(n + 7, hidden, dtype, dev)
    try:
        outs = []
        for step in range(3):   # the buffers alternate; the third call reuses the first one
            got = pr.oproj(a, w, res)
            torch.cuda.synchronize()
            assert ops.device_error(dev) is None
            assert got.shape == (n, hidden) and got.dtype == dtype
            ok, worst = close_enough(got, reference(a, w, res), floor=0.5 * k ** 0.5 * 0.25)
            assert ok, worst
            outs.append(got)
        assert outs[0].data_ptr() != outs[1].data_ptr() and outs[0].data_ptr() == outs[2].data_ptr()
        assert torch.equal(outs[0], outs[1])
        # rows given as [n, heads, head_dim] and a strided view of a wider matrix
        if k % 128 == 0:
            wide = torch.zeros((n, 2 * k), dtype=dtype, device=dev)
            wide[:, :k] = a
            got = pr.oproj(wide[:, :k], w, res)
            torch.cuda.synchronize()
            assert torch.equal(got, outs[1])
            got = pr.oproj(a.view(n, k // 128, 128), w, res)
            torch.cuda.synchronize()
            assert torch.equal(got, outs[1])
    finally:
        pr.close()


def test_argument_checks():
    dev = torch.device("cuda")
    pr = PeerReduce(64, 256, torch.bfloat16, dev)
    try:
        a = torch.zeros((8, 128), dtype=torch.bfloat16, device=dev)
        w = torch.zeros((256, 128), dtype=torch.bfloat16, device=dev)
        with pytest.raises(ValueError):
            pr.oproj(a, w[:, :64])                      # shapes disagree
        with pytest.raises(ValueError):
            pr.oproj(torch.zeros((65, 128), dtype=torch.bfloat16, device=dev), w)   # more rows than the buffers hold
        with pytest.raises(ValueError):
            pr.oproj(a.half(), w.half())                # another dtype than the buffers'
        with pytest.raises(ValueError):
            pr.oproj(a, w, torch.zeros((8, 128), dtype=torch.bfloat16, device=dev))
        a96 = torch.zeros((8, 96), dtype=torch.bfloat16, device=dev)
        with pytest.raises(ValueError):
            pr.oproj(a96, torch.zeros((256, 96), dtype=torch.bfloat16, device=dev))  # k_local not a multiple of 64
        assert pr.oproj(a[:0], w).shape == (0, 256) and pr.step == 0   # neither a refused nor an empty call takes a step number
        d = _lib.PeerReduceC()
        d.world, d.rank, d.step = 9, 0, 1
        rc = _lib.lib.piekv_oproj_allreduce(a.data_ptr(), 128, w.data_ptr(), 128, None, 0, 8, 128, 256, _lib.PIEKV_BF16,
                                            C.byref(d), None, None)
        assert rc != 0 and b"peer" in _lib.lib.piekv_last_error_string()
    finally:
        pr.close()


def test_a_rank_that_never_comes_times_out():
    """Two ranks described, one launched: the launched rank's wait for the other's partial sums runs out
    after two seconds, the error word says so, and the context stays usable."""
    dev = torch.device("cuda")
    n, k, hidden = 16, 64, 128
    lay = reduce_layout(n, hidden, 2, 2)
    mem = torch.zeros(2 * lay["nbytes"], dtype=torch.uint8, device=dev)   # "rank 1" is the second half, never run
    a = W.randn((n, k), 1, torch.bfloat16, 0.5, device=dev)
    w = W.randn((hidden, k), 2, torch.bfloat16, 0.5, device=dev)
    d = _lib.PeerReduceC()
    for r in range(2):
        base = mem.data_ptr() + r * lay["nbytes"]
        d.out[r], d.stage[r] = base + lay["out0"], base + lay["stage"]
        d.arrive[r], d.done[r] = base + lay["arrive"], base + lay["done"]
    d.stage_bytes, d.arrive_words, d.done_words = lay["stage_bytes"], lay["arrive_words"], lay["done_words"]
    d.world, d.rank, d.step = 2, 0, 1
    assert mem.data_ptr() % 256 == 0
    ops.device_error(dev)
    rc = _lib.lib.piekv_oproj_allreduce(a.data_ptr(), k, w.data_ptr(), k, None, 0, n, k, hidden, _lib.PIEKV_BF16,
                                        C.byref(d), ops._err_word(dev).data_ptr(), ops._stream(dev))
    assert rc == 0
    torch.cuda.synchronize()
    err = ops.device_error(dev)
    assert err is not None and err["code"] == _lib.PIEKV_ERR_WAIT_TIMEOUT, err
    # what rank 0 owed to rank 1 did arrive: the partial of tile 1 (rank 1 owns it) and its flags
    r1 = mem[lay["nbytes"]:]
    flags = r1[lay["arrive"]: lay["arrive"] + 4 * 16].view(torch.int32)   # slot 0: [2 senders][8 warps]
    assert flags[:8].tolist() == [1] * 8 and flags[8:16].tolist() == [0] * 8
    staged = r1[lay["stage"]: lay["stage"] + 128 * 64 * 4].view(torch.float32).view(16, 128, 4)  # sender 0, slot 0
    want = (a.float() @ w.float().t())[:, 64:128]
    got = staged[:, :n, :].permute(1, 0, 2).reshape(n, 64)
    assert torch.allclose(got, want, rtol=1e-3, atol=1e-3)
    # the context still works
    assert torch.equal(a + 0, a)
