"""The allocation-free decode entry point (piekv_decode_run_noalloc).

Who needs it: a caller that cannot give the library a workspace and must not cause an allocation -
an engine that handed all free device memory to its KV pool when it started, a thin foreign-language
binding that forwards only its own tensors, or code that runs where cudaMalloc is not permitted.
The entry point keeps its split-KV scratch in a fixed array inside the library instead.

The test drives both entry points through the C ABI on the same inputs and expects the same attention
output, on two calls in a row (the second call finds the first call's partial results and counters in
the shared array).  This file sorts last so that a run stopping at the first failure has already run
every other test.
"""
import math

import numpy as np
import pytest
import torch

from oracle import paged_kv_ref as R
from pie_b200 import _lib
from pie_b200 import workloads as W
from tests.util import dev, make_scenario

pytestmark = pytest.mark.gpu

L = _lib.lib


def _run_both(sc, ws):
    m = sc.meta
    q, pool = sc.q.cuda(), sc.pool.cuda()
    indptr, indices, last = dev(m.kv_indptr), dev(m.kv_indices), dev(m.kv_last_page_len)
    b = m.batch
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    scale = 1.0 / math.sqrt(sc.d)
    out_ws = torch.empty_like(q)
    out_na = torch.full_like(q, float("nan"))
    _lib.check(L.piekv_decode_run(q.data_ptr(), q.stride(0), q.stride(1), pool.data_ptr(), out_ws.data_ptr(), None,
                                  indptr.data_ptr(), indices.data_ptr(), last.data_ptr(), b, sc.hq, sc.hkv, sc.d, 16,
                                  sc.num_pages, _lib.PIEKV_BF16, scale, ws.data_ptr(), ws.numel(), err.data_ptr(),
                                  stream), "decode_run")
    _lib.check(L.piekv_decode_run_noalloc(q.data_ptr(), q.stride(0), q.stride(1), pool.data_ptr(), out_na.data_ptr(),
                                          None, indptr.data_ptr(), indices.data_ptr(), last.data_ptr(), b, sc.hq,
                                          sc.hkv, sc.d, 16, sc.num_pages, _lib.PIEKV_BF16, scale, err.data_ptr(),
                                          stream), "decode_run_noalloc")
    torch.cuda.synchronize()
    assert err.cpu().tolist() == [0, 0, 0, 0]
    return out_ws, out_na


def test_noalloc_matches_workspace_entry_point_twice(deterministic_decode):
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
    first = make_scenario(32, 8, 128, torch.bfloat16, [(c - 1, 1) for c in (4000, 37, 1500, 16, 900, 5)], seed=41,
                          scale=0.5)
    second = make_scenario(32, 8, 128, torch.bfloat16, [(c - 1, 1) for c in (100, 2600, 33)], seed=42, scale=0.5)
    for sc in (first, second):
        a, b = _run_both(sc, ws)
        assert torch.isfinite(b).all()
        assert (a.float() - b.float()).abs().max().item() <= 2e-2  # the tolerance of the other decode tests
        assert torch.equal(a, b)  # same kernel, same partition: the same bits
        # and both against the CPU oracle, so that a fault the two entry points share cannot hide
        m = sc.meta
        ref = R.decode_attention(sc.q, sc.pool, m.kv_indptr, m.kv_indices, m.kv_last_page_len)
        assert (b.cpu().float() - ref.float()).abs().max().item() <= 2e-2


def test_noalloc_rejects_what_does_not_fit():
    """A batch whose split-KV scratch exceeds the built-in array is refused before anything is launched.
    Real (small) device buffers are passed, so that the outcome does not hinge on the order of the checks."""
    assert L.piekv_decode_noalloc_max_bytes() == 8 << 20
    batch = 4096
    q = torch.zeros((batch, 32, 128), dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(q)
    pool = torch.zeros((4, 2, 16, 8, 128), dtype=torch.bfloat16, device="cuda")
    indptr = torch.zeros(batch + 1, dtype=torch.int32, device="cuda")  # every request empty
    indices = torch.zeros(1, dtype=torch.int32, device="cuda")
    last = torch.ones(batch, dtype=torch.int32, device="cuda")
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    for dtype_code in (_lib.PIEKV_BF16, _lib.PIEKV_F32):  # the tuned and the general kernel's dtypes alike
        rc = L.piekv_decode_run_noalloc(q.data_ptr(), q.stride(0), q.stride(1), pool.data_ptr(), out.data_ptr(), None,
                                        indptr.data_ptr(), indices.data_ptr(), last.data_ptr(), batch, 32, 8, 128, 16,
                                        4, dtype_code, 0.1, err.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc > 0
        assert b"scratch" in L.piekv_last_error_string()
    torch.cuda.synchronize()
    assert err.tolist() == [0, 0, 0, 0]
