"""CPU tests of the oracle: against golden vectors produced by the reference's own host code
(tests/golden/make_golden.py), against the reference unit test's stated expectations, and against a
dense float64 softmax(QK^T)V."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import paged_kv_ref as R
from pie_b200 import workloads as W
from tests.util import make_scenario

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _cases(npz):
    names = sorted({k.split("/")[0] for k in npz.files if "/" in k})
    return names


def test_flat_mask_matches_reference_batch_golden():
    z = np.load(os.path.join(GOLD, "reference_batch_masks.npz"))
    names = _cases(z)
    assert len(names) >= 8
    for name in names:
        g = lambda k: z[f"{name}/in/{k}"]
        mask = R.build_flat_mask(g("qo_indptr"), g("kv_page_indptr"), g("kv_last_page_lens"), int(g("page_size")),
                                 g("flattened_masks"), g("mask_indptr"))
        ref = z[f"{name}/out/mask"]
        assert mask.shape == ref.shape, name
        assert np.array_equal(mask, ref), name


def test_reference_unit_test_expectations():
    # pie/tests/worker/test_flattened_mask.py:84-88: size 80, 79 ones, bit 31 is False
    mask = R.build_flat_mask([0, 2, 3], [0, 2, 3], [16, 16], 16, [32, 32, 16], [0, 1, 2, 3])
    assert mask.size == 80
    assert int(mask.sum()) == 79
    assert not mask[31]


def test_chunk_plus_decode_rows():
    # one row of kv_len bools per query token, causal with offset kv_len - qo_len
    mask = R.build_flat_mask([0, 3, 4], [0, 1, 3], [8, 1], 16, [6, 7, 8, 17], [0, 1, 2, 3, 4])
    assert mask.size == 3 * 8 + 17
    rows = mask[:24].reshape(3, 8).astype(int).tolist()
    assert rows == [[1, 1, 1, 1, 1, 1, 0, 0], [1, 1, 1, 1, 1, 1, 1, 0], [1] * 8]
    assert int(mask.sum()) == 6 + 7 + 8 + 17


def test_seq_lens_match_cuda_dependency_golden():
    z = np.load(os.path.join(GOLD, "flashinfer_seq_lens.npz"))
    n = len([k for k in z.files if k.endswith("/seq_lens")])
    assert n >= 8
    for i in range(n):
        got = R.get_seq_lens(z[f"case_{i}/kv_indptr"], z[f"case_{i}/kv_last_page_len"], int(z[f"case_{i}/page_size"]))
        assert np.array_equal(got, z[f"case_{i}/seq_lens"]), i


def test_batch_indices_positions_config1():
    reqs = W.config1_requests()
    meta = W.decode_steps(reqs, 1)[0]
    assert meta.kv_indptr.tolist() == [0, 3, 8, 15, 16]
    assert meta.kv_last_page_len.tolist() == [6, 1, 5, 6]
    seq = R.get_seq_lens(meta.kv_indptr, meta.kv_last_page_len, 16)
    assert seq.tolist() == [38, 65, 101, 6]
    bi, pos = R.get_batch_indices_positions(meta.qo_indptr, seq, 4)
    assert bi.tolist() == [0, 1, 2, 3]
    assert pos.tolist() == [37, 64, 100, 5]


def test_positions_multi_token():
    bi, pos = R.get_batch_indices_positions([0, 3, 3, 4], [8, 0, 17], 4)
    assert bi.tolist() == [0, 0, 0, 2]
    assert pos.tolist() == [5, 6, 7, 16]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
def test_attention_against_dense(dtype, tol):
    sc = make_scenario(8, 2, 64, dtype, [(37, 1), (0, 5), (64, 3), (15, 1)], seed=3)
    m = sc.meta
    pool = sc.pool.clone()
    seq = R.get_seq_lens(m.kv_indptr, m.kv_last_page_len, 16)
    bi, pos = R.get_batch_indices_positions(m.qo_indptr, seq, sc.n)
    R.append_paged_kv_cache(sc.k, sc.v, bi, pos, pool, m.kv_indices, m.kv_indptr, m.kv_last_page_len)
    out = R.prefill_attention(sc.q, pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len, causal=True)
    for b in range(m.batch):
        k, v = R.gather_kv(pool, m.kv_indices, m.kv_indptr, m.kv_last_page_len, b)
        s, e = int(m.qo_indptr[b]), int(m.qo_indptr[b + 1])
        # the appended rows are where the page table says they are
        assert torch.equal(k[k.shape[0] - (e - s):], sc.k[s:e])
        for j in range(e - s):
            lim = k.shape[0] - (e - s) + j + 1
            ref = R.dense_attention_check(sc.q[s + j: s + j + 1], k[:lim], v[:lim], 1 / math.sqrt(sc.d))
            assert (out[s + j].double() - ref[0]).abs().max().item() < tol


def test_custom_mask_equals_causal_when_mask_is_causal():
    sc = make_scenario(4, 4, 32, torch.float32, [(5, 3), (16, 1), (0, 4)], seed=5)
    m = sc.meta
    runs, rptr = [], [0]
    for b in range(m.batch):
        qo = int(m.qo_indptr[b + 1] - m.qo_indptr[b])
        ctx = int(m.seq_lens[b]) - qo
        r, _ = R.causal_brle(ctx, qo)
        runs += r
        rptr += [rptr[-1] + i + 1 for i in range(qo)]
    mask = R.build_flat_mask(m.qo_indptr, m.kv_indptr, m.kv_last_page_len, 16, runs, rptr)
    a = R.prefill_attention(sc.q, sc.pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len, custom_mask=mask)
    b_ = R.prefill_attention(sc.q, sc.pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len, causal=True)
    assert torch.equal(a, b_)


def test_decode_is_prefill_with_one_token():
    sc = make_scenario(4, 2, 64, torch.float32, [(37, 1), (64, 1), (100, 1), (5, 1)], seed=0)
    m = sc.meta
    a = R.decode_attention(sc.q, sc.pool, m.kv_indptr, m.kv_indices, m.kv_last_page_len)
    b = R.prefill_attention(sc.q, sc.pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len, causal=True)
    assert torch.equal(a, b)


def test_rope_properties():
    inv = R.rope_inv_freq(128, 500000.0, "llama31", 8.0, 1.0, 4.0, 8192.0)
    plain = R.rope_inv_freq(128, 500000.0, "plain")
    assert inv.dtype == np.float32 and inv.shape == (64,)
    # high frequencies untouched, low frequencies divided by the scale
    assert inv[0] == plain[0] == 1.0
    assert abs(inv[-1] / plain[-1] - 1 / 8) < 1e-6
    # scale 1 makes the llama31 variant equal plain RoPE
    assert np.array_equal(R.rope_inv_freq(128, 500000.0, "llama31", 1.0), plain)
    x = W.randn((5, 3, 128), 1, torch.float32)
    c, s = R.rope_cos_sin(np.array([0, 1, 7, 100, 4095]), inv)
    y = R.apply_rope(x, c, s)
    assert torch.equal(y[0], x[0])  # position 0 is the identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)  # rotations preserve norms
    # interleaved and split-half pairings are the same rotation on permuted coordinates
    perm = torch.cat([torch.arange(0, 128, 2), torch.arange(1, 128, 2)])
    yi = R.apply_rope(x[..., torch.argsort(perm)], c, s, interleave=True)
    assert torch.equal(yi[..., perm], y)
    # table rows reproduce rope_cos_sin
    t = R.make_cos_sin_table(128, inv)
    assert np.array_equal(t[100, :64], c[3]) and np.array_equal(t[100, 64:], s[3])


def test_append_skips_out_of_range_and_copy_pages():
    pool = torch.zeros((4, 2, 4, 1, 2))
    k = torch.arange(6, dtype=torch.float32).reshape(3, 1, 2) + 1
    v = -k
    # request 0 owns page 2 only: positions 1 (ok), 5 (beyond its page list), and a bad batch slot
    R.append_paged_kv_cache(k, v, [0, 0, 0], [1, 5, 3], pool, [2], [0, 1])
    assert torch.equal(pool[2, 0, 1, 0], k[0, 0]) and torch.equal(pool[2, 1, 3, 0], v[2, 0])
    assert pool.abs().sum() == k[0].abs().sum() * 2 + k[2].abs().sum() * 2
    R.copy_pages([pool], [2], [0], [2])
    assert torch.equal(pool[0, :, :2], pool[2, :, :2]) and pool[0, :, 2:].abs().sum() == 0


def test_oracle_window_and_sinks_against_a_dense_float64_softmax():
    """Window: only keys p - W .. p (decode: p = kv_len - 1).  Sinks: softmax over [scores, sink], value of the
    sink dropped.  Both against a direct float64 evaluation."""
    import math
    from tests.util import make_scenario
    sc = make_scenario(4, 2, 64, torch.float32, [(36, 1), (99, 1)], seed=5)
    m = sc.meta
    sinks = torch.tensor([0.3, -1.0, 2.0, 0.0])
    W_ = 10
    out, lse = R.decode_attention(sc.q, sc.pool, m.kv_indptr, m.kv_indices, m.kv_last_page_len, return_lse=True,
                                  window_left=W_, sinks=sinks)
    scale = 1.0 / math.sqrt(64)
    for b in range(2):
        k, v = R.gather_kv(sc.pool, m.kv_indices, m.kv_indptr, m.kv_last_page_len, b)
        k, v = k[-(W_ + 1):].double(), v[-(W_ + 1):].double()
        for h in range(4):
            s = (k[:, h // 2] @ sc.q[b, h].double()) * scale
            z = torch.cat([s, sinks[h: h + 1].double()])
            p = torch.softmax(z, dim=0)[:-1]
            want = p @ v[:, h // 2]
            assert (out[b, h].double() - want).abs().max().item() < 1e-5
            assert abs(lse[b, h].item() - torch.logsumexp(z, 0).item()) < 1e-4
    # prefill: a window ANDed with a mask
    sc = make_scenario(2, 1, 64, torch.float32, [(20, 6)], seed=6)
    m = sc.meta
    mask = np.ones(6 * 26, dtype=bool)
    out = R.prefill_attention(sc.q, sc.pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len,
                              custom_mask=mask, window_left=3)
    k, v = R.gather_kv(sc.pool, m.kv_indices, m.kv_indptr, m.kv_last_page_len, 0)
    for j in range(6):
        lo = 20 + j - 3
        s = (k[lo:, 0].double() @ sc.q[j, 1].double()) * (1.0 / math.sqrt(64))  # the all-true mask does not bound above
        want = torch.softmax(s, 0) @ v[lo:, 0].double()
        assert (out[j, 1].double() - want).abs().max().item() < 1e-5


def test_oproj_allreduce_residual_chain():
    """The oracle's o_proj + all-reduce + residual (llama3.py:693-709): sharding the contraction changes
    nothing but roundings, and the reference's three roundings stay within three storage-type steps of
    the exact sum."""
    import torch
    from oracle import paged_kv_ref as R
    g = torch.Generator().manual_seed(5)
    n, k, hidden = 19, 256, 96
    a = (torch.randn((n, k), generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn((hidden, k), generator=g) * 0.5).to(torch.bfloat16)
    res = torch.randn((n, hidden), generator=g).to(torch.bfloat16)
    exact1 = R.oproj_allreduce_residual([a], [w], res, exact=True)
    for world in (1, 2, 4):
        kl = k // world
        ash = [a[:, r * kl:(r + 1) * kl] for r in range(world)]
        wsh = [w[:, r * kl:(r + 1) * kl] for r in range(world)]
        exact = R.oproj_allreduce_residual(ash, wsh, res, exact=True)
        assert torch.allclose(exact, exact1, rtol=0, atol=1e-9)
        got = R.oproj_allreduce_residual(ash, wsh, res)
        assert got.dtype == torch.bfloat16 and got.shape == (n, hidden)
        parts = sum((x.double() @ y.double().t()).abs() for x, y in zip(ash, wsh))
        bound = 2.0 ** -8 * (parts + 2 * exact.abs() + res.double().abs()) + 1e-6
        assert bool(((got.double() - exact).abs() <= bound).all())
    assert R.oproj_allreduce_residual([a], [w], None).shape == (n, hidden)

