"""Sliding windows, attention sinks and the cos/sin-cache RoPE call of the reference's other model families
(pie/src/pie_worker/model/olmo3.py:976-1013, gpt_oss.py:418-439,671-697,840-870) against the CPU oracle."""
import math

import numpy as np
import pytest
import torch

from oracle import paged_kv_ref as R
from pie_b200 import ops
from pie_b200 import workloads as W
from tests.util import dev, make_scenario

pytestmark = pytest.mark.gpu

TOL16, TOL32 = 2e-2, 1e-4


def _ws():
    return torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")


def _meta(m):
    return dev(m.kv_indptr), dev(m.kv_indices), dev(m.kv_last_page_len)


DECODE_SHAPES = [
    (torch.bfloat16, 32, 8, 128),   # tuned kernel, one page per stage
    (torch.bfloat16, 8, 1, 128),    # tuned kernel, eight pages per stage (the head-sharded shape)
    (torch.float16, 16, 4, 128),
    (torch.float32, 4, 2, 64),      # general kernel
]


@pytest.mark.parametrize("window", [0, 5, 16, 100, 1000, 100000])
@pytest.mark.parametrize("dtype,hq,hkv,d", DECODE_SHAPES)
def test_decode_window(dtype, hq, hkv, d, window):
    ctx = [37, 640, 16, 1, 2049, 17, 4000, 128]
    sc = make_scenario(hq, hkv, d, dtype, [(c - 1, 1) for c in ctx], seed=3 + hq, scale=0.5 if d == 128 else 1.0)
    m = sc.meta
    ref, ref_lse = R.decode_attention(sc.q, sc.pool, m.kv_indptr, m.kv_indices, m.kv_last_page_len,
                                      return_lse=True, window_left=window)
    w = ops.BatchDecodeWithPagedKVCacheWrapper(_ws(), "NHD")
    w.plan(*_meta(m), hq, hkv, d, 16, q_data_type=dtype, window_left=window)
    out, lse = w.run(sc.q.cuda(), sc.pool.cuda(), return_lse=True)
    assert ops.device_error("cuda") is None
    tol = TOL32 if dtype == torch.float32 else TOL16
    assert (out.cpu().float() - ref.float()).abs().max().item() <= tol
    assert (lse.cpu() - ref_lse).abs().max().item() <= 2e-3


def test_decode_window_many_requests_split_over_ctas_and_fused_step():
    """A windowed batch large enough that windowed page ranges are cut across CTAs, through the fused step
    (the new token's page is always inside the window), with sinks on top."""
    hq, hkv, d = 32, 8, 128
    rng = np.random.default_rng(5)
    ctx = [int(x) for x in rng.integers(1, 6000, size=96)]
    sc = make_scenario(hq, hkv, d, torch.bfloat16, [(c - 1, 1) for c in ctx], seed=9, scale=0.5)
    m = sc.meta
    window = 1023
    sinks = torch.linspace(-2.0, 3.0, hq)
    table = R.make_cos_sin_table(8192, R.rope_inv_freq(d, 500000.0, "llama31", 8.0))
    c_, s_ = table[m.pos_ids, : d // 2], table[m.pos_ids, d // 2:]
    q_r, k_r = R.apply_rope(sc.q, c_, s_), R.apply_rope(sc.k, c_, s_)
    pool_ref = sc.pool.clone()
    seq = R.get_seq_lens(m.kv_indptr, m.kv_last_page_len, 16)
    bi, kp = R.get_batch_indices_positions(m.qo_indptr, seq, m.batch)
    R.append_paged_kv_cache(k_r, sc.v, bi, kp, pool_ref, m.kv_indices, m.kv_indptr)
    ref = R.decode_attention(q_r, pool_ref, m.kv_indptr, m.kv_indices, m.kv_last_page_len, window_left=window,
                             sinks=sinks)
    w = ops.BatchDecodeWithPagedKVCacheWrapper(_ws(), "NHD")
    w.plan(*_meta(m), hq, hkv, d, 16, q_data_type=torch.bfloat16, window_left=window)
    pool = sc.pool.cuda()
    out = w.run_fused(sc.q.cuda(), sc.k.cuda(), sc.v.cuda(), dev(m.pos_ids), pool,
                      ops.RopeConfig(mode="table", cos_sin_table=dev(table)), sinks=sinks.cuda())
    assert ops.device_error("cuda") is None
    assert (out.cpu().float() - ref.float()).abs().max().item() <= TOL16
    assert torch.equal(pool.cpu().view(torch.int16), pool_ref.view(torch.int16))
    # the same plan replayed with programmatic dependent launch requested: the windowed offsets are written by
    # the launch just before, so the kernel must still wait for them
    ops.set_programmatic_dependent_launch(2)
    try:
        out2 = w.run(q_r.cuda(), pool, sinks=sinks.cuda())
    finally:
        ops.set_programmatic_dependent_launch(0)
    assert (out2.cpu().float() - ref.float()).abs().max().item() <= TOL16


@pytest.mark.parametrize("dtype,hq,hkv,d", DECODE_SHAPES)
def test_decode_sinks(dtype, hq, hkv, d):
    ctx = [37, 640, 16, 1, 5000]
    sc = make_scenario(hq, hkv, d, dtype, [(c - 1, 1) for c in ctx], seed=13, scale=0.5 if d == 128 else 1.0)
    m = sc.meta
    sinks = torch.randn(hq, generator=torch.Generator().manual_seed(1)) * 2.0
    ref, ref_lse = R.decode_attention(sc.q, sc.pool, m.kv_indptr, m.kv_indices, m.kv_last_page_len, return_lse=True,
                                      sinks=sinks)
    w = ops.BatchDecodeWithPagedKVCacheWrapper(_ws(), "NHD")
    w.plan(*_meta(m), hq, hkv, d, 16, q_data_type=dtype)
    out, lse = w.run(sc.q.cuda(), sc.pool.cuda(), return_lse=True, sinks=sinks.cuda())
    plain = w.run(sc.q.cuda(), sc.pool.cuda())
    assert ops.device_error("cuda") is None
    tol = TOL32 if dtype == torch.float32 else TOL16
    assert (out.cpu().float() - ref.float()).abs().max().item() <= tol
    assert (lse.cpu() - ref_lse).abs().max().item() <= 2e-3
    assert (out.float() - plain.float()).abs().max().item() > 1e-3  # the sinks did take probability mass


def _window_mask(reqs, window, causal):
    rows = []
    for ctx, new in reqs:
        kv = ctx + new
        for j in range(new):
            p = ctx + j
            row = np.zeros(kv, dtype=bool)
            row[max(0, p - window): (p + 1 if causal else kv)] = True
            rows.append(row)
    return np.concatenate(rows) if rows else np.zeros(0, dtype=bool)


PREFILL_REQS = [(0, 300), (511, 130), (96, 1), (1000, 257)]


@pytest.mark.parametrize("hq,hkv", [(4, 2), (3, 3)])  # two-head / one-head tensor-core kernels
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("window", [0, 7, 100, 5000])
def test_prefill_window_without_a_mask(window, causal, hq, hkv):
    sc = make_scenario(hq, hkv, 128, torch.bfloat16, PREFILL_REQS, seed=41, scale=0.5)
    m = sc.meta
    flat = _window_mask(PREFILL_REQS, window, causal)
    ref = R.prefill_attention(sc.q, sc.pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len,
                              custom_mask=flat)
    # the oracle's own window argument says the same thing as the explicit mask
    ref2 = R.prefill_attention(sc.q, sc.pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len,
                               causal=causal, window_left=window)
    assert torch.equal(ref, ref2)
    w = ops.BatchPrefillWithPagedKVCacheWrapper(_ws(), "NHD")
    w.plan(dev(m.qo_indptr), *_meta(m), hq, hkv, 128, 16, causal=causal, window_left=window,
           q_data_type=torch.bfloat16)
    out = w.run(sc.q.cuda(), sc.pool.cuda()).cpu()
    assert ops.device_error("cuda") is None
    assert (out.float() - ref.float()).abs().max().item() <= TOL16


@pytest.mark.parametrize("form", ["mask", "brle"])
@pytest.mark.parametrize("window", [3, 64, 700])
def test_prefill_window_together_with_a_custom_mask(window, form):
    """What the reference passes for sliding-window layers: the flat mask of the batch AND window_left
    (pie/src/pie_worker/model/olmo3.py:1001-1013)."""
    from pie_b200.batching import Batch
    hq, hkv = 8, 2
    reqs = [(0, 200), (300, 140), (40, 3)]
    sc = make_scenario(hq, hkv, 128, torch.bfloat16, reqs, seed=43, scale=0.5)
    m = sc.meta
    rng = np.random.default_rng(7)
    # run-length rows: random alternating runs (some holes inside the causal part)
    runs, rptr = [], [0]
    for ctx, new in reqs:
        for j in range(new):
            left = ctx + j + 1
            row = []
            while left > 0:
                r = int(min(left, rng.integers(1, 90)))
                row.append(r)
                left -= r
            runs += row
            rptr.append(len(runs))
    u = lambda a: np.asarray(a, dtype=np.uint32).tobytes()
    batch = Batch({"token_ids": u(np.arange(m.nnz)), "position_ids": u(m.pos_ids), "kv_page_indices": u(m.kv_indices),
                   "kv_page_indptr": u(m.kv_indptr), "kv_last_page_lens": u(m.kv_last_page_len),
                   "qo_indptr": u(m.qo_indptr), "flattened_masks": u(runs), "mask_indptr": u(rptr),
                   "single_token_mode": False}, 16)
    flat = batch.attention_masks
    ref = R.prefill_attention(sc.q, sc.pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len,
                              custom_mask=flat, window_left=window)
    w = ops.BatchPrefillWithPagedKVCacheWrapper(_ws(), "NHD")
    kw = dict(custom_mask=torch.from_numpy(flat).cuda()) if form == "mask" else dict(brle_mask=batch.brle_inputs("cuda"))
    w.plan(dev(m.qo_indptr), *_meta(m), hq, hkv, 128, 16, window_left=window, q_data_type=torch.bfloat16, **kw)
    out = w.run(sc.q.cuda(), sc.pool.cuda()).cpu()
    assert ops.device_error("cuda") is None
    assert (out.float() - ref.float()).abs().max().item() <= TOL16
    no_window = R.prefill_attention(sc.q, sc.pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len,
                                    custom_mask=flat)
    if window < 400:  # (the largest one spans every context here: the same result as without it)
        assert (no_window.float() - ref.float()).abs().max().item() > 1e-2  # the window did cut something


def test_prefill_window_general_kernel_fp32():
    reqs = [(10, 20), (0, 33)]
    sc = make_scenario(4, 2, 64, torch.float32, reqs, seed=47)
    m = sc.meta
    for causal in (True, False):
        ref = R.prefill_attention(sc.q, sc.pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len,
                                  causal=causal, window_left=5)
        w = ops.BatchPrefillWithPagedKVCacheWrapper(_ws(), "NHD")
        w.plan(dev(m.qo_indptr), *_meta(m), 4, 2, 64, 16, causal=causal, window_left=5, q_data_type=torch.float32)
        out = w.run(sc.q.cuda(), sc.pool.cuda()).cpu()
        assert (out - ref).abs().max().item() <= TOL32
    assert ops.device_error("cuda") is None


@pytest.mark.parametrize("hq,hkv", [(8, 2), (3, 3)])
@pytest.mark.parametrize("window", [-1, 127])
def test_attention_sink_wrapper_prefill_and_decode(window, hq, hkv):
    """The reference's sink wrapper: constructed with the window, planned like the prefill wrapper with
    causal=True, run(q, kv, sinks, scaling); the same wrapper serves decode batches."""
    dt = torch.bfloat16
    sinks = torch.randn(hq, generator=torch.Generator().manual_seed(2)) * 1.5
    scaling = 128 ** -0.5
    w = ops.BatchAttentionWithAttentionSinkWrapper(float_workspace_buffer=_ws(), kv_layout="NHD", window_left=window,
                                                   q_data_type=dt, kv_data_type=dt, head_dim_qk=128, head_dim_vo=128)
    for reqs in ([(0, 300), (511, 130), (96, 1)], [(c - 1, 1) for c in (37, 640, 16, 2000)]):
        sc = make_scenario(hq, hkv, 128, dt, reqs, seed=51, scale=0.5)
        m = sc.meta
        ref, ref_lse = R.prefill_attention(sc.q, sc.pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len,
                                           causal=True, window_left=window, sinks=sinks, sm_scale=scaling,
                                           return_lse=True)
        w.plan(dev(m.qo_indptr), *_meta(m), hq, hkv, 128, 16, causal=True, window_left=window, q_data_type=dt,
               kv_data_type=dt, non_blocking=True)
        out = w.run(sc.q.cuda(), sc.pool.cuda(), sinks.cuda(), scaling)
        assert ops.device_error("cuda") is None
        assert (out.cpu().float() - ref.float()).abs().max().item() <= TOL16
        _, lse = w.run(sc.q.cuda(), sc.pool.cuda(), sinks.cuda(), scaling, return_lse=True)
        assert (lse.cpu() - ref_lse).abs().max().item() <= 2e-3


@pytest.mark.parametrize("is_neox", [True, False])
@pytest.mark.parametrize("flat", [True, False])
def test_rope_with_cos_sin_cache(is_neox, flat):
    """apply_rope_with_cos_sin_cache_inplace(positions, query, key, head_size, cos_sin_cache, is_neox) with a
    YaRN-style table built the way the reference's models build it (cos | sin, scaled by a concentration
    factor): bit-exact against the oracle's rotation with the same table."""
    n, hq, hkv, d = 77, 8, 2, 128
    dt = torch.bfloat16
    q = W.randn((n, hq, d), 1, dt)
    k = W.randn((n, hkv, d), 2, dt)
    pos = torch.from_numpy(np.random.default_rng(3).integers(0, 4096, size=n)).to(torch.int64)
    inv = (1.0 / (150000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d)))
    fr = torch.einsum("i,j->ij", torch.arange(4096, dtype=torch.float32), inv)
    conc = 0.1 * math.log(32.0) + 1.0
    cache = torch.cat([fr.cos() * conc, fr.sin() * conc], dim=-1).to(torch.float32)
    c, s = cache[pos, : d // 2].numpy(), cache[pos, d // 2:].numpy()
    q_ref, k_ref = R.apply_rope(q, c, s, interleave=not is_neox), R.apply_rope(k, c, s, interleave=not is_neox)
    gq, gk = q.cuda(), k.cuda()
    if flat:
        ops.apply_rope_with_cos_sin_cache_inplace(positions=pos.cuda(), query=gq.view(n, -1), key=gk.view(n, -1),
                                                  head_size=d, cos_sin_cache=cache.cuda(), is_neox=is_neox)
    else:
        ops.apply_rope_with_cos_sin_cache_inplace(positions=pos.cuda().to(torch.int32), query=gq, key=gk, head_size=d,
                                                  cos_sin_cache=cache.cuda(), is_neox=is_neox)
    assert ops.device_error("cuda") is None
    assert torch.equal(gq.cpu().view(torch.int16), q_ref.view(torch.int16))
    assert torch.equal(gk.cpu().view(torch.int16), k_ref.view(torch.int16))
