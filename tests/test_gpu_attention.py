"""GPU parity of decode and prefill attention against the CPU oracle, through the reference-facing
wrappers (plan / run).  Tolerances: max-abs 2e-2 for 16-bit types, 1e-4 for fp32."""
import math

import numpy as np
import pytest
import torch

from oracle import paged_kv_ref as R
from pie_b200 import ops
from pie_b200 import workloads as W
from tests.util import dev, make_scenario

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def _workspace(nbytes=64 << 20):
    return torch.zeros(nbytes, dtype=torch.uint8, device="cuda")


def _run_decode(sc, ws=None, return_lse=False):
    m = sc.meta
    w = ops.BatchDecodeWithPagedKVCacheWrapper(ws if ws is not None else _workspace(), "NHD")
    w.plan(indptr=dev(m.kv_indptr), indices=dev(m.kv_indices), last_page_len=dev(m.kv_last_page_len),
           num_qo_heads=sc.hq, num_kv_heads=sc.hkv, head_dim=sc.d, page_size=sc.page_size,
           pos_encoding_mode="NONE", q_data_type=sc.dtype)
    return w.run(sc.q.cuda(), sc.pool.cuda(), return_lse=return_lse)


def test_config1_decode_step_fp32():
    """Config 1 end to end: RoPE -> append -> decode attention, one step, 4 requests."""
    cfg = W.CONFIG1
    reqs = W.config1_requests()
    meta = W.decode_steps(reqs, 1)[0]
    pool = W.randn(cfg.pool_shape(), 0, cfg.dtype)
    q = W.randn((4, cfg.num_qo_heads, cfg.head_dim), 1, cfg.dtype)
    k = W.randn((4, cfg.num_kv_heads, cfg.head_dim), 2, cfg.dtype)
    v = W.randn((4, cfg.num_kv_heads, cfg.head_dim), 3, cfg.dtype)
    # oracle, in the reference's op order (llama3.py:654-689); table mode so the pages are bit-exact
    inv = R.rope_inv_freq(cfg.head_dim, cfg.rope_theta, "plain")
    table = R.make_cos_sin_table(128, inv)
    c, s = table[meta.pos_ids, :32], table[meta.pos_ids, 32:]
    q_ref, k_ref = R.apply_rope(q, c, s), R.apply_rope(k, c, s)
    seq = R.get_seq_lens(meta.kv_indptr, meta.kv_last_page_len, 16)
    bi, pos = R.get_batch_indices_positions(meta.qo_indptr, seq, 4)
    ref_pool = pool.clone()
    R.append_paged_kv_cache(k_ref, v, bi, pos, ref_pool, meta.kv_indices, meta.kv_indptr, meta.kv_last_page_len)
    ref_out = R.decode_attention(q_ref, ref_pool, meta.kv_indptr, meta.kv_indices, meta.kv_last_page_len)

    gpool, gq, gk, gv = pool.cuda(), q.cuda(), k.cuda(), v.cuda()
    indptr, indices, last = dev(meta.kv_indptr), dev(meta.kv_indices), dev(meta.kv_last_page_len)
    dseq = ops.get_seq_lens(indptr, last, 16)
    dbi, dpos = ops.get_batch_indices_positions(dev(meta.qo_indptr), dseq, 4)
    rope = ops.RopeConfig(mode="table", cos_sin_table=dev(table))
    ops._rope_inplace(gq, gk, dev(meta.pos_ids), rope, "rope")
    ops.append_paged_kv_cache(gk, gv, dbi, dpos, gpool, indices, indptr, last, "NHD")
    w = ops.BatchDecodeWithPagedKVCacheWrapper(_workspace(), "NHD")
    w.plan(indptr, indices, last, cfg.num_qo_heads, cfg.num_kv_heads, cfg.head_dim, 16, pos_encoding_mode="NONE",
           q_data_type=torch.float32)
    out = w.run(gq, gpool)
    assert ops.device_error("cuda") is None
    assert torch.equal(gpool.cpu(), ref_pool)  # bit-exact pages
    assert (out.cpu() - ref_out).abs().max().item() <= 1e-4
    # plain RoPE computed on the fly agrees to fp32 rounding of cos/sin
    gq2, gk2 = q.cuda(), k.cuda()
    ops.apply_rope_pos_ids_inplace(gq2, gk2, dev(meta.pos_ids), rope_theta=cfg.rope_theta)
    assert (gk2.cpu() - k_ref).abs().max().item() < 1e-5


DECODE_CASES = [
    # (dtype, hq, hkv, d, contexts)
    (torch.bfloat16, 32, 8, 128, [37, 64, 100, 5, 1, 16, 17, 4096, 512, 33]),
    (torch.float16, 32, 8, 128, [300, 1, 2048]),
    (torch.bfloat16, 64, 8, 128, [129, 2000, 15, 16]),        # group 8 (70B shape)
    (torch.bfloat16, 32, 4, 128, [77, 1025, 16, 3]),          # 2 pages per stage
    (torch.bfloat16, 16, 2, 128, [500, 31, 32, 33, 1]),       # 4 pages per stage
    (torch.bfloat16, 8, 1, 128, [700, 5, 64, 129]),           # 8 pages per stage (70B on 8 GPUs)
    (torch.bfloat16, 16, 1, 128, [260, 9]),                   # group 16
    (torch.bfloat16, 8, 8, 128, [45, 160]),                   # MHA
    (torch.bfloat16, 12, 4, 64, [50, 7, 130]),                # general kernel (D 64)
    (torch.float32, 8, 2, 128, [50, 7, 130]),                 # general kernel (fp32)
]


@pytest.mark.parametrize("dtype,hq,hkv,d,ctx", DECODE_CASES)
def test_decode_against_oracle(dtype, hq, hkv, d, ctx):
    sc = make_scenario(hq, hkv, d, dtype, [(c - 1, 1) for c in ctx], seed=len(ctx) + hq, scale=0.5 if d == 128 else 1.0)
    m = sc.meta
    ref, ref_lse = R.decode_attention(sc.q, sc.pool, m.kv_indptr, m.kv_indices, m.kv_last_page_len, return_lse=True)
    out, lse = _run_decode(sc, return_lse=True)
    assert ops.device_error("cuda") is None
    assert (out.cpu().float() - ref.float()).abs().max().item() <= TOL[dtype]
    assert (lse.cpu() - ref_lse).abs().max().item() <= 2e-3


@pytest.mark.parametrize("deterministic", [True, False])
def test_decode_many_short_requests_and_one_long(deterministic):
    # more requests than SMs, plus one request that is split across every CTA
    ops.set_deterministic(deterministic)
    try:
        _many_short_and_one_long(deterministic)
    finally:
        ops.set_deterministic(False)


def _many_short_and_one_long(deterministic):
    ctx = [1 + (i * 7) % 40 for i in range(300)] + [20000]
    sc = make_scenario(32, 8, 128, torch.bfloat16, [(c - 1, 1) for c in ctx], seed=3, scale=0.5)
    m = sc.meta
    ref = R.decode_attention(sc.q, sc.pool, m.kv_indptr, m.kv_indices, m.kv_last_page_len)
    ws = _workspace()
    out = _run_decode(sc, ws)
    assert (out.cpu().float() - ref.float()).abs().max().item() <= 2e-2
    # the arrival counters are back at zero, so the same workspace serves the next launch
    assert int(ws[: ops.COUNTER_BYTES].view(torch.int32).abs().sum().item()) == 0
    out2 = _run_decode(sc, ws)
    if deterministic:
        assert torch.equal(out, out2)
    else:  # which SM took which pages may differ between the launches: rounding only
        assert (out.float() - out2.float()).abs().max().item() <= 4e-3
        assert (out2.cpu().float() - ref.float()).abs().max().item() <= 2e-2


def test_decode_empty_request_and_nan_in_stale_rows():
    sc = make_scenario(32, 8, 128, torch.bfloat16, [(20, 1), (0, 1), (35, 1)], seed=8, scale=0.5)
    m = sc.meta
    # request 1 loses its pages: softmax over nothing -> zeros
    ptr = m.kv_indptr.copy()
    n1 = ptr[2] - ptr[1]
    idx = np.concatenate([m.kv_indices[: ptr[1]], m.kv_indices[ptr[2]:]])
    ptr[2:] -= n1
    last = m.kv_last_page_len.copy()
    last[1] = 0
    # poison the stale rows of request 0's last page (token slots >= last_len) with NaN / Inf
    pool = sc.pool.clone()
    p_last = int(idx[ptr[1] - 1])
    pool[p_last, :, int(last[0]):] = float("nan")
    sc.pool = pool
    sc.meta = W.StepMeta(idx.astype(np.int32), ptr.astype(np.int32), last, m.qo_indptr, m.pos_ids)
    ref = R.decode_attention(sc.q, pool, ptr, idx, last)
    out = _run_decode(sc)
    assert torch.isfinite(out).all()
    assert out[1].abs().max().item() == 0
    assert (out.cpu().float() - ref.float()).abs().max().item() <= 2e-2


def test_decode_reports_bad_page_id_without_faulting():
    sc = make_scenario(32, 8, 128, torch.bfloat16, [(40, 1), (10, 1)], seed=2, scale=0.5)
    sc.meta.kv_indices[1] = sc.num_pages + 100
    out = _run_decode(sc)
    e = ops.device_error("cuda")
    assert e is not None and e["code"] == 3 and e["value"] == sc.num_pages + 100
    assert torch.isfinite(out).all()


def test_decode_tuned_and_general_kernels_agree_on_strided_q():
    sc = make_scenario(32, 8, 128, torch.bfloat16, [(c, 1) for c in (99, 1500, 16, 2)], seed=12, scale=0.5)
    m = sc.meta
    fused = torch.zeros((4, 48 * 128), dtype=torch.bfloat16, device="cuda")
    fused[:, : 32 * 128] = sc.q.cuda().reshape(4, -1)
    qv = fused[:, : 32 * 128].view(4, 32, 128)  # row stride 48*128
    w = ops.BatchDecodeWithPagedKVCacheWrapper(_workspace(), "NHD")
    w.plan(dev(m.kv_indptr), dev(m.kv_indices), dev(m.kv_last_page_len), 32, 8, 128, 16, q_data_type=torch.bfloat16)
    a = w.run(qv, sc.pool.cuda())
    # the same problem through the prefill wrapper (one token per request, causal) uses the general kernel
    p = ops.BatchPrefillWithPagedKVCacheWrapper(_workspace(), "NHD")
    p.plan(dev(m.qo_indptr), dev(m.kv_indptr), dev(m.kv_indices), dev(m.kv_last_page_len), 32, 8, 128, 16,
           causal=True, q_data_type=torch.bfloat16)
    b = p.run(qv, sc.pool.cuda())
    assert (a.float() - b.float()).abs().max().item() <= 1e-2


def test_decode_cuda_graph_replay_with_changing_tables():
    """The reference binds a decode wrapper to static index buffers, captures once and replays while
    the buffers' contents change (llama3.py:293-300,915-956)."""
    hq, hkv, d, B = 32, 8, 128, 4
    sc_a = make_scenario(hq, hkv, d, torch.bfloat16, [(c, 1) for c in (30, 700, 16, 1)], seed=1, num_pages=256, scale=0.5)
    sc_b = make_scenario(hq, hkv, d, torch.bfloat16, [(c, 1) for c in (900, 2, 65, 128)], seed=2, num_pages=256, scale=0.5)
    pool = sc_a.pool.cuda()
    indptr_buf = torch.zeros(B + 1, dtype=torch.int32, device="cuda")
    indices_buf = torch.zeros(256, dtype=torch.int32, device="cuda")
    last_buf = torch.ones(B, dtype=torch.int32, device="cuda")
    q_buf = torch.zeros((B, hq, d), dtype=torch.bfloat16, device="cuda")
    out_buf = torch.zeros_like(q_buf)
    w = ops.BatchDecodeWithPagedKVCacheWrapper(_workspace(), "NHD", use_cuda_graph=True,
                                               paged_kv_indptr_buffer=indptr_buf,
                                               paged_kv_indices_buffer=indices_buf,
                                               paged_kv_last_page_len_buffer=last_buf)

    def load(sc):
        m = sc.meta
        indptr_buf.copy_(dev(m.kv_indptr))
        indices_buf[: len(m.kv_indices)].copy_(dev(m.kv_indices))
        last_buf.copy_(dev(m.kv_last_page_len))
        q_buf.copy_(sc.q.cuda())

    load(sc_a)
    w.plan(indptr_buf, indices_buf, last_buf, hq, hkv, d, 16, q_data_type=torch.bfloat16)
    w.run(q_buf, pool, out=out_buf)  # warm-up outside capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        w.run(q_buf, pool, out=out_buf)
    for sc in (sc_b, sc_a):
        load(sc)
        g.replay()
        torch.cuda.synchronize()
        m = sc.meta
        ref = R.decode_attention(sc.q, sc_a.pool, m.kv_indptr, m.kv_indices, m.kv_last_page_len)
        assert (out_buf.cpu().float() - ref.float()).abs().max().item() <= 2e-2


def test_run_before_plan_raises_like_the_reference():
    w = ops.BatchDecodeWithPagedKVCacheWrapper(_workspace(1 << 20), "NHD")
    with pytest.raises(RuntimeError, match=r"Must call plan\(\) before run\(\)"):
        w.run(torch.zeros(1, 4, 64, device="cuda"), torch.zeros(2, 2, 16, 2, 64, device="cuda"))
    p = ops.BatchPrefillWithPagedKVCacheWrapper(_workspace(1 << 20), "NHD")
    with pytest.raises(RuntimeError, match=r"Must call plan\(\) before run\(\)"):
        p.run(torch.zeros(1, 4, 64, device="cuda"), torch.zeros(2, 2, 16, 2, 64, device="cuda"))


PREFILL_CASES = [
    (torch.bfloat16, 32, 8, 128, [(0, 40), (100, 1), (15, 2), (16, 16), (31, 33)]),
    (torch.float32, 4, 2, 64, [(5, 3), (16, 1), (0, 20)]),
    (torch.float16, 8, 8, 128, [(0, 129)]),
    (torch.bfloat16, 32, 8, 128, [(0, 300), (512, 130)]),
]


def _run_prefill(sc, custom_mask=None, causal=False):
    m = sc.meta
    w = ops.BatchPrefillWithPagedKVCacheWrapper(_workspace(), "NHD")
    w.plan(qo_indptr=dev(m.qo_indptr), paged_kv_indptr=dev(m.kv_indptr), paged_kv_indices=dev(m.kv_indices),
           paged_kv_last_page_len=dev(m.kv_last_page_len), num_qo_heads=sc.hq, num_kv_heads=sc.hkv,
           head_dim_qk=sc.d, page_size=sc.page_size,
           custom_mask=None if custom_mask is None else dev(custom_mask), causal=causal, q_data_type=sc.dtype)
    return w.run(sc.q.cuda(), sc.pool.cuda())


@pytest.mark.parametrize("dtype,hq,hkv,d,reqs", PREFILL_CASES)
@pytest.mark.parametrize("mode", ["causal", "causal_mask", "full", "random_mask"])
def test_prefill_against_oracle(dtype, hq, hkv, d, reqs, mode):
    sc = make_scenario(hq, hkv, d, dtype, reqs, seed=21, scale=0.5 if d == 128 else 1.0)
    m = sc.meta
    mask = None
    if mode == "causal_mask":
        # the production form: one attend-run per token, expanded as the reference's Batch does
        runs, rptr = [], [0]
        for b in range(m.batch):
            qo = int(m.qo_indptr[b + 1] - m.qo_indptr[b])
            r, _ = R.causal_brle(int(m.seq_lens[b]) - qo, qo)
            runs += r
            rptr += [rptr[-1] + i + 1 for i in range(qo)]
        mask = R.build_flat_mask(m.qo_indptr, m.kv_indptr, m.kv_last_page_len, 16, runs, rptr)
    elif mode == "random_mask":
        rng = np.random.default_rng(5)
        total = int(np.sum(np.diff(m.qo_indptr).astype(np.int64) * m.seq_lens))
        mask = rng.random(total) < 0.6
        # every query keeps at least its first key, so no row is fully masked
        off = 0
        for b in range(m.batch):
            qo, kv = int(m.qo_indptr[b + 1] - m.qo_indptr[b]), int(m.seq_lens[b])
            mask[off: off + qo * kv: kv] = True
            off += qo * kv
    ref = R.prefill_attention(sc.q, sc.pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len,
                              custom_mask=mask, causal=(mode == "causal"))
    out = _run_prefill(sc, mask, causal=(mode == "causal"))
    assert ops.device_error("cuda") is None
    assert (out.cpu().float() - ref.float()).abs().max().item() <= TOL[dtype]


FUSED_CASES = [
    (torch.bfloat16, 32, 8, 128, [37, 64, 100, 5, 1, 16, 17, 4096, 512, 33], "table", False),
    (torch.float16, 32, 8, 128, [300, 1, 2048], "table", False),
    (torch.bfloat16, 64, 8, 128, [129, 2000, 15, 16], "table", False),
    (torch.bfloat16, 32, 4, 128, [77, 1025, 16, 3, 1], "table", False),
    (torch.bfloat16, 8, 1, 128, [700, 5, 64, 129, 1], "table", True),
    (torch.bfloat16, 32, 8, 128, [511, 4096, 2049], "llama31", False),
    (torch.bfloat16, 32, 8, 128, [45, 160], "none", False),
    (torch.float32, 4, 2, 64, [38, 65, 101, 6], "table", False),      # config 1 through the general path
    (torch.bfloat16, 12, 4, 64, [50, 7, 130], "plain", False),        # general path, on-the-fly RoPE
]


@pytest.mark.parametrize("dtype,hq,hkv,d,ctx,mode,interleave", FUSED_CASES)
def test_fused_decode_step(dtype, hq, hkv, d, ctx, mode, interleave):
    """RoPE + append + attention in one call == the oracle's three ops in the reference's order."""
    sc = make_scenario(hq, hkv, d, dtype, [(c - 1, 1) for c in ctx], seed=hq + len(ctx), scale=0.5)
    m = sc.meta
    theta = 500000.0
    table = None
    if mode == "none":
        q_ref, k_ref = sc.q, sc.k
        cfg = ops.RopeConfig(mode="none")
    else:
        inv = R.rope_inv_freq(d, theta, "plain" if mode == "plain" else "llama31", 1.0 if mode == "plain" else 8.0)
        if mode == "table":
            table = R.make_cos_sin_table(4200, inv)
            c, s = table[m.pos_ids, : d // 2], table[m.pos_ids, d // 2:]
            cfg = ops.RopeConfig(mode="table", cos_sin_table=dev(table), interleave=interleave)
        else:
            c, s = R.rope_cos_sin(m.pos_ids, inv)
            cfg = ops.RopeConfig(mode=mode, theta=theta, scale=1.0 if mode == "plain" else 8.0, interleave=interleave)
        q_ref, k_ref = R.apply_rope(sc.q, c, s, interleave), R.apply_rope(sc.k, c, s, interleave)
    ref_pool = sc.pool.clone()
    seq = R.get_seq_lens(m.kv_indptr, m.kv_last_page_len, 16)
    bi, pos = R.get_batch_indices_positions(m.qo_indptr, seq, sc.n)
    R.append_paged_kv_cache(k_ref, sc.v, bi, pos, ref_pool, m.kv_indices, m.kv_indptr)
    ref = R.decode_attention(q_ref, ref_pool, m.kv_indptr, m.kv_indices, m.kv_last_page_len)

    pool, q, k, v = sc.pool.cuda(), sc.q.cuda(), sc.k.cuda(), sc.v.cuda()
    w = ops.BatchDecodeWithPagedKVCacheWrapper(_workspace(), "NHD")
    w.plan(dev(m.kv_indptr), dev(m.kv_indices), dev(m.kv_last_page_len), hq, hkv, d, 16, q_data_type=dtype)
    out = w.run_fused(q, k, v, dev(m.pos_ids), pool, cfg)
    assert ops.device_error("cuda") is None
    assert torch.equal(q.cpu(), sc.q) and torch.equal(k.cpu(), sc.k)  # inputs are read only
    if mode in ("table", "none"):
        assert torch.equal(pool.cpu().view(torch.uint8), ref_pool.view(torch.uint8))  # bit-exact pages
    else:
        from tests.util import ulp_diff_bf16
        assert ulp_diff_bf16(pool.cpu(), ref_pool) <= 1
    assert (out.cpu().float() - ref.float()).abs().max().item() <= TOL[dtype]
    # the separate ops on the same inputs give the same pages and (within rounding) the same output
    pool2, q2, k2 = sc.pool.cuda(), sc.q.cuda(), sc.k.cuda()
    if mode != "none":
        ops._rope_inplace(q2, k2, dev(m.pos_ids), cfg, "rope")
    ops.append_paged_kv_cache(k2, v, dev(bi), dev(pos), pool2, dev(m.kv_indices), dev(m.kv_indptr),
                              dev(m.kv_last_page_len))
    out2 = w.run(q2, pool2)
    assert torch.equal(pool2, pool)
    assert (out2.float() - out.float()).abs().max().item() <= (1e-5 if dtype == torch.float32 else 4e-3)


def test_fused_decode_many_steps_match_separate_ops():
    """Sixteen consecutive fused steps keep the pool identical to the separate-op sequence."""
    from pie_b200 import workloads as W2
    hq, hkv, d = 32, 8, 128
    reqs = W2.PagedRequests(W2.seeded_perm(256, 3))
    for c in (15, 16, 100, 1, 250):
        reqs.add(c)
    metas = W2.decode_steps(reqs, 20)
    pool_a = W2.randn((256, 2, 16, hkv, d), 5, torch.bfloat16, 0.5).cuda()
    pool_b = pool_a.clone()
    inv = R.rope_inv_freq(d, 500000.0, "llama31", 8.0)
    cfg = ops.RopeConfig(mode="table", cos_sin_table=dev(R.make_cos_sin_table(512, inv)))
    w = ops.BatchDecodeWithPagedKVCacheWrapper(_workspace(), "NHD")
    for i, m in enumerate(metas):
        q = W2.randn((5, hq, d), 100 + i, torch.bfloat16, 0.5).cuda()
        k = W2.randn((5, hkv, d), 200 + i, torch.bfloat16, 0.5).cuda()
        v = W2.randn((5, hkv, d), 300 + i, torch.bfloat16, 0.5).cuda()
        indptr, indices, last = dev(m.kv_indptr), dev(m.kv_indices), dev(m.kv_last_page_len)
        w.plan(indptr, indices, last, hq, hkv, d, 16, q_data_type=torch.bfloat16)
        oa = w.run_fused(q, k, v, dev(m.pos_ids), pool_a, cfg)
        q2, k2 = q.clone(), k.clone()
        ops._rope_inplace(q2, k2, dev(m.pos_ids), cfg, "rope")
        sl = ops.get_seq_lens(indptr, last, 16)
        bi, kp = ops.get_batch_indices_positions(dev(m.qo_indptr), sl, 5)
        ops.append_paged_kv_cache(k2, v, bi, kp, pool_b, indices, indptr, last)
        ob = w.run(q2, pool_b)
        assert torch.equal(pool_a, pool_b), i
        assert (oa.float() - ob.float()).abs().max().item() <= 4e-3
    assert ops.device_error("cuda") is None


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [True, False])
def test_prefill_tensor_core_path_multi_tile(dtype, causal):
    """Chunked-prefill mix small enough for the oracle: prompts plus chunks on a cached context,
    several 128-token kv tiles per query tile, ragged tails, GQA 4."""
    reqs = [(0, 512), (0, 130), (1024, 128), (700, 77), (0, 1), (15, 17), (256, 256)]
    sc = make_scenario(32, 8, 128, dtype, reqs, seed=33, scale=0.5)
    m = sc.meta
    ref, ref_lse = R.prefill_attention(sc.q, sc.pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len,
                                       causal=causal, return_lse=True)
    w = ops.BatchPrefillWithPagedKVCacheWrapper(_workspace(), "NHD")
    w.plan(dev(m.qo_indptr), dev(m.kv_indptr), dev(m.kv_indices), dev(m.kv_last_page_len), 32, 8, 128, 16,
           causal=causal, q_data_type=dtype)
    # strided q: a view into a wider fused buffer
    fused = torch.zeros((sc.n, 48 * 128), dtype=dtype, device="cuda")
    fused[:, : 32 * 128] = sc.q.cuda().reshape(sc.n, -1)
    out, lse = w.run(fused[:, : 32 * 128].view(sc.n, 32, 128), sc.pool.cuda(), return_lse=True)
    assert ops.device_error("cuda") is None
    assert (out.cpu().float() - ref.float()).abs().max().item() <= 2e-2
    assert (lse.cpu() - ref_lse).abs().max().item() <= 5e-3
    # the general kernel on the same problem (forced by an all-true mask for the non-causal case)
    if not causal:
        total = int(np.sum(np.diff(m.qo_indptr).astype(np.int64) * m.seq_lens))
        w.plan(dev(m.qo_indptr), dev(m.kv_indptr), dev(m.kv_indices), dev(m.kv_last_page_len), 32, 8, 128, 16,
               custom_mask=torch.ones(total, dtype=torch.bool, device="cuda"), q_data_type=dtype)
        out2 = w.run(sc.q.cuda(), sc.pool.cuda())
        assert (out2.float() - out.float()).abs().max().item() <= 1e-2


@pytest.mark.parametrize("mode", [1, 2, 3])
def test_decode_with_programmatic_dependent_launch(mode, deterministic_decode):
    """Back-to-back fused steps launched with the PDL attribute give the same pages and outputs (mode 3, whose
    promise - the kernel before wrote only into the last two pages of a request - holds for consecutive
    decode steps, lets every SM request its first pages before the previous step has finished)."""
    from pie_b200 import workloads as W2
    hq, hkv, d = 32, 8, 128
    results = {}
    for pdl in (0, mode):
        ops.set_programmatic_dependent_launch(pdl)
        try:
            reqs = W2.PagedRequests(W2.seeded_perm(4096, 3))
            ctxs = (15, 16, 1000, 1, 250, 3000, 77, 9000, 14, 12000, 31)  # page boundaries are crossed on the way
            for c in ctxs:
                reqs.add(c)
            metas = W2.decode_steps(reqs, 12)
            pool = W2.randn((4096, 2, 16, hkv, d), 5, torch.bfloat16, 0.5).cuda()
            w = ops.BatchDecodeWithPagedKVCacheWrapper(_workspace(), "NHD")
            outs = []
            q = W2.randn((len(ctxs), hq, d), 100, torch.bfloat16, 0.5).cuda()
            k = W2.randn((len(ctxs), hkv, d), 200, torch.bfloat16, 0.5).cuda()
            v = W2.randn((len(ctxs), hkv, d), 300, torch.bfloat16, 0.5).cuda()
            tabs = [(dev(m.kv_indptr), dev(m.kv_indices), dev(m.kv_last_page_len), dev(m.pos_ids)) for m in metas]
            torch.cuda.synchronize()
            for indptr, indices, last, pos in tabs:  # launched back to back, no host sync in between
                w.plan(indptr, indices, last, hq, hkv, d, 16, q_data_type=torch.bfloat16)
                outs.append(w.run_fused(q, k, v, pos, pool, ops.RopeConfig()))
            torch.cuda.synchronize()
            results[pdl] = (pool.clone(), torch.stack(outs))
        finally:
            ops.set_programmatic_dependent_launch(0)
    assert ops.device_error("cuda") is None
    assert torch.equal(results[0][0], results[mode][0])
    assert torch.equal(results[0][1], results[mode][1])


@pytest.mark.parametrize("hq,hkv", [(4, 2), (3, 3)])   # two-head kernel / one-head kernel
@pytest.mark.parametrize("causal", [True, False])
def test_prefill_ignores_nan_in_stale_rows_and_unused_pages(hq, hkv, causal):
    """A recycled page may hold anything beyond the request's last token (and pages outside every list
    anything at all): probabilities there are zero, and zero times NaN must not reach the output."""
    reqs = [(0, 300), (511, 130), (0, 5), (96, 1)]   # kv = 300, 641, 5, 97: partly filled last pages
    sc = make_scenario(hq, hkv, 128, torch.bfloat16, reqs, seed=31, scale=0.5)
    m = sc.meta
    pool = sc.pool.clone()
    used = np.zeros(sc.num_pages, dtype=bool)
    for b in range(len(reqs)):
        pages = m.kv_indices[m.kv_indptr[b]: m.kv_indptr[b + 1]]
        used[pages] = True
        last = int(m.kv_last_page_len[b])
        if last < 16:
            pool[int(pages[-1]), :, last:] = float("nan")
    pool[torch.from_numpy(~used)] = float("nan")
    ref = R.prefill_attention(sc.q, pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len, causal=causal)
    w = ops.BatchPrefillWithPagedKVCacheWrapper(_workspace(), "NHD")
    w.plan(dev(m.qo_indptr), dev(m.kv_indptr), dev(m.kv_indices), dev(m.kv_last_page_len), hq, hkv, 128, 16,
           causal=causal, q_data_type=torch.bfloat16)
    out = w.run(sc.q.cuda(), pool.cuda()).cpu()
    assert ops.device_error("cuda") is None
    assert torch.isfinite(out.float()).all()
    assert (out.float() - ref.float()).abs().max().item() <= 2e-2


@pytest.mark.parametrize("deterministic", [True, False])
@pytest.mark.parametrize("hq,hkv", [(32, 8), (8, 2), (16, 1)])   # 1, 4 and 8 page slots per stage
@pytest.mark.parametrize("ctx", [[40000], [20000, 17, 30000, 3], [5000, 5000, 5000], [70000, 66000]])
def test_decode_two_level_merge_of_long_requests(hq, hkv, ctx, deterministic):
    """Requests spread over many chunks are merged in two levels (groups of chunk pieces fold on different
    SMs, whoever completes the last group folds the groups), with and without work stealing between SMs;
    two long requests side by side share chunk boundaries; the counters and tables must come back to zero."""
    ops.set_deterministic(deterministic)
    try:
        _two_level(hq, hkv, ctx, deterministic)
    finally:
        ops.set_deterministic(False)


def _two_level(hq, hkv, ctx, deterministic):
    sc = make_scenario(hq, hkv, 128, torch.bfloat16, [(c - 1, 1) for c in ctx], seed=9, scale=0.5)
    m = sc.meta
    ref, ref_lse = R.decode_attention(sc.q, sc.pool, m.kv_indptr, m.kv_indices, m.kv_last_page_len, return_lse=True)
    ws = _workspace()
    out, lse = _run_decode(sc, ws, return_lse=True)
    assert ops.device_error("cuda") is None
    assert (out.cpu().float() - ref.float()).abs().max().item() <= 2e-2
    assert (lse.cpu() - ref_lse).abs().max().item() <= 2e-2
    assert int(ws[: ops.COUNTER_BYTES].view(torch.int32).abs().sum().item()) == 0
    out2, _ = _run_decode(sc, ws, return_lse=True)
    if deterministic:
        assert torch.equal(out, out2)
    else:
        assert (out.float() - out2.float()).abs().max().item() <= 4e-3
    assert int(ws[: ops.COUNTER_BYTES].view(torch.int32).abs().sum().item()) == 0


@pytest.mark.parametrize("hq,hkv", [(32, 8), (6, 2)])  # two heads per work item / one head per CTA
def test_prefill_work_items_with_nothing_to_attend_to(hq, hkv):
    """A request whose mask hides every key (all of its query tiles have no kv tile to visit) and a request
    without query tokens, between ordinary ones: zeros and -inf for the first, nothing for the second, the
    ordinary requests as the oracle has them.  (The persistent kernel passes such items through all its roles
    without loads or MMAs.)"""
    reqs = [(40, 150), (300, 200), (0, 0), (70, 140)]
    sc = make_scenario(hq, hkv, 128, torch.bfloat16, reqs, seed=77, scale=0.5)
    m = sc.meta
    rng = np.random.default_rng(9)
    parts = []
    for b in range(m.batch):
        qo, kv = int(m.qo_indptr[b + 1] - m.qo_indptr[b]), int(m.seq_lens[b])
        blk = rng.random((qo, kv)) < 0.5
        if qo:
            blk[:, 0] = True
        if b == 1:
            blk[:] = False  # nothing is visible to any query of this request
        parts.append(blk.reshape(-1))
    mask = np.concatenate(parts)
    ref, ref_lse = R.prefill_attention(sc.q, sc.pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len,
                                       custom_mask=mask, return_lse=True)
    w = ops.BatchPrefillWithPagedKVCacheWrapper(_workspace(), "NHD")
    w.plan(qo_indptr=dev(m.qo_indptr), paged_kv_indptr=dev(m.kv_indptr), paged_kv_indices=dev(m.kv_indices),
           paged_kv_last_page_len=dev(m.kv_last_page_len), num_qo_heads=hq, num_kv_heads=hkv, head_dim_qk=128,
           page_size=16, custom_mask=dev(mask), q_data_type=torch.bfloat16)
    out, lse = w.run(sc.q.cuda(), sc.pool.cuda(), return_lse=True)
    assert ops.device_error("cuda") is None
    s, e = int(m.qo_indptr[1]), int(m.qo_indptr[2])
    assert torch.count_nonzero(out[s:e]).item() == 0 and torch.isinf(lse[s:e]).all() and (lse[s:e] < 0).all()
    keep = np.r_[0:s, e:int(m.qo_indptr[-1])]
    assert (out.cpu().float()[keep] - ref.float()[keep]).abs().max().item() <= 2e-2
    assert (lse.cpu()[keep] - ref_lse[keep]).abs().max().item() <= 2e-2
