"""The benchmark configurations at their FULL sizes against the CPU oracle.

* config 2: 64 requests on the 32768-page (2 GiB) pool, one fused step (RoPE from a cos/sin table + append +
  decode attention): the whole pool bit-exact, outputs within 2e-2.
* config 3: 20480 query tokens (8 prompts of 2048, 8 chunks of 512 on 6144 cached tokens) through the native
  causal flag, the reference-form boolean mask and the run-length (BRLE) form: outputs within 2e-2, log-sum-exp
  within 2e-3; plus one request of 128 query tokens on a 16384-token context.
* config 5: 256 requests with the lognormal context draw, all 8 KV heads and the one-KV-head shard shape of
  an 8-way head split.

The oracle runs on the host cores; the sizes are chosen so that each case takes seconds there."""
import numpy as np
import pytest
import torch

from oracle import paged_kv_ref as R
from pie_b200 import ops
from pie_b200 import workloads as W
from pie_b200.batching import decode_brle_batch
from tests.util import dev

pytestmark = pytest.mark.gpu

TOL = 2e-2      # attention outputs, bf16 (max-abs)
TOL_LSE = 2e-3  # natural-log-sum-exp, fp32


def _table(positions: int, d: int = 128):
    return R.make_cos_sin_table(positions, R.rope_inv_freq(d, 500000.0, "llama31", 8.0))


def _oracle_decode_step(pool_cpu, q, k, v, meta, table, d=128):
    c, s = table[meta.pos_ids, : d // 2], table[meta.pos_ids, d // 2:]
    q_r, k_r = R.apply_rope(q, c, s), R.apply_rope(k, c, s)
    b = meta.batch
    seq = R.get_seq_lens(meta.kv_indptr, meta.kv_last_page_len, 16)
    bi, kp = R.get_batch_indices_positions(meta.qo_indptr, seq, b)
    R.append_paged_kv_cache(k_r, v, bi, kp, pool_cpu, meta.kv_indices, meta.kv_indptr)
    return R.decode_attention(q_r, pool_cpu, meta.kv_indptr, meta.kv_indices, meta.kv_last_page_len, return_lse=True)


def test_config2_full_size_vs_oracle():
    cfg = W.CONFIG2
    HQ, HKV, D, B = cfg.num_qo_heads, cfg.num_kv_heads, cfg.head_dim, 64
    reqs = W.config2_requests()
    meta = W.decode_steps(reqs, 1)[0]
    assert len(meta.kv_indices) > 8000 and cfg.num_pages == 32768
    pool_gpu = W.randn(cfg.pool_shape(), 7, cfg.dtype, 0.5, device="cuda")
    pool_cpu = pool_gpu.cpu()  # the same bits on both sides, stale rows and unused pages included
    q = W.randn((B, HQ, D), 8, cfg.dtype, 0.5)
    k = W.randn((B, HKV, D), 9, cfg.dtype, 0.5)
    v = W.randn((B, HKV, D), 10, cfg.dtype, 0.5)
    table = _table(8192)
    ref, ref_lse = _oracle_decode_step(pool_cpu, q, k, v, meta, table)

    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
    w = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    w.plan(dev(meta.kv_indptr), dev(meta.kv_indices), dev(meta.kv_last_page_len), HQ, HKV, D, 16,
           q_data_type=cfg.dtype)
    rope = ops.RopeConfig(mode="table", cos_sin_table=dev(table))
    out, lse = w.run_fused(q.cuda(), k.cuda(), v.cuda(), dev(meta.pos_ids), pool_gpu, rope, return_lse=True)
    assert ops.device_error("cuda") is None
    assert (out.cpu().float() - ref.float()).abs().max().item() <= TOL
    assert (lse.cpu() - ref_lse).abs().max().item() <= TOL_LSE
    # every byte of the 2 GiB pool: the 64 new rows are where the oracle put them and nothing else moved
    assert torch.equal(pool_gpu.cpu().view(torch.int16), pool_cpu.view(torch.int16))

    # the same step through the reference's separate ops (rope in place, append, decode run)
    pool2 = pool_gpu.clone()
    del pool_gpu
    meta2 = W.decode_steps(reqs, 1)[0]
    q2, k2, v2 = q.cuda(), k.cuda(), v.cuda()
    indptr, indices, last = dev(meta2.kv_indptr), dev(meta2.kv_indices), dev(meta2.kv_last_page_len)
    ops.apply_llama31_rope_pos_ids_inplace(q2, k2, dev(meta2.pos_ids))
    seq = ops.get_seq_lens(indptr, last, 16)
    bi, kp = ops.get_batch_indices_positions(dev(meta2.qo_indptr), seq, B)
    ops.append_paged_kv_cache(k2, v2, bi, kp, pool2, indices, indptr, last)
    w.plan(indptr, indices, last, HQ, HKV, D, 16, q_data_type=cfg.dtype)
    out2 = w.run(q2, pool2)
    # oracle on the library's own rotated k (on-the-fly sin/cos differs from the table by <= 1 ulp; the
    # comparison here is about the append addressing and the attention at full size)
    seq_c = R.get_seq_lens(meta2.kv_indptr, meta2.kv_last_page_len, 16)
    bi_c, kp_c = R.get_batch_indices_positions(meta2.qo_indptr, seq_c, B)
    assert np.array_equal(bi.cpu().numpy(), bi_c) and np.array_equal(kp.cpu().numpy(), kp_c)
    R.append_paged_kv_cache(k2.cpu(), v, bi_c, kp_c, pool_cpu, meta2.kv_indices, meta2.kv_indptr)
    assert torch.equal(pool2.cpu().view(torch.int16), pool_cpu.view(torch.int16))
    ref2 = R.decode_attention(q2.cpu(), pool_cpu, meta2.kv_indptr, meta2.kv_indices, meta2.kv_last_page_len)
    assert (out2.cpu().float() - ref2.float()).abs().max().item() <= TOL
    assert ops.device_error("cuda") is None


def _causal_wire_form(meta):
    """The causal-with-offset mask as the reference ships it: one attend run of position + 1 entries per
    query token (sdk/rust/inferlet/src/forward.rs:57-64), plus what Batch.__init__ derives to expand it."""
    n = meta.nnz
    counts = np.diff(meta.qo_indptr).astype(np.int64)
    seq_l = np.asarray(meta.seq_lens, dtype=np.int64)
    tok_pos = np.arange(n, dtype=np.int64) - np.repeat(meta.qo_indptr[:-1].astype(np.int64), counts) \
        + np.repeat(seq_l - counts, counts)
    runs = (tok_pos + 1).astype(np.uint32)
    rptr = np.arange(n + 1, dtype=np.int32)
    acc = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(np.repeat(seq_l, counts), out=acc[1:])
    return runs, rptr, tok_pos, acc


def test_config3_full_size_vs_oracle():
    cfg = W.CONFIG3
    HQ, HKV, D = cfg.num_qo_heads, cfg.num_kv_heads, cfg.head_dim
    meta = W.config3_meta()
    n = meta.nnz
    assert n == 20480 and int(meta.seq_lens.max()) == 6656
    pool = W.randn(cfg.pool_shape(), 31, cfg.dtype, 0.5)
    q = W.randn((n, HQ, D), 32, cfg.dtype, 0.5)
    runs, rptr, tok_pos, acc = _causal_wire_form(meta)
    flat = decode_brle_batch(runs, rptr, tok_pos, acc)  # the reference-form flat boolean mask (60.8 M entries)
    assert flat.size == 8 * 2048 * 2048 + 8 * 512 * 6656
    ref, ref_lse = R.prefill_attention(q, pool, meta.qo_indptr, meta.kv_indptr, meta.kv_indices,
                                       meta.kv_last_page_len, custom_mask=flat, return_lse=True, row_chunk=512)

    gq, gpool = q.cuda(), pool.cuda()
    m = (dev(meta.qo_indptr), dev(meta.kv_indptr), dev(meta.kv_indices), dev(meta.kv_last_page_len))
    ws = torch.zeros(128 << 20, dtype=torch.uint8, device="cuda")
    common = dict(num_qo_heads=HQ, num_kv_heads=HKV, head_dim_qk=D, page_size=16, q_data_type=cfg.dtype)
    forms = {
        "causal": dict(causal=True),
        "mask": dict(custom_mask=torch.from_numpy(flat).cuda()),
        "brle": dict(brle_mask=(torch.from_numpy(runs.view(np.int32).copy()).cuda(), dev(rptr), int(acc[-1]))),
    }
    outs = {}
    for name, kw in forms.items():
        w = ops.BatchPrefillWithPagedKVCacheWrapper(ws, "NHD")
        w.plan(*m, **common, **kw)
        out, lse = w.run(gq, gpool, return_lse=True)
        assert ops.device_error("cuda") is None, name
        assert (out.cpu().float() - ref.float()).abs().max().item() <= TOL, name
        assert (lse.cpu() - ref_lse).abs().max().item() <= TOL_LSE, name
        outs[name] = out.cpu()
    # the two mask forms describe the same bits: the same kernel must give the same result
    assert torch.equal(outs["mask"], outs["brle"])


def test_long_context_chunk_vs_oracle():
    """One request: 128 query tokens on top of 16256 cached ones (kv 16384 = 128 kv tiles per q tile)."""
    HQ, HKV, D = 32, 8, 128
    kv, qn = 16384, 128
    pages = kv // 16
    reqs = W.PagedRequests(W.seeded_perm(pages + 16, 13))
    reqs.add(kv)
    idx, ptr, last = reqs.csr()
    qo = np.array([0, qn], np.int32)
    pool = W.randn((pages + 16, 2, 16, HKV, D), 41, torch.bfloat16, 0.5)
    q = W.randn((qn, HQ, D), 42, torch.bfloat16, 0.5)
    ref, ref_lse = R.prefill_attention(q, pool, qo, ptr, idx, last, causal=True, return_lse=True, row_chunk=32)
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
    w = ops.BatchPrefillWithPagedKVCacheWrapper(ws, "NHD")
    w.plan(dev(qo), dev(ptr), dev(idx), dev(last), HQ, HKV, D, 16, causal=True, q_data_type=torch.bfloat16)
    out, lse = w.run(q.cuda(), pool.cuda(), return_lse=True)
    assert ops.device_error("cuda") is None
    assert (out.cpu().float() - ref.float()).abs().max().item() <= TOL
    assert (lse.cpu() - ref_lse).abs().max().item() <= TOL_LSE


# all heads on one GPU / the per-GPU shapes of a 2-, 4- and 8-way KV-head split (several pages per stage: the
# warps of a stage fold their partials on chip)
@pytest.mark.parametrize("shard", [1, 2, 4, 8])
def test_config5_full_batch_vs_oracle(shard):
    cfg = W.CONFIG5
    D, B = cfg.head_dim, 256
    hq, hkv = cfg.num_qo_heads // shard, cfg.num_kv_heads // shard
    num_pages = 49152  # 46.7 k pages are in use; the benchmark's pool only adds unused pages
    reqs = W.config5_requests(B, 5, num_pages)
    meta = W.decode_steps(reqs, 1)[0]
    assert meta.batch == 256 and int(meta.seq_lens.max()) > 16000 and len(meta.kv_indices) > 46000
    pool_gpu = W.randn((num_pages, 2, 16, hkv, D), 51, cfg.dtype, 0.5, device="cuda")
    pool_cpu = pool_gpu.cpu()
    q = W.randn((B, hq, D), 52, cfg.dtype, 0.5)
    k = W.randn((B, hkv, D), 53, cfg.dtype, 0.5)
    v = W.randn((B, hkv, D), 54, cfg.dtype, 0.5)
    table = _table(40000)
    ref, ref_lse = _oracle_decode_step(pool_cpu, q, k, v, meta, table)
    ws = torch.zeros(128 << 20, dtype=torch.uint8, device="cuda")
    w = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    w.plan(dev(meta.kv_indptr), dev(meta.kv_indices), dev(meta.kv_last_page_len), hq, hkv, D, 16,
           q_data_type=cfg.dtype)
    rope = ops.RopeConfig(mode="table", cos_sin_table=dev(table))
    out, lse = w.run_fused(q.cuda(), k.cuda(), v.cuda(), dev(meta.pos_ids), pool_gpu, rope, return_lse=True)
    assert ops.device_error("cuda") is None
    assert (out.cpu().float() - ref.float()).abs().max().item() <= TOL
    assert (lse.cpu() - ref_lse).abs().max().item() <= TOL_LSE
    assert torch.equal(pool_gpu.cpu().view(torch.int16), pool_cpu.view(torch.int16))
