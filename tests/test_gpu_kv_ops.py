"""GPU parity: metadata, RoPE, append, fused RoPE+append and page copy against the CPU oracle.
Everything goes through pie_b200.ops, i.e. through the C ABI of libpiekv.so."""
import numpy as np
import pytest
import torch

from oracle import paged_kv_ref as R
from pie_b200 import ops
from pie_b200 import workloads as W
from tests.util import dev, make_scenario, ulp_diff_bf16

pytestmark = pytest.mark.gpu


def _no_device_error():
    assert ops.device_error("cuda") is None


@pytest.mark.parametrize("case", [
    dict(ptr=[0, 3, 8, 15, 16], last=[6, 1, 5, 6], qo=[0, 1, 2, 3, 4], ps=16),
    dict(ptr=[0, 2, 2, 3], last=[16, 0, 5], qo=[0, 3, 3, 7], ps=16),
    dict(ptr=[0, 1], last=[1], qo=[0, 1], ps=4),
    dict(ptr=[0, 5, 9, 9, 30], last=[4, 1, 0, 3], qo=[0, 17, 18, 18, 50], ps=4),
])
def test_metadata(case):
    ptr = np.array(case["ptr"], np.int32)
    last = np.array(case["last"], np.int32)
    qo = np.array(case["qo"], np.int32)
    seq = ops.get_seq_lens(dev(ptr), dev(last), case["ps"])
    ref_seq = R.get_seq_lens(ptr, last, case["ps"])
    assert np.array_equal(seq.cpu().numpy(), ref_seq)
    bi, pos = ops.get_batch_indices_positions(dev(qo), seq, int(qo[-1]))
    rbi, rpos = R.get_batch_indices_positions(qo, ref_seq, int(qo[-1]))
    assert np.array_equal(bi.cpu().numpy(), rbi) and np.array_equal(pos.cpu().numpy(), rpos)


def test_metadata_golden_from_reference_dependency():
    import os
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "flashinfer_seq_lens.npz"))
    for i in range(8):
        got = ops.get_seq_lens(dev(z[f"case_{i}/kv_indptr"]), dev(z[f"case_{i}/kv_last_page_len"]),
                               int(z[f"case_{i}/page_size"]))
        assert np.array_equal(got.cpu().numpy(), z[f"case_{i}/seq_lens"])


ROPE_CASES = [
    (torch.bfloat16, 128, "llama31", False),
    (torch.float16, 128, "plain", False),
    (torch.float32, 64, "plain", False),
    (torch.bfloat16, 64, "llama31", True),
    (torch.float32, 96, "llama31", False),
]


@pytest.mark.parametrize("dtype,d,mode,interleave", ROPE_CASES)
def test_rope_inplace(dtype, d, mode, interleave):
    n, hq, hkv = 37, 6, 2
    theta = 500000.0 if mode == "llama31" else 10000.0
    # q and k are strided views of one fused projection output, as in the reference
    fused = W.randn((n, (hq + 2 * hkv) * d), 21, dtype)
    pos = np.array([0, 1, 2, 3, 15, 16, 17, 100, 1000, 4095, 8191, 32767] + list(range(25)), np.int32)
    inv = R.rope_inv_freq(d, theta, mode, 8.0 if mode == "llama31" else 1.0)
    c, s = R.rope_cos_sin(pos, inv)
    q_ref = R.apply_rope(fused[:, : hq * d].reshape(n, hq, d), c, s, interleave)
    k_ref = R.apply_rope(fused[:, hq * d: (hq + hkv) * d].reshape(n, hkv, d), c, s, interleave)

    g = fused.cuda()
    q = g[:, : hq * d].view(n, hq, d)
    k = g[:, hq * d: (hq + hkv) * d].view(n, hkv, d)
    v_before = g[:, (hq + hkv) * d:].clone()
    if mode == "llama31":
        ops.apply_llama31_rope_pos_ids_inplace(q=q, k=k, pos_ids=dev(pos), rope_scale=8.0, rope_theta=theta,
                                               low_freq_factor=1.0, high_freq_factor=4.0, old_context_len=8192,
                                               interleave=interleave)
    else:
        ops.apply_rope_pos_ids_inplace(q, k, dev(pos), rope_theta=theta, interleave=interleave)
    _no_device_error()
    assert torch.equal(g[:, (hq + hkv) * d:], v_before)  # v untouched
    if dtype == torch.float32:
        # on-the-fly sincosf vs numpy: a few fp32 ulp of cos/sin
        assert (q.cpu() - q_ref).abs().max().item() < 2e-5
        assert (k.cpu() - k_ref).abs().max().item() < 2e-5
    elif dtype == torch.bfloat16:
        assert ulp_diff_bf16(q.cpu(), q_ref) <= 1 and ulp_diff_bf16(k.cpu(), k_ref) <= 1
        assert (q.cpu() != q_ref).float().mean().item() < 1e-3
    else:
        assert (q.cpu().float() - q_ref.float()).abs().max().item() < 4e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_rope_table_mode_is_bit_exact(dtype):
    n, hq, hkv, d = 50, 4, 2, 128
    q0, k0 = W.randn((n, hq, d), 1, dtype), W.randn((n, hkv, d), 2, dtype)
    pos = np.arange(n, dtype=np.int32) * 83 % 4096
    inv = R.rope_inv_freq(d, 500000.0, "llama31", 8.0)
    table = R.make_cos_sin_table(4096, inv)
    c, s = table[pos, : d // 2], table[pos, d // 2:]
    q_ref, k_ref = R.apply_rope(q0, c, s), R.apply_rope(k0, c, s)
    q, k = q0.cuda(), k0.cuda()
    cfg = ops.RopeConfig(mode="table", cos_sin_table=dev(table))
    ops._rope_inplace(q, k, dev(pos), cfg, "rope table")
    assert torch.equal(q.cpu(), q_ref) and torch.equal(k.cpu(), k_ref)
    _no_device_error()


APPEND_CASES = [
    (torch.float32, 4, 2, 64, [(37, 1), (64, 1), (100, 1), (5, 1)]),          # config 1
    (torch.bfloat16, 32, 8, 128, [(0, 40), (100, 1), (15, 2), (16, 16), (31, 33)]),
    (torch.float16, 8, 1, 128, [(3, 5), (0, 1)]),
    (torch.bfloat16, 6, 3, 80, [(7, 9), (0, 3), (50, 1)]),
]


@pytest.mark.parametrize("dtype,hq,hkv,d,reqs", APPEND_CASES)
def test_append_bit_exact(dtype, hq, hkv, d, reqs):
    sc = make_scenario(hq, hkv, d, dtype, reqs, seed=7)
    m = sc.meta
    ref_pool = sc.pool.clone()
    seq = R.get_seq_lens(m.kv_indptr, m.kv_last_page_len, 16)
    rbi, rpos = R.get_batch_indices_positions(m.qo_indptr, seq, sc.n)
    R.append_paged_kv_cache(sc.k, sc.v, rbi, rpos, ref_pool, m.kv_indices, m.kv_indptr, m.kv_last_page_len)

    pool = sc.pool.cuda()
    # non-contiguous k / v rows: slices of one fused buffer
    fused = torch.cat([sc.k.reshape(sc.n, -1), sc.v.reshape(sc.n, -1)], dim=1).cuda()
    k = fused[:, : hkv * d].view(sc.n, hkv, d)
    v = fused[:, hkv * d:].view(sc.n, hkv, d)
    dseq = ops.get_seq_lens(dev(m.kv_indptr), dev(m.kv_last_page_len), 16)
    bi, pos = ops.get_batch_indices_positions(dev(m.qo_indptr), dseq, sc.n)
    ops.append_paged_kv_cache(append_key=k, append_value=v, batch_indices=bi, positions=pos, paged_kv_cache=pool,
                              kv_indices=dev(m.kv_indices), kv_indptr=dev(m.kv_indptr),
                              kv_last_page_len=dev(m.kv_last_page_len), kv_layout="NHD")
    _no_device_error()
    assert torch.equal(pool.cpu().view(torch.uint8), ref_pool.view(torch.uint8))


def test_append_reports_bad_indices_and_skips():
    sc = make_scenario(4, 2, 64, torch.bfloat16, [(3, 2), (0, 1)], seed=9)
    m = sc.meta
    pool = sc.pool.cuda()
    before = pool.clone()
    idx = m.kv_indices.copy()
    idx[0] = sc.num_pages + 5  # bad physical page for request 0
    bi = np.array([0, 0, 7], np.int32)  # third token: bad batch index
    pos = np.array([3, 4, 0], np.int32)
    ops.append_paged_kv_cache(sc.k.cuda(), sc.v.cuda(), dev(bi), dev(pos), pool, dev(idx), dev(m.kv_indptr),
                              dev(m.kv_last_page_len))
    e = ops.device_error("cuda")
    assert e is not None and e["code"] in (1, 3)
    assert torch.equal(pool, before)  # nothing was written
    assert ops.device_error("cuda") is None  # cleared


@pytest.mark.parametrize("dtype,hq,hkv,d", [(torch.bfloat16, 32, 8, 128), (torch.float32, 4, 2, 64)])
def test_fused_rope_append_table_bit_exact(dtype, hq, hkv, d):
    sc = make_scenario(hq, hkv, d, dtype, [(37, 1), (64, 1), (100, 3), (5, 1), (0, 20)], seed=4)
    m = sc.meta
    theta = 500000.0
    inv = R.rope_inv_freq(d, theta, "llama31", 8.0)
    table = R.make_cos_sin_table(256, inv)
    c, s = table[m.pos_ids, : d // 2], table[m.pos_ids, d // 2:]
    q_ref = R.apply_rope(sc.q, c, s)
    k_ref = R.apply_rope(sc.k, c, s)
    ref_pool = sc.pool.clone()
    seq = R.get_seq_lens(m.kv_indptr, m.kv_last_page_len, 16)
    rbi, rpos = R.get_batch_indices_positions(m.qo_indptr, seq, sc.n)
    R.append_paged_kv_cache(k_ref, sc.v, rbi, rpos, ref_pool, m.kv_indices, m.kv_indptr)

    pool, q, k, v = sc.pool.cuda(), sc.q.cuda(), sc.k.cuda(), sc.v.cuda()
    cfg = ops.RopeConfig(mode="table", cos_sin_table=dev(table))
    ops.rope_append_paged_kv_cache(q, k, v, dev(m.pos_ids), dev(rbi), dev(rpos), pool, dev(m.kv_indices),
                                   dev(m.kv_indptr), dev(m.kv_last_page_len), cfg, rotate_k_in_place=True)
    _no_device_error()
    assert torch.equal(pool.cpu().view(torch.uint8), ref_pool.view(torch.uint8))
    assert torch.equal(q.cpu(), q_ref) and torch.equal(k.cpu(), k_ref)
    # without rotate_k_in_place the caller's k stays as it was
    pool2, k2 = sc.pool.cuda(), sc.k.cuda()
    ops.rope_append_paged_kv_cache(None, k2, v, dev(m.pos_ids), dev(rbi), dev(rpos), pool2, dev(m.kv_indices),
                                   dev(m.kv_indptr), dev(m.kv_last_page_len), cfg)
    assert torch.equal(pool2, pool) and torch.equal(k2.cpu(), sc.k)


def test_fused_rope_append_on_the_fly_within_one_ulp():
    sc = make_scenario(32, 8, 128, torch.bfloat16, [(511, 1), (4095, 1), (2048, 4)], seed=6, scale=0.5)
    m = sc.meta
    inv = R.rope_inv_freq(128, 500000.0, "llama31", 8.0)
    c, s = R.rope_cos_sin(m.pos_ids, inv)
    k_ref = R.apply_rope(sc.k, c, s)
    ref_pool = sc.pool.clone()
    seq = R.get_seq_lens(m.kv_indptr, m.kv_last_page_len, 16)
    rbi, rpos = R.get_batch_indices_positions(m.qo_indptr, seq, sc.n)
    R.append_paged_kv_cache(k_ref, sc.v, rbi, rpos, ref_pool, m.kv_indices, m.kv_indptr)
    pool = sc.pool.cuda()
    ops.rope_append_paged_kv_cache(sc.q.cuda(), sc.k.cuda(), sc.v.cuda(), dev(m.pos_ids), dev(rbi), dev(rpos), pool,
                                   dev(m.kv_indices), dev(m.kv_indptr), dev(m.kv_last_page_len), ops.RopeConfig())
    assert ulp_diff_bf16(pool.cpu(), ref_pool) <= 1
    # V halves and untouched pages are bit-exact
    assert torch.equal(pool.cpu()[:, 1], ref_pool[:, 1])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_copy_pages(dtype):
    layers = [W.randn((12, 2, 16, 8, 128), 30 + i, dtype) for i in range(3)]
    ref = [x.clone() for x in layers]
    src, dst, valid = [0, 5, 7, 3], [1, 6, 8, 3], [8, 16, 1, 4]
    R.copy_pages(ref, src, dst, valid)
    gl = [x.cuda() for x in layers]
    ops.copy_kv_pages(gl, dev(np.array(src, np.int32)), dev(np.array(dst, np.int32)), dev(np.array(valid, np.int32)))
    _no_device_error()
    for a, b in zip(gl, ref):
        assert torch.equal(a.cpu().view(torch.uint8), b.view(torch.uint8))
    # whole pages when valid_len is omitted
    ops.copy_kv_pages(gl[0], dev(np.array([2], np.int32)), dev(np.array([9], np.int32)))
    assert torch.equal(gl[0][9], gl[0][2])
