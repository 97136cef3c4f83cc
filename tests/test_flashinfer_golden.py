"""Parity against outputs of the reference's CUDA dependency (FlashInfer), recorded on a B200 by
tests/golden/make_flashinfer_golden.py from the same seeded inputs that tests.util.make_scenario builds.
CPU part: the oracle against those outputs.  GPU part: this library against them."""
import hashlib
import importlib.util
import os

import numpy as np
import pytest
import torch

from oracle import paged_kv_ref as R
from tests.util import dev, make_scenario

HERE = os.path.dirname(__file__)
Z = np.load(os.path.join(HERE, "golden", "flashinfer_outputs.npz"))
_spec = importlib.util.spec_from_file_location("mkgold", os.path.join(HERE, "golden", "make_flashinfer_golden.py"))
_mk = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_mk)
CASES = _mk.CASES


def _t(name, key, dtype, shape):
    a = Z[f"{name}/{key}"]
    t = torch.from_numpy(a.copy())
    return t.view(dtype).reshape(shape)


def _scenario(name):
    hq, hkv, d, dtype, reqs, seed, rope = CASES[name]
    return make_scenario(hq, hkv, d, dtype, reqs, seed=seed, scale=0.5), reqs, rope


def _rope_close(a, b, src, frac=1e-2):
    """Rotated tensors agree to one rounding step of the storage type at the magnitude of the rotated pair
    (a result that nearly cancels is small, but its error is set by its inputs), and differ in few places.
    The dependency evaluates sin / cos with fast intrinsics, so single steps do differ."""
    d = src.shape[-1]
    mag = torch.hypot(src[..., : d // 2].float(), src[..., d // 2:].float())  # bound of the rotated values
    mag = torch.cat([mag, mag], dim=-1)
    step = 2.0 ** -7 if src.dtype == torch.bfloat16 else 2.0 ** -10
    assert ((a.float() - b.float()).abs() <= step * mag + 1e-7).all()
    assert (a != b).float().mean().item() <= frac


def _mask_of(m):
    total = int(np.sum(np.diff(m.qo_indptr).astype(np.int64) * m.seq_lens))
    mask = np.zeros(total, dtype=np.bool_)
    off = 0
    for b in range(m.batch):
        qn, kv = int(m.qo_indptr[b + 1] - m.qo_indptr[b]), int(m.seq_lens[b])
        for j in range(qn):
            mask[off + j * kv: off + j * kv + kv - qn + j + 1] = True
        off += qn * kv
    return mask


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_against_dependency_outputs(name):
    sc, reqs, (rmode, theta) = _scenario(name)
    m = sc.meta
    assert str(Z["flashinfer_version"]).startswith("0.6")
    seq = R.get_seq_lens(m.kv_indptr, m.kv_last_page_len, 16)
    bi, kp = R.get_batch_indices_positions(m.qo_indptr, seq, sc.n)
    assert np.array_equal(seq, Z[f"{name}/seq_lens"])
    assert np.array_equal(bi, Z[f"{name}/batch_indices"]) and np.array_equal(kp, Z[f"{name}/positions"])
    inv = R.rope_inv_freq(sc.d, theta, rmode, 8.0 if rmode == "llama31" else 1.0)
    c, s = R.rope_cos_sin(m.pos_ids, inv)
    q_rot, k_rot = R.apply_rope(sc.q, c, s), R.apply_rope(sc.k, c, s)
    gq, gk = _t(name, "q_rot", sc.dtype, sc.q.shape), _t(name, "k_rot", sc.dtype, sc.k.shape)
    _rope_close(q_rot, gq, sc.q)
    _rope_close(k_rot, gk, sc.k)
    # append: take the dependency's rotated k so that the page comparison is about data movement only
    pool = sc.pool.clone()
    R.append_paged_kv_cache(gk, sc.v, bi, kp, pool, m.kv_indices, m.kv_indptr)
    ids = torch.from_numpy(Z[f"{name}/pool_touched_ids"].astype(np.int64))
    touched = _t(name, "pool_touched", sc.dtype, (len(ids),) + tuple(pool.shape[1:]))
    assert torch.equal(pool[ids].view(torch.int16), touched.view(torch.int16))
    digest = hashlib.sha256(pool.view(torch.int16).numpy().tobytes()).hexdigest()
    assert digest == str(Z[f"{name}/pool_sha256"])  # bit-exact pool, untouched pages included
    # attention on the dependency's q / pool
    if f"{name}/decode_out" in Z.files:
        ref = R.decode_attention(gq, pool, m.kv_indptr, m.kv_indices, m.kv_last_page_len)
        got = _t(name, "decode_out", sc.dtype, sc.q.shape)
        assert (ref.float() - got.float()).abs().max().item() <= 2e-2
    ref = R.prefill_attention(gq, pool, m.qo_indptr, m.kv_indptr, m.kv_indices, m.kv_last_page_len,
                              custom_mask=_mask_of(m))
    got = _t(name, "prefill_masked_out", sc.dtype, sc.q.shape)
    assert (ref.float() - got.float()).abs().max().item() <= 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_library_against_dependency_outputs(name):
    from pie_b200 import ops

    sc, reqs, (rmode, theta) = _scenario(name)
    m = sc.meta
    q, k, v, pool = sc.q.cuda(), sc.k.cuda(), sc.v.cuda(), sc.pool.cuda()
    indptr, indices, last, qo, pos_ids = dev(m.kv_indptr), dev(m.kv_indices), dev(m.kv_last_page_len), \
        dev(m.qo_indptr), dev(m.pos_ids)
    seq = ops.get_seq_lens(indptr, last, 16)
    bi, kp = ops.get_batch_indices_positions(qo, seq, sc.n)
    assert np.array_equal(seq.cpu().numpy(), Z[f"{name}/seq_lens"])
    assert np.array_equal(bi.cpu().numpy(), Z[f"{name}/batch_indices"])
    assert np.array_equal(kp.cpu().numpy(), Z[f"{name}/positions"])
    if rmode == "llama31":
        ops.apply_llama31_rope_pos_ids_inplace(q=q, k=k, pos_ids=pos_ids, rope_scale=8.0, rope_theta=theta,
                                               low_freq_factor=1.0, high_freq_factor=4.0, old_context_len=8192)
    else:
        ops.apply_rope_pos_ids_inplace(q=q, k=k, pos_ids=pos_ids, rope_theta=theta)
    gq, gk = _t(name, "q_rot", sc.dtype, sc.q.shape), _t(name, "k_rot", sc.dtype, sc.k.shape)
    _rope_close(q.cpu(), gq, sc.q)
    _rope_close(k.cpu(), gk, sc.k)
    ops.append_paged_kv_cache(gk.cuda(), v, bi, kp, pool, indices, indptr, last, "NHD")
    digest = hashlib.sha256(pool.cpu().view(torch.int16).numpy().tobytes()).hexdigest()
    assert digest == str(Z[f"{name}/pool_sha256"])
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
    if f"{name}/decode_out" in Z.files:
        w = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
        w.plan(indptr, indices, last, sc.hq, sc.hkv, sc.d, 16, pos_encoding_mode="NONE", q_data_type=sc.dtype)
        out = w.run(gq.cuda(), pool)
        got = _t(name, "decode_out", sc.dtype, sc.q.shape)
        assert (out.cpu().float() - got.float()).abs().max().item() <= 2e-2
    wp = ops.BatchPrefillWithPagedKVCacheWrapper(ws, "NHD")
    wp.plan(qo, indptr, indices, last, sc.hq, sc.hkv, sc.d, 16, custom_mask=dev(_mask_of(m)), q_data_type=sc.dtype)
    out = wp.run(gq.cuda(), pool)
    got = _t(name, "prefill_masked_out", sc.dtype, sc.q.shape)
    assert (out.cpu().float() - got.float()).abs().max().item() <= 2e-2
    assert ops.device_error("cuda") is None


@pytest.mark.gpu
def test_library_against_the_dependency_run_live():
    """When the reference's CUDA dependency is importable on this machine, run the reference's call sequence
    (pie/src/pie_worker/model/llama3.py:660-689,745-777) live on a config-2-shaped batch and compare this
    library's results on the same inputs: metadata exact, appended pool bit-exact, decode outputs within 2e-2.
    The dependency is only called, never read."""
    try:
        import flashinfer
    except Exception as e:  # not installed, or not importable without its build tools
        pytest.skip(f"flashinfer is not importable here: {type(e).__name__}")
    from pie_b200 import ops
    from pie_b200 import workloads as W

    hq, hkv, d, batch, pages = 32, 8, 128, 64, 16384
    dt = torch.bfloat16
    reqs = W.config2_requests(batch=batch, lo=512, hi=2048, seed=1, num_pages=pages)
    m = W.decode_steps(reqs, 1)[0]
    pool = W.randn((pages, 2, 16, hkv, d), 61, dt, 0.5, device="cuda")
    q = W.randn((batch, hq, d), 62, dt, 0.5, device="cuda")
    k = W.randn((batch, hkv, d), 63, dt, 0.5, device="cuda")
    v = W.randn((batch, hkv, d), 64, dt, 0.5, device="cuda")
    indptr, indices, last, qo, pos_ids = dev(m.kv_indptr), dev(m.kv_indices), dev(m.kv_last_page_len), \
        dev(m.qo_indptr), dev(m.pos_ids)
    ws_f = torch.zeros(128 << 20, dtype=torch.uint8, device="cuda")
    try:
        fq, fk, fpool = q.clone(), k.clone(), pool.clone()
        fseq = flashinfer.get_seq_lens(indptr, last, 16)
        fbi, fkp = flashinfer.get_batch_indices_positions(qo, fseq, batch)
        flashinfer.apply_llama31_rope_pos_ids_inplace(q=fq, k=fk, pos_ids=pos_ids, rope_scale=8.0, rope_theta=5e5,
                                                      low_freq_factor=1.0, high_freq_factor=4.0, old_context_len=8192)
        flashinfer.append_paged_kv_cache(append_key=fk, append_value=v, batch_indices=fbi, positions=fkp,
                                         paged_kv_cache=fpool, kv_indices=indices, kv_indptr=indptr,
                                         kv_last_page_len=last, kv_layout="NHD")
        fw = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws_f, "NHD")
        fw.plan(indptr=indptr, indices=indices, last_page_len=last, num_qo_heads=hq, num_kv_heads=hkv, head_dim=d,
                page_size=16, pos_encoding_mode="NONE", q_data_type=dt)
        fout = fw.run(fq, fpool)
        torch.cuda.synchronize()
    except Exception as e:  # e.g. no compiler for its kernels on this machine
        pytest.skip(f"flashinfer could not run here: {type(e).__name__}: {str(e)[:120]}")
    seq = ops.get_seq_lens(indptr, last, 16)
    bi, kp = ops.get_batch_indices_positions(qo, seq, batch)
    assert torch.equal(seq, fseq.to(seq.dtype)) and torch.equal(bi, fbi.to(bi.dtype)) and torch.equal(kp, fkp.to(kp.dtype))
    mq, mk = q.clone(), k.clone()
    ops.apply_llama31_rope_pos_ids_inplace(mq, mk, pos_ids)
    _rope_close(mq.cpu(), fq.cpu(), q.cpu())
    _rope_close(mk.cpu(), fk.cpu(), k.cpu())
    mpool = pool.clone()
    ops.append_paged_kv_cache(fk, v, bi, kp, mpool, indices, indptr, last)  # the dependency's k: data movement only
    assert torch.equal(mpool.view(torch.int16), fpool.view(torch.int16))
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
    w = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    w.plan(indptr, indices, last, hq, hkv, d, 16, q_data_type=dt)
    out = w.run(fq, fpool)
    assert (out.float() - fout.float()).abs().max().item() <= 2e-2
    # and the fused step against the dependency's three separate ops
    fused = w.run_fused(q, k, v, pos_ids, pool.clone(), ops.RopeConfig())
    assert (fused.float() - fout.float()).abs().max().item() <= 2e-2
    assert ops.device_error("cuda") is None
