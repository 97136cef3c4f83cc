"""The QKV projection with RoPE + append as its epilogue (`ops.qkv_rope_append_paged_kv_cache`) against the
oracle's restatement of the reference sequence linear -> split -> RoPE -> append
(pie/src/pie_worker/model/llama3.py:627-685).

The fused kernel keeps the projection in fp32 until after the rotation (one rounding); the reference rounds
the projection to the activation type first and once more after the rotation.  The oracle below is evaluated
both ways: the kernel has to be within one rounding step of the single-rounding form and within two of the
reference's."""
import numpy as np
import pytest
import torch

from oracle import paged_kv_ref as R
from pie_b200 import ops
from pie_b200 import workloads as W
from util import dev

pytestmark = pytest.mark.gpu

# One rounding step of bf16 is 2^-8 of the value (2^-7 at the low end of a binade); a rotated element is a
# difference of products, so fp32 summation order (tensor core vs CPU) moves it by up to ~1e-6 of its
# OPERANDS, which for a result that nearly cancels is more than a step of the result: hence the absolute term,
# a step of a typical element (the projections have unit variance here).
STEP = 2.0 ** -7


def within(a, b, steps, floor=0.5):
    a, b = a.float(), b.float()
    return bool(((a - b).abs() <= steps * STEP * (b.abs() + floor)).all())


# Against the reference's order (projection rounded to the storage type BEFORE the rotation) the bound is set
# by the operands, not the result: rounding an operand of magnitude ~3 moves it by up to 2^-9 * 3, and a
# rotated element that nearly cancels inherits that in full.
OPERAND = 3.0


def _case(n_req, hq, hkv, hidden, seed, dtype=torch.bfloat16, num_pages=256):
    d = 128
    rng = np.random.default_rng(seed)
    ctx_new = [(int(rng.integers(0, 70)), int(rng.integers(1, 90))) for _ in range(n_req)]
    reqs = W.PagedRequests(W.seeded_perm(num_pages, seed), 16)
    qo, pos = [0], []
    for c, m in ctx_new:
        r = reqs.add(c, reserve=m)
        reqs.tokens[r] = c + m
        qo.append(qo[-1] + m)
        pos.extend(range(c, c + m))
    idx, ptr, last = reqs.csr()
    n = qo[-1]
    seq = R.get_seq_lens(ptr, last, 16)
    bi, kp = R.get_batch_indices_positions(np.array(qo, np.int32), seq, n)
    x = W.randn((n, hidden), seed + 1, dtype, 1.0)
    w = W.randn(((hq + 2 * hkv) * d, hidden), seed + 2, dtype, hidden ** -0.5)
    pool = W.randn((num_pages, 2, 16, hkv, d), seed + 3, dtype, 0.5)
    return dict(n=n, hq=hq, hkv=hkv, d=d, x=x, w=w, pool=pool, idx=idx, ptr=ptr, last=last,
                pos=np.array(pos, np.int32), bi=bi, kp=kp)


def _oracle(c, table, round_projection, bias=None, q_norm=None, k_norm=None, eps=1e-6):
    """(q rows, pool) of the reference sequence on the CPU; `round_projection` rounds the projection to the
    storage type before the rotation, as the reference does.  `bias`: qwen2.py:596-603; `q_norm` / `k_norm`:
    the per-head RMSNorm of qwen3.py:651-662."""
    n, hq, hkv, d = c["n"], c["hq"], c["hkv"], c["d"]
    qkv = c["x"].float() @ c["w"].float().t()
    if bias is not None:
        qkv = qkv + bias.float()
    if round_projection:
        qkv = qkv.to(c["x"].dtype).float()
    q = qkv[:, : hq * d].reshape(n, hq, d)
    k = qkv[:, hq * d: (hq + hkv) * d].reshape(n, hkv, d)
    v = qkv[:, (hq + hkv) * d:].reshape(n, hkv, d)

    def rms(t, w):
        t = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w.float()
        return t.to(c["x"].dtype).float() if round_projection else t

    if q_norm is not None:
        q = rms(q, q_norm)
    if k_norm is not None:
        k = rms(k, k_norm)
    cs, sn = table[c["pos"], :64], table[c["pos"], 64:]
    q = R.apply_rope(q, cs, sn).to(c["x"].dtype)   # float32 in: one rounding at the end
    k = R.apply_rope(k, cs, sn).to(c["x"].dtype)
    pool = c["pool"].clone()
    R.append_paged_kv_cache(k, v.to(c["x"].dtype), c["bi"], c["kp"], pool, c["idx"], c["ptr"], c["last"])
    return q, pool


@pytest.mark.parametrize("n_req,hq,hkv,hidden", [(5, 8, 2, 256), (3, 32, 8, 1024), (1, 4, 4, 64), (9, 16, 2, 4096)])
def test_qkv_rope_append_against_the_oracle(n_req, hq, hkv, hidden):
    c = _case(n_req, hq, hkv, hidden, seed=7 + hq)
    inv = R.rope_inv_freq(128, 500000.0, "llama31", 8.0)
    table = R.make_cos_sin_table(256, inv)
    pool_gpu = c["pool"].cuda()
    rope = ops.RopeConfig(mode="table", cos_sin_table=dev(table))
    q = ops.qkv_rope_append_paged_kv_cache(c["x"].cuda(), c["w"].cuda(), dev(c["pos"]), dev(c["bi"]), dev(c["kp"]),
                                           pool_gpu, dev(c["idx"]), dev(c["ptr"]), hq, hkv, rope=rope)
    torch.cuda.synchronize()
    assert ops.device_error("cuda") is None
    q1, pool1 = _oracle(c, table, round_projection=False)
    q2, pool2 = _oracle(c, table, round_projection=True)
    assert within(q.cpu(), q1, 1) and within(pool_gpu.cpu(), pool1, 1)
    assert within(q.cpu(), q2, 2, OPERAND) and within(pool_gpu.cpu(), pool2, 2, OPERAND)
    # and most elements are the single-rounding oracle's bit for bit (the rest sit next to a rounding boundary,
    # where the fp32 summation order of a long dot product decides)
    assert (q.cpu() == q1).float().mean().item() > 0.9
    # rows the step did not write are untouched
    untouched = torch.ones(c["pool"].shape[:3], dtype=torch.bool)
    for t in range(c["n"]):
        b, pos = int(c["bi"][t]), int(c["kp"][t])
        page = int(c["idx"][c["ptr"][b] + pos // 16])
        untouched[page, :, pos % 16] = False
    assert torch.equal(pool_gpu.cpu()[untouched].view(torch.int16), c["pool"][untouched].view(torch.int16))


@pytest.mark.parametrize("family", ["qwen2 (bias)", "qwen3 (q / k norm)", "both"])
def test_qkv_rope_append_with_bias_and_per_head_norm(family):
    c = _case(4, 16, 4, 512, seed=21)
    inv = R.rope_inv_freq(128, 1000000.0, "plain", 1.0)
    table = R.make_cos_sin_table(256, inv)
    bias = W.randn(((16 + 8) * 128,), 31, torch.bfloat16, 0.5) if family != "qwen3 (q / k norm)" else None
    qn = (1.0 + W.randn((128,), 32, torch.bfloat16, 0.2)) if family != "qwen2 (bias)" else None
    kn = (1.0 + W.randn((128,), 33, torch.bfloat16, 0.2)) if family != "qwen2 (bias)" else None
    pool_gpu = c["pool"].cuda()
    rope = ops.RopeConfig(mode="table", cos_sin_table=dev(table))
    q = ops.qkv_rope_append_paged_kv_cache(
        c["x"].cuda(), c["w"].cuda(), dev(c["pos"]), dev(c["bi"]), dev(c["kp"]), pool_gpu, dev(c["idx"]),
        dev(c["ptr"]), 16, 4, rope=rope, bias=None if bias is None else bias.cuda(),
        q_norm_weight=None if qn is None else qn.cuda(), k_norm_weight=None if kn is None else kn.cuda(),
        rms_norm_eps=1e-6)
    torch.cuda.synchronize()
    assert ops.device_error("cuda") is None
    q1, pool1 = _oracle(c, table, False, bias, qn, kn)
    q2, pool2 = _oracle(c, table, True, bias, qn, kn)
    assert within(q.cpu(), q1, 1) and within(pool_gpu.cpu(), pool1, 1)
    assert within(q.cpu(), q2, 3, OPERAND) and within(pool_gpu.cpu(), pool2, 3, OPERAND)
    assert not within(q.cpu(), _oracle(c, table, False)[0], 1)  # the options do something


def test_qkv_rope_append_equals_the_separate_kernels_on_a_rounded_projection():
    """Same inputs through torch's matmul + `rope_append_paged_kv_cache` (projection rounded to bf16 in between):
    within two rounding steps; and without a rotation the appended v rows are within one."""
    c = _case(4, 32, 8, 512, seed=99)
    inv = R.rope_inv_freq(128, 500000.0, "llama31", 8.0)
    table = dev(R.make_cos_sin_table(256, inv))
    rope = ops.RopeConfig(mode="table", cos_sin_table=table)
    x, w = c["x"].cuda(), c["w"].cuda()
    pool_a, pool_b = c["pool"].cuda(), c["pool"].cuda()
    args = (dev(c["pos"]), dev(c["bi"]), dev(c["kp"]))
    q_a = ops.qkv_rope_append_paged_kv_cache(x, w, *args, pool_a, dev(c["idx"]), dev(c["ptr"]), 32, 8, rope=rope)
    qkv = torch.nn.functional.linear(x, w)
    q_b, k_b, v_b = (t.reshape(c["n"], -1, 128) for t in qkv.split([32 * 128, 8 * 128, 8 * 128], dim=-1))
    ops.rope_append_paged_kv_cache(q_b, k_b, v_b, args[0], args[1], args[2], pool_b, dev(c["idx"]), dev(c["ptr"]),
                                   dev(c["last"]), rope)
    torch.cuda.synchronize()
    assert ops.device_error("cuda") is None
    assert within(q_a.cpu(), q_b.contiguous().cpu(), 2, OPERAND)
    assert within(pool_a.cpu(), pool_b.cpu(), 2, OPERAND)


def test_qkv_rope_append_rejects_what_it_cannot_do():
    c = _case(2, 8, 2, 256, seed=3)
    pool = c["pool"].cuda()
    args = (dev(c["pos"]), dev(c["bi"]), dev(c["kp"]), pool, dev(c["idx"]), dev(c["ptr"]), 8, 2)
    with pytest.raises(ValueError):
        ops.qkv_rope_append_paged_kv_cache(c["x"].cuda()[:, :200], c["w"].cuda()[:, :200], *args)  # not rows of 64
    with pytest.raises(ValueError):
        ops.qkv_rope_append_paged_kv_cache(c["x"].cuda(), c["w"].cuda()[:-128], *args)
    with pytest.raises(ValueError):
        ops.qkv_rope_append_paged_kv_cache(c["x"].cuda(), c["w"].cuda(), *args, rope=ops.RopeConfig(interleave=True))
