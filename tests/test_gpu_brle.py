"""Device-side BRLE -> bit mask (piekv_prefill_plan_brle) against the reference's own host expansion.

The golden fixtures hold, for eight batches, the wire fields and the flat boolean mask that the
reference's `pie_worker.batching.Batch` derived from them (tests/golden/make_golden.py).  The same
attention kernel is run twice, once planned from that golden flat mask and once planned from the run
lengths on the device: every output element must be identical, and both must match the CPU oracle.
A fuzz case adds rows with more than 64 runs, zero-length runs and runs past the valid length."""
import os

import numpy as np
import pytest
import torch

from oracle import paged_kv_ref as R
from pie_b200 import ops
from pie_b200 import workloads as W
from pie_b200.batching import Batch, decode_brle_batch
from tests.util import dev

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden", "reference_batch_masks.npz")


def _golden_names():
    z = np.load(GOLD)
    return sorted({k.split("/")[0] for k in z.files})


def _golden_args(z, name):
    g = lambda k: z[f"{name}/in/{k}"]
    n = int(g("qo_indptr")[-1])
    u = lambda a: np.asarray(a, dtype=np.uint32).tobytes()
    return {
        "token_ids": u(np.arange(n)), "position_ids": u(g("position_ids")),
        "kv_page_indices": u(g("kv_page_indices")), "kv_page_indptr": u(g("kv_page_indptr")),
        "kv_last_page_lens": u(g("kv_last_page_lens")), "qo_indptr": u(g("qo_indptr")),
        "flattened_masks": u(g("flattened_masks")), "mask_indptr": u(g("mask_indptr")),
        "single_token_mode": False,
    }


def _both_ways(batch: Batch, flat_mask: np.ndarray, hq: int, hkv: int, seed: int):
    """Outputs of the prefill wrapper planned from the flat mask and from the runs, plus the oracle's."""
    dtype = torch.bfloat16
    num_pages = int(batch.kv_page_indices.max()) + 2 if batch.kv_page_indices.size else 2
    pool = W.randn((num_pages, 2, 16, hkv, 128), seed, dtype, 0.5)
    n = batch.total_tokens
    q = W.randn((n, hq, 128), seed + 1, dtype, 0.5)
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
    common = dict(num_qo_heads=hq, num_kv_heads=hkv, head_dim_qk=128, page_size=16, q_data_type=dtype)
    meta = (dev(batch.qo_indptr), dev(batch.kv_page_indptr), dev(batch.kv_page_indices), dev(batch.kv_last_page_lens))
    gq, gpool = q.cuda(), pool.cuda()

    w = ops.BatchPrefillWithPagedKVCacheWrapper(ws, "NHD")
    w.plan(*meta, custom_mask=torch.from_numpy(flat_mask).cuda(), **common)
    out_flat = w.run(gq, gpool).clone()

    w2 = ops.BatchPrefillWithPagedKVCacheWrapper(ws, "NHD")
    w2.plan(*meta, brle_mask=batch.brle_inputs("cuda"), **common)
    out_brle = w2.run(gq, gpool).clone()
    assert ops.device_error("cuda") is None

    ref = R.prefill_attention(q, pool, batch.qo_indptr, batch.kv_page_indptr, batch.kv_page_indices,
                              batch.kv_last_page_lens, custom_mask=flat_mask, causal=False)
    return out_flat.cpu(), out_brle.cpu(), ref


@pytest.mark.parametrize("heads", [(4, 2), (3, 3)])  # even GQA group: two-head kernel; odd: one-head kernel
@pytest.mark.parametrize("name", _golden_names())
def test_brle_plan_matches_reference_mask(name, heads):
    z = np.load(GOLD)
    if int(z[f"{name}/in/page_size"]) != 16:
        pytest.skip("the tensor-core path has page size 16")
    batch = Batch(_golden_args(z, name), 16)
    gold = z[f"{name}/out/mask"]
    assert np.array_equal(batch.attention_masks, gold)  # the host mirror, for completeness
    out_flat, out_brle, ref = _both_ways(batch, gold, heads[0], heads[1], seed=11)
    assert torch.equal(out_flat, out_brle), name
    assert (out_brle.float() - ref.float()).abs().max().item() <= 2e-2


def test_brle_plan_fuzz_long_rows_and_odd_runs():
    rng = np.random.default_rng(5)
    page_size = 16
    qo = [37, 1, 130, 5]
    kv = [300, 17, 641, 5]          # last request: empty context; request 1: a decode-like row
    qo_indptr = np.concatenate([[0], np.cumsum(qo)]).astype(np.int32)
    npages = [-(-k // page_size) for k in kv]
    kv_indptr = np.concatenate([[0], np.cumsum(npages)]).astype(np.int32)
    perm = rng.permutation(int(kv_indptr[-1]) + 7).astype(np.int32)
    kv_indices = perm[: int(kv_indptr[-1])]
    last = np.array([(k - 1) % page_size + 1 for k in kv], dtype=np.int32)
    runs, ptr = [], [0]
    for b in range(len(qo)):
        for j in range(qo[b]):
            kind = rng.integers(0, 5)
            if kind == 0:      # plain causal: one attend run covering everything
                r = [kv[b] + 5]
            elif kind == 1:    # many short runs, more than 64 of them
                r = list(rng.integers(0, 6, size=int(rng.integers(65, 140))))
            elif kind == 2:    # starts with a zero-length attend run (i.e. with a skip)
                r = [0, int(rng.integers(1, 40)), int(rng.integers(1, 400))]
            elif kind == 3:    # nothing allowed
                r = []
            else:              # a few long runs that overshoot the row
                r = list(rng.integers(1, 300, size=int(rng.integers(1, 6))))
            runs += [int(x) for x in r]
            ptr.append(len(runs))
    pos = np.concatenate([np.arange(kv[b] - qo[b], kv[b]) for b in range(len(qo))])
    args = {
        "token_ids": list(range(int(qo_indptr[-1]))), "position_ids": [int(p) for p in pos],
        "kv_page_indices": kv_indices.tolist(), "kv_page_indptr": kv_indptr.tolist(),
        "kv_last_page_lens": last.tolist(), "qo_indptr": qo_indptr.tolist(),
        "flattened_masks": runs, "mask_indptr": ptr, "single_token_mode": False,
    }
    batch = Batch(args, page_size)
    flat = batch.attention_masks  # the numpy mirror, itself pinned to the reference's output by the golden test
    out_flat, out_brle, ref = _both_ways(batch, flat, 4, 2, seed=21)
    assert torch.equal(out_flat, out_brle)
    assert (out_brle.float() - ref.float()).abs().max().item() <= 2e-2
    # rows without any allowed key give zeros
    acc = np.concatenate([[0], np.cumsum(np.repeat(kv, qo))])
    empty = [i for i in range(len(acc) - 1) if not flat[acc[i]:acc[i + 1]].any()]
    assert empty and float(out_brle[empty].abs().max()) == 0.0


def test_brle_plan_rejects_what_it_cannot_serve():
    ws = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    w = ops.BatchPrefillWithPagedKVCacheWrapper(ws, "NHD")
    i32 = lambda *a: torch.tensor(a, dtype=torch.int32, device="cuda")
    brle = (i32(3), i32(0, 1), 3)
    with pytest.raises(ValueError):   # fp32 has no tensor-core path
        w.plan(i32(0, 1), i32(0, 1), i32(0), i32(3), 4, 2, 128, 16, brle_mask=brle, q_data_type=torch.float32)
    with pytest.raises(ValueError):   # both mask forms at once
        w.plan(i32(0, 1), i32(0, 1), i32(0), i32(3), 4, 2, 128, 16, brle_mask=brle,
               custom_mask=torch.ones(3, dtype=torch.bool, device="cuda"), q_data_type=torch.bfloat16)
