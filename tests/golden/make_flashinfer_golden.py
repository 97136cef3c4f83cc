"""Generate golden outputs of the reference's CUDA dependency (FlashInfer) on a GPU box.

Pie's worker calls `flashinfer` for this path on NVIDIA GPUs (pie/src/pie_worker/model/llama3.py:18-21,
293-313,660-689,745-791).  This script runs exactly those calls on seeded inputs (tests.util.make_scenario,
reproducible on any machine) and stores what they return, so that the parity tests can compare this
library against the dependency's own results without having it installed:

    python tests/golden/make_flashinfer_golden.py  [output.npz]

It needs a CUDA GPU and an importable `flashinfer` (it may compile its kernels on first use).  The
installed version is recorded in the file (the reference pins 0.6.1, pie/uv.lock:323-324).
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from tests.util import make_scenario  # noqa: E402

CASES = {
    # name: (hq, hkv, d, dtype, [(context, new tokens)], seed, rope)
    # the dependency dispatches its RoPE and append kernels on 16-bit types only (float32 is rejected with
    # "failed to dispatch data type"), so config 1's shapes are pinned in fp16
    "config1_shape_fp16": (4, 2, 64, torch.float16, [(37, 1), (64, 1), (100, 1), (5, 1)], 0, ("plain", 10000.0)),
    "decode_bf16": (32, 8, 128, torch.bfloat16, [(36, 1), (640, 1), (999, 1), (15, 1), (2048, 1)], 1,
                    ("llama31", 500000.0)),
    "chunk_bf16": (32, 8, 128, torch.bfloat16, [(0, 40), (100, 1), (15, 2), (16, 16), (200, 130)], 2,
                   ("llama31", 500000.0)),
}


def bits(t):
    t = t.detach().cpu().contiguous()
    return t.view(torch.int16).numpy() if t.element_size() == 2 else t.view(torch.int32).numpy()


def compact(res):
    """Keep the fixture small: of every pool only the pages that received new tokens, plus a SHA-256 of
    the whole pool (the parity test checks the untouched rest through the digest)."""
    import hashlib

    out = {}
    for key, val in res.items():
        if not key.endswith("/pool"):
            out[key] = val
            continue
        name = key.split("/")[0]
        hq, hkv, d, dtype, reqs, seed, _ = CASES[name]
        sc = make_scenario(hq, hkv, d, dtype, reqs, seed=seed, scale=0.5)
        m = sc.meta
        touched = set()
        for b, (ctx, new) in enumerate(reqs):
            for tok in range(ctx, ctx + new):
                touched.add(int(m.kv_indices[m.kv_indptr[b] + tok // 16]))
        ids = np.array(sorted(touched), dtype=np.int32)
        out[f"{name}/pool_touched_ids"] = ids
        out[f"{name}/pool_touched"] = val[ids]
        out[f"{name}/pool_sha256"] = np.array(hashlib.sha256(np.ascontiguousarray(val).tobytes()).hexdigest())
    return out


def main():
    import flashinfer

    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(__file__), "flashinfer_outputs.npz")
    dev = torch.device("cuda")
    res = {"flashinfer_version": np.array(flashinfer.__version__)}
    ws = torch.zeros(128 << 20, dtype=torch.uint8, device=dev)
    for name, (hq, hkv, d, dtype, reqs, seed, (rmode, theta)) in CASES.items():
        sc = make_scenario(hq, hkv, d, dtype, reqs, seed=seed, scale=0.5)
        m = sc.meta
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        q, k, v, pool = sc.q.to(dev), sc.k.to(dev), sc.v.to(dev), sc.pool.to(dev)
        indptr, indices, last, qo, pos_ids = t(m.kv_indptr), t(m.kv_indices), t(m.kv_last_page_len), t(m.qo_indptr), \
            t(m.pos_ids)
        seq = flashinfer.get_seq_lens(indptr, last, 16)
        bi, kp = flashinfer.get_batch_indices_positions(qo, seq, sc.n)
        if rmode == "llama31":
            flashinfer.apply_llama31_rope_pos_ids_inplace(q=q, k=k, pos_ids=pos_ids, rope_scale=8.0, rope_theta=theta,
                                                          low_freq_factor=1.0, high_freq_factor=4.0,
                                                          old_context_len=8192)
        elif rmode == "plain":
            flashinfer.apply_rope_pos_ids_inplace(q=q, k=k, pos_ids=pos_ids, rope_theta=theta)
        flashinfer.append_paged_kv_cache(append_key=k, append_value=v, batch_indices=bi, positions=kp,
                                         paged_kv_cache=pool, kv_indices=indices, kv_indptr=indptr,
                                         kv_last_page_len=last, kv_layout="NHD")
        res[f"{name}/seq_lens"] = seq.cpu().numpy()
        res[f"{name}/batch_indices"] = bi.cpu().numpy()
        res[f"{name}/positions"] = kp.cpu().numpy()
        res[f"{name}/q_rot"] = bits(q)
        res[f"{name}/k_rot"] = bits(k)
        res[f"{name}/pool"] = bits(pool)
        single = all(n == 1 for _, n in reqs)
        if single:
            try:
                w = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
                w.plan(indptr=indptr, indices=indices, last_page_len=last, num_qo_heads=hq, num_kv_heads=hkv,
                       head_dim=d, page_size=16, pos_encoding_mode="NONE", q_data_type=dtype)
                res[f"{name}/decode_out"] = bits(w.run(q, pool))
            except Exception as e:  # a dtype the dependency does not build
                print("decode unavailable for", name, type(e).__name__, str(e)[:200], flush=True)
        # prefill wrapper with the causal mask expanded the way the reference's Batch does
        total = int(np.sum(np.diff(m.qo_indptr).astype(np.int64) * m.seq_lens))
        mask = np.zeros(total, dtype=np.bool_)
        off = 0
        for b in range(m.batch):
            qn, kv = int(m.qo_indptr[b + 1] - m.qo_indptr[b]), int(m.seq_lens[b])
            for j in range(qn):
                mask[off + j * kv: off + j * kv + kv - qn + j + 1] = True
            off += qn * kv
        try:
            wp = flashinfer.BatchPrefillWithPagedKVCacheWrapper(ws, "NHD")
            wp.plan(qo_indptr=qo, paged_kv_indptr=indptr, paged_kv_indices=indices, paged_kv_last_page_len=last,
                    num_qo_heads=hq, num_kv_heads=hkv, head_dim_qk=d, page_size=16, custom_mask=t(mask),
                    q_data_type=dtype)
            res[f"{name}/prefill_masked_out"] = bits(wp.run(q, pool))
        except Exception as e:
            print("prefill unavailable for", name, type(e).__name__, str(e)[:200], flush=True)
        torch.cuda.synchronize()
        print("done", name, flush=True)
    np.savez_compressed(out_path, **compact(res))
    print("wrote", out_path, os.path.getsize(out_path))


if __name__ == "__main__":
    main()
