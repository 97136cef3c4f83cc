"""Generate the golden fixtures of tests/golden/ by running the REFERENCE's own host code.

Run where a checkout of the reference is available (read-only is enough) and name its Python source
directory, the one that holds `pie_worker/`:

    python tests/golden/make_golden.py <reference checkout>/pie/src

It imports `pie_worker.batching.Batch` (pie/src/pie_worker/batching.py) unmodified, feeds it batches in
the wire form (uint32 / float32 byte strings, pie/src/pie_worker/batching.py:61-76) and stores the inputs
together with what the reference derives from them: the flat boolean attention mask and the int32 index
tensors of `get_model_inputs`.  It also records `flashinfer.get_seq_lens` (the CUDA dependency's
sequence-length op, which runs on CPU tensors) for the same page tables.  The parity tests load the
.npz files; nothing at test time reads the reference tree.
"""
import os
import sys

import numpy as np

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("PIE_REFERENCE_SRC", "")
if not os.path.isdir(os.path.join(REF, "pie_worker")):
    raise SystemExit("usage: make_golden.py <reference checkout>/pie/src")
HERE = os.path.dirname(os.path.abspath(__file__))


def u32(x):
    return np.asarray(x, dtype=np.uint32).tobytes()


def f32(x):
    return np.asarray(x, dtype=np.float32).tobytes()


def run_batch(Batch, torch, page_size, qo_indptr, kv_page_indptr, kv_page_indices, kv_last_page_lens,
              flattened_masks, mask_indptr, position_ids, single_token_mode):
    nreq = len(qo_indptr) - 1
    ntok = qo_indptr[-1]
    args = {
        "token_ids": u32(np.arange(ntok)),
        "position_ids": u32(position_ids),
        "kv_page_indices": u32(kv_page_indices),
        "kv_page_indptr": u32(kv_page_indptr),
        "kv_last_page_lens": u32(kv_last_page_lens),
        "qo_indptr": u32(qo_indptr),
        "flattened_masks": u32(flattened_masks),
        "mask_indptr": u32(mask_indptr),
        "single_token_mode": single_token_mode,
        "adapter_indices": [None] * nreq,
        "adapter_seeds": [None] * nreq,
        "sampler_temperatures": f32([]),
        "sampler_top_k": u32([]),
        "sampler_top_p": f32([]),
        "sampler_min_p": f32([]),
        "sampler_types": u32([]),
        "request_num_samplers": u32([0] * nreq),
        "flat_output_token_indices": u32([]),
        "output_token_indptr": u32([0] * (nreq + 1)),
    }
    batch = Batch(args, kv_page_size=page_size, max_dist_size=32000, adapters={})
    inputs = batch.get_model_inputs(torch.device("cpu"))
    return {
        "mask": np.asarray(batch.attention_masks, dtype=np.bool_),
        "out_position_ids": inputs["position_ids"].numpy(),
        "out_qo_indptr": inputs["qo_indptr"].numpy(),
        "out_kv_page_indices": inputs["kv_page_indices"].numpy(),
        "out_kv_page_indptr": inputs["kv_page_indptr"].numpy(),
        "out_kv_last_page_lens": inputs["kv_last_page_lens"].numpy(),
        "total_pages": np.int64(inputs["total_pages_cpu"]),
    }


def random_case(rng, page_size, nreq, max_ctx, max_new, causal_only):
    qo, ptr, idx, last, runs, rptr, pos = [0], [0], [], [], [], [0], []
    next_page = 0
    for _ in range(nreq):
        m = int(rng.integers(1, max_new + 1))
        ctx = int(rng.integers(0, max_ctx + 1))
        total = ctx + m
        npg = -(-total // page_size)
        pages = list(range(next_page, next_page + npg))
        next_page += npg
        idx += pages
        ptr.append(ptr[-1] + npg)
        r = total % page_size
        last.append(page_size if r == 0 else r)
        qo.append(qo[-1] + m)
        for j in range(m):
            pos.append(ctx + j)
            if causal_only:
                tok_runs = [ctx + j + 1]
            else:
                # random alternating runs (first run = attend), possibly longer or shorter than the row
                tok_runs = []
                remaining = total + int(rng.integers(0, 4))
                while remaining > 0:
                    r_ = int(rng.integers(0, min(remaining, 9) + 1))
                    tok_runs.append(r_)
                    remaining -= max(r_, 1)
            runs += tok_runs
            rptr.append(rptr[-1] + len(tok_runs))
    # shuffle physical ids so the table is not the identity
    perm = rng.permutation(next_page)
    idx = [int(perm[p]) for p in idx]
    return dict(qo_indptr=qo, kv_page_indptr=ptr, kv_page_indices=idx, kv_last_page_lens=last,
                flattened_masks=runs, mask_indptr=rptr, position_ids=pos)


def main():
    sys.path.insert(0, REF)
    import torch
    from pie_worker.batching import Batch  # the reference's own code

    cases = {}
    # the reference's unit test (pie/tests/worker/test_flattened_mask.py): expects size 80, 79 ones, bit 31 off
    cases["ref_test_flattened_mask"] = dict(
        page_size=16, qo_indptr=[0, 2, 3], kv_page_indptr=[0, 2, 3], kv_page_indices=[0, 1, 2],
        kv_last_page_lens=[16, 16], flattened_masks=[32, 32, 16], mask_indptr=[0, 1, 2, 3],
        position_ids=[31, 31, 15], single_token_mode=False)
    # a 3-token chunk on a 5-token context + one decode token on 16
    cases["chunk_plus_decode"] = dict(
        page_size=16, qo_indptr=[0, 3, 4], kv_page_indptr=[0, 1, 3], kv_page_indices=[4, 9, 2],
        kv_last_page_lens=[8, 1], flattened_masks=[6, 7, 8, 17], mask_indptr=[0, 1, 2, 3, 4],
        position_ids=[5, 6, 7, 16], single_token_mode=False)
    rng = np.random.default_rng(42)
    for i in range(6):
        c = random_case(rng, page_size=16 if i % 2 == 0 else 4, nreq=int(rng.integers(1, 7)),
                        max_ctx=70, max_new=9, causal_only=(i < 2))
        c["page_size"] = 16 if i % 2 == 0 else 4
        c["single_token_mode"] = False
        cases[f"random_{i}"] = c

    out = {}
    for name, c in cases.items():
        res = run_batch(Batch, torch, **c)
        for k, v in c.items():
            out[f"{name}/in/{k}"] = np.asarray(v)
        for k, v in res.items():
            out[f"{name}/out/{k}"] = v
    np.savez_compressed(os.path.join(HERE, "reference_batch_masks.npz"), **out)

    # sequence lengths from the CUDA dependency's own op (runs on CPU tensors)
    import flashinfer
    sl = {}
    rng = np.random.default_rng(7)
    for i in range(8):
        nreq = int(rng.integers(1, 12))
        npg = rng.integers(0, 9, size=nreq)
        ptr = np.concatenate([[0], np.cumsum(npg)]).astype(np.int32)
        ps = int(rng.choice([1, 4, 16, 32]))
        last = np.where(npg > 0, rng.integers(1, ps + 1, size=nreq), rng.integers(0, 3, size=nreq)).astype(np.int32)
        got = flashinfer.get_seq_lens(torch.from_numpy(ptr), torch.from_numpy(last), ps).numpy()
        sl[f"case_{i}/kv_indptr"] = ptr
        sl[f"case_{i}/kv_last_page_len"] = last
        sl[f"case_{i}/page_size"] = np.int64(ps)
        sl[f"case_{i}/seq_lens"] = got
    sl["flashinfer_version"] = np.array(flashinfer.__version__)
    np.savez_compressed(os.path.join(HERE, "flashinfer_seq_lens.npz"), **sl)
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
