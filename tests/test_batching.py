"""Host feeder mirror (pie_b200.batching) against golden vectors produced by the reference's own
`pie_worker.batching.Batch` (tests/golden/make_golden.py)."""
import os

import numpy as np

from pie_b200.batching import Batch, decode_brle_batch

GOLD = os.path.join(os.path.dirname(__file__), "golden", "reference_batch_masks.npz")


def _args(z, name, as_bytes):
    conv = (lambda a: np.asarray(a, dtype=np.uint32).tobytes()) if as_bytes else (lambda a: list(map(int, a)))
    g = lambda k: z[f"{name}/in/{k}"]
    n = int(g("qo_indptr")[-1])
    return {
        "token_ids": conv(np.arange(n)), "position_ids": conv(g("position_ids")),
        "kv_page_indices": conv(g("kv_page_indices")), "kv_page_indptr": conv(g("kv_page_indptr")),
        "kv_last_page_lens": conv(g("kv_last_page_lens")), "qo_indptr": conv(g("qo_indptr")),
        "flattened_masks": conv(g("flattened_masks")), "mask_indptr": conv(g("mask_indptr")),
        "single_token_mode": False,
    }


def test_batch_matches_reference_golden():
    z = np.load(GOLD)
    names = sorted({k.split("/")[0] for k in z.files})
    assert len(names) >= 8
    for name in names:
        for as_bytes in (True, False):
            b = Batch(_args(z, name, as_bytes), int(z[f"{name}/in/page_size"]))
            assert np.array_equal(b.attention_masks, z[f"{name}/out/mask"]), name
            inp = b.get_model_inputs("cpu")
            for k in ("position_ids", "qo_indptr", "kv_page_indices", "kv_page_indptr", "kv_last_page_lens"):
                assert np.array_equal(inp[k].numpy(), z[f"{name}/out/out_{k}"]), (name, k)
                assert inp[k].dtype.is_floating_point is False and inp[k].element_size() == 4
            assert int(inp["total_pages_cpu"]) == int(z[f"{name}/out/total_pages"])


def test_reference_unit_test_case():
    # pie/tests/worker/test_flattened_mask.py: 80 entries, 79 set, entry 31 clear
    args = {
        "token_ids": [1, 2, 3], "position_ids": [31, 31, 15], "kv_page_indices": [0, 1, 2],
        "kv_page_indptr": [0, 2, 3], "kv_last_page_lens": [16, 16], "qo_indptr": [0, 2, 3],
        "flattened_masks": [32, 32, 16], "mask_indptr": [0, 1, 2, 3], "single_token_mode": False,
    }
    b = Batch(args, 16)
    assert b.attention_masks.size == 80 and int(b.attention_masks.sum()) == 79 and not b.attention_masks[31]


def test_brle_edge_cases():
    # zero-length runs flip the phase; runs past the valid length are cut; empty run lists give no bits
    m = decode_brle_batch([0, 3, 2, 100, 5], [0, 4, 4, 5], [6, 3, 2], [0, 8, 12, 16])
    assert m.astype(int).tolist() == [0, 0, 0, 1, 1, 0, 0, 0] + [0, 0, 0, 0] + [1, 1, 1, 0]
    assert decode_brle_batch([], [0], [], [0]).size == 0
