"""The C-ABI library loads on a machine without a GPU, exports every symbol include/piekv.h declares,
and rejects bad arguments on the host before anything is launched."""
import ctypes as C
import os
import re

import pytest
import torch

from pie_b200 import _lib, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "piekv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(piekv_[a-z0-9_]+)\s*\(", text)))


def test_header_and_bindings_agree():
    decl = _declared()
    assert len(decl) >= 13
    assert sorted(_lib.SIGNATURES) == decl
    raw = C.CDLL(str(_lib.LIB_PATH))
    for name in decl:
        assert hasattr(raw, name), name


def test_version_and_error_text():
    assert _lib.lib.piekv_version() == 103
    rc = _lib.lib.piekv_get_seq_lens(None, None, 4, 16, None, None)
    assert rc > 0
    assert b"null" in _lib.lib.piekv_last_error_string()
    rc = _lib.lib.piekv_get_seq_lens(None, None, 4, 0, None, None)
    assert rc > 0 and b"page_size" in _lib.lib.piekv_last_error_string()
    with pytest.raises(ValueError):
        _lib.check(rc, "x")


def test_host_side_argument_checks_without_gpu():
    L = _lib.lib
    one = C.c_void_p(16)
    # heads not divisible
    rc = L.piekv_decode_run(one, 128, 128, one, one, None, one, one, one, 1, 6, 4, 128, 16, 8, 2, 1.0, one, 1 << 20,
                            None, None)
    assert rc > 0 and b"multiple" in L.piekv_last_error_string()
    # unknown dtype
    rc = L.piekv_decode_run(one, 128, 128, one, one, None, one, one, one, 1, 8, 4, 128, 16, 8, 9, 1.0, one, 1 << 20,
                            None, None)
    assert rc > 0 and b"dtype" in L.piekv_last_error_string()
    # rope_inplace without rope params
    rc = L.piekv_rope_inplace(one, one, 128, 128, 128, 128, one, 1, 1, 1, 128, 2, None, None, None)
    assert rc > 0
    # odd head_dim
    rp = _lib.RopeParams()
    rp.mode = _lib.ROPE_PLAIN
    rp.theta = 1e4
    rc = L.piekv_rope_inplace(one, one, 128, 128, 128, 128, one, 1, 1, 1, 127, 2, C.byref(rp), None, None)
    assert rc > 0 and b"head_dim" in L.piekv_last_error_string()
    # copy_pages without layers
    rc = L.piekv_copy_pages(None, 0, one, one, None, 1, 16, 8, 128, 4, 2, None, None)
    assert rc > 0
    assert L.piekv_decode_workspace_bytes(64, 32, 8, 128) > 65536
    assert L.piekv_decode_counter_bytes(64) == ops.COUNTER_BYTES


def test_ops_reject_cpu_tensors_like_the_reference_facade():
    i = torch.zeros(3, dtype=torch.int32)
    with pytest.raises(ValueError, match="CUDA"):
        ops.get_seq_lens(i, i, 16)
    with pytest.raises(ValueError, match="CUDA"):
        ops.BatchDecodeWithPagedKVCacheWrapper(torch.zeros(1 << 20, dtype=torch.uint8))
    q = torch.zeros(2, 4, 64)
    with pytest.raises(ValueError):
        ops.apply_rope_pos_ids_inplace(q, q, i[:2])
    with pytest.raises(ValueError, match="NHD"):
        ops.append_paged_kv_cache(q, q, i, i, torch.zeros(1, 2, 16, 4, 64), i, i, i, kv_layout="HND")


def test_struct_mirrors_have_the_size_the_library_reports():
    import ctypes as C

    from pie_b200 import _lib
    assert _lib.lib.piekv_abi_sizeof(0) == C.sizeof(_lib.RopeParams)
    assert _lib.lib.piekv_abi_sizeof(1) == C.sizeof(_lib.PeerOutputsC)
    assert _lib.lib.piekv_abi_sizeof(2) == C.sizeof(_lib.AttnOptions)
    assert _lib.lib.piekv_abi_sizeof(3) == C.sizeof(_lib.WireBatch)
    assert _lib.lib.piekv_abi_sizeof(4) == C.sizeof(_lib.QkvOptions)
    assert _lib.lib.piekv_abi_sizeof(5) == C.sizeof(_lib.PeerReduceC)
    assert _lib.lib.piekv_abi_sizeof(99) == -1


def test_ops_refuse_tensors_of_a_device_that_is_not_current(monkeypatch):
    """The library launches on the current CUDA device; tensors of another GPU must raise instead of being
    paired with a foreign stream.  Checked on the host with the two torch queries replaced."""
    class FakeStream:
        cuda_stream = 0

    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda device=None: FakeStream())
    assert ops._stream(torch.device("cuda", 0)) == 0
    assert ops._stream(torch.device("cuda")) == 0
    with pytest.raises(ValueError, match="current CUDA device"):
        ops._stream(torch.device("cuda", 1))
