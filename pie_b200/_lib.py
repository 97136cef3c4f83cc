"""ctypes binding of libpiekv.so (the C ABI declared in include/piekv.h).

The library is the only implementation: there is no Python or CPU fallback.  If the shared
object is missing or a symbol is absent, import fails with an explicit error.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libpiekv.so"

PIEKV_F32, PIEKV_F16, PIEKV_BF16 = 0, 1, 2
ROPE_NONE, ROPE_PLAIN, ROPE_LLAMA31, ROPE_TABLE = 0, 1, 2, 3
OPT_PDL = 0
OPT_WORK_STEALING = 1

PIEKV_ERR_WAIT_TIMEOUT = 5
STATUS_OUT_OF_PAGES = 8
ERR_NAMES = {
    0: "ok",
    1: "batch index out of range",
    2: "position beyond the request's page list",
    3: "physical page id out of range",
    4: "kv_last_page_len out of range",
    5: "bounded on-chip wait timed out",
    6: "RoPE table position out of range",
    7: "non-monotone indptr",
    8: "device page table: not enough free pages",
    9: "device page table: request row full / too many pages in one call",
    10: "device page table: bad slot",
}


class RopeParams(C.Structure):
    """Mirror of `piekv_rope_params`."""

    _fields_ = [
        ("mode", C.c_int32),
        ("interleave", C.c_int32),
        ("theta", C.c_float),
        ("scale", C.c_float),
        ("low_freq_factor", C.c_float),
        ("high_freq_factor", C.c_float),
        ("old_context_len", C.c_float),
        ("table_len", C.c_int32),
        ("cos_sin_table", C.c_void_p),
    ]


class AttnOptions(C.Structure):
    """Mirror of `piekv_attn_options`."""

    _fields_ = [("window_left", C.c_int32), ("reserved", C.c_int32), ("sinks", C.c_void_p)]


class WireBatch(C.Structure):
    """Mirror of `piekv_wire_batch`."""

    _fields_ = [(n, C.c_int64) for n in ("token_ids", "position_ids", "kv_page_indices", "kv_page_indptr",
                                         "kv_last_page_lens", "qo_indptr", "flattened_masks", "mask_indptr")] + \
               [(n, C.c_int32) for n in ("nnz", "batch", "total_pages", "num_runs")]


class QkvOptions(C.Structure):
    """Mirror of `piekv_qkv_options`."""

    _fields_ = [("bias", C.c_void_p), ("q_norm_weight", C.c_void_p), ("k_norm_weight", C.c_void_p),
                ("rms_eps", C.c_float), ("reserved", C.c_int32)]


MAX_PEERS = 8
PEER_HANDLE_BYTES = 64


class PeerOutputsC(C.Structure):
    """Mirror of `piekv_peer_outputs`."""

    _fields_ = [
        ("out", C.c_void_p * MAX_PEERS),
        ("flags", C.c_void_p * MAX_PEERS),
        ("world", C.c_int32),
        ("rank", C.c_int32),
        ("row_heads", C.c_int32),
        ("step", C.c_int32),
        ("step_counter", C.c_void_p),
        ("out_alt", C.c_void_p * MAX_PEERS),
    ]


class PeerReduceC(C.Structure):
    """Mirror of `piekv_peer_reduce`."""

    _fields_ = [
        ("out", C.c_void_p * MAX_PEERS),
        ("stage", C.c_void_p * MAX_PEERS),
        ("arrive", C.c_void_p * MAX_PEERS),
        ("done", C.c_void_p * MAX_PEERS),
        ("stage_bytes", C.c_int64),
        ("arrive_words", C.c_int64),
        ("done_words", C.c_int64),
        ("world", C.c_int32),
        ("rank", C.c_int32),
        ("step", C.c_int32),
        ("flags", C.c_int32),
    ]


REDUCE_PARTIALS_16BIT = 1

_p = C.c_void_p
_i32 = C.c_int32
_i64 = C.c_int64
_f32 = C.c_float

# name -> (restype, argtypes); must list every function declared in include/piekv.h
SIGNATURES = {
    "piekv_version": (C.c_int, []),
    "piekv_last_error_string": (C.c_char_p, []),
    "piekv_set_option": (C.c_int, [_i32, _i32]),
    "piekv_get_seq_lens": (C.c_int, [_p, _p, _i32, _i32, _p, _p]),
    "piekv_get_batch_indices_positions": (C.c_int, [_p, _p, _i32, _i32, _p, _p, _p]),
    "piekv_metadata": (C.c_int, [_p, _p, _p, _i32, _i32, _i32, _p, _p, _p, _p]),
    "piekv_rope_inplace": (
        C.c_int,
        [_p, _p, _i64, _i64, _i64, _i64, _p, _i32, _i32, _i32, _i32, _i32, C.POINTER(RopeParams), _p, _p],
    ),
    "piekv_rope_append": (
        C.c_int,
        [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _p, _p, _p, _p, _p, _p, _p,
         _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, C.POINTER(RopeParams), _i32, _p, _p],
    ),
    "piekv_qkv_rope_append": (
        C.c_int,
        [_p, _i64, _p, _i64, _p, _p, _p, _p, _p, _p, _p, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32,
         C.POINTER(RopeParams), _p, _p],
    ),
    "piekv_qkv_rope_append_opt": (
        C.c_int,
        [_p, _i64, _p, _i64, _p, _p, _p, _p, _p, _p, _p, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32,
         C.POINTER(RopeParams), _p, _p, C.POINTER(QkvOptions)],
    ),
    "piekv_oproj_allreduce_sizes": (C.c_int, [_i32, _i32, _i32, C.POINTER(C.c_int64)]),
    "piekv_oproj_tile_cols": (_i32, [_i32, _i32]),
    "piekv_oproj_allreduce": (
        C.c_int,
        [_p, _i64, _p, _i64, _p, _i64, _i32, _i32, _i32, _i32, C.POINTER(PeerReduceC), _p, _p],
    ),
    "piekv_decode_workspace_bytes": (_i64, [_i32, _i32, _i32, _i32]),
    "piekv_decode_counter_bytes": (_i64, [_i32]),
    "piekv_decode_run": (
        C.c_int,
        [_p, _i64, _i64, _p, _p, _p, _p, _p, _p, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _p, _i64, _p, _p],
    ),
    "piekv_decode_run_opt": (
        C.c_int,
        [_p, _i64, _i64, _p, _p, _p, _p, _p, _p, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _p, _i64, _p, _p,
         C.POINTER(AttnOptions)],
    ),
    "piekv_decode_step_fused_opt": (
        C.c_int,
        [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _p, _p, _p, _p, _p, _p, _p,
         _i32, _i32, _i32, _i32, _i32, _i32, _i32, C.POINTER(RopeParams), _f32, _p, _i64, _p, _p,
         C.POINTER(AttnOptions)],
    ),
    "piekv_prefill_plan_opt": (
        C.c_int,
        [_p, _p, _p, _p, _p, _p, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _p, _i64, _p, _p],
    ),
    "piekv_prefill_run_opt": (
        C.c_int,
        [_p, _i64, _i64, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32,
         _i32, _i32, _f32, _p, _i64, _p, _p, C.POINTER(AttnOptions)],
    ),
    "piekv_decode_noalloc_max_bytes": (_i64, []),
    "piekv_decode_run_noalloc": (
        C.c_int,
        [_p, _i64, _i64, _p, _p, _p, _p, _p, _p, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _p, _p],
    ),
    "piekv_decode_step_fused": (
        C.c_int,
        [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _p, _p, _p, _p, _p, _p, _p,
         _i32, _i32, _i32, _i32, _i32, _i32, _i32, C.POINTER(RopeParams), _f32, _p, _i64, _p, _p],
    ),
    "piekv_peer_alloc": (C.c_int, [_i64, C.POINTER(C.c_void_p), _p]),
    "piekv_peer_open": (C.c_int, [_p, C.POINTER(C.c_void_p)]),
    "piekv_peer_close": (C.c_int, [_p]),
    "piekv_peer_free": (C.c_int, [_p]),
    "piekv_decode_step_fused_peer": (
        C.c_int,
        [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _p, _p, _p, _p, _p, _p, _i32, _i32, _i32, _i32, _i32,
         _i32, _i32, C.POINTER(RopeParams), _f32, _p, _i64, _p, _p],
    ),
    "piekv_peer_wait": (C.c_int, [_p, _i32, _i32, _p, _p]),
    "piekv_peer_wait_counted": (C.c_int, [_p, _i32, _p, _p, _p]),
    "piekv_batch_from_wire": (C.c_int, [_p, C.POINTER(WireBatch), _i32, _p, _p, _p, _p, _p, _p]),
    "piekv_prefill_export_mask": (C.c_int, [_p, _p, _p, _i64, _i32, _i32, _i32, _i32, _p, _i64, _p, _p]),
    "piekv_pagestate_bytes": (_i64, [_i32, _i32, _i32]),
    "piekv_pagestate_init": (C.c_int, [_p, _i64, _i32, _i32, _i32, _i32, _p]),
    "piekv_pagestate_adjust": (C.c_int, [_p, _i32, _i32, _i32, _i32, _p, _p, _i32, _i32, _p, _p, _p, _p, _p, _p]),
    "piekv_pagestate_release": (C.c_int, [_p, _i32, _i32, _i32, _i32, _p, _i32, _p, _p]),
    "piekv_pagestate_fork": (C.c_int, [_p, _i32, _i32, _i32, _i32, _p, _p, _i32, _p, _p, _p, _p, _p]),
    "piekv_pages_create": (C.c_void_p, [_i32]),
    "piekv_pages_destroy": (None, [_p]),
    "piekv_pages_available": (_i32, [_p]),
    "piekv_pages_refcount": (_i32, [_p, _i32]),
    "piekv_pages_owned": (_i32, [_p, C.c_uint64]),
    "piekv_pages_alloc": (C.c_int, [_p, C.c_uint64, _i32, _p]),
    "piekv_pages_last_victims": (_i32, [_p, _p, _i32]),
    "piekv_pages_free": (C.c_int, [_p, C.c_uint64, _p, _i32]),
    "piekv_pages_share": (C.c_int, [_p, C.c_uint64, _p, _i32]),
    "piekv_pages_cleanup": (C.c_int, [_p, C.c_uint64]),
    "piekv_pages_export": (C.c_int, [_p, C.c_uint64, _p, _i32, C.c_char_p]),
    "piekv_pages_import": (_i32, [_p, C.c_char_p, _p, _i32]),
    "piekv_pages_release_exported": (C.c_int, [_p, C.c_char_p]),
    "piekv_abi_sizeof": (_i32, [_i32]),
    "piekv_prefill_workspace_bytes": (_i64, [_i32, _i32, _i32, _i32, _i32, _i64]),
    "piekv_prefill_plan": (
        C.c_int,
        [_p, _p, _p, _p, _i64, _i32, _i32, _i32, _i32, _i32, _p, _i64, _p, _p],
    ),
    "piekv_prefill_plan_brle": (
        C.c_int,
        [_p, _p, _p, _p, _p, _i64, _i32, _i32, _i32, _i32, _p, _i64, _p, _p],
    ),
    "piekv_prefill_run": (
        C.c_int,
        [_p, _i64, _i64, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32,
         _i32, _i32, _f32, _p, _i64, _p, _p],
    ),
    "piekv_copy_pages": (
        C.c_int,
        [C.POINTER(C.c_void_p), _i32, _p, _p, _p, _i32, _i32, _i32, _i32, _i32, _i32, _p, _p],
    ),
}


class PiekvError(RuntimeError):
    """A libpiekv call returned a non-zero status."""


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python pie_b200/build.py` "
            "(nvcc, sm_100a). pie_b200 has no fallback implementation."
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:  # pragma: no cover
            raise ImportError(f"{LIB_PATH} does not export {name}; rebuild it") from e
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(status: int, what: str) -> None:
    """Raise on a non-zero status, with the library's message."""
    if status == 0:
        return
    msg = lib.piekv_last_error_string()
    text = msg.decode("utf-8", "replace") if msg else ""
    if status > 0:
        raise ValueError(f"{what}: {text}")
    raise PiekvError(f"{what}: {text} (status {status})")
