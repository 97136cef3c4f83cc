"""pie_b200: B200 (sm_100a) implementation of Pie's paged KV-cache hot path.

`import pie_b200.ops as ops` is a drop-in for the operator API the reference's Python worker
imports at pie/src/pie_worker/model/llama3.py:18-21: fused RoPE + K/V append into pages,
page-gather decode and prefill attention, page copy for fork.  The CUDA kernels live in
libpiekv.so (C ABI: include/piekv.h); importing this package fails if the library is missing.
"""
__version__ = "0.1.0"

from . import ops  # noqa: F401  (loads libpiekv.so; raises ImportError if it is not built)
from .ops import (  # noqa: F401
    BatchDecodeWithPagedKVCacheWrapper,
    BatchPrefillWithPagedKVCacheWrapper,
    RopeConfig,
    append_paged_kv_cache,
    apply_llama31_rope_pos_ids_inplace,
    apply_rope_pos_ids_inplace,
    copy_kv_pages,
    device_error,
    get_batch_indices_positions,
    get_seq_lens,
    rope_append_paged_kv_cache,
)

__all__ = [
    "ops",
    "BatchPrefillWithPagedKVCacheWrapper",
    "BatchDecodeWithPagedKVCacheWrapper",
    "apply_rope_pos_ids_inplace",
    "apply_llama31_rope_pos_ids_inplace",
    "append_paged_kv_cache",
    "get_seq_lens",
    "get_batch_indices_positions",
    "rope_append_paged_kv_cache",
    "copy_kv_pages",
    "RopeConfig",
    "device_error",
]
