"""Paged-KV operator API of the reference, backed by libpiekv.so.

This module keeps the names and keyword arguments that Pie's Python worker uses at its
single op seam (`from flashinfer import ...` / `flashinfer_metal as ops`,
pie/src/pie_worker/model/llama3.py:18-21; exported names
pie/src/flashinfer_metal/__init__.py:14-37), so `import pie_b200.ops as ops` is a drop-in
for that path:

    get_seq_lens, get_batch_indices_positions,
    apply_rope_pos_ids_inplace, apply_llama31_rope_pos_ids_inplace,
    append_paged_kv_cache,
    BatchDecodeWithPagedKVCacheWrapper, BatchPrefillWithPagedKVCacheWrapper

plus the fused / extended entry points this library adds (`rope_append_paged_kv_cache`,
`copy_kv_pages`).  Every function forwards raw device pointers and the current CUDA stream
to the C ABI; nothing here computes on the host and there is no fallback path.
Error behaviour follows the reference facade: wrong device / dtype / shape raise
`ValueError`, `run()` before `plan()` raises `RuntimeError("Must call plan() before run()")`
(pie/src/flashinfer_metal/ops.py:186-190,208-209).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import RopeParams, check, lib

__all__ = [
    "BatchPrefillWithPagedKVCacheWrapper",
    "BatchDecodeWithPagedKVCacheWrapper",
    "BatchAttentionWithAttentionSinkWrapper",
    "apply_rope_pos_ids_inplace",
    "apply_rope_with_cos_sin_cache_inplace",
    "apply_llama31_rope_pos_ids_inplace",
    "append_paged_kv_cache",
    "get_seq_lens",
    "get_batch_indices_positions",
    "rope_append_paged_kv_cache",
    "copy_kv_pages",
    "RopeConfig",
    "device_error",
    "COUNTER_BYTES",
]

COUNTER_BYTES = 65536  # head of every workspace: split-KV arrival counters, kept zero

_DTYPES = {torch.float32: _lib.PIEKV_F32, torch.float16: _lib.PIEKV_F16, torch.bfloat16: _lib.PIEKV_BF16}


# ---------------------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------------------
def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise ValueError(f"{name} must be a torch.Tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise ValueError(f"{name} must be on a CUDA device, got {t.device}")


def _require_i32(t: torch.Tensor, name: str) -> None:
    _require_cuda(t, name)
    if t.dtype != torch.int32:
        raise ValueError(f"{name} must be int32, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _dtype_code(dt: torch.dtype, name: str) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise ValueError(f"{name}: unsupported dtype {dt} (float32, float16, bfloat16)") from None


def _stream(device: torch.device) -> int:
    """Stream handle for a launch on `device`.  The library launches on the CURRENT CUDA device (and looks
    its SM count and built-in scratch up for that device), so tensors of another GPU are refused instead of
    being paired with a foreign stream.  The reference worker pins one device per process
    (pie/src/pie_worker/model/llama3.py:732-733)."""
    cur = torch.cuda.current_device()
    idx = device.index if device.index is not None else cur
    if idx != cur:
        raise ValueError(f"tensors live on cuda:{idx} but the current CUDA device is cuda:{cur}; "
                         f"call torch.cuda.set_device({idx}) (or use `with torch.cuda.device({idx})`) first")
    return torch.cuda.current_stream(device).cuda_stream


def _rows(t: torch.Tensor, name: str) -> Tuple[int, int]:
    """(token stride, head stride) in elements of a [n, H, D] tensor whose last axis is contiguous."""
    if t.dim() != 3:
        raise ValueError(f"{name} must be [tokens, heads, head_dim], got shape {tuple(t.shape)}")
    if t.shape[2] > 1 and t.stride(2) != 1:
        raise ValueError(f"{name}: head_dim axis must be contiguous")
    return t.stride(0), t.stride(1)


_ERR_WORDS: dict = {}


def _err_word(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    w = _ERR_WORDS.get(key)
    if w is None:
        w = torch.zeros(4, dtype=torch.int32, device=device)
        _ERR_WORDS[key] = w
    return w


def device_error(device=None, clear: bool = True) -> Optional[dict]:
    """Read the device error word (synchronises).  None when no kernel reported a fault."""
    device = torch.device(device if device is not None else "cuda")
    w = _err_word(device)
    vals = w.cpu().tolist()
    if vals[0] == 0:
        return None
    if clear:
        w.zero_()
    return {
        "code": vals[0],
        "what": _lib.ERR_NAMES.get(vals[0], "unknown"),
        "kernel": vals[1],
        "index": vals[2],
        "value": vals[3],
    }


def set_programmatic_dependent_launch(mode: int) -> None:
    """0 off, 1 on, 2 on with the promise that the page-table arrays are not written by the kernel that
    runs immediately before a decode call, 3 with the further promise that that kernel wrote at most into
    the last two pages of any request (the previous decode step of the same requests); see PIEKV_OPT_PDL in
    include/piekv.h."""
    check(lib.piekv_set_option(_lib.OPT_PDL, int(mode)), "set_option")


def set_work_stealing(on: bool) -> None:
    """False (default): the tuned decode kernel keeps every SM to its own page range and equal inputs give
    bit-identical outputs.  True: SMs that finish early take over work of slower ones; the grouping of the
    partial results, hence the last bits, may then differ between launches.  See PIEKV_OPT_WORK_STEALING."""
    check(lib.piekv_set_option(_lib.OPT_WORK_STEALING, 1 if on else 0), "set_option")


def set_deterministic(on: bool) -> None:
    """`set_work_stealing(not on)`."""
    set_work_stealing(not on)


def _check_pool(pool: torch.Tensor, name: str = "paged_kv_cache"):
    if isinstance(pool, (tuple, list)):
        raise ValueError(f"{name}: separate (k_cache, v_cache) tensors are not supported; pass the "
                         "combined [pages, 2, page_size, kv_heads, head_dim] tensor")
    _require_cuda(pool, name)
    if pool.dim() != 5 or pool.shape[1] != 2:
        raise ValueError(f"{name} must be [pages, 2, page_size, kv_heads, head_dim], got {tuple(pool.shape)}")
    if not pool.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return pool.shape[0], pool.shape[2], pool.shape[3], pool.shape[4]


@dataclass
class RopeConfig:
    """Rotary-embedding parameters (defaults: the reference's Llama-3 model config,
    pie/src/pie_worker/model/llama3.py:167-173).  `mode`: "none" | "plain" | "llama31" | "table"."""

    mode: str = "llama31"
    theta: float = 500000.0
    scale: float = 8.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    old_context_len: float = 8192.0
    interleave: bool = False
    cos_sin_table: Optional[torch.Tensor] = None  # fp32 [positions, head_dim]: cos | sin

    def to_c(self, head_dim: int) -> RopeParams:
        modes = {"none": _lib.ROPE_NONE, "plain": _lib.ROPE_PLAIN, "llama31": _lib.ROPE_LLAMA31,
                 "table": _lib.ROPE_TABLE}
        if self.mode not in modes:
            raise ValueError(f"unknown rope mode {self.mode!r}")
        rp = RopeParams()
        rp.mode = modes[self.mode]
        rp.interleave = 1 if self.interleave else 0
        rp.theta = float(self.theta)
        rp.scale = float(self.scale)
        rp.low_freq_factor = float(self.low_freq_factor)
        rp.high_freq_factor = float(self.high_freq_factor)
        rp.old_context_len = float(self.old_context_len)
        rp.table_len = 0
        rp.cos_sin_table = None
        if self.mode == "table":
            t = self.cos_sin_table
            if t is None:
                raise ValueError("rope mode 'table' needs cos_sin_table")
            _require_cuda(t, "cos_sin_table")
            if t.dtype != torch.float32 or t.dim() != 2 or t.shape[1] != head_dim or not t.is_contiguous():
                raise ValueError("cos_sin_table must be contiguous float32 [positions, head_dim]")
            rp.table_len = t.shape[0]
            rp.cos_sin_table = t.data_ptr()
        return rp


# ---------------------------------------------------------------------------------------
# metadata
# ---------------------------------------------------------------------------------------
def get_seq_lens(kv_page_indptr: torch.Tensor, kv_last_page_lens: torch.Tensor, page_size: int) -> torch.Tensor:
    """Sequence length of every request from its page count and last-page fill.

    Reference call: pie/src/pie_worker/model/llama3.py:745-749."""
    _require_i32(kv_page_indptr, "kv_page_indptr")
    _require_i32(kv_last_page_lens, "kv_last_page_lens")
    batch = kv_page_indptr.shape[0] - 1
    if kv_last_page_lens.shape[0] < batch:
        raise ValueError("kv_last_page_lens shorter than the batch")
    out = torch.empty(batch, dtype=torch.int32, device=kv_page_indptr.device)
    check(lib.piekv_get_seq_lens(kv_page_indptr.data_ptr(), kv_last_page_lens.data_ptr(), batch, int(page_size),
                                 out.data_ptr(), _stream(out.device)), "get_seq_lens")
    return out


def get_batch_indices_positions(append_indptr: torch.Tensor, seq_lens: torch.Tensor, nnz: int
                                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Request index and KV slot of every appended token.

    Reference call: pie/src/pie_worker/model/llama3.py:751-755."""
    _require_i32(append_indptr, "append_indptr")
    _require_i32(seq_lens, "seq_lens")
    batch = append_indptr.shape[0] - 1
    dev = append_indptr.device
    bi = torch.empty(nnz, dtype=torch.int32, device=dev)
    pos = torch.empty(nnz, dtype=torch.int32, device=dev)
    check(lib.piekv_get_batch_indices_positions(append_indptr.data_ptr(), seq_lens.data_ptr(), batch, int(nnz),
                                                bi.data_ptr(), pos.data_ptr(), _stream(dev)),
          "get_batch_indices_positions")
    return bi, pos


# ---------------------------------------------------------------------------------------
# RoPE / append
# ---------------------------------------------------------------------------------------
def _rope_inplace(q, k, pos_ids, cfg: RopeConfig, who: str) -> None:
    _require_cuda(q, "q")
    _require_cuda(k, "k")
    _require_i32(pos_ids, "pos_ids")
    if q.dtype != k.dtype:
        raise ValueError(f"{who}: q and k dtypes differ ({q.dtype} vs {k.dtype})")
    qs, ks = _rows(q, "q"), _rows(k, "k")
    n, hq, d = q.shape
    if k.shape[0] != n or k.shape[2] != d or pos_ids.shape[0] != n:
        raise ValueError(f"{who}: q {tuple(q.shape)}, k {tuple(k.shape)}, pos_ids {tuple(pos_ids.shape)} disagree")
    rp = cfg.to_c(d)
    check(lib.piekv_rope_inplace(q.data_ptr(), k.data_ptr(), qs[0], qs[1], ks[0], ks[1], pos_ids.data_ptr(), n, hq,
                                 k.shape[1], d, _dtype_code(q.dtype, who), C.byref(rp),
                                 _err_word(q.device).data_ptr(), _stream(q.device)), who)


def apply_rope_pos_ids_inplace(q: torch.Tensor, k: torch.Tensor, pos_ids: torch.Tensor,
                               rotary_dim: Optional[int] = None, interleave: bool = False,
                               rope_scale: float = 1.0, rope_theta: float = 10000.0) -> None:
    """Plain rotary embedding in place (reference call: pie/src/pie_worker/model/qwen3.py:665-670)."""
    if rotary_dim is not None and rotary_dim != q.shape[-1]:
        raise ValueError("rotary_dim smaller than head_dim is not supported")
    cfg = RopeConfig(mode="plain", theta=rope_theta, scale=rope_scale, interleave=interleave)
    _rope_inplace(q, k, pos_ids, cfg, "apply_rope_pos_ids_inplace")


def apply_llama31_rope_pos_ids_inplace(q: torch.Tensor, k: torch.Tensor, pos_ids: torch.Tensor,
                                       rotary_dim: Optional[int] = None, interleave: bool = False,
                                       rope_scale: float = 8.0, rope_theta: float = 500000.0,
                                       low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                                       old_context_len: int = 8192) -> None:
    """Llama-3.1 rotary embedding in place (reference call: pie/src/pie_worker/model/llama3.py:660-669)."""
    if rotary_dim is not None and rotary_dim != q.shape[-1]:
        raise ValueError("rotary_dim smaller than head_dim is not supported")
    cfg = RopeConfig(mode="llama31", theta=rope_theta, scale=rope_scale, low_freq_factor=low_freq_factor,
                     high_freq_factor=high_freq_factor, old_context_len=float(old_context_len),
                     interleave=interleave)
    _rope_inplace(q, k, pos_ids, cfg, "apply_llama31_rope_pos_ids_inplace")


def apply_rope_with_cos_sin_cache_inplace(positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor,
                                          head_size: int, cos_sin_cache: torch.Tensor, is_neox: bool = True) -> None:
    """Rotary embedding in place from a precomputed table, as the YaRN-scaled model families call it
    (pie/src/pie_worker/model/gpt_oss.py:671-678, mistral3.py:838-845, olmo3.py:797-804).

    `cos_sin_cache` is float32 [max_position, rotary_dim]: cos in the first half of a row, sin in the second
    (any attention-temperature factor already multiplied in, gpt_oss.py:540-547).  `query` / `key` are
    [n, heads, head_size] or flattened [n, heads * head_size]; `is_neox=True` pairs element i with
    i + head_size / 2, False pairs (2i, 2i + 1).  Positions may be int32 or int64."""
    _require_cuda(query, "query")
    _require_cuda(key, "key")
    _require_cuda(positions, "positions")
    _require_cuda(cos_sin_cache, "cos_sin_cache")
    if positions.dtype not in (torch.int32, torch.int64):
        raise ValueError(f"positions must be int32 or int64, got {positions.dtype}")
    pos = positions if positions.dtype == torch.int32 else positions.to(torch.int32)
    pos = pos.contiguous()
    if cos_sin_cache.dtype != torch.float32 or cos_sin_cache.dim() != 2:
        raise ValueError("cos_sin_cache must be float32 [max_position, rotary_dim]")
    if cos_sin_cache.shape[1] != head_size:
        raise ValueError(f"rotary_dim {cos_sin_cache.shape[1]} smaller than head_size {head_size} is not supported")

    def heads(t, name):
        if t.dim() == 3:
            if t.shape[2] != head_size:
                raise ValueError(f"{name}: last axis {t.shape[2]} differs from head_size {head_size}")
            return t
        if t.dim() != 2 or t.shape[1] % head_size != 0:
            raise ValueError(f"{name} must be [n, heads, head_size] or [n, heads * head_size], got {tuple(t.shape)}")
        if t.shape[1] > 1 and t.stride(1) != 1:
            raise ValueError(f"{name}: the flattened head axis must be contiguous")
        return t.as_strided((t.shape[0], t.shape[1] // head_size, head_size), (t.stride(0), head_size, 1),
                            t.storage_offset())

    cfg = RopeConfig(mode="table", cos_sin_table=cos_sin_cache.contiguous(), interleave=not is_neox)
    _rope_inplace(heads(query, "query"), heads(key, "key"), pos, cfg, "apply_rope_with_cos_sin_cache_inplace")


def _append(q, k, v, pos_ids, batch_indices, positions, pool, kv_indices, kv_indptr, kv_last_page_len,
            cfg: Optional[RopeConfig], rotate_k_in_place: bool, who: str) -> None:
    _require_cuda(k, "append_key")
    _require_cuda(v, "append_value")
    _require_i32(batch_indices, "batch_indices")
    _require_i32(positions, "positions")
    _require_i32(kv_indices, "kv_indices")
    _require_i32(kv_indptr, "kv_indptr")
    _require_i32(kv_last_page_len, "kv_last_page_len")
    num_pages, page_size, hkv, d = _check_pool(pool)
    ks, vs = _rows(k, "append_key"), _rows(v, "append_value")
    n = k.shape[0]
    if tuple(k.shape) != (n, hkv, d) or tuple(v.shape) != (n, hkv, d):
        raise ValueError(f"{who}: key {tuple(k.shape)} / value {tuple(v.shape)} do not match the cache "
                         f"[*, {hkv}, {d}]")
    if k.dtype != pool.dtype or v.dtype != pool.dtype:
        raise ValueError(f"{who}: key/value dtype {k.dtype}/{v.dtype} differs from the cache dtype {pool.dtype}")
    if batch_indices.shape[0] < n or positions.shape[0] < n:
        raise ValueError(f"{who}: batch_indices / positions shorter than the number of tokens")
    batch = kv_indptr.shape[0] - 1
    rp = None
    q_ptr, qs, hq, pos_ptr = None, (0, 0), 0, None
    if cfg is not None and cfg.mode != "none":
        rp = cfg.to_c(d)
        _require_i32(pos_ids, "pos_ids")
        pos_ptr = pos_ids.data_ptr()
        if q is not None:
            _require_cuda(q, "q")
            qs = _rows(q, "q")
            if q.shape[0] != n or q.shape[2] != d or q.dtype != pool.dtype:
                raise ValueError(f"{who}: q {tuple(q.shape)} {q.dtype} does not match key / cache")
            q_ptr, hq = q.data_ptr(), q.shape[1]
    check(lib.piekv_rope_append(q_ptr, k.data_ptr(), v.data_ptr(), qs[0], qs[1], ks[0], ks[1], vs[0], vs[1], pos_ptr,
                                batch_indices.data_ptr(), positions.data_ptr(), pool.data_ptr(),
                                kv_indices.data_ptr(), kv_indptr.data_ptr(), kv_last_page_len.data_ptr(), n, batch,
                                hq, hkv, d, page_size, num_pages, _dtype_code(pool.dtype, who),
                                C.byref(rp) if rp is not None else None, 1 if rotate_k_in_place else 0,
                                _err_word(pool.device).data_ptr(), _stream(pool.device)), who)


def append_paged_kv_cache(append_key: torch.Tensor, append_value: torch.Tensor, batch_indices: torch.Tensor,
                          positions: torch.Tensor, paged_kv_cache: torch.Tensor, kv_indices: torch.Tensor,
                          kv_indptr: torch.Tensor, kv_last_page_len: torch.Tensor, kv_layout: str = "NHD") -> None:
    """Scatter new K/V rows into their pages (reference call: pie/src/pie_worker/model/llama3.py:675-685)."""
    if kv_layout != "NHD":
        raise ValueError(f"kv_layout {kv_layout!r} is not supported (NHD only)")
    _append(None, append_key, append_value, None, batch_indices, positions, paged_kv_cache, kv_indices, kv_indptr,
            kv_last_page_len, None, False, "append_paged_kv_cache")


def rope_append_paged_kv_cache(q: Optional[torch.Tensor], k: torch.Tensor, v: torch.Tensor, pos_ids: torch.Tensor,
                               batch_indices: torch.Tensor, positions: torch.Tensor, paged_kv_cache: torch.Tensor,
                               kv_indices: torch.Tensor, kv_indptr: torch.Tensor, kv_last_page_len: torch.Tensor,
                               rope: RopeConfig, rotate_k_in_place: bool = False) -> None:
    """RoPE (q in place, k on the way to the cache) fused with the append: one launch for the
    reference's two ops at pie/src/pie_worker/model/llama3.py:660-685."""
    _append(q, k, v, pos_ids, batch_indices, positions, paged_kv_cache, kv_indices, kv_indptr, kv_last_page_len,
            rope, rotate_k_in_place, "rope_append_paged_kv_cache")


def qkv_rope_append_paged_kv_cache(x: torch.Tensor, w_qkv: torch.Tensor, pos_ids: torch.Tensor,
                                   batch_indices: torch.Tensor, positions: torch.Tensor,
                                   paged_kv_cache: torch.Tensor, kv_indices: torch.Tensor, kv_indptr: torch.Tensor,
                                   num_qo_heads: int, num_kv_heads: int, rope: Optional[RopeConfig] = None,
                                   q_out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                                   q_norm_weight: Optional[torch.Tensor] = None,
                                   k_norm_weight: Optional[torch.Tensor] = None,
                                   rms_norm_eps: float = 1e-6) -> torch.Tensor:
    """The QKV projection with RoPE and the append as its epilogue: `x` [n, hidden] times `w_qkv`
    [(Hq + 2 Hkv) * 128, hidden] (the fused weight of pie/src/pie_worker/model/llama3.py:627-630, as
    `torch.nn.functional.linear` takes it); rotated q comes back as [n, Hq, 128], rotated k and v go straight
    into the paged cache.  The projection output itself is never written to memory, and the fp32 accumulator is
    rounded once, after the rotation (the reference rounds the projection first).  One launch for
    llama3.py:627-685 when no adapter edits q / k / v in between.  head_dim 128, 16-bit types, hidden a
    multiple of 64.

    `bias` [(Hq + 2 Hkv) * 128] is added to the projection (pie/src/pie_worker/model/qwen2.py:596-603);
    `q_norm_weight` / `k_norm_weight` [128] apply the per-head RMSNorm of qwen3.py:651-662 to q / k before
    the rotation (`rms_norm_eps` as there)."""
    _require_cuda(x, "x")
    _require_cuda(w_qkv, "w_qkv")
    _require_i32(pos_ids, "pos_ids")
    _require_i32(batch_indices, "batch_indices")
    _require_i32(positions, "positions")
    _require_i32(kv_indices, "kv_indices")
    _require_i32(kv_indptr, "kv_indptr")
    num_pages, page_size, hkv, d = _check_pool(paged_kv_cache)
    if x.dim() != 2 or w_qkv.dim() != 2 or x.stride(1) != 1 or w_qkv.stride(1) != 1:
        raise ValueError("x and w_qkv must be 2-D with contiguous rows")
    n, hidden = x.shape
    if hkv != num_kv_heads or d != 128:
        raise ValueError(f"the cache holds {hkv} kv heads of dim {d}; expected {num_kv_heads} of dim 128")
    if tuple(w_qkv.shape) != ((num_qo_heads + 2 * num_kv_heads) * d, hidden):
        raise ValueError(f"w_qkv shape {tuple(w_qkv.shape)} differs from "
                         f"({(num_qo_heads + 2 * num_kv_heads) * d}, {hidden})")
    if not (x.dtype == w_qkv.dtype == paged_kv_cache.dtype):
        raise ValueError("x, w_qkv and the cache must share one dtype")
    if pos_ids.shape[0] < n or batch_indices.shape[0] < n or positions.shape[0] < n:
        raise ValueError("pos_ids / batch_indices / positions shorter than the token count")
    if q_out is None:
        q_out = torch.empty((n, num_qo_heads, d), dtype=x.dtype, device=x.device)
    elif tuple(q_out.shape) != (n, num_qo_heads, d) or q_out.dtype != x.dtype or not q_out.is_contiguous():
        raise ValueError("q_out must be a contiguous [n, num_qo_heads, 128] tensor of x's dtype")
    rp = (rope if rope is not None else RopeConfig()).to_c(d)
    opt = None
    if bias is not None or q_norm_weight is not None or k_norm_weight is not None:
        opt = _lib.QkvOptions()
        for name, t, numel in (("bias", bias, (num_qo_heads + 2 * num_kv_heads) * d),
                               ("q_norm_weight", q_norm_weight, d), ("k_norm_weight", k_norm_weight, d)):
            if t is not None:
                _require_cuda(t, name)
                if t.dtype != x.dtype or t.numel() != numel or not t.is_contiguous():
                    raise ValueError(f"{name} must be a contiguous tensor of {numel} elements of x's dtype")
            setattr(opt, name, t.data_ptr() if t is not None else None)
        opt.rms_eps = float(rms_norm_eps)
        opt.reserved = 0
    check(lib.piekv_qkv_rope_append_opt(x.data_ptr(), x.stride(0), w_qkv.data_ptr(), w_qkv.stride(0),
                                        q_out.data_ptr(), pos_ids.data_ptr(), batch_indices.data_ptr(),
                                        positions.data_ptr(), paged_kv_cache.data_ptr(), kv_indices.data_ptr(),
                                        kv_indptr.data_ptr(), n, kv_indptr.shape[0] - 1, hidden, num_qo_heads,
                                        num_kv_heads, d, page_size, num_pages,
                                        _dtype_code(x.dtype, "qkv_rope_append_paged_kv_cache"), rp,
                                        _err_word(x.device).data_ptr(), _stream(x.device),
                                        C.byref(opt) if opt is not None else None),
          "qkv_rope_append_paged_kv_cache")
    return q_out


def copy_kv_pages(kv_cache_at_layer: Sequence[torch.Tensor], src_pages: torch.Tensor, dst_pages: torch.Tensor,
                  valid_len: Optional[torch.Tensor] = None) -> None:
    """Copy the first `valid_len[j]` token rows (default: all) of page src[j] to page dst[j] in every
    layer's pool: copy-on-write of a partially filled last page when a context forks.  The reference
    drops and recomputes that page instead (sdk/rust/inferlet/src/context.rs:147-225)."""
    if isinstance(kv_cache_at_layer, torch.Tensor):
        kv_cache_at_layer = [kv_cache_at_layer]
    if len(kv_cache_at_layer) == 0:
        raise ValueError("copy_kv_pages: no layers")
    _require_i32(src_pages, "src_pages")
    _require_i32(dst_pages, "dst_pages")
    if src_pages.shape != dst_pages.shape:
        raise ValueError("copy_kv_pages: src_pages and dst_pages differ in length")
    if valid_len is not None:
        _require_i32(valid_len, "valid_len")
        if valid_len.shape != src_pages.shape:
            raise ValueError("copy_kv_pages: valid_len length differs from src_pages")
    shape0 = None
    for i, pool in enumerate(kv_cache_at_layer):
        s = _check_pool(pool, f"kv_cache_at_layer[{i}]")
        if shape0 is None:
            shape0, dt0 = s, pool.dtype
        elif s != shape0 or pool.dtype != dt0:
            raise ValueError("copy_kv_pages: layers differ in shape or dtype")
    num_pages, page_size, hkv, d = shape0
    ptrs = (C.c_void_p * len(kv_cache_at_layer))(*[p.data_ptr() for p in kv_cache_at_layer])
    dev = kv_cache_at_layer[0].device
    check(lib.piekv_copy_pages(ptrs, len(kv_cache_at_layer), src_pages.data_ptr(), dst_pages.data_ptr(),
                               valid_len.data_ptr() if valid_len is not None else None, src_pages.shape[0],
                               page_size, hkv, d, num_pages, _dtype_code(dt0, "copy_kv_pages"),
                               _err_word(dev).data_ptr(), _stream(dev)), "copy_kv_pages")


# ---------------------------------------------------------------------------------------
# attention wrappers
# ---------------------------------------------------------------------------------------
def _check_workspace(ws: torch.Tensor) -> None:
    _require_cuda(ws, "workspace_buffer")
    if ws.dtype != torch.uint8 or ws.dim() != 1 or not ws.is_contiguous():
        raise ValueError("workspace_buffer must be a contiguous 1-D uint8 tensor")
    if ws.numel() < COUNTER_BYTES:
        raise ValueError(f"workspace_buffer must hold at least {COUNTER_BYTES} bytes")


def _attn_options(window_left: int, sinks: Optional[torch.Tensor], num_qo_heads: int):
    """ctypes `piekv_attn_options` (or None when there is neither a window nor sinks)."""
    if window_left < 0 and sinks is None:
        return None
    o = _lib.AttnOptions()
    o.window_left = int(window_left) if window_left >= 0 else -1
    o.reserved = 0
    o.sinks = None
    if sinks is not None:
        _require_cuda(sinks, "sinks")
        if sinks.dtype != torch.float32 or sinks.dim() != 1 or sinks.shape[0] != num_qo_heads or \
                not sinks.is_contiguous():
            raise ValueError(f"sinks must be a contiguous float32 tensor of {num_qo_heads} entries (one per query "
                             f"head), got {tuple(sinks.shape)} {sinks.dtype}")
        o.sinks = sinks.data_ptr()
    return o


class BatchDecodeWithPagedKVCacheWrapper:
    """One query token per request against its paged K/V.

    Reference construction and use: pie/src/pie_worker/model/llama3.py:293-300 (CUDA-graph form
    bound to static index buffers), 311-313, plan 766-777, run 689.  `plan()` only records the
    index tensors: the work partition is computed on the device inside `run()`, so the same planned
    wrapper can be replayed from a CUDA graph while the buffers' contents change."""

    def __init__(self, float_workspace_buffer: torch.Tensor, kv_layout: str = "NHD", use_cuda_graph: bool = False,
                 use_tensor_cores: bool = False, paged_kv_indptr_buffer: Optional[torch.Tensor] = None,
                 paged_kv_indices_buffer: Optional[torch.Tensor] = None,
                 paged_kv_last_page_len_buffer: Optional[torch.Tensor] = None, **_ignored) -> None:
        if kv_layout != "NHD":
            raise ValueError(f"kv_layout {kv_layout!r} is not supported (NHD only)")
        _check_workspace(float_workspace_buffer)
        self.workspace_buffer = float_workspace_buffer
        self.kv_layout = kv_layout
        self.use_cuda_graph = use_cuda_graph
        self._fixed = None
        if use_cuda_graph:
            for name, t in (("paged_kv_indptr_buffer", paged_kv_indptr_buffer),
                            ("paged_kv_indices_buffer", paged_kv_indices_buffer),
                            ("paged_kv_last_page_len_buffer", paged_kv_last_page_len_buffer)):
                if t is None:
                    raise ValueError(f"{name} is required when use_cuda_graph=True")
                _require_i32(t, name)
            self._fixed = (paged_kv_indptr_buffer, paged_kv_indices_buffer, paged_kv_last_page_len_buffer)
        # split-KV arrival counters live at the head of the workspace and must start at zero
        float_workspace_buffer[:COUNTER_BYTES].zero_()
        self._plan = None

    def plan(self, indptr: torch.Tensor, indices: torch.Tensor, last_page_len: torch.Tensor, num_qo_heads: int,
             num_kv_heads: int, head_dim: int, page_size: int, pos_encoding_mode: str = "NONE",
             window_left: int = -1, logits_soft_cap: Optional[float] = None,
             q_data_type: torch.dtype = torch.float16, kv_data_type: Optional[torch.dtype] = None,
             data_type: Optional[torch.dtype] = None, sm_scale: Optional[float] = None, **_ignored) -> None:
        _require_i32(indptr, "indptr")
        _require_i32(indices, "indices")
        _require_i32(last_page_len, "last_page_len")
        if pos_encoding_mode != "NONE":
            raise ValueError("pos_encoding_mode other than 'NONE' is not supported; apply RoPE before the append")
        if logits_soft_cap not in (None, 0.0):
            raise ValueError("logits_soft_cap is not supported")
        if window_left is None or window_left < -1:
            raise ValueError("window_left must be -1 (no window) or >= 0")
        if num_qo_heads % num_kv_heads != 0:
            raise ValueError(f"num_qo_heads {num_qo_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if kv_data_type is not None and kv_data_type != q_data_type:
            raise ValueError("kv_data_type must equal q_data_type")
        batch = indptr.shape[0] - 1
        if last_page_len.shape[0] < batch:
            raise ValueError("last_page_len shorter than the batch")
        if self._fixed is not None:
            fi, fx, fl = self._fixed
            if fi.shape[0] != batch + 1 or fl.shape[0] < batch:
                raise ValueError("batch size differs from the buffers this CUDA-graph wrapper was bound to")
            if fi.data_ptr() != indptr.data_ptr():
                fi.copy_(indptr, non_blocking=True)
            if fx.data_ptr() != indices.data_ptr():
                if indices.shape[0] > fx.shape[0]:
                    raise ValueError("indices longer than paged_kv_indices_buffer")
                fx[: indices.shape[0]].copy_(indices, non_blocking=True)
            if fl.data_ptr() != last_page_len.data_ptr():
                fl[:batch].copy_(last_page_len[:batch], non_blocking=True)
            indptr, indices, last_page_len = fi, fx, fl
        need = lib.piekv_decode_workspace_bytes(batch, num_qo_heads, num_kv_heads, head_dim)
        if self.workspace_buffer.numel() < need:
            raise ValueError(f"workspace_buffer too small: {self.workspace_buffer.numel()} < {need} bytes")
        self._plan = dict(indptr=indptr, indices=indices, last_page_len=last_page_len, batch=batch,
                          hq=int(num_qo_heads), hkv=int(num_kv_heads), d=int(head_dim), page_size=int(page_size),
                          dtype=q_data_type, window_left=int(window_left),
                          sm_scale=float(sm_scale) if sm_scale is not None else 1.0 / math.sqrt(head_dim))

    def run(self, q: torch.Tensor, paged_kv_cache: torch.Tensor, out: Optional[torch.Tensor] = None,
            return_lse: bool = False, sinks: Optional[torch.Tensor] = None, sm_scale: Optional[float] = None):
        """`sinks` (float32 [num_qo_heads]) and `sm_scale` are extensions: per-head attention-sink logits and
        a scale that overrides the planned one (the sink wrapper of the reference passes both at run time)."""
        if self._plan is None:
            raise RuntimeError("Must call plan() before run()")
        pl = self._plan
        _require_cuda(q, "q")
        num_pages, page_size, hkv, d = _check_pool(paged_kv_cache)
        qs = _rows(q, "q")
        if tuple(q.shape) != (pl["batch"], pl["hq"], pl["d"]):
            raise ValueError(f"q shape {tuple(q.shape)} differs from the plan "
                             f"({pl['batch']}, {pl['hq']}, {pl['d']})")
        if (page_size, hkv, d) != (pl["page_size"], pl["hkv"], pl["d"]):
            raise ValueError("paged_kv_cache shape differs from the plan")
        if q.dtype != paged_kv_cache.dtype:
            raise ValueError(f"q dtype {q.dtype} differs from the cache dtype {paged_kv_cache.dtype}")
        if out is None:
            out = torch.empty((pl["batch"], pl["hq"], pl["d"]), dtype=q.dtype, device=q.device)
        elif tuple(out.shape) != tuple(q.shape) or out.dtype != q.dtype or not out.is_contiguous():
            raise ValueError("out must be a contiguous tensor shaped and typed like q")
        lse = torch.empty((pl["batch"], pl["hq"]), dtype=torch.float32, device=q.device) if return_lse else None
        ws = self.workspace_buffer
        opt = _attn_options(pl["window_left"], sinks, pl["hq"])
        check(lib.piekv_decode_run_opt(q.data_ptr(), qs[0], qs[1], paged_kv_cache.data_ptr(), out.data_ptr(),
                                       lse.data_ptr() if lse is not None else None, pl["indptr"].data_ptr(),
                                       pl["indices"].data_ptr(), pl["last_page_len"].data_ptr(), pl["batch"],
                                       pl["hq"], pl["hkv"], pl["d"], pl["page_size"], num_pages,
                                       _dtype_code(q.dtype, "decode run"),
                                       float(sm_scale) if sm_scale is not None else pl["sm_scale"], ws.data_ptr(),
                                       ws.numel(), _err_word(q.device).data_ptr(), _stream(q.device),
                                       C.byref(opt) if opt is not None else None), "BatchDecode.run")
        return (out, lse) if return_lse else out

    forward = run

    def _fused_inputs(self, q, k, v, pos_ids, paged_kv_cache):
        """Checks shared by the fused entry points; returns (plan, num_pages, d, batch, q / k / v row strides)."""
        if self._plan is None:
            raise RuntimeError("Must call plan() before run()")
        pl = self._plan
        for t, name in ((q, "q"), (k, "k"), (v, "v")):
            _require_cuda(t, name)
        _require_i32(pos_ids, "pos_ids")
        num_pages, page_size, hkv, d = _check_pool(paged_kv_cache)
        qs, ks, vs = _rows(q, "q"), _rows(k, "k"), _rows(v, "v")
        b = pl["batch"]
        if tuple(q.shape) != (b, pl["hq"], pl["d"]) or tuple(k.shape) != (b, pl["hkv"], pl["d"]) \
                or tuple(v.shape) != tuple(k.shape) or pos_ids.shape[0] < b:
            raise ValueError(f"q {tuple(q.shape)} / k {tuple(k.shape)} / v {tuple(v.shape)} differ from the plan")
        if (page_size, hkv, d) != (pl["page_size"], pl["hkv"], pl["d"]):
            raise ValueError("paged_kv_cache shape differs from the plan")
        return pl, num_pages, d, b, qs, ks, vs

    def run_fused(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pos_ids: torch.Tensor,
                  paged_kv_cache: torch.Tensor, rope: Optional["RopeConfig"] = None,
                  out: Optional[torch.Tensor] = None, return_lse: bool = False,
                  sinks: Optional[torch.Tensor] = None):
        """One decode step in a single launch: RoPE of q and of the new k at `pos_ids`, append of k / v
        into the last slot of every request's last page, attention over all pages.  Equivalent to the
        reference's per-layer sequence at pie/src/pie_worker/model/llama3.py:660-689, except that q and
        k are read only (not rotated in place).  The planned page table must already include the new
        token, as it does in the reference."""
        pl, num_pages, d, b, qs, ks, vs = self._fused_inputs(q, k, v, pos_ids, paged_kv_cache)
        if not (q.dtype == k.dtype == v.dtype == paged_kv_cache.dtype):
            raise ValueError("q, k, v and the cache must share one dtype")
        if out is None:
            out = torch.empty((b, pl["hq"], pl["d"]), dtype=q.dtype, device=q.device)
        elif tuple(out.shape) != tuple(q.shape) or out.dtype != q.dtype or not out.is_contiguous():
            raise ValueError("out must be a contiguous tensor shaped and typed like q")
        lse = torch.empty((b, pl["hq"]), dtype=torch.float32, device=q.device) if return_lse else None
        rp = (rope if rope is not None else RopeConfig()).to_c(d)
        ws = self.workspace_buffer
        opt = _attn_options(pl["window_left"], sinks, pl["hq"])
        check(lib.piekv_decode_step_fused_opt(q.data_ptr(), k.data_ptr(), v.data_ptr(), qs[0], qs[1], ks[0], ks[1],
                                              vs[0], vs[1], pos_ids.data_ptr(), paged_kv_cache.data_ptr(),
                                              out.data_ptr(), lse.data_ptr() if lse is not None else None,
                                              pl["indptr"].data_ptr(), pl["indices"].data_ptr(),
                                              pl["last_page_len"].data_ptr(), b, pl["hq"], pl["hkv"], pl["d"],
                                              pl["page_size"], num_pages, _dtype_code(q.dtype, "fused decode"),
                                              C.byref(rp), pl["sm_scale"], ws.data_ptr(), ws.numel(),
                                              _err_word(q.device).data_ptr(), _stream(q.device),
                                              C.byref(opt) if opt is not None else None),
              "BatchDecode.run_fused")
        return (out, lse) if return_lse else out

    def run_fused_peer(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pos_ids: torch.Tensor,
                       paged_kv_cache: torch.Tensor, peers, rope: Optional["RopeConfig"] = None,
                       counted: bool = False) -> torch.Tensor:
        """`run_fused` for head-sharded ranks (the reference's tensor parallelism,
        pie/src/pie_worker/model/llama3.py:607-610): this rank's heads are stored into the output rows of
        every rank by the kernel itself (`peers`: a `pie_b200.parallel.PeerOutputs`), the wait for the
        other ranks' rows is queued on the stream, and the full [batch, all heads, head_dim] tensor of
        this rank is returned.  Takes the place of attention followed by an NCCL collective.

        `counted=True` takes the step number from the device-side counter of `peers` instead of a launch
        argument, which makes the two launches capturable in a CUDA graph that is replayed step after step;
        call `peers.advance(n)` after every replay of a graph that holds n such steps (an eager counted
        call advances by itself).  Do not mix counted and uncounted steps on one `PeerOutputs`."""
        pl, num_pages, d, b, qs, ks, vs = self._fused_inputs(q, k, v, pos_ids, paged_kv_cache)
        if not (q.dtype == k.dtype == v.dtype == paged_kv_cache.dtype == peers.dtype):
            raise ValueError("q, k, v, the cache and the peer buffers must share one dtype")
        if b > peers.batch_max or d != peers.head_dim or pl["hq"] * peers.world > peers.row_heads:
            raise ValueError("peer buffers are too small for this plan")
        if pl["window_left"] >= 0:
            raise ValueError("run_fused_peer does not take a sliding window")
        if b == 0:
            # Nothing would be launched, so no flag would be raised: every rank (they share the page tables)
            # skips the step number and the wait instead of spinning until the wait's time limit.
            return peers.full(0)
        rp = (rope if rope is not None else RopeConfig()).to_c(d)
        ws = self.workspace_buffer
        desc = peers.counted_descriptor() if counted else peers.begin_step()
        check(lib.piekv_decode_step_fused_peer(q.data_ptr(), k.data_ptr(), v.data_ptr(), qs[0], qs[1], ks[0], ks[1],
                                               vs[0], vs[1], pos_ids.data_ptr(), paged_kv_cache.data_ptr(),
                                               C.byref(desc), pl["indptr"].data_ptr(), pl["indices"].data_ptr(),
                                               pl["last_page_len"].data_ptr(), b, pl["hq"], pl["hkv"], pl["d"],
                                               pl["page_size"], num_pages, _dtype_code(q.dtype, "fused decode"),
                                               C.byref(rp), pl["sm_scale"], ws.data_ptr(), ws.numel(),
                                               _err_word(q.device).data_ptr(), _stream(q.device)),
              "BatchDecode.run_fused_peer")
        if counted:
            peers.wait_counted()
            if not torch.cuda.is_current_stream_capturing():
                peers.advance()
        else:
            peers.wait()
        return peers.full(b)


class BatchPrefillWithPagedKVCacheWrapper:
    """Packed variable-length (prefill / chunked / multi-token) attention over paged K/V.

    Reference construction and use: pie/src/pie_worker/model/llama3.py:307-309, plan 779-791,
    run 689.  `custom_mask` is the flat boolean mask of pie/src/pie_worker/batching.py:113-135:
    for every query token a row of kv_len_b entries.

    Extension: `plan(..., brle_mask=(runs, indptr, mask_bits))` takes the mask in its wire form (per
    query token a list of alternating attend / skip run lengths, `pie_b200.batching.Batch.brle_inputs`)
    and builds the bit-packed mask on the device; the flat boolean mask is never materialised."""

    def __init__(self, float_workspace_buffer: torch.Tensor, kv_layout: str = "NHD", **_ignored) -> None:
        if kv_layout != "NHD":
            raise ValueError(f"kv_layout {kv_layout!r} is not supported (NHD only)")
        _check_workspace(float_workspace_buffer)
        self.workspace_buffer = float_workspace_buffer
        self.kv_layout = kv_layout
        float_workspace_buffer[:COUNTER_BYTES].zero_()
        self._plan = None

    def plan(self, qo_indptr: torch.Tensor, paged_kv_indptr: torch.Tensor, paged_kv_indices: torch.Tensor,
             paged_kv_last_page_len: torch.Tensor, num_qo_heads: int, num_kv_heads: int, head_dim_qk: int,
             page_size: int, head_dim_vo: Optional[int] = None, custom_mask: Optional[torch.Tensor] = None,
             packed_custom_mask: Optional[torch.Tensor] = None, causal: bool = False,
             pos_encoding_mode: str = "NONE", window_left: int = -1, logits_soft_cap: Optional[float] = None,
             sm_scale: Optional[float] = None, q_data_type: torch.dtype = torch.float16,
             kv_data_type: Optional[torch.dtype] = None, brle_mask=None, **_ignored) -> None:
        _require_i32(qo_indptr, "qo_indptr")
        _require_i32(paged_kv_indptr, "paged_kv_indptr")
        _require_i32(paged_kv_indices, "paged_kv_indices")
        _require_i32(paged_kv_last_page_len, "paged_kv_last_page_len")
        if pos_encoding_mode != "NONE":
            raise ValueError("pos_encoding_mode other than 'NONE' is not supported; apply RoPE before the append")
        if logits_soft_cap not in (None, 0.0):
            raise ValueError("logits_soft_cap is not supported")
        if window_left < -1:
            raise ValueError("window_left must be -1 (no window) or >= 0")
        if packed_custom_mask is not None:
            raise ValueError("packed_custom_mask is not supported; pass the boolean custom_mask")
        if head_dim_vo is not None and head_dim_vo != head_dim_qk:
            raise ValueError("head_dim_vo must equal head_dim_qk")
        if num_qo_heads % num_kv_heads != 0:
            raise ValueError(f"num_qo_heads {num_qo_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if kv_data_type is not None and kv_data_type != q_data_type:
            raise ValueError("kv_data_type must equal q_data_type")
        if paged_kv_indptr.shape[0] != qo_indptr.shape[0]:
            raise ValueError("qo_indptr and paged_kv_indptr describe different batch sizes")
        mask = None
        if custom_mask is not None:
            _require_cuda(custom_mask, "custom_mask")
            if custom_mask.dtype not in (torch.bool, torch.uint8) or not custom_mask.is_contiguous():
                raise ValueError("custom_mask must be a contiguous bool (or uint8) tensor")
            mask = custom_mask.view(torch.uint8) if custom_mask.dtype == torch.bool else custom_mask
            causal = False  # the mask alone decides, as in the reference
        brle = None
        if brle_mask is not None:
            if custom_mask is not None:
                raise ValueError("pass either custom_mask or brle_mask, not both")
            runs, run_indptr, mask_bits = brle_mask
            _require_cuda(runs, "brle runs")
            _require_i32(run_indptr, "brle indptr")
            if runs.dtype not in (torch.int32, torch.uint32) or not runs.is_contiguous():
                raise ValueError("brle runs must be a contiguous int32 / uint32 tensor")
            if page_size != 16 or head_dim_qk != 128 or q_data_type not in (torch.float16, torch.bfloat16):
                raise ValueError("brle_mask needs the tensor-core prefill path (fp16/bf16, head_dim 128, page size 16)")
            if run_indptr.shape[0] < 1:
                raise ValueError("brle indptr must have nnz + 1 entries")
            brle = (runs, run_indptr, int(mask_bits))
            causal = False
        window_entries = 0
        if window_left >= 0 and custom_mask is None and brle is None:
            # A window without a mask becomes a packed mask on the device (the query at position p sees keys
            # p - window_left .. p, or .. kv_len - 1 when not causal); kv tiles outside every window of a query
            # tile are then skipped through the mask summary.  Its size needs sum(qo_len * kv_len): one small
            # device reduction read back here (plan() is a host-synchronous call in the reference as well).
            if page_size == 16 and head_dim_qk == 128 and q_data_type in (torch.float16, torch.bfloat16):
                counts = (qo_indptr[1:] - qo_indptr[:-1]).to(torch.int64)
                seq = get_seq_lens(paged_kv_indptr, paged_kv_last_page_len, page_size).to(torch.int64)
                window_entries = int((counts * seq).sum().item())
        batch = qo_indptr.shape[0] - 1
        self._plan = dict(qo_indptr=qo_indptr, indptr=paged_kv_indptr, indices=paged_kv_indices,
                          last_page_len=paged_kv_last_page_len, batch=batch, hq=int(num_qo_heads),
                          hkv=int(num_kv_heads), d=int(head_dim_qk), page_size=int(page_size), mask=mask,
                          mask_bytes=int(mask.numel()) if mask is not None else (brle[2] if brle else window_entries),
                          brle=brle, causal=bool(causal), dtype=q_data_type, planned_for=None,
                          window_left=int(window_left),
                          sm_scale=float(sm_scale) if sm_scale is not None else 1.0 / math.sqrt(head_dim_qk))

    def _device_plan(self, n: int, num_pages: int) -> None:
        """Build the work list (and pack the mask) on the device once per plan(); later run() calls
        of the same batch - one per layer in the reference - reuse it."""
        pl = self._plan
        key = (n, num_pages)
        if pl["planned_for"] == key:
            return
        ws = self.workspace_buffer
        need = lib.piekv_prefill_workspace_bytes(pl["batch"], n, pl["hq"], pl["d"], num_pages, pl["mask_bytes"])
        if ws.numel() < need:
            raise ValueError(f"workspace_buffer too small: {ws.numel()} < {need} bytes")
        dev = pl["qo_indptr"].device
        runs_ptr = rptr_ptr = None
        if pl["brle"] is not None:
            runs, run_indptr, _ = pl["brle"]
            if run_indptr.shape[0] != n + 1:
                raise ValueError(f"brle indptr has {run_indptr.shape[0]} entries for {n} query tokens")
            runs_ptr, rptr_ptr = runs.data_ptr(), run_indptr.data_ptr()
        check(lib.piekv_prefill_plan_opt(pl["qo_indptr"].data_ptr(), pl["indptr"].data_ptr(),
                                         pl["last_page_len"].data_ptr(),
                                         pl["mask"].data_ptr() if pl["mask"] is not None else None, runs_ptr, rptr_ptr,
                                         pl["mask_bytes"], 1 if pl["causal"] else 0, pl["window_left"], pl["batch"], n,
                                         pl["page_size"], num_pages, ws.data_ptr(), ws.numel(),
                                         _err_word(dev).data_ptr(), _stream(dev)), "BatchPrefill.plan")
        pl["planned_for"] = key

    def run(self, q: torch.Tensor, paged_kv_cache: torch.Tensor, out: Optional[torch.Tensor] = None,
            return_lse: bool = False, sinks: Optional[torch.Tensor] = None, sm_scale: Optional[float] = None):
        """`sinks` (float32 [num_qo_heads]) and `sm_scale` are extensions, see the decode wrapper's run()."""
        if self._plan is None:
            raise RuntimeError("Must call plan() before run()")
        pl = self._plan
        _require_cuda(q, "q")
        num_pages, page_size, hkv, d = _check_pool(paged_kv_cache)
        qs = _rows(q, "q")
        n = q.shape[0]
        if tuple(q.shape[1:]) != (pl["hq"], pl["d"]):
            raise ValueError(f"q shape {tuple(q.shape)} differs from the plan (*, {pl['hq']}, {pl['d']})")
        if (page_size, hkv, d) != (pl["page_size"], pl["hkv"], pl["d"]):
            raise ValueError("paged_kv_cache shape differs from the plan")
        if q.dtype != paged_kv_cache.dtype:
            raise ValueError(f"q dtype {q.dtype} differs from the cache dtype {paged_kv_cache.dtype}")
        if out is None:
            out = torch.empty((n, pl["hq"], pl["d"]), dtype=q.dtype, device=q.device)
        elif tuple(out.shape) != tuple(q.shape) or out.dtype != q.dtype or not out.is_contiguous():
            raise ValueError("out must be a contiguous tensor shaped and typed like q")
        lse = torch.empty((n, pl["hq"]), dtype=torch.float32, device=q.device) if return_lse else None
        ws = self.workspace_buffer
        self._device_plan(n, num_pages)
        opt = _attn_options(pl["window_left"], sinks, pl["hq"])
        check(lib.piekv_prefill_run_opt(q.data_ptr(), qs[0], qs[1], paged_kv_cache.data_ptr(), out.data_ptr(),
                                        lse.data_ptr() if lse is not None else None, pl["qo_indptr"].data_ptr(),
                                        pl["indptr"].data_ptr(), pl["indices"].data_ptr(),
                                        pl["last_page_len"].data_ptr(),
                                        pl["mask"].data_ptr() if pl["mask"] is not None else None, pl["mask_bytes"],
                                        1 if pl["causal"] else 0, 2 if pl["brle"] is not None else 1, pl["batch"], n,
                                        pl["hq"], pl["hkv"], pl["d"],
                                        pl["page_size"], num_pages, _dtype_code(q.dtype, "prefill run"),
                                        float(sm_scale) if sm_scale is not None else pl["sm_scale"], ws.data_ptr(),
                                        ws.numel(), _err_word(q.device).data_ptr(), _stream(q.device),
                                        C.byref(opt) if opt is not None else None), "BatchPrefill.run")
        return (out, lse) if return_lse else out

    forward = run

    def export_custom_mask(self, num_query_tokens: int, num_pages: int) -> torch.Tensor:
        """The mask this plan holds on the device (from bytes, run lengths and / or a window) in the reference's
        flat boolean form (pie/src/pie_worker/batching.py:113-135): for checking a device-built mask against
        the reference's, or for a consumer that still wants that tensor."""
        if self._plan is None:
            raise RuntimeError("Must call plan() before run()")
        pl = self._plan
        if pl["page_size"] != 16:
            raise ValueError("the packed mask exists for page size 16 only")
        self._device_plan(int(num_query_tokens), int(num_pages))
        flat = torch.zeros(pl["mask_bytes"], dtype=torch.uint8, device=pl["qo_indptr"].device)
        ws = self.workspace_buffer
        check(lib.piekv_prefill_export_mask(pl["qo_indptr"].data_ptr(), pl["indptr"].data_ptr(),
                                            pl["last_page_len"].data_ptr(), pl["mask_bytes"], pl["batch"],
                                            int(num_query_tokens), 16, int(num_pages), ws.data_ptr(), ws.numel(),
                                            flat.data_ptr(), _stream(flat.device)), "BatchPrefill.export_custom_mask")
        return flat.view(torch.bool)


class BatchAttentionWithAttentionSinkWrapper(BatchPrefillWithPagedKVCacheWrapper):
    """Paged attention with per-head attention sinks and an optional sliding window fixed at construction.

    Reference construction and use: pie/src/pie_worker/model/gpt_oss.py:418-439 (two wrappers, one with
    `window_left = sliding_window - 1`, one without), plan 840-870 (the prefill wrapper's positional
    arguments with `causal=True` and the same window), run 693-697: `run(q, kv_cache_layer, sinks, scaling)`.
    The head's sink logit joins the softmax normaliser only.  Decode batches (one query token per request)
    go through the same planned call."""

    def __init__(self, float_workspace_buffer: torch.Tensor, kv_layout: str = "NHD", window_left: int = -1,
                 q_data_type: Optional[torch.dtype] = None, kv_data_type: Optional[torch.dtype] = None,
                 head_dim_qk: Optional[int] = None, head_dim_vo: Optional[int] = None, **_ignored) -> None:
        super().__init__(float_workspace_buffer, kv_layout)
        if head_dim_qk is not None and head_dim_vo is not None and head_dim_qk != head_dim_vo:
            raise ValueError("head_dim_vo must equal head_dim_qk")
        if kv_data_type is not None and q_data_type is not None and kv_data_type != q_data_type:
            raise ValueError("kv_data_type must equal q_data_type")
        self._window_left = int(window_left)
        self._q_data_type = q_data_type

    def plan(self, qo_indptr, paged_kv_indptr, paged_kv_indices, paged_kv_last_page_len, num_qo_heads, num_kv_heads,
             head_dim_qk, page_size, causal: bool = False, window_left: Optional[int] = None,
             q_data_type: Optional[torch.dtype] = None, kv_data_type: Optional[torch.dtype] = None,
             non_blocking: bool = True, **kw) -> None:
        wl = self._window_left if window_left is None else int(window_left)
        dt = q_data_type or self._q_data_type or torch.float16
        super().plan(qo_indptr, paged_kv_indptr, paged_kv_indices, paged_kv_last_page_len, num_qo_heads, num_kv_heads,
                     head_dim_qk, page_size, causal=causal, window_left=wl, q_data_type=dt, kv_data_type=kv_data_type,
                     **kw)

    def run(self, q: torch.Tensor, paged_kv_cache: torch.Tensor, sinks: Optional[torch.Tensor] = None,
            sm_scale: Optional[float] = None, out: Optional[torch.Tensor] = None, return_lse: bool = False):
        if sinks is not None and sinks.dtype != torch.float32:
            sinks = sinks.to(torch.float32)
        return super().run(q, paged_kv_cache, out=out, return_lse=return_lse, sinks=sinks, sm_scale=sm_scale)

    forward = run
