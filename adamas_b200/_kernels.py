"""Operator module with the surface of the reference's pybind extension ``adamas._kernels``
(adamas/ops/csrc/bsk_ops.cu:4-21, declarations adamas/ops/csrc/bsk_ops.h:23-124).

Same function names, argument order and meaning, and the same error behaviour (bad shapes,
dtypes or devices raise ``RuntimeError``, as ``TORCH_CHECK`` does).  Each function checks its
tensors and hands raw device pointers to the C ABI in ``libadamas_b200.so``; torch is used for
memory and streams only.  All launches go to torch's current CUDA stream.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import _lib
from ._lib import lib

NHD, HND = 0, 1
DEFAULT_THRESHOLDS = (-10.0, 0.0, 10.0)


# ----------------------------------------------------------------------------------------------
# checks (the reference's CHECK_INPUT / CHECK_DIM / CHECK_EQ, pytorch_extension_utils.h:52-66)
# ----------------------------------------------------------------------------------------------
def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_input(t: torch.Tensor, name: str, dim: Optional[int] = None) -> None:
    _require(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _require(t.is_cuda, f"{name} must be a CUDA tensor")
    _require(t.is_contiguous(), f"{name} must be contiguous")
    if dim is not None:
        _require(t.dim() == dim, f"{name} must be a {dim}D tensor")


def _check_rows(t: torch.Tensor, name: str) -> None:
    """2-D CUDA tensor whose rows are dense; the row stride may exceed the row length or be 0
    (one row shared by all heads)."""
    _require(isinstance(t, torch.Tensor) and t.is_cuda, f"{name} must be a CUDA tensor")
    _require(t.dim() == 2, f"{name} must be a 2D tensor")
    _require(t.size(1) <= 1 or t.stride(1) == 1, f"{name} must have unit stride along its rows")
    _require(t.size(0) <= 1 or t.stride(0) == 0 or t.stride(0) >= t.size(1), f"{name} has overlapping rows")


def _dtype_code(dtype: torch.dtype, what: str) -> int:
    if dtype == torch.float16:
        return _lib.F16
    if dtype == torch.bfloat16:
        return _lib.BF16
    raise RuntimeError(f"{what} failed to dispatch with dtype {dtype}")


def _value_format(dtype: torch.dtype, what: str) -> int:
    if dtype == torch.float16:
        return _lib.VAL_F16
    if dtype in (torch.int16, torch.uint16):
        return _lib.VAL_U16
    raise RuntimeError(f"{what} failed to dispatch with dtype {dtype}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
    """The current CUDA stream of the current device as a raw handle."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _nhd_only(layout: int) -> None:
    _require(int(layout) == NHD, "only the NHD layout is implemented (the reference's controller always uses it)")


# ----------------------------------------------------------------------------------------------
# stage 1
# ----------------------------------------------------------------------------------------------
def hadamard_transform(x: torch.Tensor, inplace: bool = False, scale: Optional[float] = None) -> torch.Tensor:
    """Stand-in for ``faster_hadamard_transform.hadamard_transform`` (call sites
    adamas/models/Adamas.py:120,150): Walsh-Hadamard transform of the last dimension (128),
    scaled by 1/sqrt(128) unless `scale` is given, result in x.dtype."""
    _check_input(x, "x")
    _require(x.size(-1) == 128, "hadamard_transform supports a last dimension of 128")
    y = x if inplace else torch.empty_like(x)
    rows = x.numel() // 128
    s = 1.0 / math.sqrt(128.0) if scale is None else float(scale)
    _lib.check(lib.adamas_hadamard_transform(_ptr(x), _ptr(y), rows, 128, s,
                                             _dtype_code(x.dtype, "hadamard_transform"), _stream()),
               "hadamard_transform")
    return y


def apply_rope_in_place(q: torch.Tensor, k: torch.Tensor, past_kv_len: int, rope_scale: float = 1.0,
                        rope_theta: float = 1e4) -> None:
    """adamas/ops/csrc/page.cu:228-269.  q [N,Hq,D], k [N,Hk,D] rotated in place; token s has
    position past_kv_len + s; linear position scaling by rope_scale."""
    _check_input(q, "q", 3)
    _check_input(k, "k", 3)
    _require(q.size(0) == k.size(0) and q.size(2) == k.size(2) == 128 and q.dtype == k.dtype,
             "q and k must be [N, H, 128] of one dtype")
    _lib.check(lib.adamas_apply_rope_in_place(_ptr(q), _ptr(k), q.size(0), q.size(1), k.size(1), 128,
                                              int(past_kv_len), float(rope_scale), float(rope_theta),
                                              _dtype_code(q.dtype, "apply_rope_in_place"), _stream()),
               "apply_rope_in_place")


def bucketize_pack(h: torch.Tensor, o: torch.Tensor, thresholds=None) -> None:
    """o[..., w] = packed 2-bit buckets of h[..., 8w:8w+8] (kernels/include/decode/decode_page.cuh:380-398)."""
    _check_input(h, "h")
    _check_input(o, "o")
    _require(h.size(-1) == 128 and o.size(-1) == 16, "h must end in 128 and o in 16")
    _require(o.element_size() == 2 and o.numel() * 8 == h.numel(), "o must hold one 16-bit word per 8 values")
    _lib.check(lib.adamas_bucketize_pack(_ptr(h), _ptr(o), h.numel() // 128, 128, _lib.thresholds_arg(thresholds),
                                         _dtype_code(h.dtype, "bucketize_pack"), _stream()), "bucketize_pack")


def pack_2bit(h: torch.Tensor, o: torch.Tensor, past_kv_len: int = 0) -> None:
    """adamas/ops/csrc/page.cu:271-298 under its reference name: o[..., w] = packed 2-bit codes of the
    already transformed values h[..., 8w:8w+8] (default thresholds).  `past_kv_len` is accepted for
    the reference's signature; the packing does not depend on it."""
    bucketize_pack(h, o)


def histogram_scratch(num_heads: int, device) -> torch.Tensor:
    """A zeroed scratch table for decode_step / select_attend: per head 16 histograms of 512 32-bit
    counts, then the slots through which the thread blocks of a head pass their partial results.
    Every call that uses it leaves the histograms all zero, so one table serves all steps of a
    sequence; calls that may overlap on the GPU need separate tables."""
    return torch.zeros(num_heads, _lib.HIST_WORDS_PER_HEAD, dtype=torch.int32, device=device)


def histogram_counts(hist: torch.Tensor) -> torch.Tensor:
    """The [H, 16, 512] histogram part of a histogram_scratch table."""
    return hist.view(hist.size(0), -1)[:, : 16 * 512].view(hist.size(0), 16, 512)


def _check_hist(hist: Optional[torch.Tensor], num_heads: int) -> Optional[torch.Tensor]:
    if hist is not None:
        _require(hist.is_cuda and hist.is_contiguous() and hist.dtype == torch.int32
                 and hist.numel() >= num_heads * _lib.HIST_WORDS_PER_HEAD,
                 "hist must be a contiguous int32 CUDA tensor made by histogram_scratch(H)")
    return hist


def select_attend_slices(n: int, k: int, num_heads: int) -> int:
    """Thread blocks per head (= histogram slices) select_attend uses for rows of n distances."""
    out = ctypes.c_int(0)
    _lib.check(lib.adamas_select_attend_slices(int(n), int(k), int(num_heads), ctypes.byref(out)), "select_attend_slices")
    return out.value


def _check_append(k, v, kv_data, kv_indices, hadamard_data, hadamard_indices, layout):
    _nhd_only(layout)
    _check_input(k, "k", 3)
    _check_input(v, "v", 3)
    _check_input(kv_data, "kv_data", 5)
    _check_input(kv_indices, "kv_indices", 1)
    _check_input(hadamard_data, "hadamard_data", 5)
    _check_input(hadamard_indices, "hadamard_indices", 1)
    _require(kv_indices.dtype == torch.int32, "kv_indices must be int32")
    _require(hadamard_indices.dtype == torch.int32, "hadamard_indices must be int32")
    num_heads, head_dim = k.size(1), k.size(2)
    _require(tuple(v.shape) == tuple(k.shape), "k and v must have the same shape")
    page_size = kv_data.size(2)
    _require(kv_data.size(1) == 2 and kv_data.size(3) == num_heads and kv_data.size(4) == head_dim,
             "kv_data must be [pages, 2, page_size, num_heads, head_dim]")
    _require(hadamard_data.size(1) == 1 and hadamard_data.size(2) == page_size
             and hadamard_data.size(3) == num_heads and hadamard_data.size(4) == head_dim // 8,
             "hadamard_data must be [pages, 1, page_size, num_heads, head_dim/8]")
    _require(kv_data.dtype == k.dtype and v.dtype == k.dtype, "k, v and kv_data must share a dtype")
    _require(hadamard_data.element_size() == 2, "hadamard_data must have 16-bit elements")
    return num_heads, head_dim, page_size


def _query_heads(q, k, name: str) -> int:
    """Query heads of q [1, Hq, D] over the cache heads of k [1, H, D]: Hq a multiple of H (grouped-query
    attention when larger; the reference supports Hq == H only, kernels/include/decode/decode_handler.cuh:83)."""
    _require(q.dim() == 3 and q.size(0) == 1 and q.size(2) == k.size(2) and q.dtype == k.dtype
             and q.size(1) >= k.size(1) and q.size(1) % k.size(1) == 0,
             f"{name}: q must be [1, Hq, D] in k.dtype with Hq a multiple of the cache's heads")
    return q.size(1)


def append_kv_cache_decode(k, v, h, o, kv_data, kv_indices, kv_indptr, kv_last_page_len, kv_last_page_idx,
                           hadamard_data, hadamard_indices, hadamard_indptr, hadamard_last_page_len,
                           hadamard_last_page_idx, layout, thresholds=None) -> None:
    """adamas/ops/csrc/page.cu:6-109.  k, v [1,H,D]; h [2,H,D] = Hadamard(q), Hadamard(k);
    o [1,H,D/8] receives the packed query code.  The indptr tensors are [0, len(indices)]."""
    num_heads, head_dim, page_size = _check_append(k, v, kv_data, kv_indices, hadamard_data, hadamard_indices, layout)
    _check_input(h, "h", 3)
    _check_input(o, "o", 3)
    _require(k.size(0) == 1 and v.size(0) == 1 and h.size(0) == 2 and o.size(0) == 1, "decode appends one token")
    _require(h.size(1) == num_heads and h.size(2) == head_dim and h.dtype == k.dtype, "h must be [2, H, D] in k.dtype")
    _require(o.size(1) == num_heads and o.size(2) == head_dim // 8 and o.element_size() == 2, "o must be [1, H, D/8] 16-bit")
    _lib.check(lib.adamas_append_decode(
        _ptr(k), _ptr(v), _ptr(h), _ptr(o),
        _ptr(kv_data), _ptr(kv_indices), kv_indices.numel(), int(kv_last_page_len),
        _ptr(hadamard_data), _ptr(hadamard_indices), hadamard_indices.numel(), int(hadamard_last_page_len),
        num_heads, head_dim, page_size, _lib.thresholds_arg(thresholds),
        _dtype_code(k.dtype, "Append_kv_cache_decode"), _stream()), "Append_kv_cache_decode")


def append_kv_cache_decode_fused(q, k, v, o, kv_data, kv_indices, kv_last_page_len, hadamard_data,
                                 hadamard_indices, hadamard_last_page_len, layout=NHD, scale=None,
                                 thresholds=None, rope=None) -> None:
    """One launch for torch.cat((q, k)) + hadamard_transform + append_kv_cache_decode
    (adamas/models/Adamas.py:145-161).  With rope=(rope_scale, rope_theta), or a frequency table
    {"inv_freq": tensor[64], "mscale": float}, q and k arrive un-rotated and are rotated in place first
    (also replaces apply_rope_in_place, Adamas.py:113).  q may have a multiple of k's heads."""
    num_heads, head_dim, page_size = _check_append(k, v, kv_data, kv_indices, hadamard_data, hadamard_indices, layout)
    _check_input(q, "q", 3)
    _check_input(o, "o", 3)
    _require(k.size(0) == 1, "k, v must be [1, H, D]")
    q_heads = _query_heads(q, k, "append_kv_cache_decode_fused")
    _require(o.size(1) == q_heads and o.size(2) == head_dim // 8 and o.element_size() == 2, "o must be [1, Hq, D/8] 16-bit")
    s = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
    if rope is not None:
        rs, rt, inv_freq, mscale = _rope_args(rope)
        _lib.check(lib.adamas_append_decode_rope_fused(
            _ptr(q), _ptr(k), _ptr(v), _ptr(o),
            _ptr(kv_data), _ptr(kv_indices), kv_indices.numel(), int(kv_last_page_len),
            _ptr(hadamard_data), _ptr(hadamard_indices), hadamard_indices.numel(), int(hadamard_last_page_len),
            num_heads, q_heads, head_dim, page_size, s, _lib.thresholds_arg(thresholds), rs if inv_freq is None else 1.0,
            rt if inv_freq is None else 1e4, _ptr(inv_freq), mscale,
            _dtype_code(k.dtype, "append_kv_cache_decode_rope_fused"), _stream()), "append_kv_cache_decode_rope_fused")
        return
    _lib.check(lib.adamas_append_decode_fused(
        _ptr(q), _ptr(k), _ptr(v), _ptr(o),
        _ptr(kv_data), _ptr(kv_indices), kv_indices.numel(), int(kv_last_page_len),
        _ptr(hadamard_data), _ptr(hadamard_indices), hadamard_indices.numel(), int(hadamard_last_page_len),
        num_heads, q_heads, head_dim, page_size, s, _lib.thresholds_arg(thresholds),
        _dtype_code(k.dtype, "append_kv_cache_decode_fused"), _stream()), "append_kv_cache_decode_fused")


def append_kv_cache_prefill(k, v, h, kv_data, kv_indices, kv_indptr, kv_last_page_len, kv_last_page_idx,
                            hadamard_data, hadamard_indices, hadamard_indptr, hadamard_last_page_len,
                            hadamard_last_page_idx, layout, scale=None, thresholds=None) -> None:
    """adamas/ops/csrc/page.cu:111-226.  k, v, h [N,H,D]; h = Hadamard(k).  Passing h=None
    computes the transform inside the same launch."""
    num_heads, head_dim, page_size = _check_append(k, v, kv_data, kv_indices, hadamard_data, hadamard_indices, layout)
    if h is not None:
        _check_input(h, "h", 3)
        _require(tuple(h.shape) == tuple(k.shape) and h.dtype == k.dtype, "h must match k")
    s = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
    _lib.check(lib.adamas_append_prefill(
        _ptr(k), _ptr(v), _ptr(h), k.size(0),
        _ptr(kv_data), _ptr(kv_indices), kv_indices.numel(), int(kv_last_page_len),
        _ptr(hadamard_data), _ptr(hadamard_indices), hadamard_indices.numel(), int(hadamard_last_page_len),
        num_heads, head_dim, page_size, s, _lib.thresholds_arg(thresholds),
        _dtype_code(k.dtype, "Append_kv_cache_prefill"), _stream()), "Append_kv_cache_prefill")


# ----------------------------------------------------------------------------------------------
# stage 2
# ----------------------------------------------------------------------------------------------
def estimate_attn_score(q, o, metadata_data, metadata_indices, metadata_indptr, metadata_last_page_len,
                        metadata_last_page_idx, layout, metric: str = "l1", exclude_last: bool = True,
                        hist: Optional[torch.Tensor] = None, hist_slices: int = 0) -> None:
    """adamas/ops/csrc/estimate.cu:6-84.  q [1,H,D/8] packed query code; o [H, n] with
    n = (pages-1)*page_size + last_page_len - 1 (newest token excluded); o.dtype float16 stores the
    distances as fp16 (reference), int16 as integers.  exclude_last=False covers every cached token
    (a sequence shard that does not hold the newest token).  `hist` (a zeroed histogram_scratch(H))
    additionally receives the per-slice counts that select_attend(..., hist_ready=True) reads;
    hist_slices = select_attend_slices(n, k, H) of that call."""
    _nhd_only(layout)
    _check_input(q, "q", 3)
    _check_rows(o, "o")
    _check_input(metadata_data, "hadamard_data", 5)
    _check_input(metadata_indices, "hadamard_indices", 1)
    _require(q.size(0) == 1, "q.size(0) must be 1")
    _require(metadata_indices.dtype == torch.int32, "hadamard_indices must be int32")
    q_heads, code_words = q.size(1), q.size(2)
    page_size = metadata_data.size(2)
    num_heads = metadata_data.size(3)          # heads of the cache; q_heads is a multiple of it
    _require(q_heads >= num_heads and q_heads % num_heads == 0 and metadata_data.size(4) == code_words
             and code_words == 16, "hadamard_data must be [pages, 1, page_size, num_heads, 16], q [1, Hq, 16]")
    _require(q.element_size() == 2 and metadata_data.element_size() == 2, "codes must be 16-bit words")
    n = (metadata_indices.numel() - 1) * page_size + int(metadata_last_page_len) - (1 if exclude_last else 0)
    _require(o.size(0) == q_heads and o.size(1) == n, f"o must be [{q_heads}, {n}]")
    _lib.check(lib.adamas_estimate(
        _ptr(q), _ptr(metadata_data), _ptr(metadata_indices), metadata_indices.numel(),
        int(metadata_last_page_len), page_size, num_heads, q_heads, code_words * 8, _ptr(o), o.stride(0),
        _value_format(o.dtype, "Estimate_attn_score"),
        {"l1": _lib.METRIC_L1, "xor": _lib.METRIC_XOR}[metric], 1 if exclude_last else 0,
        _ptr(_check_hist(hist, q_heads)), int(hist_slices), _stream()),
        "Estimate_attn_score")


# ----------------------------------------------------------------------------------------------
# stage 3
# ----------------------------------------------------------------------------------------------
def topk_filtering(estimated_value, estimated_indices, d_out, indices_out, buf, page_budget) -> None:
    """adamas/ops/csrc/topk.cu:7-46.  Selects the `page_budget` smallest entries of every row of
    estimated_value [H, n] and writes their values to d_out [H, k] and the matching entries of
    estimated_indices [H, n] to indices_out [H, k].  `buf` (the reference's radix scratch) is
    accepted and unused.  Unlike the reference the result is deterministic: equal values are taken
    lowest position first and rows are emitted in ascending position order."""
    _check_rows(estimated_value, "estimated_value")
    _check_rows(estimated_indices, "estimated_indices")
    _check_rows(d_out, "d_out")
    _check_rows(indices_out, "indices_out")
    _require(d_out.stride(0) == indices_out.stride(0), "d_out and indices_out must share a row stride")
    rows, n = estimated_value.shape
    k = int(page_budget)
    _require(tuple(estimated_indices.shape) == (rows, n), "estimated_indices must match estimated_value")
    _require(estimated_indices.dtype == torch.int32 and indices_out.dtype == torch.int32, "indices must be int32")
    _require(n >= k, "num_pages must be >= page_budget")
    _require(d_out.size(1) == k and indices_out.size(1) == k, "outputs must have page_budget columns")
    _require(d_out.size(0) == rows and indices_out.size(0) == rows, "outputs must have one row per head")
    _require(d_out.dtype == estimated_value.dtype, "d_out must have the dtype of estimated_value")
    _lib.check(lib.adamas_topk(
        _ptr(estimated_value), _value_format(estimated_value.dtype, "Top-k filtering"), estimated_value.stride(0), n,
        _ptr(estimated_indices), estimated_indices.stride(0), 1, rows, k,
        _ptr(d_out), _ptr(indices_out), indices_out.stride(0), _stream()), "Top-k filtering")


def topk_select(values, k, indices_out, values_out=None, page_table=None, page_size=1) -> None:
    """Token-granular select used when page_size > 1: positions p of the k smallest values per row
    are mapped through one page table shared by all rows, out = page_table[p // page_size] *
    page_size + p % page_size (or p itself when page_table is None)."""
    _check_rows(values, "values")
    _check_rows(indices_out, "indices_out")
    rows, n = values.shape
    _require(indices_out.dtype == torch.int32 and indices_out.size(0) == rows and indices_out.size(1) >= k,
             "indices_out must be int32 [rows, >=k]")
    if values_out is not None:
        _check_rows(values_out, "values_out")
        _require(values_out.dtype == values.dtype and values_out.stride(0) == indices_out.stride(0),
                 "values_out must match values.dtype and the row stride of indices_out")
    if page_table is not None:
        _check_input(page_table, "page_table", 1)
        _require(page_table.dtype == torch.int32 and page_table.numel() * page_size >= n, "page_table too short")
    _lib.check(lib.adamas_topk(
        _ptr(values), _value_format(values.dtype, "topk_select"), values.stride(0), n,
        _ptr(page_table), 0, int(page_size), rows, int(k),
        _ptr(values_out), _ptr(indices_out), indices_out.stride(0), _stream()), "topk_select")


# ----------------------------------------------------------------------------------------------
# stage 4
# ----------------------------------------------------------------------------------------------
class BatchDecodeWithPagedKVCachePyTorchWrapper:
    """adamas/ops/csrc/bsk_ops.h:95-124, adamas/ops/csrc/approx_attn.cu:27-151."""

    def __init__(self, layout: int):
        _nhd_only(layout)
        self._layout = int(layout)
        self._handle = ctypes.c_void_p()
        _lib.check(lib.adamas_decode_handler_create(ctypes.byref(self._handle)), "BatchDecodeWithPagedKVCache")
        self._started = False
        self._planned_tokens = 0
        self._cfg = None

    def __del__(self):
        h = getattr(self, "_handle", None)
        if h and lib is not None:          # `lib` is already gone when the interpreter shuts down
            try:
                lib.adamas_decode_handler_destroy(h)
            except Exception:
                pass
            self._handle = None

    def begin_forward(self, indptr, num_qo_heads, num_kv_heads, head_dim, page_size, empty_data) -> None:
        _require(indptr.dim() == 1 and indptr.dtype == torch.int32 and indptr.is_contiguous(),
                 "indptr must be a contiguous 1D int32 tensor")
        _require(num_qo_heads >= num_kv_heads >= 1 and num_qo_heads % num_kv_heads == 0,
                 "num_qo_heads must be a multiple of num_kv_heads")
        self._cfg = (int(num_qo_heads), int(head_dim), int(page_size),
                     _dtype_code(empty_data.dtype, "BatchDecodeWithPagedKVCache"))
        self._kv_heads = int(num_kv_heads)
        self._batch = max(1, indptr.numel() - 1)      # the reference's indptr has one entry per sequence, plus one
        self._started = True
        self._planned_tokens = 0   # scratch is sized on the first forward, from the index tensor

    def end_forward(self) -> None:
        self._started = False
        _lib.check(lib.adamas_decode_end_forward(self._handle), "BatchDecodeWithPagedKVCache")

    def forward(self, q, o, paged_kv_data, paged_kv_indices, paged_kv_indptr, paged_kv_last_page_len,
                paged_kv_last_page_idx, rope_scale=1.0, rope_theta=1e4, token_granular: bool = False,
                lse: Optional[torch.Tensor] = None, tail_len: Optional[int] = None,
                o_f32: Optional[torch.Tensor] = None) -> None:
        """q, o [1,H,D]; paged_kv_indices [H, n] per-head page ids (the reference's meaning: each
        page is attended in full, then the last page's last_page_len entries).  With
        token_granular=True the entries are physical token slots (page*page_size + entry) and only
        the newest token is appended; negative entries are holes.  `tail_len` overrides the number of
        trailing entries of the last page that are always attended (0: none, for a shard that does
        not hold the newest token).  With `o_f32` (float32 [H, D], needs `lse`) the result is written
        there unrounded instead of into `o` (partial result of a sequence shard)."""
        if not self._started:
            raise RuntimeError("BatchDecodeWithPagedKVCache failed with error: forward called before begin_forward")
        _check_input(q, "q", 3)
        if o_f32 is None:
            _check_input(o, "o", 3)
        _check_input(paged_kv_data, "paged_kv_data", 5)
        _check_rows(paged_kv_indices, "paged_kv_indices")
        num_heads, head_dim, page_size, dt = self._cfg
        _require(q.size(0) == 1 and q.size(1) == num_heads and q.size(2) == head_dim, "q must be [1, H, D]")
        _require(o_f32 is not None or (tuple(o.shape) == tuple(q.shape) and o.dtype == q.dtype), "o must match q")
        _require(paged_kv_data.size(1) == 2 and paged_kv_data.size(2) == page_size
                 and paged_kv_data.size(3) == self._kv_heads and paged_kv_data.size(4) == head_dim,
                 "paged_kv_data must be [pages, 2, page_size, H_kv, D]")
        _require(paged_kv_indices.size(0) == num_heads and paged_kv_indices.dtype == torch.int32,
                 "paged_kv_indices must be int32 [H, n]")
        _require(_dtype_code(q.dtype, "BatchDecodeWithPagedKVCache") == dt and paged_kv_data.dtype == q.dtype,
                 "dtype differs from begin_forward")
        n_idx = paged_kv_indices.size(1)
        unit = 1 if token_granular else page_size
        tail = 1 if token_granular else int(paged_kv_last_page_len)
        if tail_len is not None:
            tail = int(tail_len)
        n_tokens = n_idx * unit + tail
        if n_tokens > self._planned_tokens:
            _lib.check(lib.adamas_decode_begin_forward(self._handle, n_tokens, self._batch, self._kv_heads, num_heads,
                                                       head_dim, page_size, dt, _stream()), "BatchDecodeWithPagedKVCache")
            self._planned_tokens = n_tokens
        if lse is not None:
            _require(lse.is_cuda and lse.dtype == torch.float32 and lse.numel() == num_heads and lse.is_contiguous(),
                     "lse must be a contiguous float32 CUDA tensor of H elements")
        if o_f32 is not None:
            _require(lse is not None and o_f32.is_cuda and o_f32.dtype == torch.float32 and o_f32.is_contiguous()
                     and o_f32.numel() == num_heads * head_dim, "o_f32 must be float32 [H, D] and lse given")
            _lib.check(lib.adamas_decode_forward_partial(
                self._handle, _ptr(q), _ptr(o_f32), _ptr(lse), _ptr(paged_kv_data), _ptr(paged_kv_indices),
                paged_kv_indices.stride(0), n_idx, unit, int(paged_kv_last_page_idx), int(paged_kv_last_page_len),
                tail, 1.0 / math.sqrt(head_dim), _stream()), "BatchDecodeWithPagedKVCache")
            return
        _lib.check(lib.adamas_decode_forward(
            self._handle, _ptr(q), _ptr(o), _ptr(lse), _ptr(paged_kv_data), _ptr(paged_kv_indices),
            paged_kv_indices.stride(0), n_idx, unit, int(paged_kv_last_page_idx), int(paged_kv_last_page_len), tail,
            1.0 / math.sqrt(head_dim), _stream()), "BatchDecodeWithPagedKVCache")


    def dense_step_dev(self, q, k, v, o, q_code, kv_data, kv_indices, hadamard_data, hadamard_indices,
                       seq_len: torch.Tensor, max_seq_len: int, scale: Optional[float] = None, thresholds=None,
                       rope=None, lse: Optional[torch.Tensor] = None) -> None:
        """The dense layers' decode step with the sequence length in device memory (see
        decode_step_dev): fused append (with the rotary embedding when `rope` is given) and attention
        over all seq_len tokens, shaped by max_seq_len only, so that it can be captured in a graph."""
        if not self._started:
            raise RuntimeError("BatchDecodeWithPagedKVCache failed with error: dense step called before begin_forward")
        num_heads, head_dim, page_size = _check_append(k, v, kv_data, kv_indices, hadamard_data, hadamard_indices, NHD)
        cfg_heads, cfg_dim, cfg_ps, dt = self._cfg
        _check_input(q, "q", 3)
        _check_input(o, "o", 3)
        _check_input(q_code, "q_code", 3)
        _check_seq_len(seq_len)
        q_heads = _query_heads(q, k, "dense_step_dev")
        _require((q_heads, num_heads, head_dim, page_size) == (cfg_heads, self._kv_heads, cfg_dim, cfg_ps)
                 and _dtype_code(k.dtype, "dense_step_dev") == dt, "cache geometry differs from begin_forward")
        _require(tuple(q.shape) == tuple(o.shape) and k.size(0) == 1, "q, o must be [1, Hq, D], k, v [1, H, D]")
        _require(kv_indices.numel() * page_size >= max_seq_len, "the page table must have room for max_seq_len tokens")
        if max_seq_len > self._planned_tokens:
            _lib.check(lib.adamas_decode_begin_forward(self._handle, int(max_seq_len), self._batch, num_heads, q_heads,
                                                       head_dim, page_size, dt, _stream()), "BatchDecodeWithPagedKVCache")
            self._planned_tokens = int(max_seq_len)
        s = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
        rs, rt, inv_freq, mscale = _rope_args(rope)
        _lib.check(lib.adamas_dense_step_dev(
            self._handle, _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), _ptr(q_code), _ptr(kv_data),
            _ptr(kv_indices), _ptr(hadamard_data), _ptr(hadamard_indices), _ptr(seq_len), int(max_seq_len),
            num_heads, q_heads, head_dim, page_size, dt, s, _lib.thresholds_arg(thresholds), rs, rt, _ptr(inv_freq),
            mscale, 1.0 / math.sqrt(head_dim), _stream()), "dense_step_dev")

    def dense_step_batch_dev(self, q, k, v, o, q_code, seqs, seq_lens, max_seq_len: int, page_size: int,
                              scale: Optional[float] = None, thresholds=None, rope=None,
                              lse: Optional[torch.Tensor] = None) -> None:
        """dense_step_dev for several sequences in the same launches (shapes as decode_step_batch_dev).  The
        wrapper must have been begun with an indptr of batch + 1 entries."""
        if not self._started:
            raise RuntimeError("BatchDecodeWithPagedKVCache failed with error: dense step called before begin_forward")
        batch, num_heads, q_heads = _check_batch(q, k, v, o, q_code, seqs, seq_lens, "dense_step_batch_dev")
        cfg_heads, cfg_dim, cfg_ps, dt = self._cfg
        _require((q_heads, num_heads, 128, int(page_size)) == (cfg_heads, self._kv_heads, cfg_dim, cfg_ps)
                 and _dtype_code(k.dtype, "dense_step_batch_dev") == dt and batch <= self._batch,
                 "cache geometry or batch differs from begin_forward")
        if max_seq_len > self._planned_tokens:
            _lib.check(lib.adamas_decode_begin_forward(self._handle, int(max_seq_len), self._batch, num_heads, q_heads,
                                                       128, cfg_ps, dt, _stream()), "BatchDecodeWithPagedKVCache")
            self._planned_tokens = int(max_seq_len)
        s = 1.0 / math.sqrt(128.0) if scale is None else float(scale)
        rs, rt, inv_freq, mscale = _rope_args(rope)
        _lib.check(lib.adamas_dense_step_batch_dev(
            self._handle, _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), _ptr(q_code), _ptr(seqs), _ptr(seq_lens), batch,
            int(max_seq_len), num_heads, q_heads, 128, cfg_ps, dt, s, _lib.thresholds_arg(thresholds), rs, rt,
            _ptr(inv_freq), mscale, 1.0 / math.sqrt(128.0), _stream()), "dense_step_batch_dev")



def set_max_cluster(blocks: int) -> None:
    """Upper bound (1, 2, 4, 8) on the thread blocks that share one head in select_attend /
    decode_step: 8 is fastest for a single sequence, smaller values let calls of several sequences
    on different streams overlap."""
    _lib.check(lib.adamas_set_max_cluster(int(blocks)), "set_max_cluster")


def set_estimate_blocks_per_sm(blocks: int) -> None:
    """1 or 2 (default) resident blocks of the estimate kernel per SM; 1 leaves room for kernels of other
    sequences running on other streams."""
    _lib.check(lib.adamas_set_estimate_blocks_per_sm(int(blocks)), "set_estimate_blocks_per_sm")


def set_fused_append(enable: bool) -> None:
    """decode_step with the append folded into the estimate launch (two launches, the default for 16,
    32 or 64 heads) or as three launches; the results are identical."""
    _lib.check(lib.adamas_set_fused_append(int(bool(enable))), "set_fused_append")


def select_attend(dist: torch.Tensor, k: int, q: torch.Tensor, o: Optional[torch.Tensor], kv_data: torch.Tensor,
                  kv_indices: torch.Tensor, last_page_len: int, last_page_idx: int,
                  indices_out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None,
                  hist: Optional[torch.Tensor] = None, hist_ready: bool = False,
                  ext_cut: Optional[torch.Tensor] = None, o_f32: Optional[torch.Tensor] = None) -> None:
    """Top-k and sparse attention in one launch (replaces topk_filtering + the decode wrapper's
    forward, adamas/models/Adamas.py:185-200).  dist int16 [H, n] integer distances with rows on
    16-byte boundaries; q, o [1,H,D]; kv_indices int32 page table; indices_out optional int32
    [H, >=k] receiving the winners' token slots.  last_page_len = 0: no newest token is attended.
    hist: a histogram_scratch(H) (made for the call when None); hist_ready: an estimate call has
    already counted the distances into it.  ext_cut int32 [H, 2]: cut distance and number of
    cut-valued winners of this call per head, decided elsewhere.  o_f32 float32 [H, D] (+ lse):
    unrounded partial result."""
    _check_rows(dist, "dist")
    _check_input(q, "q", 3)
    if o is not None:
        _check_input(o, "o", 3)
    _check_input(kv_data, "kv_data", 5)
    _check_input(kv_indices, "kv_indices", 1)
    _require(dist.dtype in (torch.int16, torch.uint16), "dist must hold 16-bit integer distances")
    h, n = dist.shape
    _require(q.size(0) == 1 and q.size(1) == h and q.size(2) == 128, "q must be [1, H, 128]")
    _require(o is not None or o_f32 is not None, "o or o_f32 must be given")
    _require(o is None or (tuple(o.shape) == tuple(q.shape) and o.dtype == q.dtype), "o must match q")
    page_size = kv_data.size(2)
    kv_heads = kv_data.size(3)
    _require(kv_data.size(1) == 2 and h >= kv_heads >= 1 and h % kv_heads == 0 and kv_data.size(4) == 128
             and kv_data.dtype == q.dtype,
             "kv_data must be [pages, 2, page_size, H_kv, 128] in q.dtype, with H a multiple of H_kv")
    _require(kv_indices.dtype == torch.int32 and kv_indices.numel() * page_size >= n, "page table too short")
    out_stride = 0
    if indices_out is not None:
        _check_rows(indices_out, "indices_out")
        _require(indices_out.dtype == torch.int32 and indices_out.size(0) == h and indices_out.size(1) >= k,
                 "indices_out must be int32 [H, >=k]")
        out_stride = indices_out.stride(0)
    if lse is not None:
        _require(lse.is_cuda and lse.dtype == torch.float32 and lse.numel() == h and lse.is_contiguous(),
                 "lse must be a contiguous float32 CUDA tensor of H elements")
    if o_f32 is not None:
        _require(lse is not None and o_f32.is_cuda and o_f32.dtype == torch.float32 and o_f32.is_contiguous()
                 and o_f32.numel() == h * 128, "o_f32 must be float32 [H, 128] and lse given")
    if ext_cut is not None:
        _require(ext_cut.is_cuda and ext_cut.dtype == torch.int32 and ext_cut.is_contiguous()
                 and tuple(ext_cut.shape) == (h, 2), "ext_cut must be a contiguous int32 CUDA tensor [H, 2]")
    if hist is None:
        _require(not hist_ready, "hist_ready needs the table an estimate call has filled")
        hist = histogram_scratch(h, dist.device)
    _lib.check(lib.adamas_select_attend(
        _ptr(dist), dist.stride(0), n, int(k), _ptr(q), _ptr(o), _ptr(o_f32), _ptr(lse), _ptr(kv_data),
        _ptr(kv_indices), page_size, kv_heads, h, 128, _dtype_code(q.dtype, "select_attend"), int(last_page_idx),
        int(last_page_len), _ptr(_check_hist(hist, h)), 1 if hist_ready else 0, _ptr(ext_cut),
        _ptr(indices_out), out_stride, 1.0 / math.sqrt(128.0), _stream()), "select_attend")


def decode_step(q, k, v, o, q_code, kv_data, kv_indices, kv_last_page_len, kv_last_page_idx, hadamard_data,
                hadamard_indices, hadamard_last_page_len, budget: int, dist_scratch: torch.Tensor,
                hist: torch.Tensor, indices_out: Optional[torch.Tensor] = None,
                lse: Optional[torch.Tensor] = None, scale: Optional[float] = None, thresholds=None,
                rope=None) -> None:
    """One layer's decode step in one call: append + estimate, select + attend (two launches for 16, 32
    or 64 heads, else three, for what adamas/models/Adamas.py:145-200 does with seven).  Needs context > budget.  `hist`: a histogram_scratch(H), all zero between steps.  With
    rope=(rope_scale, rope_theta) or {"inv_freq": tensor[64], "mscale": float} q and k arrive un-rotated
    and are rotated in place first.  q, o may have a multiple of k's heads (grouped-query attention)."""
    num_heads, head_dim, page_size = _check_append(k, v, kv_data, kv_indices, hadamard_data, hadamard_indices, NHD)
    _check_input(q, "q", 3)
    _check_input(o, "o", 3)
    _check_input(q_code, "q_code", 3)
    _check_rows(dist_scratch, "dist_scratch")
    q_heads = _query_heads(q, k, "decode_step")
    _require(tuple(q.shape) == tuple(o.shape) and k.size(0) == 1, "q, o must be [1, Hq, D], k, v [1, H, D]")
    _require(q_code.element_size() == 2 and q_code.numel() == q_heads * head_dim // 8, "q_code must be [1, Hq, D/8] 16-bit")
    _require(dist_scratch.element_size() == 2 and dist_scratch.size(0) == q_heads, "dist_scratch must be 16-bit [Hq, n]")
    out_stride = 0
    if indices_out is not None:
        _check_rows(indices_out, "indices_out")
        _require(indices_out.dtype == torch.int32 and indices_out.size(0) == q_heads
                 and indices_out.size(1) >= budget - 1, "indices_out must be int32 [Hq, >=budget-1]")
        out_stride = indices_out.stride(0)
    s = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
    rs, rt, inv_freq, mscale = _rope_args(rope)
    _lib.check(lib.adamas_decode_step(
        _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), _ptr(q_code),
        _ptr(kv_data), _ptr(kv_indices), kv_indices.numel(), int(kv_last_page_len), int(kv_last_page_idx),
        _ptr(hadamard_data), _ptr(hadamard_indices), hadamard_indices.numel(), int(hadamard_last_page_len),
        num_heads, q_heads, head_dim, page_size, _dtype_code(k.dtype, "decode_step"), int(budget),
        _ptr(dist_scratch), dist_scratch.stride(0), _ptr(_check_hist(hist, q_heads)), _ptr(indices_out), out_stride, s,
        _lib.thresholds_arg(thresholds), rs, rt, _ptr(inv_freq), mscale, 1.0 / math.sqrt(head_dim), _stream()),
        "decode_step")


def _rope_args(rope):
    """rope: None | (rope_scale, rope_theta) | {"inv_freq": float32 CUDA tensor [64], "mscale": float}."""
    if rope is None:
        return 0.0, 0.0, None, 1.0
    if isinstance(rope, dict):
        t = rope["inv_freq"]
        _require(t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and t.numel() == 64,
                 "rope inv_freq must be a contiguous float32 CUDA tensor of 64 elements")
        return 0.0, 0.0, t, float(rope.get("mscale", 1.0))
    return float(rope[0]), float(rope[1]), None, 1.0


def _check_seq_len(seq_len: torch.Tensor, count: int = 1) -> None:
    _require(isinstance(seq_len, torch.Tensor) and seq_len.is_cuda and seq_len.dtype == torch.int32
             and seq_len.is_contiguous() and seq_len.numel() == count,
             f"seq_len must be a contiguous int32 CUDA tensor of {count} element(s)")


def decode_step_dev(q, k, v, o, q_code, kv_data, kv_indices, hadamard_data, hadamard_indices,
                    seq_len: torch.Tensor, max_seq_len: int, budget: int, dist_scratch: torch.Tensor,
                    hist: torch.Tensor, indices_out: Optional[torch.Tensor] = None,
                    lse: Optional[torch.Tensor] = None, scale: Optional[float] = None, thresholds=None,
                    rope=None) -> None:
    """decode_step with the sequence length (tokens in the caches, the new one included) in device
    memory: the launches depend on max_seq_len only, so a CUDA graph captured once serves every token
    (advance `seq_len` with seq_len_advance at the end of each token's work).  kv_indices /
    hadamard_indices: the page tables, with an entry for every page the current length needs."""
    num_heads, head_dim, page_size = _check_append(k, v, kv_data, kv_indices, hadamard_data, hadamard_indices, NHD)
    _check_input(q, "q", 3)
    _check_input(o, "o", 3)
    _check_input(q_code, "q_code", 3)
    _check_rows(dist_scratch, "dist_scratch")
    _check_seq_len(seq_len)
    q_heads = _query_heads(q, k, "decode_step_dev")
    _require(tuple(q.shape) == tuple(o.shape) and k.size(0) == 1, "q, o must be [1, Hq, D], k, v [1, H, D]")
    _require(q_code.element_size() == 2 and q_code.numel() == q_heads * head_dim // 8, "q_code must be [1, Hq, D/8] 16-bit")
    _require(dist_scratch.element_size() == 2 and dist_scratch.size(0) == q_heads
             and dist_scratch.size(1) >= max_seq_len - 1, "dist_scratch must be 16-bit [Hq, >= max_seq_len - 1]")
    _require(kv_indices.numel() * page_size >= max_seq_len and hadamard_indices.numel() * page_size >= max_seq_len,
             "the page tables must have room for max_seq_len tokens")
    out_stride = 0
    if indices_out is not None:
        _check_rows(indices_out, "indices_out")
        _require(indices_out.dtype == torch.int32 and indices_out.size(0) == q_heads
                 and indices_out.size(1) >= budget - 1, "indices_out must be int32 [Hq, >=budget-1]")
        out_stride = indices_out.stride(0)
    s = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
    rs, rt, inv_freq, mscale = _rope_args(rope)
    _lib.check(lib.adamas_decode_step_dev(
        _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), _ptr(q_code), _ptr(kv_data), _ptr(kv_indices),
        _ptr(hadamard_data), _ptr(hadamard_indices), _ptr(seq_len), int(max_seq_len), num_heads, q_heads, head_dim,
        page_size, _dtype_code(k.dtype, "decode_step_dev"), int(budget), _ptr(dist_scratch),
        dist_scratch.stride(0), _ptr(_check_hist(hist, q_heads)), _ptr(indices_out), out_stride, s,
        _lib.thresholds_arg(thresholds), rs, rt, _ptr(inv_freq), mscale, 1.0 / math.sqrt(head_dim), _stream()),
        "decode_step_dev")


def seq_len_advance(seq_len: torch.Tensor, delta: int = 1) -> None:
    """seq_len += delta on the device (every element: one per sequence of a batch), as one launch
    ordered against its neighbours in the stream."""
    _check_seq_len(seq_len, seq_len.numel())
    _lib.check(lib.adamas_seq_len_advance(_ptr(seq_len), seq_len.numel(), int(delta), _stream()), "seq_len_advance")


# ----------------------------------------------------------------------------------------------
# several sequences in one launch
# ----------------------------------------------------------------------------------------------
def dist_histograms(dist: torch.Tensor, hist: torch.Tensor, slices: int) -> None:
    """Counts the integer distance rows `dist` [H, n] into the histogram scratch (`slices` per-slice
    histograms per row): what estimate_attn_score(..., hist=...) does on the side, as a launch of its own."""
    _check_rows(dist, "dist")
    _require(dist.dtype in (torch.int16, torch.uint16), "dist must hold 16-bit integer distances")
    h, n = dist.shape
    _lib.check(lib.adamas_dist_histograms(_ptr(dist), dist.stride(0), n, h, int(slices), _ptr(_check_hist(hist, h)),
                                          _stream()), "dist_histograms")


def sequence_descriptors(kv_datas, code_datas, kv_tables, code_tables) -> torch.Tensor:
    """Device array of adamas_seq_desc_t for one layer: int64 [batch, 4] holding, per sequence, the
    addresses of its KV cache, code cache, KV page table and code page table.  The tensors must stay
    alive (and in place) for as long as the array is used."""
    rows = []
    for kv, cd, kt, ct in zip(kv_datas, code_datas, kv_tables, code_tables):
        _check_input(kv, "kv_data", 5)
        _check_input(cd, "hadamard_data", 5)
        _require(kt.is_cuda and ct.is_cuda and kt.dtype == torch.int32 and ct.dtype == torch.int32
                 and kt.is_contiguous() and ct.is_contiguous(), "page tables must be contiguous int32 CUDA tensors")
        rows.append([kv.data_ptr(), cd.data_ptr(), kt.data_ptr(), ct.data_ptr()])
    _require(len(rows) >= 1, "no sequences")
    return torch.tensor(rows, dtype=torch.int64).to(kv_datas[0].device)


def _check_batch(q, k, v, o, q_code, seqs, seq_lens, name):
    _check_input(q, "q", 3)
    _check_input(k, "k", 3)
    _check_input(v, "v", 3)
    _check_input(o, "o", 3)
    _check_input(q_code, "q_code", 3)
    batch = seqs.size(0)
    _require(seqs.is_cuda and seqs.dtype == torch.int64 and seqs.is_contiguous() and seqs.dim() == 2 and seqs.size(1) == 4,
             "seqs must be the int64 [batch, 4] array sequence_descriptors() makes")
    _check_seq_len(seq_lens, batch)
    _require(k.size(0) == batch and tuple(v.shape) == tuple(k.shape) and k.size(2) == 128 and k.dtype == q.dtype == v.dtype,
             f"{name}: k, v must be [batch, H, 128] in q.dtype")
    num_heads = k.size(1)
    q_heads = q.size(1)
    _require(q.size(0) == batch and q.size(2) == 128 and q_heads >= num_heads and q_heads % num_heads == 0
             and tuple(o.shape) == tuple(q.shape) and o.dtype == q.dtype, f"{name}: q, o must be [batch, Hq, 128]")
    _require(q_code.element_size() == 2 and q_code.numel() == batch * q_heads * 16, "q_code must be [batch, Hq, 16] 16-bit")
    return batch, num_heads, q_heads


def decode_step_batch_dev(q, k, v, o, q_code, seqs: torch.Tensor, seq_lens: torch.Tensor, max_seq_len: int,
                          page_size: int, budget: int, dist_scratch: torch.Tensor, hist: torch.Tensor,
                          indices_out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None,
                          scale: Optional[float] = None, thresholds=None, rope=None) -> None:
    """decode_step_dev for several sequences in the same launches.  q, o [batch, Hq, 128]; k, v
    [batch, H, 128]; q_code [batch, Hq, 16]; seqs: sequence_descriptors() of this layer; seq_lens int32
    [batch]; dist_scratch 16-bit [batch * Hq, >= max_seq_len - 1]; hist: histogram_scratch(batch * Hq);
    indices_out int32 [batch * Hq, >= budget - 1]."""
    batch, num_heads, q_heads = _check_batch(q, k, v, o, q_code, seqs, seq_lens, "decode_step_batch_dev")
    _check_rows(dist_scratch, "dist_scratch")
    rows = batch * q_heads
    _require(dist_scratch.element_size() == 2 and dist_scratch.size(0) == rows and dist_scratch.size(1) >= max_seq_len - 1,
             "dist_scratch must be 16-bit [batch * Hq, >= max_seq_len - 1]")
    out_stride = 0
    if indices_out is not None:
        _check_rows(indices_out, "indices_out")
        _require(indices_out.dtype == torch.int32 and indices_out.size(0) == rows and indices_out.size(1) >= budget - 1,
                 "indices_out must be int32 [batch * Hq, >= budget - 1]")
        out_stride = indices_out.stride(0)
    if lse is not None:
        _require(lse.is_cuda and lse.dtype == torch.float32 and lse.numel() == rows and lse.is_contiguous(),
                 "lse must be a contiguous float32 CUDA tensor of batch * Hq elements")
    s = 1.0 / math.sqrt(128.0) if scale is None else float(scale)
    rs, rt, inv_freq, mscale = _rope_args(rope)
    _lib.check(lib.adamas_decode_step_batch_dev(
        _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), _ptr(q_code), _ptr(seqs), _ptr(seq_lens), batch,
        int(max_seq_len), num_heads, q_heads, 128, int(page_size), _dtype_code(k.dtype, "decode_step_batch_dev"),
        int(budget), _ptr(dist_scratch), dist_scratch.stride(0), _ptr(_check_hist(hist, rows)), _ptr(indices_out),
        out_stride, s, _lib.thresholds_arg(thresholds), rs, rt, _ptr(inv_freq), mscale, 1.0 / math.sqrt(128.0),
        _stream()), "decode_step_batch_dev")


def apply_rope_table_in_place(q: torch.Tensor, k: torch.Tensor, past_kv_len: int, inv_freq: torch.Tensor,
                              mscale: float = 1.0) -> None:
    """apply_rope_in_place with a table of 64 rotation frequencies and a factor on the rotated values
    (YaRN-scaled models) instead of (rope_scale, rope_theta)."""
    _check_input(q, "q", 3)
    _check_input(k, "k", 3)
    _require(q.size(0) == k.size(0) and q.size(2) == k.size(2) == 128 and q.dtype == k.dtype,
             "q and k must be [N, H, 128] of one dtype")
    _, _, t, ms = _rope_args({"inv_freq": inv_freq, "mscale": mscale})
    _lib.check(lib.adamas_apply_rope_table_in_place(_ptr(q), _ptr(k), q.size(0), q.size(1), k.size(1), 128,
                                                    int(past_kv_len), _ptr(t), ms,
                                                    _dtype_code(q.dtype, "apply_rope_table_in_place"), _stream()),
               "apply_rope_table_in_place")


def append_estimate(q, k, v, q_code, kv_data, kv_indices, kv_last_page_len, hadamard_data, hadamard_indices,
                    hadamard_last_page_len, dist: torch.Tensor, scale: Optional[float] = None,
                    thresholds=None, hist: Optional[torch.Tensor] = None, hist_slices: int = 0) -> None:
    """Decode append and distance estimate in one launch (16, 32 or 64 heads; q and k after RoPE): what
    append_kv_cache_decode_fused followed by estimate_attn_score do, with integer (16-bit) distances
    in `dist` [H, >= context-1]."""
    num_heads, head_dim, page_size = _check_append(k, v, kv_data, kv_indices, hadamard_data, hadamard_indices, NHD)
    _check_input(q, "q", 3)
    _check_input(q_code, "q_code", 3)
    _check_rows(dist, "dist")
    _require(tuple(q.shape) == tuple(k.shape) and k.size(0) == 1, "q, k, v must be [1, H, D]")
    _require(q_code.element_size() == 2 and q_code.numel() == num_heads * head_dim // 8, "q_code must be [1, H, D/8] 16-bit")
    _require(dist.element_size() == 2 and dist.size(0) == num_heads, "dist must be 16-bit [H, n]")
    s = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
    _lib.check(lib.adamas_append_estimate(
        _ptr(q), _ptr(k), _ptr(v), _ptr(q_code),
        _ptr(kv_data), _ptr(kv_indices), kv_indices.numel(), int(kv_last_page_len),
        _ptr(hadamard_data), _ptr(hadamard_indices), hadamard_indices.numel(), int(hadamard_last_page_len),
        num_heads, head_dim, page_size, _dtype_code(k.dtype, "append_estimate"),
        _ptr(dist), dist.stride(0), s, _lib.thresholds_arg(thresholds), _ptr(_check_hist(hist, num_heads)),
        int(hist_slices), _stream()), "append_estimate")


def hist_rowsum(hist: torch.Tensor, slices: int, out: torch.Tensor) -> None:
    """out [H, 512] int32 = sum of the first `slices` histogram rows per head of a histogram_scratch
    table an estimate call has filled (a sequence shard's histogram, ready to be exchanged)."""
    h = out.size(0)
    _check_hist(hist, h)
    _require(out.is_cuda and out.dtype == torch.int32 and out.is_contiguous() and tuple(out.shape) == (h, 512),
             "out must be a contiguous int32 CUDA tensor [H, 512]")
    _lib.check(lib.adamas_hist_rowsum(_ptr(hist), h, int(slices), _ptr(out), _stream()), "hist_rowsum")


def global_cut(all_hists: torch.Tensor, shard: int, k: int, ext_cut: torch.Tensor) -> None:
    """all_hists [G, H, 512] int32 (the shards' histograms, ascending token ranges) -> ext_cut [H, 2]
    int32 for shard `shard`: the cut distance of the k smallest distances of the whole sequence and
    this shard's share of the cut-valued elements."""
    _require(all_hists.is_cuda and all_hists.dtype == torch.int32 and all_hists.is_contiguous()
             and all_hists.dim() == 3 and all_hists.size(2) == 512, "all_hists must be int32 [G, H, 512]")
    g, h, _ = all_hists.shape
    _require(ext_cut.is_cuda and ext_cut.dtype == torch.int32 and ext_cut.is_contiguous()
             and tuple(ext_cut.shape) == (h, 2), "ext_cut must be a contiguous int32 CUDA tensor [H, 2]")
    _lib.check(lib.adamas_global_cut(_ptr(all_hists), g, int(shard), h, int(k), _ptr(ext_cut), _stream()), "global_cut")


def merge_states(o_parts: torch.Tensor, lse_parts: torch.Tensor, o: torch.Tensor,
                 lse: Optional[torch.Tensor] = None) -> None:
    """o_parts [P,H,D] fp32 normalised partial outputs, lse_parts [P,H] base-2 -> o [H,D] (or [1,H,D])."""
    _check_input(o_parts, "o_parts", 3)
    _check_input(lse_parts, "lse_parts", 2)
    _check_input(o, "o")
    p, h, d = o_parts.shape
    _require(o_parts.dtype == torch.float32 and lse_parts.dtype == torch.float32, "partials must be float32")
    _require(tuple(lse_parts.shape) == (p, h) and o.numel() == h * d, "shape mismatch")
    _lib.check(lib.adamas_merge_states(_ptr(o_parts), _ptr(lse_parts), p, h, d, _ptr(o), _ptr(lse),
                                       _dtype_code(o.dtype, "merge_states"), _stream()), "merge_states")
