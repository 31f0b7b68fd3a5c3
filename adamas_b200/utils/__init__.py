"""Host runtime of the decode path with the operator names of the reference's ``adamas.utils``
(adamas/utils/__init__.py:11-24)."""
from typing import Optional

import torch

from .. import _kernels
from .controller import InferenceController
from .decode_wrapper import BatchDecodeWithPagedKVCacheWrapper
from .kv_cache import KvCache
from .sequence_batch import SequenceBatch
from .utils import TensorLayout

__all__ = [
    "TensorLayout",
    "KvCache",
    "InferenceController",
    "BatchDecodeWithPagedKVCacheWrapper",
    "apply_rope_in_place",
    "append_kvh",
    "append_qkv_fused",
    "decode_estimate",
    "decode_topk",
    "decode_sparse_attn",
    "decode_step",
    "decode_step_dev",
    "seq_len_advance",
    "SequenceBatch",
]


def apply_rope_in_place(q: torch.Tensor, k: torch.Tensor, past_kv_len: int, rope_scale: Optional[float] = None,
                        rope_theta: Optional[float] = None):
    """Rotary embedding of q, k [N,H,D] in place (adamas/utils/__init__.py:26-53)."""
    _kernels.apply_rope_in_place(q, k, past_kv_len, 1.0 if rope_scale is None else rope_scale,
                                 1e4 if rope_theta is None else rope_theta)


def append_kvh(k: torch.Tensor, v: torch.Tensor, h: Optional[torch.Tensor], iController: InferenceController,
               layer_idx: int):
    """Append new keys/values and their 2-bit codes (adamas/utils/__init__.py:94-157).

    k, v [N,H,D].  Prefill (N > 1): h [N,H,D] = hadamard_transform(k), or None to have the
    transform computed in the same launch.  Decode (N == 1): h [2,H,D] =
    hadamard_transform(cat(q, k)); returns the packed query code [1,H,D/8].
    """
    seq_len, num_heads, head_dim = k.shape
    c = iController
    if seq_len > 1:
        _kernels.append_kv_cache_prefill(
            k, v, h,
            c.kv_cache.buf_layer(layer_idx), c.kv_indices_with_last, None, c.kv_cache.last_page_len,
            c.kv_last_page_idx,
            c.hadamard_cache.buf_layer(layer_idx), c.hadamard_indices, None, c.hadamard_cache.last_page_len,
            c.hadamard_last_page_idx, c.layout)
        return None
    o = torch.empty(seq_len, num_heads, head_dim // 8, dtype=h.dtype, device=h.device)
    _kernels.append_kv_cache_decode(
        k, v, h, o,
        c.kv_cache.buf_layer(layer_idx), c.kv_indices_with_last, None, c.kv_cache.last_page_len,
        c.kv_last_page_idx,
        c.hadamard_cache.buf_layer(layer_idx), c.hadamard_indices, None, c.hadamard_cache.last_page_len,
        c.hadamard_last_page_idx, c.layout)
    return o


def append_qkv_fused(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, iController: InferenceController,
                     layer_idx: int, scale: Optional[float] = None,
                     out: Optional[torch.Tensor] = None, rope=None) -> torch.Tensor:
    """Decode-step append with the Hadamard transform inside: replaces torch.cat((q, k)),
    hadamard_transform and append_kvh (adamas/models/Adamas.py:145-161) with one launch.
    Returns the packed query code [1,H,D/8] (written into `out` when given).  rope=(rope_scale,
    rope_theta): q and k are un-rotated and get rotated in place inside the same launch."""
    c = iController
    o = out if out is not None else torch.empty(1, q.size(1), k.size(2) // 8, dtype=k.dtype, device=k.device)
    _kernels.append_kv_cache_decode_fused(
        q, k, v, o, c.kv_cache.buf_layer(layer_idx), c.kv_indices_with_last, c.kv_cache.last_page_len,
        c.hadamard_cache.buf_layer(layer_idx), c.hadamard_indices, c.hadamard_cache.last_page_len,
        c.layout, scale, rope=rope)
    return o


def decode_estimate(q: torch.Tensor, iController: InferenceController, layer_idx: int,
                    metric: str = "l1") -> torch.Tensor:
    """Distance of the packed query code q [1,H,D/8] to every cached key code except the newest
    token's -> [H, seqlen-1] (adamas/utils/__init__.py:203-237)."""
    c = iController
    o = c.estimate_buffer(c.hadamard_cache.seqlen - 1)
    _kernels.estimate_attn_score(q, o, c.hadamard_cache.buf_layer(layer_idx), c.hadamard_indices, None,
                                 c.hadamard_cache.last_page_len, c.hadamard_last_page_idx, c.layout, metric)
    return o


def decode_topk(estimated_attn_score: torch.Tensor, iController: InferenceController):
    """Pick the budget-1 smallest distances per head; results land in iController.topk_dout_buffer /
    topk_dindices_buffer (adamas/utils/__init__.py:239-269).  At page_size 1 the indices are page ids
    as in the reference; otherwise physical token slots page*page_size + entry."""
    c = iController
    k = c.inference_token_budget - 1
    _kernels.topk_select(estimated_attn_score, k, c.topk_dindices_buffer, c.topk_dout_buffer,
                         page_table=c.kv_indices_with_last, page_size=c.page_size)


def decode_sparse_attn(q: torch.Tensor, iController: InferenceController, layer_idx: int,
                       topk_indices: torch.Tensor, rope_scale: Optional[float] = None,
                       rope_theta: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention over the selected pages/tokens plus the newest token
    (adamas/utils/__init__.py:271-308).  q [1,H,D] -> o [1,H,D].  `topk_indices` is either
    iController.topk_dindices_buffer (selected tokens) or iController.kv_indices_without_last (all
    pages: the dense path).  The result is written into `out` when given."""
    c = iController
    o = out if out is not None else torch.empty_like(q)
    token_granular = c.page_size > 1 and topk_indices is not c.kv_indices_without_last
    c._decode_handler.forward(q, o, c.kv_cache.buf_layer(layer_idx), topk_indices, None,
                              c.kv_cache.last_page_len, c.kv_last_page_idx, rope_scale, rope_theta,
                              token_granular=token_granular)
    return o


def decode_step(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, iController: InferenceController,
                layer_idx: int, out: Optional[torch.Tensor] = None, record_indices: bool = True,
                scale: Optional[float] = None, rope=None) -> torch.Tensor:
    """The whole decode branch of the attention module (adamas/models/Adamas.py:145-200: cat,
    Hadamard, append, estimate, top-k, sparse attention) in one call and two or three launches.

    q, k, v [1,H,D] after RoPE, or before it with rope=(rope_scale, rope_theta): q and k are then
    rotated in place by the append launch (apply_rope_in_place, Adamas.py:113).  Returns o [1,H,D].  When the context still fits in the budget
    (iController.need_estimate() is False, e.g. the dense first layers) it appends and attends to
    every page instead.  With record_indices the selected token slots are also written to
    iController.topk_dindices_buffer, as decode_topk would."""
    c = iController
    o = out if out is not None else torch.empty_like(q)
    if not c.need_estimate():
        append_qkv_fused(q, k, v, c, layer_idx, scale=scale, rope=rope)
        return decode_sparse_attn(q, c, layer_idx, c.kv_indices_without_last, out=o)
    n = c.hadamard_cache.seqlen - 1
    _kernels.decode_step(
        q, k, v, o, c.q_code_scratch(k.dtype), c.kv_cache.buf_layer(layer_idx), c.kv_indices_with_last,
        c.kv_cache.last_page_len, c.kv_last_page_idx, c.hadamard_cache.buf_layer(layer_idx), c.hadamard_indices,
        c.hadamard_cache.last_page_len, c.inference_token_budget, c.distance_scratch(n), c.hist_scratch,
        indices_out=c.topk_dindices_buffer if record_indices else None, scale=scale, rope=rope)
    return o


def decode_step_dev(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, iController: InferenceController,
                    layer_idx: int, out: Optional[torch.Tensor] = None, dense: bool = False,
                    scale: Optional[float] = None, rope=None) -> torch.Tensor:
    """decode_step whose launches do not depend on the sequence length: the kernels read it from
    iController.seq_len_dev, so the call can be captured in a CUDA graph once and replayed for every
    token (the reference re-plans on the host every step: adamas/utils/controller.py:82-131,
    kernels/include/decode/decode_handler.cuh:73-121).  Per token the host still reserves cache room
    (prepare_hadamard(1), which uploads a new page number when a page fills up); the device length is
    advanced with seq_len_advance at the END of the token's work (or set with sync_seq_len()).

    dense=True: append and attend to every token (the first layers of the reference's model);
    otherwise the sparse step at the controller's token budget, which needs a longer context.
    rope: None, (rope_scale, rope_theta) or {"inv_freq": tensor[64], "mscale": float}."""
    c = iController
    o = out if out is not None else torch.empty_like(q)
    kv_table = c.kv_cache.table_all()
    code_table = c.hadamard_cache.table_all()
    if dense:
        c._decode_handler.dense_step_dev(q, k, v, o, c.q_code_scratch(k.dtype), c.kv_cache.buf_layer(layer_idx),
                                         kv_table, c.hadamard_cache.buf_layer(layer_idx), code_table, c.seq_len_dev,
                                         c.max_seq_len, scale=scale, rope=rope)
        return o
    _kernels.decode_step_dev(q, k, v, o, c.q_code_scratch(k.dtype), c.kv_cache.buf_layer(layer_idx), kv_table,
                             c.hadamard_cache.buf_layer(layer_idx), code_table, c.seq_len_dev, c.max_seq_len,
                             c.token_budget(), c.distance_scratch(c.max_seq_len - 1), c.hist_scratch,
                             scale=scale, rope=rope)
    return o


def seq_len_advance(iController: InferenceController, delta: int = 1) -> None:
    """iController.seq_len_dev += delta on the device (one capturable launch)."""
    _kernels.seq_len_advance(iController.seq_len_dev, delta)
