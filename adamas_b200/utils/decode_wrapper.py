"""Host-side owner of a decode-attention handler.

Same public surface as the reference's wrapper (adamas/utils/decode_wrapper.py:11-86: construct with a
layout name, begin_forward once per model forward, forward once per layer, end_forward), so the
controller and the model code drive it unchanged.  What it owns is different: no FlashInfer plan, but
the native handler of this library (split plan and partial-result scratch, sized once per head count
and batch), which is also what the graph-replayable dense steps run on.
"""
from __future__ import annotations

import contextlib
from typing import Iterator, Optional

import torch

from .. import _kernels
from .utils import TensorLayout

_DEFAULT_ROPE_SCALE = 1.0
_DEFAULT_ROPE_THETA = 1e4


def _layout_code(name: str) -> int:
    """'NHD' / 'HND' -> TensorLayout value; anything else is a KeyError, as in the reference."""
    try:
        return getattr(TensorLayout, name)
    except AttributeError:
        raise KeyError("Invalide kv_layout {}".format(name)) from None


class BatchDecodeWithPagedKVCacheWrapper:
    def __init__(self, kv_layout: str = "NHD"):
        self.kv_layout = kv_layout
        self._wrapper = _kernels.BatchDecodeWithPagedKVCachePyTorchWrapper(_layout_code(kv_layout))

    # ---- the reference's protocol -----------------------------------------------------------------
    def begin_forward(self, indptr: torch.Tensor, num_qo_heads: int, num_kv_heads: int, head_dim: int,
                      page_size: int, data_type) -> None:
        """Once per model forward, before the layers.  `indptr` has one entry per sequence plus one
        ([0, budget] for the single sequence of the reference); `data_type` is the cache's dtype, which
        travels as an empty tensor like in the reference's binding.  num_qo_heads may be a multiple of
        num_kv_heads (grouped-query attention)."""
        dtype_carrier = torch.empty(0, dtype=data_type)
        self._wrapper.begin_forward(indptr, num_qo_heads, num_kv_heads, head_dim, page_size, dtype_carrier)

    def end_forward(self) -> None:
        """After the last layer.  The scratch stays allocated for the next forward."""
        self._wrapper.end_forward()

    @contextlib.contextmanager
    def forward_pass(self, indptr: torch.Tensor, num_qo_heads: int, num_kv_heads: int, head_dim: int,
                     page_size: int, data_type) -> Iterator["BatchDecodeWithPagedKVCacheWrapper"]:
        """begin_forward ... end_forward as a context."""
        self.begin_forward(indptr, num_qo_heads, num_kv_heads, head_dim, page_size, data_type)
        try:
            yield self
        finally:
            self.end_forward()

    def forward(self, q: torch.Tensor, o: torch.Tensor, paged_kv_data: torch.Tensor,
                paged_kv_indices: torch.Tensor, paged_kv_indptr: Optional[torch.Tensor],
                paged_kv_last_page_len: int, paged_kv_last_page_idx: int,
                rope_scale: Optional[float] = None, rope_theta: Optional[float] = None, *,
                token_granular: bool = False, lse: Optional[torch.Tensor] = None) -> None:
        """One layer's attention over the listed pages (or, token_granular, token slots) plus the newest
        token.  rope_scale / rope_theta are part of the reference's signature; the rotation itself
        happens in the append, not here."""
        self._wrapper.forward(
            q, o, paged_kv_data, paged_kv_indices, paged_kv_indptr, paged_kv_last_page_len, paged_kv_last_page_idx,
            _DEFAULT_ROPE_SCALE if rope_scale is None else rope_scale,
            _DEFAULT_ROPE_THETA if rope_theta is None else rope_theta,
            token_granular=token_granular, lse=lse)

    # ---- steps with the sequence length in device memory ------------------------------------------
    def dense_step_dev(self, *args, **kwargs) -> None:
        """Append and attention over every token of one sequence
        (_kernels.BatchDecodeWithPagedKVCachePyTorchWrapper.dense_step_dev)."""
        self._wrapper.dense_step_dev(*args, **kwargs)

    def dense_step_batch_dev(self, *args, **kwargs) -> None:
        """The same for several sequences in the same launches (begin_forward with an indptr of batch + 1
        entries first)."""
        self._wrapper.dense_step_batch_dev(*args, **kwargs)
