"""Python face of the decode-attention handler (adamas/utils/decode_wrapper.py)."""
from typing import Optional

import torch

from .. import _kernels
from .utils import TensorLayout


def _check_kv_layout(kv_layout: str):
    if not hasattr(TensorLayout, kv_layout):
        raise KeyError("Invalide kv_layout {}".format(kv_layout))


class BatchDecodeWithPagedKVCacheWrapper:
    """Owns the split plan and the partial-result scratch that are reused by every layer of a
    decode step (begin_forward ... forward x layers ... end_forward)."""

    def __init__(self, kv_layout: str = "NHD"):
        _check_kv_layout(kv_layout)
        self.kv_layout = kv_layout
        self._wrapper = _kernels.BatchDecodeWithPagedKVCachePyTorchWrapper(getattr(TensorLayout, kv_layout))

    def begin_forward(self, indptr: torch.Tensor, num_qo_heads: int, num_kv_heads: int, head_dim: int,
                      page_size: int, data_type):
        empty_data = torch.empty(0, dtype=data_type)   # carries the dtype, as in the reference
        self._wrapper.begin_forward(indptr, num_qo_heads, num_kv_heads, head_dim, page_size, empty_data)

    def end_forward(self):
        self._wrapper.end_forward()

    def forward(self, q: torch.Tensor, o: torch.Tensor, paged_kv_data: torch.Tensor,
                paged_kv_indices: torch.Tensor, paged_kv_indptr: torch.Tensor, paged_kv_last_page_len: int,
                paged_kv_last_page_idx: int, rope_scale: Optional[float] = None,
                rope_theta: Optional[float] = None, token_granular: bool = False,
                lse: Optional[torch.Tensor] = None):
        if rope_scale is None:
            rope_scale = 1.0
        if rope_theta is None:
            rope_theta = 1e4
        self._wrapper.forward(q, o, paged_kv_data, paged_kv_indices, paged_kv_indptr, paged_kv_last_page_len,
                              paged_kv_last_page_idx, rope_scale, rope_theta, token_granular=token_granular,
                              lse=lse)

    def dense_step_dev(self, *args, **kwargs):
        """Dense decode step with the sequence length on the device (see
        _kernels.BatchDecodeWithPagedKVCachePyTorchWrapper.dense_step_dev)."""
        self._wrapper.dense_step_dev(*args, **kwargs)
