"""Several sequences of one cache geometry decoded by the same launches.

The reference serves one sequence per InferenceController and one per model call
(adamas/models/Adamas.py:83 asserts batch size 1); a server that holds several sequences loops over
them.  SequenceBatch keeps the controllers as they are (each sequence owns its caches and page tables)
and adds what a batched step needs: per layer a device array of the sequences' cache addresses, one
array of device-resident lengths, and scratch with one row per (sequence, head).  A step is then
shaped by (batch, max_seq_len) only and can be captured in one CUDA graph for all sequences.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import _kernels
from .controller import InferenceController
from .decode_wrapper import BatchDecodeWithPagedKVCacheWrapper


class SequenceBatch:
    def __init__(self, controllers: Sequence[InferenceController]):
        assert len(controllers) >= 1
        c0 = controllers[0]
        for c in controllers:
            assert (c.num_heads, c.num_q_heads, c.head_dim, c.page_size, c.dtype, c.max_seq_len, c.token_budget()) == \
                   (c0.num_heads, c0.num_q_heads, c0.head_dim, c0.page_size, c0.dtype, c0.max_seq_len, c0.token_budget()), \
                   "the sequences of a batch share one cache geometry, capacity and budget"
        self.controllers: List[InferenceController] = list(controllers)
        self.batch = len(controllers)
        self.device = c0.device
        self.num_heads, self.num_q_heads = c0.num_heads, c0.num_q_heads
        self.page_size, self.max_seq_len, self.dtype = c0.page_size, c0.max_seq_len, c0.dtype
        rows = self.batch * self.num_q_heads
        layers = c0.kv_cache.pool.num_layers
        kv_tables = [c.kv_cache.table_all() for c in controllers]
        code_tables = [c.hadamard_cache.table_all() for c in controllers]
        self._seqs = [_kernels.sequence_descriptors([c.kv_cache.buf_layer(l) for c in controllers],
                                                    [c.hadamard_cache.buf_layer(l) for c in controllers],
                                                    kv_tables, code_tables) for l in range(layers)]
        self.seq_lens = torch.zeros(self.batch, dtype=torch.int32, device=self.device)
        self._q_code = torch.empty(self.batch, self.num_q_heads, c0.head_dim // 8, dtype=self.dtype, device=self.device)
        cap = (self.max_seq_len - 1 + 7) // 8 * 8
        self._dist = torch.empty(rows, cap, dtype=torch.int16, device=self.device)
        self._hist = _kernels.histogram_scratch(rows, self.device)
        self._dense = BatchDecodeWithPagedKVCacheWrapper("NHD")
        self._dense.begin_forward(torch.zeros(self.batch + 1, dtype=torch.int32), self.num_q_heads, self.num_heads,
                                  c0.head_dim, self.page_size, self.dtype)

    def prepare(self, new_tokens: int = 1) -> None:
        """Reserve cache room in every sequence and upload the page numbers of pages opened by that."""
        for c in self.controllers:
            c.prepare_hadamard(new_tokens)
            c.kv_cache.table_all()
            c.hadamard_cache.table_all()

    def sync_seq_lens(self) -> None:
        """seq_lens := the host's lengths (after prepare: the lengths the coming step works on)."""
        self.seq_lens.copy_(torch.tensor([c.kv_cache.seqlen for c in self.controllers], dtype=torch.int32))

    def all_sparse(self) -> bool:
        """Every sequence is longer than the token budget (what the sparse step needs)."""
        return all(c.kv_cache.seqlen > c.token_budget() for c in self.controllers)

    def decode_step_dev(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layer_idx: int,
                        out: Optional[torch.Tensor] = None, dense: bool = False, scale: Optional[float] = None,
                        rope=None, indices_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """utils.decode_step_dev for the whole batch: q [batch, Hq, D], k, v [batch, H, D] -> o [batch, Hq, D]."""
        o = out if out is not None else torch.empty_like(q)
        c0 = self.controllers[0]
        if dense:
            self._dense.dense_step_batch_dev(q, k, v, o, self._q_code, self._seqs[layer_idx], self.seq_lens,
                                                      self.max_seq_len, self.page_size, scale=scale, rope=rope)
            return o
        _kernels.decode_step_batch_dev(q, k, v, o, self._q_code, self._seqs[layer_idx], self.seq_lens,
                                       self.max_seq_len, self.page_size, c0.token_budget(),
                                       self._dist[:, : self.max_seq_len - 1], self._hist, indices_out=indices_out,
                                       scale=scale, rope=rope)
        return o

    def advance(self, delta: int = 1) -> None:
        """Every device-resident length += delta (one capturable launch)."""
        _kernels.seq_len_advance(self.seq_lens, delta)
