"""Paged cache storage for one sequence: the buffer layout and bookkeeping of the reference's
KvPool / KvCache (adamas/utils/kv_cache.py), with the page table additionally mirrored on the
device so that a decode step uploads only the page ids that are new."""
from __future__ import annotations

import heapq

import torch

from .utils import TensorLayout


class KvPool:
    """One buffer [num_layers, capacity, items, block_len, num_heads, head_dim] shared by all
    layers (adamas/utils/kv_cache.py:21-24) and a free list of page numbers.  Pages are handed out
    lowest number first."""

    def __init__(self, num_layers: int, num_heads: int, head_dim: int, capacity: int, items: int,
                 block_len: int, dtype: torch.dtype, device):
        self._layout = TensorLayout.NHD
        self._buf = torch.empty((num_layers, capacity, items, block_len, num_heads, head_dim),
                                dtype=dtype, device=device)
        self._free = list(range(capacity))
        heapq.heapify(self._free)
        self._in_use = set()

    layout = property(lambda self: self._layout)
    buf = property(lambda self: self._buf)
    num_layers = property(lambda self: self._buf.shape[0])
    capacity = property(lambda self: self._buf.shape[1])
    block_len = property(lambda self: self._buf.shape[3])
    num_free_blocks = property(lambda self: len(self._free))

    def alloc_block(self) -> int:
        if not self._free:
            raise RuntimeError("KvPool is out of pages")
        idx = heapq.heappop(self._free)
        self._in_use.add(idx)
        return idx

    def free_block(self, idx: int) -> None:
        assert 0 <= idx < self.capacity
        assert idx in self._in_use
        self._in_use.remove(idx)
        heapq.heappush(self._free, idx)


class KvCache:
    """Key-value (or code) cache of one sequence (adamas/utils/kv_cache.py:66-135)."""

    def __init__(self, num_layers, num_heads, head_dim, max_seq_len: int, page_size, items,
                 dtype: torch.dtype, device):
        if max_seq_len <= 0:
            raise ValueError("init_len must be non-negative")
        self._pool = KvPool(num_layers=num_layers, num_heads=num_heads, head_dim=head_dim,
                            capacity=(max_seq_len + page_size - 1) // page_size, items=items,
                            block_len=page_size, dtype=dtype, device=device)
        self._indicies = []
        self._seqlen = 0
        self._table = torch.zeros(self._pool.capacity, dtype=torch.int32, device=device)
        # host mirror of the table; pinned when the table lives on a GPU, so that new entries travel
        # with an asynchronous copy (a copy from pageable memory would wait for the stream to drain,
        # i.e. for the decode steps already queued, every time a sequence grows by a page)
        self._host_table = torch.zeros(self._pool.capacity, dtype=torch.int32)
        if self._table.is_cuda:
            self._host_table = self._host_table.pin_memory()
        self._uploaded = 0

    pool = property(lambda self: self._pool)
    seqlen = property(lambda self: self._seqlen)
    indicies = property(lambda self: self._indicies)

    @property
    def last_page_len(self) -> int:
        return (self._seqlen - 1) % self._pool.block_len + 1

    def buf_layer(self, layer_idx: int) -> torch.Tensor:
        assert layer_idx < self._pool.num_layers
        return self._pool.buf[layer_idx]

    def append_seq(self, seq_len: int) -> int:
        """Reserve room for seq_len more tokens; returns the number of pages added."""
        if seq_len <= 0:
            return 0
        block = self._pool.block_len
        need = (self._seqlen + seq_len + block - 1) // block
        added = need - len(self._indicies)
        for _ in range(added):
            self._indicies.append(self._pool.alloc_block())
        self._seqlen += seq_len
        return added

    def table_device(self) -> torch.Tensor:
        """int32 device tensor [num_pages] of physical page numbers, in logical order (a view of a
        persistent buffer; only entries added since the last call are copied to the device)."""
        n = len(self._indicies)
        if self._uploaded < n:
            # every entry of the mirror is written once, before the copy that reads it is queued
            self._host_table[self._uploaded:n] = torch.tensor(self._indicies[self._uploaded:n], dtype=torch.int32)
            self._table[self._uploaded:n].copy_(self._host_table[self._uploaded:n], non_blocking=True)
            self._uploaded = n
        return self._table[:n]

    def table_all(self) -> torch.Tensor:
        """The whole persistent table buffer (capacity entries; entries beyond the current page count
        are not meaningful), after uploading any new entries: what a kernel that takes the sequence
        length from device memory indexes."""
        self.table_device()
        return self._table

    def release(self) -> None:
        """Give all pages back."""
        self._seqlen = 0
        for idx in self._indicies:
            self._pool.free_block(idx)
        self._indicies.clear()
        if self._table.is_cuda and self._uploaded:
            torch.cuda.current_stream(self._table.device).synchronize()   # copies out of the mirror have landed
        self._uploaded = 0
